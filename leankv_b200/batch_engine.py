"""Batched long-context decode on the TurboQuant paged pool.

B sequences advance one token per step. At batch > 1 the reference runs its projections dense
(``leankv/teal/patching.py:155-157`` — TEAL's gather only pays at one row), so the projections
here are library GEMMs over the same ``[in][out]`` weights; what this module adds is the KV side:
every sequence's K/V go through rotate + 3-bit quantize + pack on append and attention runs on
the packed pages of all sequences in one launch (``leankv/turboquant/cache.py:102-189`` without
ever forming the fp16 copy). Sequences are independent, so a multi-GPU run gives each rank its
own slice of the batch and needs no collective.

Positions, the per-sequence block table and the flat page table live on the device; one step is
captured in a CUDA graph.
"""

from __future__ import annotations

import math
from typing import Optional, Sequence

import torch

from . import _native
from .engine import PAGE, DecodeEngine, DecoderConfig


class BatchDecodeEngine(DecodeEngine):
    """Full (unsharded) weights + a paged 3-bit pool shared by ``batch`` sequences."""

    def __init__(self, cfg: DecoderConfig, weights: dict, device, batch: int, max_seq_len: int = 4352,
                 tq_seed: int = 42):
        # single-sequence buffers of the parent are not needed: build the shared parts by hand
        if cfg.head_dim != 128 or cfg.num_q_heads != 4 * cfg.num_kv_heads:
            raise RuntimeError("BatchDecodeEngine needs head_dim 128 and 4 query heads per kv head")
        if batch < 1:
            raise ValueError("batch must be >= 1")
        from .turboquant.codebook import get_codebook_tensors
        from .turboquant.rotation import generate_rotation_matrix

        self.cfg, self.dev = cfg, torch.device(device)
        self.tp_rank, self.tp_size, self.group = 0, 1, None
        self.xchg = None
        self.lib = _native.lib()
        self.nq, self.nkv, self.inter = cfg.num_q_heads, cfg.num_kv_heads, cfg.intermediate_size
        self.n_qkv = (self.nq + 2 * self.nkv) * 128
        self.B = batch
        self.max_seq_len = max_seq_len
        self.pps = (max_seq_len + PAGE - 1) // PAGE          # pages per sequence
        self.max_pages = self.pps * batch                    # pages in each layer's pool
        L, dev, H = cfg.num_layers, self.dev, cfg.hidden_size

        # gate and up as one [H][2I] matrix so the MLP's first half is a single GEMM
        self.w = weights
        for lw in weights["layers"]:
            if "wgu_t" not in lw:
                lw["wgu_t"] = torch.cat([lw["wgate_t"], lw["wup_t"]], dim=1).contiguous()
                lw["wgate_t"], lw["wup_t"] = lw["wgu_t"][:, :self.inter], lw["wgu_t"][:, self.inter:]

        self.Pi_k = [generate_rotation_matrix(128, dev, torch.float32, tq_seed + 2 * l).contiguous() for l in range(L)]
        self.Pi_v = [generate_rotation_matrix(128, dev, torch.float32, tq_seed + 2 * l + 1).contiguous() for l in range(L)]
        self.Pi_k_t = [m.t().contiguous() for m in self.Pi_k]
        self.Pi_v_t = [m.t().contiguous() for m in self.Pi_v]
        cents, bounds = get_codebook_tensors(128, 3, "cpu")
        self.centroids_host = cents.float().contiguous()
        self._prefill_ws = None
        self.centroids = self.centroids_host.to(dev)
        self.bounds = bounds[1:-1].float().contiguous().to(dev)

        self.pools = [torch.zeros(self.max_pages, 2, self.nkv, _native.TQ_CHUNK_BYTES, dtype=torch.uint8,
                                  device=dev) for _ in range(L)]
        # every sequence owns pps pages, scattered over the pool
        perm = torch.randperm(self.max_pages, generator=torch.Generator().manual_seed(tq_seed))
        self.block_table = perm.to(torch.int32).reshape(batch, self.pps).contiguous().to(dev)

        i32 = lambda n: torch.zeros(n, dtype=torch.int32, device=dev)
        self.pos, self.steps = i32(batch), i32(batch)
        self.kv_indptr, self.kv_page_indices, self.kv_last = i32(batch + 1), i32(self.max_pages), i32(batch)
        half = lambda *s: torch.zeros(*s, dtype=torch.float16, device=dev)
        self.h, self.x = half(batch, H), half(batch, H)
        self.qkv, self.attn, self.o = half(batch, self.n_qkv), half(batch, self.nq * 128), half(batch, H)
        self.q_rot = torch.zeros(batch, self.nq, 128, dtype=torch.float32, device=dev)
        self.gate_up, self.mlp_h, self.down = half(batch, 2 * self.inter), half(batch, self.inter), half(batch, H)
        self.logits = half(batch, cfg.vocab_size)
        self.tokens = torch.zeros(batch, dtype=torch.int64, device=dev)
        self.history_cap = max_seq_len + 8
        self.history = torch.zeros(batch, self.history_cap, dtype=torch.int64, device=dev)
        self.inv_freq = (1.0 / (cfg.rope_theta ** (torch.arange(0, 128, 2, dtype=torch.int64).float() / 128))
                         ).to(dev).contiguous()
        with torch.cuda.device(dev):
            need = self.lib.leankv_tq_decode_attn_workspace_bytes(batch, self.nq, self.nkv, self.pps)
            self.ws_attn = torch.zeros(need + 256, dtype=torch.uint8, device=dev)
        self.graph = None
        self.launches_per_step = 0       # kernels of this library
        self.gemms_per_step = 0          # library GEMMs

    @classmethod
    def random_init(cls, cfg: DecoderConfig, device, batch: int, seed: int = 0, **kw) -> "BatchDecodeEngine":
        dev = torch.device(device)
        return cls(cfg, DecodeEngine.random_weights(cfg, dev, seed), dev, batch, **kw)

    # ── one step ─────────────────────────────────────────────────────────

    def _mm(self, a, w, out):
        torch.matmul(a, w, out=out)
        self.gemms_per_step += 1

    def _norm_rows(self, delta, w):
        rc = self.lib.leankv_rmsnorm_rows_f16(self.h.data_ptr(), _native.ptr(delta), w.data_ptr(),
                                              self.x.data_ptr(), self.B, self.cfg.hidden_size, self.cfg.rms_eps,
                                              self._st())
        _native.check(rc, "rmsnorm_rows")
        self.launches_per_step += 1

    def _step_launches(self) -> None:
        cfg, lib, st, B = self.cfg, self.lib, self._st, self.B
        self.launches_per_step = self.gemms_per_step = 0
        _native.check(lib.leankv_batch_decode_begin(
            self.w["embed"].data_ptr(), self.tokens.data_ptr(), self.h.data_ptr(), cfg.hidden_size, cfg.vocab_size,
            B, self.pos.data_ptr(), self.block_table.data_ptr(), self.pps, self.kv_indptr.data_ptr(),
            self.kv_page_indices.data_ptr(), self.kv_last.data_ptr(), st()), "batch_decode_begin")
        self.launches_per_step += 1
        self._norm_rows(None, self.w["layers"][0]["ln1"])
        for l, lw in enumerate(self.w["layers"]):
            self._mm(self.x, lw["wqkv_t"], self.qkv)
            _native.check(lib.leankv_batch_qkv_post(
                self.qkv.data_ptr(), B, self.inv_freq.data_ptr(), self.pos.data_ptr(), self.kv_indptr.data_ptr(),
                self.Pi_k_t[l].data_ptr(), self.Pi_v_t[l].data_ptr(), self.bounds.data_ptr(),
                self.pools[l].data_ptr(), self.max_pages, self.kv_page_indices.data_ptr(), self.nq, self.nkv,
                self.q_rot.data_ptr(), st()), "batch_qkv_post")
            _native.check(lib.leankv_tq_decode_attn_rotated(
                self.q_rot.data_ptr(), self.attn.data_ptr(), B, self.nq, self.nkv, self.pools[l].data_ptr(),
                self.max_pages, self.kv_indptr.data_ptr(), self.kv_page_indices.data_ptr(),
                self.kv_last.data_ptr(), self.pps, self.Pi_v[l].data_ptr(), self.centroids_host.data_ptr(),
                1.0 / math.sqrt(128.0), self.ws_attn.data_ptr(), self.ws_attn.numel(), _native.ATTN_EARLY_FETCH,
                st()), "decode_attn_rotated")
            self.launches_per_step += 2
            self._mm(self.attn, lw["wo_t"], self.o)
            self._norm_rows(self.o, lw["ln2"])                       # h += o ; x = norm(h)
            self._mm(self.x, lw["wgu_t"], self.gate_up)
            _native.check(lib.leankv_silu_mul_f16(self.gate_up.data_ptr(), self.mlp_h.data_ptr(), B, self.inter,
                                                  st()), "silu_mul")
            self.launches_per_step += 1
            self._mm(self.mlp_h, lw["wdown_t"], self.down)
            nxt = self.w["layers"][l + 1]["ln1"] if l + 1 < cfg.num_layers else self.w["final_norm"]
            self._norm_rows(self.down, nxt)                          # h += down ; x = norm(h)
        self._mm(self.x, self.w["lm_head_t"], self.logits)
        _native.check(lib.leankv_batch_decode_end(self.logits.data_ptr(), cfg.vocab_size, B, self.tokens.data_ptr(),
                                                  self.history.data_ptr(), self.history_cap, self.pos.data_ptr(),
                                                  self.steps.data_ptr(), st()), "batch_decode_end")
        self.launches_per_step += 1

    def capture(self) -> None:
        with torch.cuda.device(self.dev):
            snap = (self.pos.clone(), self.steps.clone(), self.tokens.clone(), self.history.clone())
            # the throw-away warm-up step overwrites one slot per sequence in every pool: keep those pages
            touched = self.block_table.gather(1, (self.pos // PAGE).clamp(max=self.pps - 1).long().unsqueeze(1))
            touched = touched.reshape(-1).long()
            saved = [p[touched].clone() for p in self.pools]
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                self._step_launches()
            torch.cuda.current_stream().wait_stream(side)
            torch.cuda.synchronize()
            self.pos.copy_(snap[0]); self.steps.copy_(snap[1]); self.tokens.copy_(snap[2]); self.history.copy_(snap[3])
            for p, s in zip(self.pools, saved):
                p[touched] = s
            self.graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(self.graph, capture_error_mode="thread_local"):
                self._step_launches()

    # ── prefill / generate ───────────────────────────────────────────────

    @torch.no_grad()
    def prefill(self, prompts, attention: str = "packed", chunk: Optional[int] = None) -> torch.Tensor:
        """``prompts``: int64 [B][T] (equal lengths). Fills every sequence's pages with a prompt pass
        (library GEMMs, one sequence at a time, ``chunk`` tokens per pass) and leaves the first generated
        token of each ready for ``step``. ``attention``: "packed" = causal attention on the packed pages,
        "dense" = de-quantize + library attention (whole prompt per pass only); see
        ``DecodeEngine.prefill``."""
        ids = torch.as_tensor(prompts, device=self.dev)
        if ids.dim() != 2 or ids.shape[0] != self.B:
            raise ValueError("prompts must be [batch][T]")
        T = ids.shape[1]
        if T < 1 or T >= self.max_seq_len:
            raise ValueError("prompt length must be in [1, max_seq_len)")
        if chunk is None:
            chunk = T
        if chunk < 1 or (attention == "dense" and chunk < T):
            raise ValueError("chunk must be positive; the dense route handles whole prompts only")
        with torch.cuda.device(self.dev):
            for p in self.pools:
                p.zero_()
            last = []
            for b in range(self.B):
                for s0 in range(0, T, chunk):
                    x = self._dense_forward(ids[b, s0:s0 + chunk], write_cache=True,
                                            page_indices=self.block_table[b], start_pos=s0, attention=attention)
                last.append(x)
            if attention == "packed":
                self._check_prefill_status()
            logits = torch.stack(last) @ self.w["lm_head_t"]
            tok = torch.argmax(logits.float(), dim=-1)
            self.tokens.copy_(tok)
            self.history.zero_()
            self.history[:, 0] = tok
            self.pos.fill_(T)
            self.steps.fill_(1)
            self.prefill_logits = logits
        return tok

    @torch.no_grad()
    def generate(self, prompts, max_new_tokens: int) -> torch.Tensor:
        """Greedy generation for the whole batch; returns int64 [B][max_new_tokens]."""
        self.prefill(prompts)
        n_steps = max(min(max_new_tokens - 1, self.max_seq_len - int(self.pos[0]) - 1), 0)
        with torch.cuda.device(self.dev):
            for _ in range(n_steps):
                self.step()
            self.check_status()
        return self.history[:, :1 + n_steps].clone()

    def kv_bytes_per_sequence(self, n_tokens: int) -> int:
        """Pool bytes one sequence of ``n_tokens`` occupies: whole pages, K and V, every layer and kv head."""
        return ((n_tokens + PAGE - 1) // PAGE) * 2 * self.cfg.num_layers * self.nkv * _native.TQ_CHUNK_BYTES


def partition_batch(total: int, world_size: int, rank: int) -> range:
    """The sequences rank ``rank`` serves when ``total`` independent sequences are split over
    ``world_size`` ranks: contiguous, sizes differing by at most one, no sequence on two ranks."""
    if not 0 <= rank < world_size:
        raise ValueError("rank out of range")
    base, extra = divmod(total, world_size)
    start = rank * base + min(rank, extra)
    return range(start, start + base + (1 if rank < extra else 0))
