"""Batch-1 decode loop for Llama/Mistral-shaped models on the two leankv hot paths.

The reference speeds up HuggingFace ``generate`` by patching seven projections per block
(TEAL) and swapping the KV cache (TurboQuant); everything between those two hooks stays
HF Python. At B200 speeds a 7B decode step is ~1 ms, so this module drives the same block
structure directly: every projection is a sparse GEMV launch (q/k/v fused into one launch,
gate/up fused with SiLU), K/V are rotated+quantized+packed on append, attention runs on the
packed pages, and one whole step — including position / page-table bookkeeping and the
greedy argmax — is captured in a CUDA graph and replayed per token. Tensor parallelism
splits q/k/v/gate/up by output columns and o/down by input rows; the two sums per block are taken
inside the row-parallel GEMV kernels over peer memory (``LEANKV_TP_EXCHANGE=nccl`` selects a separate
NCCL all-reduce launch after o_proj and down_proj instead).

Under tensor parallelism the output head is split over the vocabulary and the ranks exchange their
arg-max inside the step's last kernel.

Prefill (prompt processing) uses dense projections, like the reference's kernel mode
(``leankv/teal/patching.py:178-180``: library GEMMs), whole or in chunks; every chunk is quantized
into the pool first and its causal attention then runs on the packed pages
(``leankv_tq_prefill_attn``), so no fp16 copy of the sequence is ever formed. ``attention="dense"``
keeps the reference's route (de-quantize + library attention).
"""

from __future__ import annotations

import ctypes
import math
import os
from dataclasses import dataclass
from typing import Optional

import torch
import torch.nn.functional as F

from . import _native
from .teal.sparse_fns import compute_threshold_for_sparsity
from .turboquant.codebook import get_codebook_tensors
from .turboquant.rotation import generate_rotation_matrix

PROJ_NAMES = ["q_proj", "k_proj", "v_proj", "o_proj", "gate_proj", "up_proj", "down_proj"]
PAGE = _native.TQ_PAGE_TOKENS


@dataclass
class DecoderConfig:
    vocab_size: int = 32768
    hidden_size: int = 4096
    intermediate_size: int = 14336
    num_layers: int = 32
    num_q_heads: int = 32
    num_kv_heads: int = 8
    head_dim: int = 128
    rope_theta: float = 1e6
    rms_eps: float = 1e-5

    @classmethod
    def mistral_7b(cls) -> "DecoderConfig":
        """Mistral-7B-v0.3 architecture."""
        return cls()

    @classmethod
    def llama3_8b(cls) -> "DecoderConfig":
        return cls(vocab_size=128256, rope_theta=5e5)

    @classmethod
    def from_hf(cls, c) -> "DecoderConfig":
        return cls(vocab_size=c.vocab_size, hidden_size=c.hidden_size,
                   intermediate_size=c.intermediate_size, num_layers=c.num_hidden_layers,
                   num_q_heads=c.num_attention_heads,
                   num_kv_heads=getattr(c, "num_key_value_heads", c.num_attention_heads),
                   head_dim=getattr(c, "head_dim", None) or c.hidden_size // c.num_attention_heads,
                   rope_theta=float(getattr(c, "rope_theta", None)
                                    or (getattr(c, "rope_parameters", None) or {}).get("rope_theta", 1e4)),
                   rms_eps=c.rms_norm_eps)


def _rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    xf = x.float()
    return w * (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)).to(x.dtype)


def _rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """x [T, H, 128]; cos/sin [T, 1, 128] in x.dtype; rotate_half form."""
    half = x.shape[-1] // 2
    rot = torch.cat((-x[..., half:], x[..., :half]), dim=-1)
    return x * cos + rot * sin


class DecodeEngine:
    """Owns the (sharded) weights in kernel layout, the paged 3-bit KV pool and the step graph."""

    def __init__(self, cfg: DecoderConfig, weights: dict, device, max_seq_len: int = 1024,
                 thresholds: Optional[dict] = None, tp_rank: int = 0, tp_size: int = 1, group=None,
                 tq_seed: int = 42):
        if cfg.head_dim != 128 or cfg.num_q_heads != 4 * cfg.num_kv_heads:
            raise RuntimeError("DecodeEngine needs head_dim 128 and 4 query heads per kv head")
        if cfg.num_kv_heads % tp_size or cfg.intermediate_size % (8 * tp_size):
            raise RuntimeError("tensor-parallel size must divide the kv heads and intermediate size")
        self.cfg, self.dev = cfg, torch.device(device)
        self.tp_rank, self.tp_size, self.group = tp_rank, tp_size, group
        self.w = weights
        self.lib = _native.lib()
        self.nq = cfg.num_q_heads // tp_size
        self.nkv = cfg.num_kv_heads // tp_size
        self.inter = cfg.intermediate_size // tp_size
        self.n_qkv = (self.nq + 2 * self.nkv) * 128
        self.max_seq_len = max_seq_len
        self.max_pages = (max_seq_len + PAGE - 1) // PAGE
        L, dev = cfg.num_layers, self.dev

        # per-layer rotations: seed + 2l for K, seed + 2l + 1 for V (leankv/turboquant/cache.py:59-71)
        self.Pi_k = [generate_rotation_matrix(128, dev, torch.float32, tq_seed + 2 * l).contiguous() for l in range(L)]
        self.Pi_v = [generate_rotation_matrix(128, dev, torch.float32, tq_seed + 2 * l + 1).contiguous() for l in range(L)]
        self.Pi_k_t = [m.t().contiguous() for m in self.Pi_k]
        self.Pi_v_t = [m.t().contiguous() for m in self.Pi_v]
        cents, bounds = get_codebook_tensors(128, 3, "cpu")
        self.centroids_host = cents.float().contiguous()
        self._prefill_ws = None
        self.centroids = self.centroids_host.to(dev)
        self.bounds = bounds[1:-1].float().contiguous().to(dev)

        # paged pool, one tensor per layer; the sequence's pages are assigned up front in a
        # shuffled order so that the page table is exercised
        self.pools = [torch.zeros(self.max_pages, 2, self.nkv, _native.TQ_CHUNK_BYTES, dtype=torch.uint8,
                                  device=dev) for _ in range(L)]
        perm = torch.randperm(self.max_pages, generator=torch.Generator().manual_seed(tq_seed))
        self.page_indices = perm.to(torch.int32).to(dev)

        half = lambda n: torch.zeros(n, dtype=torch.float16, device=dev)
        self.h, self.x, self.h2 = half(cfg.hidden_size), half(cfg.hidden_size), half(cfg.hidden_size)
        self.qkv, self.q_rope, self.k_rope = half(self.n_qkv), half(self.nq * 128), half(self.nkv * 128)
        self.attn, self.o = half(self.nq * 128), half(cfg.hidden_size)
        self.q_rot = torch.zeros(self.nq * 128, dtype=torch.float32, device=dev)
        self.fused_post = True   # False: rope / append / query rotation as separate launches
        self.fused_norm = True   # False: RMSNorm + residual add as launches of their own
        self.mlp_h, self.down = half(self.inter), half(cfg.hidden_size)
        self.logits = half(cfg.vocab_size)
        self.token = torch.zeros(1, dtype=torch.int64, device=dev)
        self.history_cap = max_seq_len + 8
        self.history = torch.zeros(self.history_cap, dtype=torch.int64, device=dev)
        self.state = torch.zeros(8, dtype=torch.int32, device=dev)
        self.active_elems = torch.zeros(1, dtype=torch.int64, device=dev)
        self.inv_freq = (1.0 / (cfg.rope_theta ** (torch.arange(0, 128, 2, dtype=torch.int64).float() / 128))
                         ).to(dev).contiguous()

        shapes = [(self.n_qkv, cfg.hidden_size), (cfg.hidden_size, self.nq * 128),
                  (cfg.hidden_size, self.inter), (cfg.vocab_size, cfg.hidden_size)]
        with torch.cuda.device(dev):
            need = max(self.lib.leankv_sparse_gemv_workspace_bytes(n, z) for n, z in shapes)
            need = max(need, self.lib.leankv_sparse_swiglu_workspace_bytes(self.inter, cfg.hidden_size))
            self.ws_gemv = torch.zeros(need + 256, dtype=torch.uint8, device=dev)
            need = self.lib.leankv_tq_decode_attn_workspace_bytes(1, self.nq, self.nkv, self.max_pages)
            self.ws_attn = torch.zeros(need + 256, dtype=torch.uint8, device=dev)
        # Tensor parallel: the o / down projections sum their partial products over peer memory inside
        # the GEMV kernel (LEANKV_TP_EXCHANGE=nccl keeps a separate NCCL all-reduce launch instead).
        self.xchg = None
        if tp_size > 1 and os.environ.get("LEANKV_TP_EXCHANGE", "peer") != "nccl":
            from .peer_exchange import PeerExchange

            self.xchg = PeerExchange(dev, tp_rank, tp_size, group, n_slots=2 * L + 1, max_cols=cfg.hidden_size)
        # Output head split over the vocabulary (needs the peer exchange for the arg-max): the decode step
        # streams 1 / tp_size of it and the ranks exchange {best value, index}. The full matrix stays for the
        # prompt pass and the parity references.
        self.lm_head_local = None
        if self.xchg is not None and cfg.vocab_size % (8 * tp_size) == 0 and \
                os.environ.get("LEANKV_TP_LM_HEAD", "sharded") != "replicated":
            vl = cfg.vocab_size // tp_size
            self.vocab_local, self.vocab_offset = vl, tp_rank * vl
            self.lm_head_local = self.w["lm_head_t"][:, self.vocab_offset:self.vocab_offset + vl].contiguous()
        self.set_thresholds(thresholds)
        self.graph = None
        self.launches_per_step = 0
        self._pinned_token = torch.zeros(1, dtype=torch.int64).pin_memory() if torch.cuda.is_available() else None
        self._pinned_status = torch.zeros(2, dtype=torch.int32).pin_memory() if torch.cuda.is_available() else None

    # ── construction helpers ─────────────────────────────────────────────

    @staticmethod
    def shard_weights(full: dict, cfg: DecoderConfig, tp_rank: int, tp_size: int) -> dict:
        """Slice HF-layout weights ([out, in] per projection) for one rank and lay them out for the kernels."""
        nq, nkv, it = cfg.num_q_heads // tp_size, cfg.num_kv_heads // tp_size, cfg.intermediate_size // tp_size
        qs, ks, ms = slice(tp_rank * nq * 128, (tp_rank + 1) * nq * 128), \
            slice(tp_rank * nkv * 128, (tp_rank + 1) * nkv * 128), slice(tp_rank * it, (tp_rank + 1) * it)
        out = {"embed": full["embed"].contiguous(), "final_norm": full["final_norm"].contiguous(),
               "lm_head_t": full["lm_head"].t().contiguous(), "layers": []}
        for lw in full["layers"]:
            qkv = torch.cat([lw["q_proj"][qs], lw["k_proj"][ks], lw["v_proj"][ks]], dim=0)
            out["layers"].append({
                "ln1": lw["ln1"].contiguous(), "ln2": lw["ln2"].contiguous(),
                "wqkv_t": qkv.t().contiguous(),                       # [hidden][q|k|v columns]
                "wo_t": lw["o_proj"][:, qs].t().contiguous(),         # [local q dims][hidden]
                "wgate_t": lw["gate_proj"][ms].t().contiguous(),
                "wup_t": lw["up_proj"][ms].t().contiguous(),
                "wdown_t": lw["down_proj"][:, ms].t().contiguous(),   # [local inter][hidden]
            })
        return out

    @classmethod
    def from_hf(cls, model, **kw) -> "DecodeEngine":
        """Build from a HuggingFace Llama/Mistral ``*ForCausalLM`` (weights are copied and re-laid out)."""
        cfg = DecoderConfig.from_hf(model.config)
        full = {"embed": model.model.embed_tokens.weight.data.half(),
                "final_norm": model.model.norm.weight.data.half(),
                "lm_head": model.lm_head.weight.data.half(), "layers": []}
        for layer in model.model.layers:
            lw = {"ln1": layer.input_layernorm.weight.data.half(),
                  "ln2": layer.post_attention_layernorm.weight.data.half()}
            for p in PROJ_NAMES:
                parent = layer.self_attn if p in ("q_proj", "k_proj", "v_proj", "o_proj") else layer.mlp
                lw[p] = getattr(parent, p).weight.data.half()
            full["layers"].append(lw)
        tp_rank, tp_size = kw.get("tp_rank", 0), kw.get("tp_size", 1)
        device = kw.pop("device", model.device)
        return cls(cfg, cls.shard_weights(full, cfg, tp_rank, tp_size), device, **kw)

    @classmethod
    def random_init(cls, cfg: DecoderConfig, device, seed: int = 0, tp_rank: int = 0, tp_size: int = 1,
                    **kw) -> "DecodeEngine":
        """Random fp16 weights ~ N(0, 0.02) generated on the device directly in kernel layout.

        Every rank draws the full-size tensor of each projection from the same seeded stream and
        keeps its slice, so that the sharded model equals the single-GPU one.
        """
        dev = torch.device(device)
        return cls(cfg, cls.random_weights(cfg, dev, seed, tp_rank, tp_size), dev, tp_rank=tp_rank,
                   tp_size=tp_size, **kw)

    @staticmethod
    def random_weights(cfg: DecoderConfig, dev, seed: int = 0, tp_rank: int = 0, tp_size: int = 1) -> dict:
        """The weight dict of ``random_init`` (kernel layout, this rank's slices)."""
        gen = torch.Generator(device=dev).manual_seed(seed)
        nq, nkv, it = cfg.num_q_heads // tp_size, cfg.num_kv_heads // tp_size, cfg.intermediate_size // tp_size
        H = cfg.hidden_size

        def draw(rows, cols):
            return (torch.randn(rows, cols, generator=gen, device=dev, dtype=torch.float32) * 0.02).half()

        def cols(t, start, n):
            return t[:, start:start + n]

        w = {"embed": draw(cfg.vocab_size, H), "lm_head_t": draw(H, cfg.vocab_size),
             "final_norm": torch.ones(H, dtype=torch.float16, device=dev), "layers": []}
        for _ in range(cfg.num_layers):
            q_t, k_t, v_t = draw(H, cfg.num_q_heads * 128), draw(H, cfg.num_kv_heads * 128), draw(H, cfg.num_kv_heads * 128)
            wqkv_t = torch.cat([cols(q_t, tp_rank * nq * 128, nq * 128), cols(k_t, tp_rank * nkv * 128, nkv * 128),
                                cols(v_t, tp_rank * nkv * 128, nkv * 128)], dim=1).contiguous()
            del q_t, k_t, v_t
            o_t = draw(cfg.num_q_heads * 128, H)
            g_t, u_t = draw(H, cfg.intermediate_size), draw(H, cfg.intermediate_size)
            d_t = draw(cfg.intermediate_size, H)
            w["layers"].append({
                "ln1": torch.ones(H, dtype=torch.float16, device=dev),
                "ln2": torch.ones(H, dtype=torch.float16, device=dev),
                "wqkv_t": wqkv_t,
                "wo_t": o_t[tp_rank * nq * 128:(tp_rank + 1) * nq * 128].contiguous(),
                "wgate_t": cols(g_t, tp_rank * it, it).contiguous(),
                "wup_t": cols(u_t, tp_rank * it, it).contiguous(),
                "wdown_t": d_t[tp_rank * it:(tp_rank + 1) * it].contiguous(),
            })
            del o_t, g_t, u_t, d_t
        return w

    # ── thresholds ───────────────────────────────────────────────────────

    def set_thresholds(self, thresholds: Optional[dict]) -> None:
        """``{layer: {proj_name: t}}`` as ``apply_teal`` takes it; missing entries / None = dense (t < 0)."""
        self.thresholds = []
        for l in range(self.cfg.num_layers):
            src = (thresholds or {}).get(l, {})
            t = {p: float(src.get(p, 0.0)) for p in PROJ_NAMES}
            # t <= 0 disables TEAL for that projection in the reference; -1 keeps exact zeros too
            self.thresholds.append({p: (v if v > 0 else -1.0) for p, v in t.items()})
        self.graph = None

    def _qkv_segments(self, l: int) -> _native.Segments:
        t = self.thresholds[l]
        segs = _native.Segments()
        ends = (self.nq * 128, (self.nq + self.nkv) * 128, self.n_qkv)
        if t["q_proj"] == t["k_proj"] == t["v_proj"]:
            segs.n_segments = 1
            segs.seg_end[0], segs.threshold[0] = self.n_qkv, t["q_proj"]
        elif ends[0] % 256 == 0 and ends[1] % 256 == 0:
            segs.n_segments = 3
            for i, p in enumerate(("q_proj", "k_proj", "v_proj")):
                segs.seg_end[i], segs.threshold[i] = ends[i], t[p]
        else:
            raise RuntimeError("distinct q/k/v thresholds need 256-aligned projection widths on this rank")
        return segs

    # ── kernel launches (all on the current stream) ──────────────────────

    def _st(self) -> int:
        return torch.cuda.current_stream().cuda_stream

    def _gemv(self, wt, x, y, t, segs=None, residual=None, norm_w=None):
        """y = [residual +] Wt^T . mask_t(x); with ``norm_w`` the kernel first applies RMSNorm(x; norm_w)."""
        z, n = wt.shape
        if segs is None:
            segs = _native.Segments()
            segs.n_segments = 1
            segs.seg_end[0], segs.threshold[0] = n, t
        if norm_w is not None:
            rc = self.lib.leankv_sparse_gemv_rmsnorm_f16(wt.data_ptr(), x.data_ptr(), norm_w.data_ptr(),
                                                         self.cfg.rms_eps, y.data_ptr(), n, z, ctypes.byref(segs),
                                                         _native.ptr(residual), self.ws_gemv.data_ptr(),
                                                         self.ws_gemv.numel(), self.active_elems.data_ptr(),
                                                         self._st())
        else:
            rc = self.lib.leankv_sparse_gemv_seg_f16(wt.data_ptr(), x.data_ptr(), y.data_ptr(), n, z,
                                                     ctypes.byref(segs), None, _native.ptr(residual),
                                                     self.ws_gemv.data_ptr(), self.ws_gemv.numel(),
                                                     self.active_elems.data_ptr(), self._st())
        _native.check(rc, "sparse gemv")
        self.launches_per_step += 1

    def _gemv_allreduce(self, wt, x, y, t, residual, slot):
        """y = residual + sum over ranks of Wt_r^T . mask_t(x_r): GEMV and exchange in one kernel."""
        z, n = wt.shape
        rc = self.lib.leankv_sparse_gemv_allreduce_f16(wt.data_ptr(), x.data_ptr(), y.data_ptr(), n, z, t,
                                                       _native.ptr(residual), self.ws_gemv.data_ptr(),
                                                       self.ws_gemv.numel(), self.active_elems.data_ptr(),
                                                       ctypes.byref(self.xchg.c), slot, self._st())
        _native.check(rc, "sparse gemv + all-reduce")
        self.launches_per_step += 1

    def _norm(self, delta, w):
        rc = self.lib.leankv_rmsnorm_f16(self.h.data_ptr(), _native.ptr(delta), w.data_ptr(), self.x.data_ptr(),
                                         self.cfg.hidden_size, self.cfg.rms_eps, self._st())
        _native.check(rc, "rmsnorm")
        self.launches_per_step += 1

    def _allreduce(self, t):
        if self.tp_size > 1:
            torch.distributed.all_reduce(t, group=self.group)
            self.launches_per_step += 1

    def _layer_launches(self, l: int, probe=None) -> None:
        """Block ``l`` of one decode step: expects ``self.x`` = input-normed hidden state and the decode
        state words set; leaves the residual stream in ``self.h`` and the next norm's output in ``self.x``.
        ``probe(stage)`` (eager debugging / tests only) is called after each stage's launch with the name
        of the buffer that stage just wrote: "qkv", "attn", "o", "x", "mlp_h", "down"."""
        probe = probe or (lambda stage: None)
        cfg, lib, st = self.cfg, self.lib, self._st
        sp = self.state.data_ptr()
        lw, t = self.w["layers"][l], self.thresholds[l]
        fused_norm = self.fused_norm
        if fused_norm:   # RMSNorm of the residual stream happens inside the projection kernels
            self._gemv(lw["wqkv_t"], self.h, self.qkv, 0.0, self._qkv_segments(l), norm_w=lw["ln1"])
        else:
            self._gemv(lw["wqkv_t"], self.x, self.qkv, 0.0, self._qkv_segments(l))
        probe("qkv")
        if self.fused_post:
            # rope(q, k) + rotate/quantize/pack of k, v into the page + query rotation: one launch
            _native.check(lib.leankv_decode_qkv_post(self.qkv.data_ptr(), self.inv_freq.data_ptr(), sp,
                                                     self.Pi_k_t[l].data_ptr(), self.Pi_v_t[l].data_ptr(),
                                                     self.bounds.data_ptr(), self.pools[l].data_ptr(),
                                                     self.max_pages, self.page_indices.data_ptr(), self.nq,
                                                     self.nkv, self.q_rot.data_ptr(), st()), "decode_qkv_post")
            _native.check(lib.leankv_tq_decode_attn_rotated(
                self.q_rot.data_ptr(), self.attn.data_ptr(), 1, self.nq, self.nkv, self.pools[l].data_ptr(),
                self.max_pages, sp + 8, self.page_indices.data_ptr(), sp + 16, self.max_pages,
                self.Pi_v[l].data_ptr(), self.centroids_host.data_ptr(), 1.0 / math.sqrt(128.0),
                self.ws_attn.data_ptr(), self.ws_attn.numel(), _native.ATTN_EARLY_FETCH, st()), "decode_attn_rotated")
            self.launches_per_step += 2
        else:
            _native.check(lib.leankv_rope_f16(self.qkv.data_ptr(), self.inv_freq.data_ptr(), sp,
                                              self.q_rope.data_ptr(), self.k_rope.data_ptr(), self.nq, self.nkv,
                                              128, st()), "rope")
            v_ptr = self.qkv.data_ptr() + (self.nq + self.nkv) * 128 * 2
            _native.check(lib.leankv_tq_pool_append(self.k_rope.data_ptr(), v_ptr, 1, self.nkv, 1,
                                                    self.Pi_k[l].data_ptr(), self.Pi_v[l].data_ptr(),
                                                    self.bounds.data_ptr(), self.pools[l].data_ptr(),
                                                    self.max_pages, sp + 8, self.page_indices.data_ptr(),
                                                    sp + 20, st()), "pool_append")
            _native.check(lib.leankv_tq_decode_attn(self.q_rope.data_ptr(), self.attn.data_ptr(), 1, self.nq,
                                                    self.nkv, self.pools[l].data_ptr(), self.max_pages, sp + 8,
                                                    self.page_indices.data_ptr(), sp + 16, self.max_pages,
                                                    self.Pi_k[l].data_ptr(), self.Pi_v[l].data_ptr(),
                                                    self.centroids_host.data_ptr(), 1.0 / math.sqrt(128.0),
                                                    self.ws_attn.data_ptr(), self.ws_attn.numel(), st()),
                          "decode_attn")
            self.launches_per_step += 4     # rope, append, query rotation, attention
        probe("attn")
        if fused_norm:
            # Single rank: h += o_proj(attn) in place.
            # Tensor parallel, peer exchange: the same two launches, each summing the ranks' partial
            # products over peer memory before it adds the residual stream (6 kernels per block).
            # Tensor parallel, NCCL: every rank writes its partial product to a second buffer, rank 0
            # alone adds the residual stream to its partial, and an all-reduce launch leaves the updated
            # stream on every rank (6 kernels + 2 all-reduces per block).
            if self.xchg is not None:
                self._gemv_allreduce(lw["wo_t"], self.attn, self.h, t["o_proj"], self.h, 2 * l)
                rc = lib.leankv_sparse_swiglu_rmsnorm_f16(
                    lw["wgate_t"].data_ptr(), lw["wup_t"].data_ptr(), self.h.data_ptr(), lw["ln2"].data_ptr(),
                    cfg.rms_eps, self.mlp_h.data_ptr(), self.inter, cfg.hidden_size, t["gate_proj"], t["up_proj"],
                    self.ws_gemv.data_ptr(), self.ws_gemv.numel(), self.active_elems.data_ptr(), st())
                _native.check(rc, "sparse swiglu")
                self.launches_per_step += 1
                probe("mlp_h")
                self._gemv_allreduce(lw["wdown_t"], self.mlp_h, self.h, t["down_proj"], self.h, 2 * l + 1)
                return
            tp = self.tp_size > 1
            h_mid = self.h2 if tp else self.h
            res = self.h if (not tp or self.tp_rank == 0) else None
            self._gemv(lw["wo_t"], self.attn, h_mid, t["o_proj"], residual=res)
            self._allreduce(h_mid)
            rc = lib.leankv_sparse_swiglu_rmsnorm_f16(
                lw["wgate_t"].data_ptr(), lw["wup_t"].data_ptr(), h_mid.data_ptr(), lw["ln2"].data_ptr(),
                cfg.rms_eps, self.mlp_h.data_ptr(), self.inter, cfg.hidden_size, t["gate_proj"], t["up_proj"],
                self.ws_gemv.data_ptr(), self.ws_gemv.numel(), self.active_elems.data_ptr(), st())
            _native.check(rc, "sparse swiglu")
            self.launches_per_step += 1
            probe("mlp_h")
            res = h_mid if (not tp or self.tp_rank == 0) else None
            self._gemv(lw["wdown_t"], self.mlp_h, self.h, t["down_proj"], residual=res)  # h = h_mid + down_proj(..)
            self._allreduce(self.h)
            return
        self._gemv(lw["wo_t"], self.attn, self.o, t["o_proj"])
        self._allreduce(self.o)
        probe("o")
        self._norm(self.o, lw["ln2"])
        probe("x")
        rc = lib.leankv_sparse_swiglu_f16(lw["wgate_t"].data_ptr(), lw["wup_t"].data_ptr(), self.x.data_ptr(),
                                          self.mlp_h.data_ptr(), self.inter, cfg.hidden_size, t["gate_proj"],
                                          t["up_proj"], self.ws_gemv.data_ptr(), self.ws_gemv.numel(),
                                          self.active_elems.data_ptr(), st())
        _native.check(rc, "sparse swiglu")
        self.launches_per_step += 1
        probe("mlp_h")
        self._gemv(lw["wdown_t"], self.mlp_h, self.down, t["down_proj"])
        self._allreduce(self.down)
        probe("down")
        nxt = self.w["layers"][l + 1]["ln1"] if l + 1 < cfg.num_layers else self.w["final_norm"]
        self._norm(self.down, nxt)

    def _step_launches(self) -> None:
        """One decode step: consumes ``self.token`` at position state[0], leaves the next token there."""
        cfg, lib, st = self.cfg, self.lib, self._st
        sp = self.state.data_ptr()
        self.launches_per_step = 0
        _native.check(lib.leankv_decode_begin(self.w["embed"].data_ptr(), self.token.data_ptr(), self.h.data_ptr(),
                                              cfg.hidden_size, cfg.vocab_size, sp, st()), "decode_begin")
        self.launches_per_step += 1
        fused_norm = self.fused_norm
        sharded_head = self.lm_head_local is not None and fused_norm
        if self.xchg is not None and fused_norm and not sharded_head:
            self.xchg.advance(st())        # with a sharded head the step's last kernel moves the epoch on
            self.launches_per_step += 1
        if not fused_norm:
            self._norm(None, self.w["layers"][0]["ln1"])
        for l in range(cfg.num_layers):
            self._layer_launches(l)
        if sharded_head:
            mine = self.logits[self.vocab_offset:self.vocab_offset + self.vocab_local]
            self._gemv(self.lm_head_local, self.h, mine, -1.0, norm_w=self.w["final_norm"])
            _native.check(lib.leankv_decode_end_sharded(mine.data_ptr(), self.vocab_local, self.vocab_offset,
                                                        self.token.data_ptr(), self.history.data_ptr(),
                                                        self.history_cap, sp, ctypes.byref(self.xchg.c),
                                                        2 * cfg.num_layers, st()), "decode_end_sharded")
            self.launches_per_step += 1
            return
        if fused_norm:
            self._gemv(self.w["lm_head_t"], self.h, self.logits, -1.0, norm_w=self.w["final_norm"])
        else:
            self._gemv(self.w["lm_head_t"], self.x, self.logits, -1.0)
        _native.check(lib.leankv_decode_end(self.logits.data_ptr(), cfg.vocab_size, self.token.data_ptr(),
                                            self.history.data_ptr(), self.history_cap, sp, st()), "decode_end")
        self.launches_per_step += 1

    def capture(self) -> None:
        """Capture one decode step into a CUDA graph (a throw-away eager step warms everything up first)."""
        with torch.cuda.device(self.dev):
            snap = (self.state.clone(), self.token.clone(), self.history.clone(),
                    [p.clone() for p in self.pools], self.active_elems.clone())
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                self._step_launches()
            torch.cuda.current_stream().wait_stream(side)
            torch.cuda.synchronize()
            self.state.copy_(snap[0]); self.token.copy_(snap[1]); self.history.copy_(snap[2])
            for p, s in zip(self.pools, snap[3]):
                p.copy_(s)
            self.active_elems.copy_(snap[4])
            self.graph = torch.cuda.CUDAGraph()
            # thread_local: the NCCL watchdog thread (tensor parallel runs) may touch CUDA while we capture
            with torch.cuda.graph(self.graph, capture_error_mode="thread_local"):
                self._step_launches()
            # capture does not execute; state is unchanged
            if self.tp_size > 1:
                # the in-kernel exchange waits a bounded time for its peers: start the replays together
                torch.cuda.synchronize()
                torch.distributed.barrier(group=self.group)

    def full_logits(self) -> torch.Tensor:
        """Logits of the last decode step over the whole vocabulary (fp16 [vocab]). With the output head
        split over tensor-parallel ranks ``self.logits`` holds only this rank's slice up to date: the
        slices are gathered here (a collective: every rank must call it)."""
        if self.lm_head_local is None:
            return self.logits
        mine = self.logits[self.vocab_offset:self.vocab_offset + self.vocab_local].contiguous()
        parts = [torch.empty_like(mine) for _ in range(self.tp_size)]
        torch.distributed.all_gather(parts, mine, group=self.group)
        return torch.cat(parts)

    def status_words(self) -> tuple[int, int]:
        """(exchange status, attention status) read from the device: non-zero once a bounded wait inside
        the in-kernel all-reduce / the attention kernel's page copies has given up, or a page id was out
        of range. Synchronises the device."""
        ex = int(self.xchg.status.item()) if self.xchg is not None else 0
        at = int(self.ws_attn[:4].view(torch.int32).item())
        return ex, at

    def check_status(self) -> None:
        """Raise if any kernel of this engine has reported a failed wait or a bad page id. The exchange
        status is sticky and switches later polls off, so results computed after it was set are
        meaningless: callers must not use them."""
        ex, at = self.status_words()
        if ex or at:
            raise RuntimeError(f"decode kernels reported a failure: exchange status {ex} "
                               f"(1 = a peer's partial sum never arrived), attention status {at} "
                               f"(1 = page copy wait gave up, 2 = page id out of range)")

    def step(self, use_graph: bool = True) -> None:
        if use_graph:
            if self.graph is None:
                self.capture()
            self.graph.replay()
        else:
            with torch.cuda.device(self.dev):
                self._step_launches()

    # ── prefill ──────────────────────────────────────────────────────────

    def _check_prefill_status(self) -> None:
        st = ctypes.c_int(0)
        _native.check(self.lib.leankv_tq_decode_attn_status(self._prefill_ws.data_ptr(), ctypes.byref(st)),
                      "attn_status")
        if st.value != 0:
            raise RuntimeError(f"prefill attention reported status {st.value} "
                               "(1 = a bounded wait ran out, 2 = page id outside the pool)")

    def _dense_forward(self, ids: torch.Tensor, write_cache: bool, collect: Optional[dict] = None,
                       page_indices: Optional[torch.Tensor] = None, start_pos: int = 0,
                       attention: str = "dense"):
        """Pass over ``ids`` (a prompt, or the chunk of it that starts at ``start_pos``) with library
        GEMMs for the projections. Returns the final hidden state of the last token.
        ``page_indices``: the pages of the sequence being filled (default: the engine's single sequence).
        ``attention``: "packed" = causal attention straight on the packed pages
        (``leankv_tq_prefill_attn``; needs ``write_cache``), "dense" = de-quantize the whole sequence to
        fp16 and call the library's attention (only for a chunk that starts at 0)."""
        from .turboquant.quantizer import MSEQuantized, TurboQuantMSE  # noqa: F401

        cfg, T = self.cfg, ids.numel()
        pages = self.page_indices if page_indices is None else page_indices
        if attention not in ("dense", "packed"):
            raise ValueError("attention must be 'dense' or 'packed'")
        if attention == "packed" and not write_cache:
            raise ValueError("packed attention reads the pool: it needs write_cache")
        if attention == "dense" and start_pos != 0:
            raise ValueError("the dense route handles whole prompts only")
        if attention == "packed":
            need = self.lib.leankv_tq_prefill_attn_workspace_bytes(T, start_pos, self.nq, self.nkv)
            if self._prefill_ws is None or self._prefill_ws.numel() < need:
                self._prefill_ws = torch.zeros(need, dtype=torch.uint8, device=self.dev)
            attn_out = torch.empty(T, self.nq, 128, dtype=torch.float16, device=self.dev)
        pos = torch.arange(start_pos, start_pos + T, device=self.dev).float()
        ang = torch.outer(pos, self.inv_freq)
        emb = torch.cat((ang, ang), dim=-1)
        cos, sin = emb.cos().half().unsqueeze(1), emb.sin().half().unsqueeze(1)
        h = self.w["embed"][ids]
        n_pages = (start_pos + T + PAGE - 1) // PAGE
        indptr = torch.tensor([0, n_pages], dtype=torch.int32, device=self.dev)
        start = torch.full((1,), start_pos, dtype=torch.int32, device=self.dev)

        def note(l, name, t):
            if collect is not None:
                collect.setdefault(l, {})[name] = t

        for l, lw in enumerate(self.w["layers"]):
            x = _rmsnorm(h, lw["ln1"], cfg.rms_eps)
            for p in ("q_proj", "k_proj", "v_proj"):
                note(l, p, x)
            qkv = x @ lw["wqkv_t"]
            q = _rope(qkv[:, :self.nq * 128].reshape(T, self.nq, 128), cos, sin)
            k = _rope(qkv[:, self.nq * 128:(self.nq + self.nkv) * 128].reshape(T, self.nkv, 128), cos, sin)
            v = qkv[:, (self.nq + self.nkv) * 128:].reshape(T, self.nkv, 128)
            kh = k.transpose(0, 1).contiguous().unsqueeze(0)     # [1, nkv, T, 128]
            vh = v.transpose(0, 1).contiguous().unsqueeze(0)
            if write_cache:
                rc = self.lib.leankv_tq_pool_append(kh.data_ptr(), vh.data_ptr(), 1, self.nkv, T,
                                                    self.Pi_k[l].data_ptr(), self.Pi_v[l].data_ptr(),
                                                    self.bounds.data_ptr(), self.pools[l].data_ptr(),
                                                    self.max_pages, indptr.data_ptr(),
                                                    pages.data_ptr(), start.data_ptr(), self._st())
                _native.check(rc, "pool_append")
                if attention == "dense":
                    kh, vh = self._dense_kv(l, T, pages)
            else:
                kh, vh = self._roundtrip(kh, l, 0), self._roundtrip(vh, l, 1)
            if attention == "packed":
                qc = q.contiguous()
                rc = self.lib.leankv_tq_prefill_attn(qc.data_ptr(), attn_out.data_ptr(), T, start_pos,
                                                     self.nq, self.nkv, self.pools[l].data_ptr(),
                                                     self.max_pages, pages.data_ptr(),
                                                     self.Pi_k[l].data_ptr(), self.Pi_v[l].data_ptr(),
                                                     self.centroids_host.data_ptr(), 1.0 / math.sqrt(128.0),
                                                     self._prefill_ws.data_ptr(), self._prefill_ws.numel(),
                                                     self._st())
                _native.check(rc, "prefill_attn")
                a = attn_out.reshape(T, self.nq * 128)
            else:
                a = F.scaled_dot_product_attention(q.transpose(0, 1).unsqueeze(0), kh, vh, is_causal=True,
                                                   enable_gqa=True)
                a = a.squeeze(0).transpose(0, 1).reshape(T, self.nq * 128)
            note(l, "o_proj", a)
            o = a @ lw["wo_t"]
            self._allreduce(o)
            h = h + o
            x = _rmsnorm(h, lw["ln2"], cfg.rms_eps)
            note(l, "gate_proj", x)
            note(l, "up_proj", x)
            m = F.silu(x @ lw["wgate_t"]) * (x @ lw["wup_t"])
            note(l, "down_proj", m)
            d = m @ lw["wdown_t"]
            self._allreduce(d)
            h = h + d
        return _rmsnorm(h[-1], self.w["final_norm"], cfg.rms_eps)

    @torch.no_grad()
    def dense_step_reference(self, token: int, pos: int) -> torch.Tensor:
        """Logits of the decode step that fed ``token`` at position ``pos``, recomputed with library
        GEMMs and library attention over the pool as that step left it (positions 0 .. pos, de-quantized
        to fp16). It reads the very codes the step wrote, so the two differ by rounding only, never by a
        code that fell on the other side of a decision boundary. Thresholds are not applied: meaningful
        for a step taken with TEAL off. For parity checks."""
        cfg = self.cfg
        with torch.cuda.device(self.dev):
            ang = float(pos) * self.inv_freq
            emb = torch.cat((ang, ang), dim=-1)
            cos, sin = emb.cos().half().reshape(1, 1, 128), emb.sin().half().reshape(1, 1, 128)
            h = self.w["embed"][token].reshape(1, -1)
            for l, lw in enumerate(self.w["layers"]):
                x = _rmsnorm(h, lw["ln1"], cfg.rms_eps)
                q = _rope((x @ lw["wqkv_t"])[:, :self.nq * 128].reshape(1, self.nq, 128), cos, sin)
                kh, vh = self._dense_kv(l, pos + 1)
                a = F.scaled_dot_product_attention(q.transpose(0, 1).unsqueeze(0), kh, vh, enable_gqa=True)
                o = a.squeeze(0).transpose(0, 1).reshape(1, self.nq * 128) @ lw["wo_t"]
                if self.tp_size > 1:
                    torch.distributed.all_reduce(o, group=self.group)
                h = h + o
                x = _rmsnorm(h, lw["ln2"], cfg.rms_eps)
                d = (F.silu(x @ lw["wgate_t"]) * (x @ lw["wup_t"])) @ lw["wdown_t"]
                if self.tp_size > 1:
                    torch.distributed.all_reduce(d, group=self.group)
                h = h + d
            return (_rmsnorm(h[0], self.w["final_norm"], cfg.rms_eps) @ self.w["lm_head_t"]).float()

    def _dense_kv(self, l: int, T: int, page_indices: Optional[torch.Tensor] = None):
        """fp16 K_hat, V_hat [1, nkv, T, 128] of layer ``l`` de-quantized from the pool."""
        outs = []
        n_pages = (T + PAGE - 1) // PAGE
        pages = (self.page_indices if page_indices is None else page_indices)[:n_pages].contiguous()
        for which, Pi in ((0, self.Pi_k[l]), (1, self.Pi_v[l])):
            idx = torch.empty(self.nkv, T, 64, dtype=torch.uint8, device=self.dev)
            norms = torch.empty(self.nkv, T, dtype=torch.float32, device=self.dev)
            rc = self.lib.leankv_tq_pool_unpack(self.pools[l].data_ptr(), self.max_pages, self.nkv,
                                                pages.data_ptr(), T, which,
                                                idx.data_ptr(), norms.data_ptr(), self._st())
            _native.check(rc, "pool_unpack")
            out = torch.empty(1, self.nkv, T, 128, dtype=torch.float16, device=self.dev)
            rc = self.lib.leankv_tq_dequantize(idx.data_ptr(), norms.data_ptr(), self.nkv * T, 128, 3,
                                               Pi.data_ptr(), self.centroids.data_ptr(), out.data_ptr(), 0,
                                               self._st())
            _native.check(rc, "dequantize")
            outs.append(out)
        return outs

    def _roundtrip(self, x, l, which):
        """Quantize + de-quantize without touching the pool (used by the calibration pass)."""
        Pi = (self.Pi_k if which == 0 else self.Pi_v)[l]
        n = x.numel() // 128
        idx = torch.empty(n, 64, dtype=torch.uint8, device=self.dev)
        norms = torch.empty(n, dtype=torch.float32, device=self.dev)
        x = x.contiguous()
        _native.check(self.lib.leankv_tq_quantize(x.data_ptr(), 0, n, 128, 3, Pi.data_ptr(),
                                                  self.bounds.data_ptr(), idx.data_ptr(), norms.data_ptr(),
                                                  self._st()), "quantize")
        norms = norms.half().float()
        out = torch.empty_like(x)
        _native.check(self.lib.leankv_tq_dequantize(idx.data_ptr(), norms.data_ptr(), n, 128, 3, Pi.data_ptr(),
                                                    self.centroids.data_ptr(), out.data_ptr(), 0, self._st()),
                      "dequantize")
        return out

    @torch.no_grad()
    def calibrate_thresholds(self, prompt_ids, sparsity: float = 0.4) -> dict:
        """Per-projection thresholds = the ``sparsity`` quantile of |input activation| over the prompt
        (``compute_threshold_for_sparsity``, leankv/teal/sparse_fns.py:47-69). Row-parallel inputs
        (o_proj, down_proj) are gathered across tensor-parallel ranks so every rank gets the same value."""
        ids = torch.as_tensor(prompt_ids, device=self.dev).reshape(-1)
        collect: dict = {}
        with torch.cuda.device(self.dev):
            self._dense_forward(ids, write_cache=False, collect=collect)
        thresholds = {}
        for l, acts in collect.items():
            thresholds[l] = {}
            for p, a in acts.items():
                if self.tp_size > 1 and p in ("o_proj", "down_proj"):
                    parts = [torch.empty_like(a) for _ in range(self.tp_size)]
                    torch.distributed.all_gather(parts, a.contiguous(), group=self.group)
                    a = torch.cat(parts, dim=-1)
                thresholds[l][p] = compute_threshold_for_sparsity(a.float(), sparsity)
        self.set_thresholds(thresholds)
        return thresholds

    @torch.no_grad()
    def prefill(self, prompt_ids, chunk: Optional[int] = None, attention: str = "packed") -> int:
        """Process the prompt, fill the pool, and leave the first generated token ready for ``step``.
        ``chunk``: tokens per pass (default: the whole prompt in one); every chunk is quantized into the
        pool first and then attends to the packed pages of everything up to itself, so no fp16 K/V
        of more than one chunk ever exists. ``attention="dense"`` (whole prompt only) de-quantizes the
        sequence and uses the library's attention instead, as the reference does
        (leankv/turboquant/cache.py:136-142)."""
        ids = torch.as_tensor(prompt_ids, device=self.dev).reshape(-1)
        T = ids.numel()
        if T < 1 or T >= self.max_seq_len:
            raise ValueError("prompt length must be in [1, max_seq_len)")
        if chunk is None:
            chunk = T
        if chunk < 1:
            raise ValueError("chunk must be positive")
        if attention == "dense" and chunk < T:
            raise ValueError("the dense route handles whole prompts only")
        with torch.cuda.device(self.dev):
            for p in self.pools:
                p.zero_()
            for s0 in range(0, T, chunk):
                x = self._dense_forward(ids[s0:s0 + chunk], write_cache=True, start_pos=s0,
                                        attention=attention)
            if attention == "packed":
                self._check_prefill_status()
            logits = x @ self.w["lm_head_t"]
            tok = torch.argmax(logits.float()).reshape(1)
            self.token.copy_(tok)
            self.history.zero_()
            self.history[0] = tok[0]
            self.state.zero_()
            self.state[0], self.state[1] = T, 1
            self.prefill_logits = logits
        return int(tok.item())

    @torch.no_grad()
    def generate(self, prompt_ids, max_new_tokens: int, stream_to_host: bool = True) -> list[int]:
        """Greedy generation. With ``stream_to_host`` every token is copied to pinned host memory and
        waited for before the next step is launched (what an interactive caller sees); without it the
        steps are enqueued back to back and the tokens are read once at the end."""
        first = self.prefill(prompt_ids)
        n_steps = min(max_new_tokens - 1, self.max_seq_len - len(prompt_ids) - 1)
        out = [first]
        with torch.cuda.device(self.dev):
            if self.graph is None:
                self.capture()
            for _ in range(max(n_steps, 0)):
                self.graph.replay()
                if stream_to_host:
                    self._pinned_token.copy_(self.token, non_blocking=True)
                    self._pinned_status[0:1].copy_(self.ws_attn[:4].view(torch.int32), non_blocking=True)
                    if self.xchg is not None:
                        self._pinned_status[1:2].copy_(self.xchg.status, non_blocking=True)
                    torch.cuda.current_stream().synchronize()
                    if int(self._pinned_status[0]) or int(self._pinned_status[1]):
                        self.check_status()
                    out.append(int(self._pinned_token[0]))
            if not stream_to_host:
                out = self.history[:1 + max(n_steps, 0)].tolist()
            self.check_status()
        return out

    def bytes_streamed(self) -> int:
        """Weight bytes the sparse GEMVs have streamed since the counter was last zeroed."""
        return 2 * int(self.active_elems.item())

    def kv_bytes_per_token(self) -> int:
        """Pool bytes per cached token on this rank: K and V, every layer and local kv head, 50 B per vector."""
        return 2 * self.cfg.num_layers * self.nkv * 50
