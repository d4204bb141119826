"""Helpers shared by the GPU tests: raw C-ABI calls for the paged TurboQuant pool."""

import ctypes
import math

import numpy as np
import torch

from leankv_b200 import _native
from leankv_b200.turboquant import codebook, rotation


class RawPool:
    """One layer's pool driven directly through the C ABI (no PagedKVCache logic in between)."""

    def __init__(self, n_pages, n_kv_heads, device, seed_k=42, seed_v=43):
        self.lib = _native.lib()
        self.dev = device
        self.n_pages, self.H = n_pages, n_kv_heads
        assert self.lib.leankv_tq_pool_bytes(n_pages, n_kv_heads) == n_pages * 2 * n_kv_heads * 800
        self.pool = torch.zeros(n_pages, 2, n_kv_heads, 800, dtype=torch.uint8, device=device)
        self.Pi_k = rotation.generate_rotation_matrix(128, device, torch.float32, seed_k).contiguous()
        self.Pi_v = rotation.generate_rotation_matrix(128, device, torch.float32, seed_v).contiguous()
        cents, bounds = codebook.get_codebook_tensors(128, 3, "cpu")
        self.centroids_host = cents.contiguous()
        self.centroids = cents.to(device)
        self.bounds = bounds[1:-1].contiguous().to(device)
        self.ws = None

    def i32(self, values):
        return torch.tensor(list(values), dtype=torch.int32, device=self.dev)

    def append(self, k, v, indptr, indices, start_pos):
        """k, v: [B, H, T, 128] fp16 on the device; page table / start positions as python lists."""
        B, H, T, _ = k.shape
        ip, ix, sp = self.i32(indptr), self.i32(indices), self.i32(start_pos)
        k, v = k.contiguous(), v.contiguous()      # keep the copies alive until the launch has been queued
        rc = self.lib.leankv_tq_pool_append(k.data_ptr(), v.data_ptr(), B, H, T,
                                            self.Pi_k.data_ptr(), self.Pi_v.data_ptr(), self.bounds.data_ptr(),
                                            self.pool.data_ptr(), self.n_pages, ip.data_ptr(), ix.data_ptr(),
                                            sp.data_ptr(), torch.cuda.current_stream().cuda_stream)
        _native.check(rc, "leankv_tq_pool_append")
        torch.cuda.synchronize()

    def unpack(self, pages, n_tokens, which):
        ix = self.i32(pages)
        idx = torch.empty(self.H, n_tokens, 64, dtype=torch.uint8, device=self.dev)
        norms = torch.empty(self.H, n_tokens, dtype=torch.float32, device=self.dev)
        rc = self.lib.leankv_tq_pool_unpack(self.pool.data_ptr(), self.n_pages, self.H, ix.data_ptr(),
                                            n_tokens, which, idx.data_ptr(), norms.data_ptr(),
                                            torch.cuda.current_stream().cuda_stream)
        _native.check(rc, "leankv_tq_pool_unpack")
        torch.cuda.synchronize()
        return idx.cpu().numpy(), norms.cpu().numpy()

    def prefill_attention(self, q, seq_pages, start_pos):
        """q [T, Hq, 128] fp16: the chunk of prompt tokens at positions start_pos.. -> out [T, Hq, 128]."""
        T, Hq, _ = q.shape
        need = self.lib.leankv_tq_prefill_attn_workspace_bytes(T, start_pos, Hq, self.H)
        ws = torch.zeros(need, dtype=torch.uint8, device=self.dev)
        q = q.contiguous()
        out = torch.empty_like(q)
        pg = self.i32(seq_pages)
        rc = self.lib.leankv_tq_prefill_attn(q.data_ptr(), out.data_ptr(), T, start_pos, Hq, self.H,
                                             self.pool.data_ptr(), self.n_pages, pg.data_ptr(),
                                             self.Pi_k.data_ptr(), self.Pi_v.data_ptr(),
                                             self.centroids_host.data_ptr(), 1.0 / math.sqrt(128.0),
                                             ws.data_ptr(), ws.numel(), torch.cuda.current_stream().cuda_stream)
        _native.check(rc, "leankv_tq_prefill_attn")
        torch.cuda.synchronize()
        st = ctypes.c_int(0)
        _native.check(self.lib.leankv_tq_decode_attn_status(ws.data_ptr(), ctypes.byref(st)), "status")
        assert st.value == 0
        return out

    def attention(self, q, indptr, indices, last_len, max_pages=None):
        """q [B, Hq, 128] fp16 -> out [B, Hq, 128] fp16."""
        B, Hq, _ = q.shape
        if max_pages is None:
            max_pages = max(1, max(indptr[b + 1] - indptr[b] for b in range(B)))
        need = self.lib.leankv_tq_decode_attn_workspace_bytes(B, Hq, self.H, max_pages)
        if self.ws is None or self.ws.numel() < need:
            self.ws = torch.zeros(need, dtype=torch.uint8, device=self.dev)
        q = q.contiguous()
        out = torch.empty_like(q)
        ip, ix, ll = self.i32(indptr), self.i32(indices if len(indices) else [0]), self.i32(last_len)
        rc = self.lib.leankv_tq_decode_attn(q.data_ptr(), out.data_ptr(), B, Hq, self.H,
                                            self.pool.data_ptr(), self.n_pages, ip.data_ptr(), ix.data_ptr(),
                                            ll.data_ptr(), max_pages, self.Pi_k.data_ptr(), self.Pi_v.data_ptr(),
                                            self.centroids_host.data_ptr(), 1.0 / math.sqrt(128.0),
                                            self.ws.data_ptr(), self.ws.numel(),
                                            torch.cuda.current_stream().cuda_stream)
        _native.check(rc, "leankv_tq_decode_attn")
        torch.cuda.synchronize()
        return out

    def status(self):
        import ctypes

        val = ctypes.c_int(-1)
        _native.check(self.lib.leankv_tq_decode_attn_status(self.ws.data_ptr(), ctypes.byref(val)), "status")
        return val.value


def oracle_attention_from_pool(rp: RawPool, q, seq_pages, seq_lens):
    """Reference path on the CPU: codes/norms read back from the pool -> de-quantize (torch, as
    quantizer.py:131-137) -> fp16 K_hat/V_hat (cache.py:176-181) -> fp32 softmax attention."""
    from oracle import turboquant as otq

    B = q.shape[0]
    T = max(seq_lens)
    k_hat = torch.zeros(B, rp.H, T, 128, dtype=torch.float16)
    v_hat = torch.zeros_like(k_hat)
    cents = rp.centroids.cpu()
    for b in range(B):
        if seq_lens[b] == 0:
            continue
        for which, dst, Pi in ((0, k_hat, rp.Pi_k.cpu()), (1, v_hat, rp.Pi_v.cpu())):
            idx, norms = rp.unpack(seq_pages[b], seq_lens[b], which)
            deq = otq.dequantize(torch.from_numpy(idx), torch.from_numpy(norms), Pi, cents, 3, 128)
            dst[b, :, :seq_lens[b]] = deq.half()
    return otq.kv_attention(q.cpu(), k_hat, v_hat, 128 ** -0.5, lengths=seq_lens)
