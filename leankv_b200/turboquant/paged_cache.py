"""Paged TurboQuant KV cache with fused decode attention (API of ``leankv/turboquant/paged_cache.py``).

The reference class of this name keeps fp16 pages and hands them to FlashInfer. This one
keeps **3-bit TurboQuant pages** (48 bytes of codes + an fp16 norm per 128-d vector, 16
tokens per page) and runs decode attention directly on the packed pages with the sm_100a
kernel behind ``leankv_tq_decode_attn``; FlashInfer is not needed. Page-table conventions
(``kv_indptr`` / ``kv_page_indices`` / ``kv_last_page_len`` int32, LIFO free list, one
page table shared by all layers) are the reference's (``paged_cache.py:78,96-115,215-233``).

The page table lives on the device: a free-page stack, a block table (pages of each sequence in
order) and the sequence lengths are advanced by one small kernel per step
(``leankv_paged_table_step``), which also rebuilds the flat arrays the append and attention calls
read. The host only mirrors the lengths as integers (HF asks for them every step, and pool
exhaustion is raised before anything is launched); it builds no per-token lists or tensors.

``update`` appends through the fused rotate+quantize+pack kernel and, for HF
compatibility, returns dense K/V de-quantized from the pages; ``decode_attention`` is the
fast path.
"""

from __future__ import annotations

import math

import torch

from .. import _native
from .quantizer import TurboQuantMSE

PAGE = _native.TQ_PAGE_TOKENS


class PagedKVCache:
    """Page pool of 3-bit TurboQuant KV + fused paged decode attention."""

    is_compileable = False
    layer_type = None

    def __init__(self, num_layers: int = 32, num_kv_heads: int = 8, num_q_heads: int = 32,
                 head_dim: int = 128, page_size: int = 16, max_pages: int = 2048,
                 dtype: torch.dtype = torch.float16, device=None, bits: int = 3, seed: int = 42):
        if head_dim != _native.TQ_DIM or page_size != PAGE or bits != 3:
            raise RuntimeError("PagedKVCache kernels need head_dim=128, page_size=16, bits=3")
        self.num_layers = num_layers
        self.num_kv_heads = num_kv_heads
        self.num_q_heads = num_q_heads
        self.head_dim = head_dim
        self.page_size = page_size
        self.max_pages = max_pages
        self.bits = bits
        self._dtype = dtype
        self._device = torch.device(device) if device is not None else torch.device("cuda")
        self._seen_tokens = 0

        # [layer][page][K|V][kv head][800 bytes]; zero pages decode to finite values
        self.kv_data = torch.zeros(num_layers, max_pages, 2, num_kv_heads, _native.TQ_CHUNK_BYTES,
                                   dtype=torch.uint8, device=self._device)
        # same per-layer rotations as TurboQuantCache (seed + 2i for K, seed + 2i + 1 for V)
        self.key_quantizers = [TurboQuantMSE(head_dim, bits, self._device, torch.float32, seed + 2 * i)
                               for i in range(num_layers)]
        self.val_quantizers = [TurboQuantMSE(head_dim, bits, self._device, torch.float32,
                                             seed + 2 * i + 1) for i in range(num_layers)]
        self._centroids_host = self.key_quantizers[0].centroids.float().cpu().contiguous()
        self._bounds = self.key_quantizers[0].decision_boundaries.float().contiguous()

        self._seq_lengths: list[int] = []     # host mirror of the device lengths (plain integers)
        self._batch_size = 0
        self._free_count = max_pages          # host mirror of the free stack's height
        self._workspace = None
        self.fused_decode = False             # set by hf_attention.enable_paged_attention
        self.fused_prefill = False            # likewise: prompt passes attend on the packed pages too
        self._prefill_ws = None
        self._alloc_tables(0)

    # ── page table (device) ─────────────────────────────────────────────

    def _alloc_tables(self, batch_cap: int):
        """(Re)allocate the per-sequence device arrays for ``batch_cap`` sequences, keeping their content.
        The first call also creates the free stack (LIFO like the reference's list: page
        ``max_pages - 1`` is handed out first)."""
        dev, i32 = self._device, torch.int32
        old_table = getattr(self, "_block_table", None)
        old_len = getattr(self, "_seq_len_dev", None)
        rows = max(batch_cap, 1)
        self._batch_cap = batch_cap
        self._pps_cap = self.max_pages                       # a single sequence may take the whole pool
        self._block_table = torch.zeros(rows, self._pps_cap, dtype=i32, device=dev)
        self._seq_len_dev = torch.zeros(rows, dtype=i32, device=dev)
        self._kv_indptr = torch.zeros(rows + 1, dtype=i32, device=dev)
        self._kv_last = torch.zeros(rows, dtype=i32, device=dev)
        self._start_dev = torch.zeros(rows, dtype=i32, device=dev)
        if old_table is None:
            self._free_stack = torch.arange(self.max_pages, dtype=i32, device=dev)
            self._free_top = torch.full((1,), self.max_pages, dtype=i32, device=dev)
            self._kv_page_indices = torch.zeros(self.max_pages, dtype=i32, device=dev)
            self._status = torch.zeros(1, dtype=i32, device=dev)
        else:
            n = old_table.shape[0]
            self._block_table[:n] = old_table
            self._seq_len_dev[:n] = old_len
        self._meta_batch = -1                                # batch size the flat arrays were built for

    def _ensure_batch_size(self, batch_size: int):
        if batch_size > self._batch_cap:
            self._alloc_tables(batch_size)
        while len(self._seq_lengths) < batch_size:
            self._seq_lengths.append(0)
        self._batch_size = max(self._batch_size, batch_size)

    def _table_step(self, t_new: int, batch: int):
        """Advance every sequence by ``t_new`` tokens on the device and rebuild the flat arrays."""
        with torch.cuda.device(self._device):
            rc = _native.lib().leankv_paged_table_step(
                t_new, batch, self._seq_len_dev.data_ptr(), self._block_table.data_ptr(), self._pps_cap,
                self._free_stack.data_ptr(), self._free_top.data_ptr(), self._kv_indptr.data_ptr(),
                self._kv_page_indices.data_ptr(), self._kv_last.data_ptr(), self._start_dev.data_ptr(),
                self._status.data_ptr(), _native.current_stream())
        _native.check(rc, "leankv_paged_table_step")
        self._meta_batch = batch

    def _allocate_page(self) -> int:
        """Pop one page off the free stack (the reference's method of this name, ``paged_cache.py:96-103``).
        The step kernel does this for whole batches; this single-page form reads the id back to the host."""
        if self._free_count == 0:
            raise RuntimeError(
                f"PagedKVCache: out of pages ({self.max_pages} used). "
                f"Increase max_pages or reduce batch/sequence length.")
        page = int(self._free_stack[self._free_count - 1])
        self._free_top -= 1
        self._free_count -= 1
        return page

    def _free_sequence_pages(self, batch_idx: int):
        """Return a sequence's pages to the stack (in order, so that the last one is reused first)."""
        n = math.ceil(self._seq_lengths[batch_idx] / PAGE)
        if n:
            top = self._free_count                               # stack height == free pages
            self._free_stack[top:top + n] = self._block_table[batch_idx, :n]
            self._free_top += n
            self._free_count += n
        self._seq_len_dev[batch_idx] = 0
        self._seq_lengths[batch_idx] = 0
        self._meta_batch = -1

    def _device_meta(self, batch_size: int):
        """(kv_indptr, kv_page_indices, kv_last_page_len) int32 on the device."""
        if self._meta_batch != batch_size:
            self._ensure_batch_size(batch_size)
            self._table_step(0, batch_size)                      # rebuild only
        return self._kv_indptr, self._kv_page_indices, self._kv_last

    def page_table_status(self) -> int:
        """Device status word of the page table (0 = clean, 1 = pool exhausted, 2 = block table row full)."""
        return int(self._status.item())

    # ── appends ────────────────────────────────────────────────────────

    def update(self, key_states: torch.Tensor, value_states: torch.Tensor, layer_idx: int,
               cache_kwargs=None):
        """Quantize-append ``[B, Hkv, T_new, D]`` K/V of one layer; return dense ``(K, V)``.

        With ``fused_decode`` set (``hf_attention.enable_paged_attention``) a one-token update only
        appends and hands the new token's own K/V back as a placeholder: the registered attention
        function answers from the packed pages and never looks at it. With ``fused_prefill`` set as
        well the same holds for prompt chunks (``prefill_attention``)."""
        self.append(layer_idx, key_states, value_states)
        if self.fused_decode and (key_states.shape[2] == 1 or self.fused_prefill):
            return key_states, value_states
        return self._gather_kv(layer_idx, key_states.shape[0])

    def append(self, layer_idx: int, key_states: torch.Tensor, value_states: torch.Tensor):
        """Quantize-append without building dense tensors (use with ``decode_attention``)."""
        _native.require_cuda(key_states, "key_states")
        batch, _, t_new, _ = key_states.shape
        if layer_idx == 0:
            # the page table is shared by all layers: pages are assigned once per step, on the device;
            # the host checks the pool size with integer arithmetic first (same error as the reference)
            self._seen_tokens += t_new
            self._ensure_batch_size(batch)
            need = sum(math.ceil((n + t_new) / PAGE) - math.ceil(n / PAGE) for n in self._seq_lengths[:batch])
            if need > self._free_count:
                raise RuntimeError(
                    f"PagedKVCache: out of pages ({self.max_pages} used). "
                    f"Increase max_pages or reduce batch/sequence length.")
            self._table_step(t_new, batch)
            self._free_count -= need
            for b in range(batch):
                self._seq_lengths[b] += t_new
        indptr, flat, _ = self._device_meta(batch)
        start = self._start_dev          # written by the table step, shared by all layers
        k = key_states.to(torch.float16).contiguous()
        v = value_states.to(torch.float16).contiguous()
        kq, vq = self.key_quantizers[layer_idx], self.val_quantizers[layer_idx]
        with torch.cuda.device(self._device):
            rc = _native.lib().leankv_tq_pool_append(
                k.data_ptr(), v.data_ptr(), batch, self.num_kv_heads, t_new, kq._consts()[0].data_ptr(),
                vq._consts()[0].data_ptr(), self._bounds.data_ptr(), self.kv_data[layer_idx].data_ptr(),
                self.max_pages, indptr.data_ptr(), flat.data_ptr(), start.data_ptr(),
                _native.current_stream())
        _native.check(rc, "leankv_tq_pool_append")

    def unpack_sequence(self, layer_idx: int, batch_idx: int, which: int):
        """Codes (uint8 [Hkv, T, 64], reference nibble format) and norms (fp32 [Hkv, T]) of one sequence."""
        t = self._seq_lengths[batch_idx]
        pages = self._block_table[batch_idx, :max(math.ceil(t / PAGE), 1)]      # device view, no host list
        idx = torch.empty(self.num_kv_heads, t, 64, dtype=torch.uint8, device=self._device)
        norms = torch.empty(self.num_kv_heads, t, dtype=torch.float32, device=self._device)
        with torch.cuda.device(self._device):
            rc = _native.lib().leankv_tq_pool_unpack(
                self.kv_data[layer_idx].data_ptr(), self.max_pages, self.num_kv_heads,
                pages.data_ptr(), t, which, idx.data_ptr(), norms.data_ptr(), _native.current_stream())
        _native.check(rc, "leankv_tq_pool_unpack")
        return idx, norms

    def _gather_kv(self, layer_idx: int, batch_size: int):
        """Dense ``[B, Hkv, max_seq, D]`` K and V de-quantized from the pages (zero padded)."""
        from .quantizer import MSEQuantized

        max_seq = max(self._seq_lengths[:batch_size])
        keys = torch.zeros(batch_size, self.num_kv_heads, max_seq, self.head_dim, dtype=self._dtype,
                           device=self._device)
        values = torch.zeros_like(keys)
        for b in range(batch_size):
            t = self._seq_lengths[b]
            if t == 0:
                continue
            for which, quant, dst in ((0, self.key_quantizers[layer_idx], keys),
                                      (1, self.val_quantizers[layer_idx], values)):
                idx, norms = self.unpack_sequence(layer_idx, b, which)
                dst[b, :, :t] = quant.dequantize(MSEQuantized(idx, norms, self.bits)).to(self._dtype)
        return keys, values

    # ── fused decode attention ─────────────────────────────────────────

    def decode_attention(self, layer_idx: int, query: torch.Tensor) -> torch.Tensor:
        """``softmax(q K_hat^T / sqrt(d)) V_hat`` over the packed pages; query/out ``[B, Hq, D]``."""
        _native.require_cuda(query, "query")
        batch = query.shape[0]
        indptr, flat, last = self._device_meta(batch)
        max_pages_seq = max(math.ceil(n / PAGE) for n in self._seq_lengths[:batch])
        q = query.to(torch.float16).contiguous()
        out = torch.empty_like(q)
        lib = _native.lib()
        with torch.cuda.device(self._device):
            need = lib.leankv_tq_decode_attn_workspace_bytes(batch, self.num_q_heads, self.num_kv_heads,
                                                             max_pages_seq)
            if self._workspace is None or self._workspace.numel() < need:
                self._workspace = torch.zeros(max(need, 1 << 20), dtype=torch.uint8, device=self._device)
            kq, vq = self.key_quantizers[layer_idx], self.val_quantizers[layer_idx]
            rc = lib.leankv_tq_decode_attn(
                q.data_ptr(), out.data_ptr(), batch, self.num_q_heads, self.num_kv_heads,
                self.kv_data[layer_idx].data_ptr(), self.max_pages, indptr.data_ptr(), flat.data_ptr(),
                last.data_ptr(), max_pages_seq, kq._consts()[0].data_ptr(), vq._consts()[0].data_ptr(),
                self._centroids_host.data_ptr(), 1.0 / math.sqrt(self.head_dim),
                self._workspace.data_ptr(), self._workspace.numel(), _native.current_stream())
        _native.check(rc, "leankv_tq_decode_attn")
        return out if query.dtype == torch.float16 else out.to(query.dtype)

    def prefill_attention(self, layer_idx: int, query: torch.Tensor) -> torch.Tensor:
        """Causal attention of the chunk that ``update`` / ``append`` has just added, over the packed
        pages of everything up to each token: ``query`` ``[B, Hq, T, D]`` -> ``[B, Hq, T, D]``. The T tokens
        are the last T of every sequence. Replaces ``update`` (de-quantize the history) + eager attention
        on a prompt pass (leankv/turboquant/cache.py:136-142)."""
        _native.require_cuda(query, "query")
        batch, _, t_new, _ = query.shape
        lib = _native.lib()
        out = torch.empty(batch, t_new, self.num_q_heads, self.head_dim, dtype=torch.float16, device=self._device)
        kq, vq = self.key_quantizers[layer_idx], self.val_quantizers[layer_idx]
        with torch.cuda.device(self._device):
            for b in range(batch):
                n = self._seq_lengths[b]
                start = n - t_new
                if start < 0:
                    raise RuntimeError("prefill_attention: the chunk has not been appended to this sequence")
                need = lib.leankv_tq_prefill_attn_workspace_bytes(t_new, start, self.num_q_heads, self.num_kv_heads)
                if self._prefill_ws is None or self._prefill_ws.numel() < need:
                    self._prefill_ws = torch.zeros(need, dtype=torch.uint8, device=self._device)
                q = query[b].transpose(0, 1).to(torch.float16).contiguous()          # [T, Hq, D]
                pages = self._block_table[b, :math.ceil(n / PAGE)]
                rc = lib.leankv_tq_prefill_attn(
                    q.data_ptr(), out[b].data_ptr(), t_new, start, self.num_q_heads, self.num_kv_heads,
                    self.kv_data[layer_idx].data_ptr(), self.max_pages, pages.data_ptr(),
                    kq._consts()[0].data_ptr(), vq._consts()[0].data_ptr(), self._centroids_host.data_ptr(),
                    1.0 / math.sqrt(self.head_dim), self._prefill_ws.data_ptr(), self._prefill_ws.numel(),
                    _native.current_stream())
                _native.check(rc, "leankv_tq_prefill_attn")
        out = out.transpose(1, 2)
        return out if query.dtype == torch.float16 else out.to(query.dtype)

    def kernel_status(self) -> int:
        """Status words of the attention kernels' bounded waits, decode and prefill OR-ed (0 = clean)."""
        import ctypes

        status = 0
        for ws in (self._workspace, self._prefill_ws):
            if ws is None:
                continue
            val = ctypes.c_int(0)
            _native.check(_native.lib().leankv_tq_decode_attn_status(ws.data_ptr(), ctypes.byref(val)),
                          "leankv_tq_decode_attn_status")
            status |= val.value
        return status

    # ── HF cache surface ───────────────────────────────────────────────

    def get_seq_length(self, layer_idx: int = 0) -> int:
        return max(self._seq_lengths[:self._batch_size]) if self._batch_size > 0 else 0

    def get_mask_sizes(self, query_length: int, layer_idx: int = 0):
        return self.get_seq_length(layer_idx) + query_length, 0

    def get_max_cache_shape(self, *args, **kwargs):
        return None

    def get_max_length(self):
        return self.max_pages * self.page_size

    def has_previous_state(self, layer_idx=None):
        return any(s > 0 for s in self._seq_lengths)

    def crop(self, max_length):
        pass

    def batch_repeat_interleave(self, repeats):
        pass

    def batch_select_indices(self, indices):
        pass

    def reorder_cache(self, beam_idx):
        pass

    def reset(self):
        self._seq_lengths = []
        self._batch_size = 0
        self._seen_tokens = 0
        self._free_count = self.max_pages
        self._block_table = None
        self._alloc_tables(0)
        self.kv_data.zero_()

    @property
    def seen_tokens(self):
        return self._seen_tokens

    @property
    def key_cache(self):
        return [torch.empty(0, device=self._device)] * self.num_layers

    @property
    def value_cache(self):
        return [torch.empty(0, device=self._device)] * self.num_layers

    @property
    def is_initialized(self):
        return any(s > 0 for s in self._seq_lengths)

    @property
    def is_sliding(self):
        return [False] * self.num_layers

    @property
    def max_batch_size(self):
        return self._batch_size

    @property
    def max_cache_len(self):
        return max(self._seq_lengths) if self._seq_lengths else 0

    def __len__(self):
        return self.num_layers if any(s > 0 for s in self._seq_lengths) else 0

    def __getitem__(self, layer_idx):
        return self._gather_kv(layer_idx, self._batch_size)

    def __iter__(self):
        for i in range(self.num_layers):
            yield self._gather_kv(i, self._batch_size)

    def __bool__(self):
        return True

    # ── diagnostics ────────────────────────────────────────────────────

    def get_pages_used(self) -> int:
        return self.max_pages - self._free_count

    def bytes_per_page(self) -> int:
        """Bytes one page occupies in one layer (K and V, all kv heads)."""
        return 2 * self.num_kv_heads * _native.TQ_CHUNK_BYTES

    def get_memory_usage_mb(self) -> float:
        return self.get_pages_used() * self.bytes_per_page() * self.num_layers / 1e6

    def get_total_pool_mb(self) -> float:
        return self.kv_data.numel() * self.kv_data.element_size() / 1e6

    def print_memory_report(self):
        seq_len = max(self._seq_lengths) if self._seq_lengths else 0
        print(f"[PagedKVCache] pages={self.get_pages_used()}/{self.max_pages}, "
              f"pool={self.get_total_pool_mb():.1f} MB, used={self.get_memory_usage_mb():.1f} MB, "
              f"batch={self._batch_size}, seq_len={seq_len}")
