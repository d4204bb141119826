"""HuggingFace-compatible TurboQuant KV cache (API of ``leankv/turboquant/cache.py``).

Same storage model as the reference: the newest ``hot_buffer_size`` tokens of every layer
stay in fp16; older tokens are flushed to a cold store of packed codes + norms; ``update``
returns dense ``(K, V)`` = de-quantized cold tokens followed by the hot tokens, which is
what HF attention expects from ``past_key_values.update``.

Differences in mechanism, not in results: quantize / de-quantize run on the sm_100a
kernels (``leankv_tq_quantize`` / ``leankv_tq_dequantize``), cold de-quantization writes
fp16 directly, and the cold store grows geometrically instead of by ``torch.cat`` per
flush. Codes of a token do not depend on when it was flushed.
"""

from __future__ import annotations

import torch

from .. import _native
from .quantizer import MSEQuantized, TurboQuantMSE


class _ColdStore:
    """Codes [B, H, cap, packed] + norms [B, H, cap] with amortised O(1) append along tokens."""

    def __init__(self):
        self.indices = None
        self.norms = None
        self.length = 0

    def append(self, q: MSEQuantized) -> None:
        new = q.indices.shape[2]
        if self.indices is None or self.length + new > self.indices.shape[2]:
            cap = max(2 * (self.length + new), 256)
            b, h, _, p = q.indices.shape
            idx = torch.empty((b, h, cap, p), dtype=torch.uint8, device=q.indices.device)
            nrm = torch.empty((b, h, cap), dtype=q.norms.dtype, device=q.norms.device)
            if self.indices is not None:
                idx[:, :, :self.length] = self.indices[:, :, :self.length]
                nrm[:, :, :self.length] = self.norms[:, :, :self.length]
            self.indices, self.norms = idx, nrm
        self.indices[:, :, self.length:self.length + new] = q.indices
        self.norms[:, :, self.length:self.length + new] = q.norms
        self.length += new

    def view(self, bits: int) -> MSEQuantized | None:
        if self.length == 0:
            return None
        return MSEQuantized(indices=self.indices[:, :, :self.length],
                            norms=self.norms[:, :, :self.length], bits=bits)

    def nbytes(self) -> int:
        if self.length == 0:
            return 0
        b, h, _, p = self.indices.shape
        return b * h * self.length * (p * self.indices.element_size() + self.norms.element_size())


class TurboQuantCache:
    """Hybrid KV cache: compressed cold storage + fp16 hot buffer (``cache.py:27-351``)."""

    is_compileable = False
    layer_type = None

    def __init__(self, bits: int = 3, head_dim: int = 128, num_layers: int = 32,
                 hot_buffer_size: int = 64, device=None, dtype: torch.dtype = torch.float16,
                 seed: int = 42):
        self.bits = bits
        self.head_dim = head_dim
        self.num_layers = num_layers
        self.hot_buffer_size = hot_buffer_size
        self._device = torch.device(device) if device is not None else torch.device(
            "cuda" if torch.cuda.is_available() else "cpu")
        self._dtype = dtype
        self._seen_tokens = 0
        self._seq_lengths = [0] * num_layers
        # Distinct rotations per layer and per K/V: seeds seed+2i and seed+2i+1 (cache.py:59-71).
        self.key_quantizers = [
            TurboQuantMSE(dim=head_dim, bits=bits, device=self._device, dtype=torch.float32,
                          seed=seed + 2 * i) for i in range(num_layers)]
        self.val_quantizers = [
            TurboQuantMSE(dim=head_dim, bits=bits, device=self._device, dtype=torch.float32,
                          seed=seed + 2 * i + 1) for i in range(num_layers)]
        self._init_storage()

    def _init_storage(self):
        n = self.num_layers
        self._cold_k = [_ColdStore() for _ in range(n)]
        self._cold_v = [_ColdStore() for _ in range(n)]
        self._hot_keys: list[torch.Tensor | None] = [None] * n
        self._hot_values: list[torch.Tensor | None] = [None] * n

    # reference-named views of the cold store
    @property
    def _cold_keys(self):
        return [s.view(self.bits) for s in self._cold_k]

    @property
    def _cold_values(self):
        return [s.view(self.bits) for s in self._cold_v]

    @property
    def _cold_lengths(self):
        return [s.length for s in self._cold_k]

    # ── core ────────────────────────────────────────────────────────────

    def update(self, key_states: torch.Tensor, value_states: torch.Tensor, layer_idx: int,
               cache_kwargs=None):
        """Append ``[B, H, T_new, D]`` keys/values of one layer; return dense ``(K, V)``."""
        _native.require_cuda(key_states, "key_states")
        new_len = key_states.shape[2]
        if layer_idx == 0:
            self._seen_tokens += new_len
        self._seq_lengths[layer_idx] += new_len

        k_new = key_states.to(self._dtype)
        v_new = value_states.to(self._dtype)
        if self._hot_keys[layer_idx] is None:
            self._hot_keys[layer_idx], self._hot_values[layer_idx] = k_new, v_new
        else:
            self._hot_keys[layer_idx] = torch.cat([self._hot_keys[layer_idx], k_new], dim=2)
            self._hot_values[layer_idx] = torch.cat([self._hot_values[layer_idx], v_new], dim=2)
        if self._hot_keys[layer_idx].shape[2] > self.hot_buffer_size:
            self._flush_to_cold(layer_idx)
        return self._get_full_cache(layer_idx)

    def _flush_to_cold(self, layer_idx: int):
        """Quantize everything but the newest ``hot_buffer_size`` tokens into the cold store."""
        hot_k, hot_v = self._hot_keys[layer_idx], self._hot_values[layer_idx]
        flush_len = hot_k.shape[2] - self.hot_buffer_size
        # fp16 rows are widened inside the kernel: same values as .float() in cache.py:141-142
        ki, kn = self.key_quantizers[layer_idx]._quantize_impl(hot_k[:, :, :flush_len])
        vi, vn = self.val_quantizers[layer_idx]._quantize_impl(hot_v[:, :, :flush_len])
        self._cold_k[layer_idx].append(MSEQuantized(indices=ki, norms=kn, bits=self.bits))
        self._cold_v[layer_idx].append(MSEQuantized(indices=vi, norms=vn, bits=self.bits))
        self._hot_keys[layer_idx] = hot_k[:, :, flush_len:].contiguous()
        self._hot_values[layer_idx] = hot_v[:, :, flush_len:].contiguous()

    def _merge_quantized(self, a: MSEQuantized, b: MSEQuantized) -> MSEQuantized:
        """Concatenate two quantized blocks along the token dimension."""
        return MSEQuantized(indices=torch.cat([a.indices, b.indices], dim=2),
                            norms=torch.cat([a.norms, b.norms], dim=2), bits=a.bits)

    def _dequant_cold(self, quantizer: TurboQuantMSE, store: _ColdStore) -> torch.Tensor:
        q = store.view(self.bits)
        idx = q.indices.contiguous()
        norms = q.norms.float().contiguous()
        b, h, t, _ = idx.shape
        out = torch.empty((b, h, t, self.head_dim), dtype=torch.float16, device=idx.device)
        Pi, cents, _ = quantizer._consts()
        with torch.cuda.device(idx.device):
            rc = _native.lib().leankv_tq_dequantize(idx.data_ptr(), norms.data_ptr(), b * h * t,
                                                    self.head_dim, self.bits, Pi.data_ptr(),
                                                    cents.data_ptr(), out.data_ptr(), 0,
                                                    _native.current_stream())
        _native.check(rc, "leankv_tq_dequantize")
        return out if self._dtype == torch.float16 else out.to(self._dtype)

    def _get_full_cache(self, layer_idx: int):
        """Dense K and V of one layer: de-quantized cold tokens, then the hot tokens."""
        hot_k, hot_v = self._hot_keys[layer_idx], self._hot_values[layer_idx]
        if self._cold_k[layer_idx].length == 0:
            return hot_k, hot_v
        cold_k = self._dequant_cold(self.key_quantizers[layer_idx], self._cold_k[layer_idx])
        cold_v = self._dequant_cold(self.val_quantizers[layer_idx], self._cold_v[layer_idx])
        return torch.cat([cold_k, hot_k], dim=2), torch.cat([cold_v, hot_v], dim=2)

    # ── what HF generation calls ────────────────────────────────────────

    def get_seq_length(self, layer_idx: int = 0) -> int:
        return self._seq_lengths[layer_idx] if layer_idx < len(self._seq_lengths) else 0

    def get_mask_sizes(self, query_length: int, layer_idx: int = 0):
        return self.get_seq_length(layer_idx) + query_length, 0

    def get_max_cache_shape(self, *args, **kwargs):
        return None

    def get_max_length(self):
        return None

    def has_previous_state(self, layer_idx=None):
        if layer_idx is not None:
            return layer_idx < len(self._seq_lengths) and self._seq_lengths[layer_idx] > 0
        return any(s > 0 for s in self._seq_lengths)

    def crop(self, max_length: int):
        pass

    def batch_repeat_interleave(self, repeats: int):
        pass

    def batch_select_indices(self, indices: torch.Tensor):
        pass

    def reorder_cache(self, beam_idx: torch.LongTensor):
        pass

    def reset(self):
        self._init_storage()
        self._seq_lengths = [0] * self.num_layers
        self._seen_tokens = 0

    # ── properties ──────────────────────────────────────────────────────

    def _n_live_layers(self) -> int:
        return sum(1 for s in self._seq_lengths if s > 0)

    @property
    def seen_tokens(self):
        return self._seen_tokens

    @property
    def key_cache(self):
        return [torch.empty(0, device=self._device)] * self._n_live_layers()

    @property
    def value_cache(self):
        return [torch.empty(0, device=self._device)] * self._n_live_layers()

    @property
    def is_initialized(self):
        return self._n_live_layers() > 0

    @property
    def is_sliding(self):
        return [False] * self.num_layers

    @property
    def max_batch_size(self):
        return next((k.shape[0] for k in self._hot_keys if k is not None), 0)

    @property
    def max_cache_len(self):
        return max(self._seq_lengths) if self._seq_lengths else 0

    # ── container protocol ──────────────────────────────────────────────

    def __len__(self) -> int:
        return self._n_live_layers()

    def __getitem__(self, layer_idx: int):
        if self._seq_lengths[layer_idx] > 0:
            return self._get_full_cache(layer_idx)
        raise IndexError(f"Layer {layer_idx} not in cache")

    def __iter__(self):
        for i in range(self.num_layers):
            if self._seq_lengths[i] > 0:
                yield self._get_full_cache(i)

    def __bool__(self):
        return True

    def to_legacy_cache(self):
        return tuple(self._get_full_cache(i) for i in range(self.num_layers)
                     if self._seq_lengths[i] > 0)

    # ── diagnostics ─────────────────────────────────────────────────────

    def get_compressed_memory_bytes(self) -> int:
        """Bytes of live cold storage (codes + norms), K and V."""
        return sum(s.nbytes() for s in self._cold_k) + sum(s.nbytes() for s in self._cold_v)

    def get_hot_memory_bytes(self) -> int:
        return sum(t.numel() * t.element_size()
                   for t in self._hot_keys + self._hot_values if t is not None)

    def get_total_cache_bytes(self) -> int:
        return self.get_compressed_memory_bytes() + self.get_hot_memory_bytes()

    def get_fp16_equivalent_bytes(self) -> int:
        """Size of the same cache held entirely in fp16."""
        elems = 0
        for i, s in enumerate(self._seq_lengths):
            if s > 0 and self._hot_keys[i] is not None:
                b, h = self._hot_keys[i].shape[:2]
                elems += 2 * b * h * s * self.head_dim   # K and V
        return elems * 2

    def get_compression_ratio(self) -> float:
        actual = self.get_total_cache_bytes()
        return self.get_fp16_equivalent_bytes() / actual if actual else 0.0

    def print_memory_report(self):
        seq_len = max(self._seq_lengths) if self._seq_lengths else 0
        cold_len = max(self._cold_lengths) if self._cold_lengths else 0
        print(f"[TurboQuantCache] seq={seq_len} (cold={cold_len}, hot={seq_len - cold_len}), "
              f"actual={self.get_total_cache_bytes() / 1e6:.1f} MB "
              f"(cold={self.get_compressed_memory_bytes() / 1e6:.1f} + "
              f"hot={self.get_hot_memory_bytes() / 1e6:.1f}), "
              f"FP16 equiv={self.get_fp16_equivalent_bytes() / 1e6:.1f} MB, "
              f"ratio={self.get_compression_ratio():.1f}x")
