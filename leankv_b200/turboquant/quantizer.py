"""TurboQuant quantizers with the call surface of ``leankv/turboquant/quantizer.py``.

``TurboQuantMSE.quantize`` / ``dequantize`` run the sm_100a kernels behind
``leankv_tq_quantize`` / ``leankv_tq_dequantize``; tensors must live on a CUDA device
(there is no CPU fallback). Formats are the reference's: ``indices`` is uint8, two 4-bit
fields per byte for 3- and 4-bit codes (low nibble = even coordinate,
``quantizer.py:38-62``), ``norms`` are the vectors' L2 norms.
"""

from __future__ import annotations

import math
from typing import NamedTuple

import torch

from .. import _native
from .codebook import get_codebook_tensors
from .rotation import generate_qjl_matrix, generate_rotation_matrix


class MSEQuantized(NamedTuple):
    """Result of :meth:`TurboQuantMSE.quantize`."""

    indices: torch.Tensor   # (..., packed_len) uint8
    norms: torch.Tensor     # (...,) L2 norms
    bits: int


class ProdQuantized(NamedTuple):
    """Result of :meth:`TurboQuantProd.quantize`."""

    mse_indices: torch.Tensor
    qjl_signs: torch.Tensor
    residual_norms: torch.Tensor
    norms: torch.Tensor
    mse_bits: int


def _field_layout(bits: int) -> tuple[int, int]:
    """(fields per byte, field width) of the reference packing; (1, 8) = unpacked."""
    if bits == 1:
        return 8, 1
    if bits == 2:
        return 4, 2
    if bits <= 4:
        return 2, 4
    return 1, 8


def _pack_indices(indices: torch.Tensor, bits: int) -> torch.Tensor:
    """Pack integer codes into uint8 (layout of ``quantizer.py:38-62``)."""
    per_byte, width = _field_layout(bits)
    codes = indices.to(torch.uint8)
    if per_byte == 1:
        return codes
    d = codes.shape[-1]
    pad = (-d) % per_byte
    if pad:
        codes = torch.nn.functional.pad(codes, (0, pad), value=0)
    codes = codes.reshape(*codes.shape[:-1], -1, per_byte).to(torch.int32)
    weights = torch.tensor([1 << (width * i) for i in range(per_byte)], device=codes.device,
                           dtype=torch.int32)
    return (codes * weights).sum(dim=-1).to(torch.uint8)


def _unpack_indices(packed: torch.Tensor, bits: int, d: int) -> torch.Tensor:
    """Inverse of :func:`_pack_indices`; returns int64 codes of length ``d``."""
    per_byte, width = _field_layout(bits)
    if per_byte == 1:
        return packed.long()
    shifts = torch.arange(per_byte, device=packed.device, dtype=torch.int32) * width
    fields = (packed.to(torch.int32).unsqueeze(-1) >> shifts) & ((1 << width) - 1)
    return fields.reshape(*packed.shape[:-1], -1)[..., :d].long()


class TurboQuantMSE(torch.nn.Module):
    """MSE-optimal TurboQuant (Algorithm 1): rotate, scalar-quantize each coordinate.

    Buffers ``Pi`` [d, d], ``centroids`` [2^bits], ``boundaries`` [2^bits + 1] and
    ``decision_boundaries`` [2^bits - 1] match ``quantizer.py:96-117``.
    """

    def __init__(self, dim: int, bits: int = 3, device=None, dtype: torch.dtype = torch.float32,
                 seed: int = 42):
        super().__init__()
        self.dim = dim
        self.bits = bits
        self.n_clusters = 2**bits
        self.device = torch.device(device) if device is not None else torch.device(
            "cuda" if torch.cuda.is_available() else "cpu")
        self.register_buffer("Pi", generate_rotation_matrix(dim, self.device, dtype, seed=seed))
        centroids, boundaries = get_codebook_tensors(dim, bits, self.device, dtype)
        self.register_buffer("centroids", centroids)
        self.register_buffer("boundaries", boundaries)
        self.register_buffer("decision_boundaries", boundaries[1:-1].contiguous())

    def _consts(self):
        """(Pi, centroids, decision boundaries) as fp32 row-major device tensors for the kernels.

        Cached on the module: callers pass raw pointers to asynchronous launches, so these
        must not be temporaries that die before the kernel runs."""
        key = (self.Pi.data_ptr(), self.Pi.device)
        if getattr(self, "_consts_key", None) != key:
            self._consts_val = (self.Pi.float().contiguous(), self.centroids.float().contiguous(),
                                self.decision_boundaries.float().contiguous())
            self._consts_key = key
        return self._consts_val

    def _check(self, t: torch.Tensor, what: str) -> None:
        _native.require_cuda(t, what)
        if self.dim != _native.TQ_DIM or not 1 <= self.bits <= 4:
            raise RuntimeError(
                f"TurboQuantMSE kernels support dim=128 and bits 1..4, got dim={self.dim} bits={self.bits}")

    def _quantize_impl(self, x: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
        """(indices uint8 (..., packed_len), norms fp32 (...)) for fp16 or fp32 ``x``."""
        self._check(x, "x")
        if x.shape[-1] != self.dim:
            raise ValueError(f"last dimension must be {self.dim}, got {tuple(x.shape)}")
        lead = x.shape[:-1]
        xk = x if x.dtype in (torch.float16, torch.float32) else x.float()
        xk = xk.reshape(-1, self.dim).contiguous()
        n = xk.shape[0]
        lib = _native.lib()
        plen = lib.leankv_tq_packed_len(self.dim, self.bits)
        indices = torch.empty((n, plen), dtype=torch.uint8, device=x.device)
        norms = torch.empty((n,), dtype=torch.float32, device=x.device)
        Pi, _, bounds = self._consts()
        with torch.cuda.device(x.device):
            rc = lib.leankv_tq_quantize(xk.data_ptr(), 0 if xk.dtype == torch.float16 else 1, n,
                                        self.dim, self.bits, Pi.data_ptr(), bounds.data_ptr(),
                                        indices.data_ptr(), norms.data_ptr(),
                                        _native.current_stream())
        _native.check(rc, "leankv_tq_quantize")
        return indices.reshape(*lead, plen), norms.reshape(lead)

    def quantize(self, x: torch.Tensor) -> MSEQuantized:
        """Quantize vectors ``x`` of shape (..., d).

        fp16 and fp32 inputs are read by the kernel directly (fp16 is widened exactly, so
        ``quantize(x.half())`` and ``quantize(x.half().float())`` give the same codes);
        other dtypes are widened to fp32 first. Norms are returned in ``x.dtype`` like
        ``x.norm(dim=-1)``.
        """
        indices, norms = self._quantize_impl(x)
        if x.dtype != torch.float32:
            norms = norms.to(x.dtype)
        return MSEQuantized(indices=indices, norms=norms, bits=self.bits)

    def dequantize(self, q: MSEQuantized) -> torch.Tensor:
        """Reconstruct fp32 vectors (..., d) from codes and norms."""
        self._check(q.indices, "q.indices")
        lead = q.indices.shape[:-1]
        idx = q.indices.reshape(-1, q.indices.shape[-1]).contiguous()
        norms = q.norms.reshape(-1).float().contiguous()
        n = idx.shape[0]
        out = torch.empty((n, self.dim), dtype=torch.float32, device=idx.device)
        Pi, cents, _ = self._consts()
        with torch.cuda.device(idx.device):
            rc = _native.lib().leankv_tq_dequantize(idx.data_ptr(), norms.data_ptr(), n, self.dim,
                                                    q.bits, Pi.data_ptr(), cents.data_ptr(),
                                                    out.data_ptr(), 1, _native.current_stream())
        _native.check(rc, "leankv_tq_dequantize")
        return out.reshape(*lead, self.dim)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        """Quantize then dequantize."""
        return self.dequantize(self.quantize(x))


class TurboQuantProd(torch.nn.Module):
    """Inner-product TurboQuant (Algorithm 2, ``quantizer.py:144-237``).

    (b-1)-bit MSE quantization on the CUDA kernels plus one QJL sign bit per coordinate of
    the residual. The residual projection and sign packing are plain torch ops: nothing on
    the decode path of the reference uses this class (its cache imports only the MSE
    quantizer, ``cache.py:24``).
    """

    def __init__(self, dim: int, bits: int = 3, device=None, dtype: torch.dtype = torch.float32,
                 seed: int = 42):
        super().__init__()
        if bits < 2:
            raise AssertionError(
                "Inner product TurboQuant requires at least 2 bits (1 for MSE + 1 for QJL)")
        self.dim = dim
        self.bits = bits
        self.device = torch.device(device) if device is not None else torch.device(
            "cuda" if torch.cuda.is_available() else "cpu")
        self.mse_quantizer = TurboQuantMSE(dim=dim, bits=bits - 1, device=self.device, dtype=dtype,
                                           seed=seed)
        self.register_buffer("S", generate_qjl_matrix(dim, self.device, dtype, seed=seed + 1000))
        self.qjl_scale = math.sqrt(math.pi / 2.0) / dim

    def _pack_qjl_signs(self, projected: torch.Tensor) -> torch.Tensor:
        return _pack_indices((projected > 0).to(torch.uint8), 1)

    def _unpack_qjl_signs(self, packed: torch.Tensor) -> torch.Tensor:
        return 2.0 * _unpack_indices(packed, 1, self.dim).float() - 1.0

    def quantize(self, x: torch.Tensor) -> ProdQuantized:
        mse_q = self.mse_quantizer.quantize(x)
        residual = x - self.mse_quantizer.dequantize(mse_q)
        projected = torch.matmul(residual.float(), self.S.T)
        return ProdQuantized(mse_indices=mse_q.indices, qjl_signs=self._pack_qjl_signs(projected),
                             residual_norms=residual.norm(dim=-1), norms=mse_q.norms,
                             mse_bits=mse_q.bits)

    def dequantize(self, q: ProdQuantized) -> torch.Tensor:
        x_mse = self.mse_quantizer.dequantize(
            MSEQuantized(indices=q.mse_indices, norms=q.norms, bits=q.mse_bits))
        x_qjl = torch.matmul(self._unpack_qjl_signs(q.qjl_signs), self.S)
        return x_mse + x_qjl * (self.qjl_scale * q.residual_norms.unsqueeze(-1))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.dequantize(self.quantize(x))
