"""Sparse GEMV entry points (API of ``leankv/teal/kernels/sparse_gemv.py``) on the sm_100a kernels.

``sparse_gemv(x, weight, threshold)`` computes ``y = (x * (|x| > threshold)) @ weight.T``
for a single token, reading only the weight columns of surviving input channels.
``weight`` must be in the layout ``prepare_weight_for_sparse_gemv`` returns: logical
``[N, D]`` with strides ``(1, N)``, i.e. each input channel's N weights contiguous.
"""

from __future__ import annotations

import torch

from ... import _native

_workspaces: dict[tuple[int, int], torch.Tensor] = {}


def _workspace(device: torch.device, nbytes: int) -> torch.Tensor:
    """Zero-initialised split-K scratch, one per (device, stream), grown on demand."""
    key = (device.index if device.index is not None else torch.cuda.current_device(),
           _native.current_stream())
    ws = _workspaces.get(key)
    if ws is None or ws.numel() < nbytes:
        ws = torch.zeros(max(nbytes, 1 << 20), dtype=torch.uint8, device=device)
        _workspaces[key] = ws
    return ws


def _weight_as_rows(weight: torch.Tensor) -> tuple[int, int]:
    if weight.dim() != 2:
        raise ValueError("weight must be 2-D [N, D]")
    n, z = weight.shape
    if weight.dtype != torch.float16:
        raise TypeError("sparse_gemv needs fp16 weights")
    if weight.stride() != (1, n) and not (z == 1 or n == 1):
        raise ValueError(
            "weight must be column-major (strides (1, N)); convert it once with "
            "prepare_weight_for_sparse_gemv")
    return n, z


def sparse_gemv(x: torch.Tensor, weight: torch.Tensor, threshold: float,
                sparsity_bin: int = 5) -> torch.Tensor:
    """B=1 sparse GEMV. ``x``: [1, 1, D]; returns [1, 1, N] in ``x.dtype``.

    ``sparsity_bin`` is accepted for compatibility (the reference uses it as an autotune
    key); the CUDA kernel has no tuning state and ignores it.
    """
    _native.require_cuda(x, "x")
    _native.require_cuda(weight, "weight")
    n, z = _weight_as_rows(weight)
    xin = x.reshape(1, z)
    xh = xin if xin.dtype == torch.float16 else xin.to(torch.float16)
    xh = xh.contiguous()
    y = torch.empty(1, n, device=x.device, dtype=torch.float16)
    lib = _native.lib()
    with torch.cuda.device(x.device):
        nbytes = lib.leankv_sparse_gemv_workspace_bytes(n, z)
        ws = _workspace(x.device, nbytes)
        rc = lib.leankv_sparse_gemv_f16(weight.data_ptr(), xh.data_ptr(), y.data_ptr(), n, z,
                                        float(threshold), None, None, ws.data_ptr(), ws.numel(),
                                        None, _native.current_stream())
    _native.check(rc, "leankv_sparse_gemv_f16")
    out = y.reshape(1, 1, n)
    return out if x.dtype == torch.float16 else out.to(x.dtype)


def sparse_swiglu(x: torch.Tensor, gate_weight: torch.Tensor, up_weight: torch.Tensor,
                  gate_threshold: float, up_threshold: float) -> torch.Tensor:
    """Fused ``silu(gate(x_s)) * up(x_s)`` for one token; both weights column-major [N, D].

    The reference has no counterpart kernel: it runs ``sparse_gemv`` twice and the
    activation product in two more elementwise kernels. Rounding points are the same.
    """
    _native.require_cuda(x, "x")
    n, z = _weight_as_rows(gate_weight)
    if _weight_as_rows(up_weight) != (n, z):
        raise ValueError("gate and up weights must have the same shape")
    xh = x.reshape(1, z).to(torch.float16).contiguous()
    y = torch.empty(1, n, device=x.device, dtype=torch.float16)
    lib = _native.lib()
    with torch.cuda.device(x.device):
        nbytes = lib.leankv_sparse_swiglu_workspace_bytes(n, z)
        ws = _workspace(x.device, nbytes)
        rc = lib.leankv_sparse_swiglu_f16(gate_weight.data_ptr(), up_weight.data_ptr(),
                                          xh.data_ptr(), y.data_ptr(), n, z, float(gate_threshold),
                                          float(up_threshold), ws.data_ptr(), ws.numel(), None,
                                          _native.current_stream())
    _native.check(rc, "leankv_sparse_swiglu_f16")
    out = y.reshape(1, 1, n)
    return out if x.dtype == torch.float16 else out.to(x.dtype)


def batched_sparse_gemm(x: torch.Tensor, weight: torch.Tensor, threshold: float,
                        sparsity_bin: int = 5) -> torch.Tensor:
    """B>1 variant: every row of ``x`` [B, D] gets its own mask; returns [B, N].

    One GEMV launch per row. The reference's patching never takes this path (it uses a
    dense matmul for B>1, ``patching.py:178-180``); it exists for API completeness.
    """
    rows = [sparse_gemv(x[i].reshape(1, 1, -1), weight, threshold, sparsity_bin).reshape(1, -1)
            for i in range(x.shape[0])]
    return torch.cat(rows, dim=0)


def prepare_weight_for_sparse_gemv(weight: torch.Tensor) -> torch.Tensor:
    """Re-lay ``weight`` [N, D] so that each input channel's N weights are contiguous.

    The result has the same shape and values, strides ``(1, N)``.
    """
    n, z = weight.shape
    out = torch.empty_strided((n, z), (1, n), dtype=weight.dtype, device=weight.device)
    out.copy_(weight)
    return out
