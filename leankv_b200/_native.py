"""ctypes binding of ``libleankv_b200.so`` (the C ABI declared in ``include/leankv_b200.h``).

There is no CPU or PyTorch fallback behind these calls: if the library is missing or a
kernel reports an error, a ``RuntimeError`` is raised.
"""

from __future__ import annotations

import ctypes
import os
from ctypes import (POINTER, Structure, c_char_p, c_float, c_int, c_int32, c_longlong, c_size_t,
                    c_uint8, c_ulonglong, c_void_p)

_PKG_DIR = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG_DIR, "libleankv_b200.so")

MAX_SEGMENTS = 4
TQ_PAGE_TOKENS = 16
TQ_DIM = 128
TQ_CHUNK_BYTES = 800
ATTN_EARLY_FETCH = 1


class Segments(Structure):
    """Mirror of ``leankv_segments_t``."""

    _fields_ = [
        ("n_segments", c_int),
        ("seg_end", c_int * MAX_SEGMENTS),
        ("threshold", c_float * MAX_SEGMENTS),
    ]


MAX_RANKS = 8


class Xchg(Structure):
    """Mirror of ``leankv_xchg_t``."""

    _fields_ = [
        ("world", c_int), ("rank", c_int),
        ("n_slots", c_int), ("max_cols", c_int),
        ("max_wait_iters", c_int),
        ("recv", c_void_p * MAX_RANKS),
        ("epoch", c_void_p),
        ("status", c_void_p),
    ]


# name -> (restype, argtypes); every symbol the header declares appears here.
SIGNATURES = {
    "leankv_strerror": (c_char_p, [c_int]),
    "leankv_abi_version": (c_int, []),
    "leankv_last_cuda_error": (c_char_p, []),
    "leankv_sparse_gemv_workspace_bytes": (c_size_t, [c_int, c_int]),
    "leankv_sparse_gemv_f16": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_float,
                                       c_void_p, c_void_p, c_void_p, c_size_t, c_void_p, c_void_p]),
    "leankv_sparse_gemv_seg_f16": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int,
                                           POINTER(Segments), c_void_p, c_void_p, c_void_p,
                                           c_size_t, c_void_p, c_void_p]),
    "leankv_sparse_gemv_rmsnorm_f16": (c_int, [c_void_p, c_void_p, c_void_p, c_float, c_void_p, c_int, c_int,
                                               POINTER(Segments), c_void_p, c_void_p, c_size_t, c_void_p,
                                               c_void_p]),
    "leankv_sparse_swiglu_rmsnorm_f16": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_float, c_void_p,
                                                 c_int, c_int, c_float, c_float, c_void_p, c_size_t,
                                                 c_void_p, c_void_p]),
    "leankv_sparse_gemv_f16_static": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_float, c_void_p]),
    "leankv_sparse_swiglu_workspace_bytes": (c_size_t, [c_int, c_int]),
    "leankv_sparse_swiglu_f16": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int,
                                         c_float, c_float, c_void_p, c_size_t, c_void_p, c_void_p]),
    "leankv_tq_packed_len": (c_int, [c_int, c_int]),
    "leankv_tq_quantize": (c_int, [c_void_p, c_int, c_longlong, c_int, c_int, c_void_p, c_void_p,
                                   c_void_p, c_void_p, c_void_p]),
    "leankv_tq_dequantize": (c_int, [c_void_p, c_void_p, c_longlong, c_int, c_int, c_void_p,
                                     c_void_p, c_void_p, c_int, c_void_p]),
    "leankv_tq_pool_bytes": (c_size_t, [c_int, c_int]),
    "leankv_tq_pool_append": (c_int, [c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p,
                                      c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p,
                                      c_void_p]),
    "leankv_tq_band_stats": (c_int, [POINTER(c_ulonglong), c_int]),
    "leankv_tq_pool_unpack": (c_int, [c_void_p, c_int, c_int, c_void_p, c_int, c_int, c_void_p,
                                      c_void_p, c_void_p]),
    "leankv_tq_decode_attn_workspace_bytes": (c_size_t, [c_int, c_int, c_int, c_int]),
    "leankv_tq_decode_attn": (c_int, [c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_int,
                                      c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
                                      c_void_p, c_float, c_void_p, c_size_t, c_void_p]),
    "leankv_tq_decode_attn_rotated": (c_int, [c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_int,
                                              c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
                                              c_float, c_void_p, c_size_t, c_int, c_void_p]),
    "leankv_decode_qkv_post": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                       c_void_p, c_int, c_void_p, c_int, c_int, c_void_p, c_void_p]),
    "leankv_tq_decode_attn_status": (c_int, [c_void_p, POINTER(c_int)]),
    "leankv_tq_prefill_attn_workspace_bytes": (c_size_t, [c_int, c_int, c_int, c_int]),
    "leankv_tq_prefill_attn": (c_int, [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_int,
                                       c_void_p, c_void_p, c_void_p, c_void_p, c_float, c_void_p, c_size_t,
                                       c_void_p]),
    "leankv_rmsnorm_f16": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_float, c_void_p]),
    "leankv_decode_begin": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p]),
    "leankv_rope_f16": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                                c_void_p]),
    "leankv_decode_end": (c_int, [c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p]),
    "leankv_decode_end_sharded": (c_int, [c_void_p, c_int, c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
                                          c_int, c_void_p]),
    "leankv_tq_append_status": (c_int, [POINTER(c_int)]),
    "leankv_xchg_recv_bytes": (c_size_t, [c_int, c_int, c_int]),
    "leankv_xchg_advance": (c_int, [c_void_p, c_void_p]),
    "leankv_sparse_gemv_allreduce_f16": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_float, c_void_p,
                                                 c_void_p, c_size_t, c_void_p, c_void_p, c_int, c_void_p]),
    "leankv_ipc_alloc": (c_int, [c_size_t, POINTER(c_void_p), c_char_p]),
    "leankv_ipc_open": (c_int, [c_char_p, POINTER(c_void_p)]),
    "leankv_ipc_close": (c_int, [c_void_p]),
    "leankv_ipc_free": (c_int, [c_void_p]),
    "leankv_rmsnorm_rows_f16": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_float, c_void_p]),
    "leankv_batch_decode_begin": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p,
                                          c_int, c_void_p, c_void_p, c_void_p, c_void_p]),
    "leankv_batch_qkv_post": (c_int, [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                      c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_void_p, c_void_p]),
    "leankv_paged_table_step": (c_int, [c_int, c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p,
                                        c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]),
    "leankv_silu_mul_f16": (c_int, [c_void_p, c_void_p, c_int, c_int, c_void_p]),
    "leankv_batch_decode_end": (c_int, [c_void_p, c_int, c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
                                        c_void_p]),
}

_lib = None


def lib() -> ctypes.CDLL:
    """Load the shared library once; raise if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m leankv_b200.build` "
                "(leankv_b200 has no CPU or PyTorch fallback)")
        handle = ctypes.CDLL(LIB_PATH)
        for name, (restype, argtypes) in SIGNATURES.items():
            fn = getattr(handle, name)   # AttributeError if the build is stale
            fn.restype = restype
            fn.argtypes = argtypes
        _lib = handle
    return _lib


def check(code: int, what: str) -> None:
    """Raise ``RuntimeError`` for a negative status code."""
    if code == 0:
        return
    handle = lib()
    msg = handle.leankv_strerror(code).decode()
    if code == -4:
        msg += ": " + handle.leankv_last_cuda_error().decode()
    raise RuntimeError(f"{what} failed: {msg} (code {code})")


def ptr(t) -> int | None:
    """Device address of a torch tensor (None passes NULL)."""
    return None if t is None else t.data_ptr()


def current_stream() -> int:
    import torch

    return torch.cuda.current_stream().cuda_stream


def require_cuda(t, name: str) -> None:
    if not t.is_cuda:
        raise RuntimeError(
            f"{name} must be a CUDA tensor: leankv_b200 runs only on the GPU (no CPU fallback)")
