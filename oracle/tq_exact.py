"""ctypes front end of ``tq_exact.c`` (test infrastructure): builds it with gcc on demand."""

from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_DIR = os.path.dirname(os.path.abspath(__file__))
_BUILD = os.path.join(_DIR, "_build")
_lib = None


def _cpu_has_fma() -> bool:
    try:
        with open("/proc/cpuinfo") as f:
            return " fma " in f.read().replace("\n", " ")
    except OSError:
        return False


def build(force: bool = False) -> str:
    """Compile tq_exact.c into oracle/_build/. -ffp-contract=off: only the written fma calls fuse."""
    os.makedirs(_BUILD, exist_ok=True)
    fma = _cpu_has_fma()
    out = os.path.join(_BUILD, "libtq_exact_fma.so" if fma else "libtq_exact.so")
    src = os.path.join(_DIR, "tq_exact.c")
    if force or not os.path.exists(out) or os.path.getmtime(out) < os.path.getmtime(src):
        cmd = ["gcc", "-O2", "-ffp-contract=off", "-fopenmp", "-shared", "-fPIC", src, "-o", out, "-lm"]
        if fma:
            cmd.insert(1, "-mfma")
        subprocess.run(cmd, check=True)
    return out


def lib():
    global _lib
    if _lib is None:
        _lib = ctypes.CDLL(build())
    return _lib


def quantize(x: np.ndarray, Pi: np.ndarray, bounds: np.ndarray):
    """x float32 (n,128) -> codes uint8 (n,128), norms f32 (n), y f32 (n,128), margin f32 (n,128)."""
    x = np.ascontiguousarray(x, dtype=np.float32).reshape(-1, 128)
    Pi = np.ascontiguousarray(Pi, dtype=np.float32)
    bounds = np.ascontiguousarray(bounds, dtype=np.float32)
    n = x.shape[0]
    codes = np.empty((n, 128), np.uint8)
    norms = np.empty(n, np.float32)
    y = np.empty((n, 128), np.float32)
    margin = np.empty((n, 128), np.float32)
    P = ctypes.c_void_p
    lib().tq_exact_quantize(P(x.ctypes.data), ctypes.c_long(n), P(Pi.ctypes.data), P(bounds.ctypes.data),
                            ctypes.c_int(len(bounds)), P(codes.ctypes.data), P(norms.ctypes.data),
                            P(y.ctypes.data), P(margin.ctypes.data))
    return codes, norms, y, margin


def dequantize(codes: np.ndarray, norms: np.ndarray, Pi: np.ndarray, centroids: np.ndarray):
    codes = np.ascontiguousarray(codes, dtype=np.uint8).reshape(-1, 128)
    norms = np.ascontiguousarray(norms, dtype=np.float32).reshape(-1)
    Pi = np.ascontiguousarray(Pi, dtype=np.float32)
    centroids = np.ascontiguousarray(centroids, dtype=np.float32)
    out = np.empty((codes.shape[0], 128), np.float32)
    P = ctypes.c_void_p
    lib().tq_exact_dequantize(P(codes.ctypes.data), P(norms.ctypes.data), ctypes.c_long(codes.shape[0]),
                              P(Pi.ctypes.data), P(centroids.ctypes.data), P(out.ctypes.data))
    return out


if __name__ == "__main__":
    print(build(force=True))
