"""Lloyd-Max scalar codebooks for TurboQuant (host side, offline).

After a random rotation every coordinate of a unit vector in R^d has density
``f(x) = Gamma(d/2) / (sqrt(pi) Gamma((d-1)/2)) * (1 - x^2)^((d-3)/2)`` on [-1, 1]. The
codebook is the fixed point of the Lloyd-Max iteration for that density, with the same
initialisation, quadrature and stopping rule as ``leankv/turboquant/codebook.py:62-131``
so that centroids and decision boundaries agree with the reference to double-precision
round-off (the fp32 boundaries are kernel constants: a one-ulp difference would flip codes).

The codebook is not a GPU computation; the kernels receive its 2^bits centroids and
2^bits - 1 decision boundaries as fp32 constants.
"""

from __future__ import annotations

import json
import os

import numpy as np
import torch

_CODEBOOK_CACHE: dict[tuple[int, int], dict] = {}
# JSON files here use the reference's schema (centroids, boundaries, mse_per_coord,
# mse_total, d, bits), so a file written by either implementation can be read by both.
_CODEBOOK_DIR = os.path.join(os.path.dirname(__file__), "codebooks")


def beta_pdf(x: np.ndarray, d: int) -> np.ndarray:
    """Density of one coordinate of a uniform point on the sphere S^(d-1)."""
    from scipy import special

    if d <= 2:
        raise ValueError(f"Dimension d={d} too small, need d >= 3")
    log_norm = special.gammaln(d / 2.0) - 0.5 * np.log(np.pi) - special.gammaln((d - 1) / 2.0)
    x = np.clip(x, -1 + 1e-15, 1 - 1e-15)
    return np.exp(log_norm + ((d - 3) / 2.0) * np.log(1 - x**2))


def _cell_edges(centroids: np.ndarray) -> np.ndarray:
    """Nearest-centroid cells on [-1, 1]: -1, the midpoints, +1."""
    edges = np.empty(len(centroids) + 1)
    edges[0], edges[-1] = -1.0, 1.0
    edges[1:-1] = (centroids[:-1] + centroids[1:]) / 2.0
    return edges


def _cell_mean(lo: float, hi: float, d: int) -> float:
    from scipy import integrate

    first, _ = integrate.quad(lambda x: x * beta_pdf(np.array([x]), d)[0], lo, hi)
    mass, _ = integrate.quad(lambda x: beta_pdf(np.array([x]), d)[0], lo, hi)
    return (lo + hi) / 2.0 if mass < 1e-30 else first / mass


def _distortion(centroids: np.ndarray, d: int) -> float:
    from scipy import integrate

    edges = _cell_edges(centroids)
    total = 0.0
    for i, c in enumerate(centroids):
        part, _ = integrate.quad(lambda x, c=c: (x - c) ** 2 * beta_pdf(np.array([x]), d)[0],
                                 edges[i], edges[i + 1])
        total += part
    return total


def compute_lloyd_max_codebook(d: int, bits: int, max_iter: int = 200, tol: float = 1e-12) -> dict:
    """Continuous 1-D k-means on the rotated-coordinate density (2^bits levels)."""
    levels = 2**bits
    grid = np.linspace(-1 + 1e-10, 1 - 1e-10, 10000)
    cdf = np.cumsum(beta_pdf(grid, d)) * (grid[1] - grid[0])
    cdf /= cdf[-1]
    # start from the mid-quantile of each of `levels` equal-probability cells
    q_edges = np.linspace(0, 1, levels + 1)
    centroids = np.array([
        grid[min(np.searchsorted(cdf, (q_edges[i] + q_edges[i + 1]) / 2.0), len(grid) - 1)]
        for i in range(levels)
    ])

    previous = float("inf")
    cost = previous
    for _ in range(max_iter):
        edges = _cell_edges(centroids)
        centroids = np.array([_cell_mean(edges[i], edges[i + 1], d) for i in range(levels)])
        cost = _distortion(centroids, d)
        if abs(previous - cost) < tol:
            break
        previous = cost

    return {
        "centroids": centroids.tolist(),
        "boundaries": _cell_edges(centroids).tolist(),
        "mse_per_coord": float(cost),
        "mse_total": float(cost * d),
        "d": d,
        "bits": bits,
    }


def get_codebook(d: int, bits: int) -> dict:
    """Codebook for (d, bits): memory cache, then the JSON cache, then computed."""
    key = (d, bits)
    if key in _CODEBOOK_CACHE:
        return _CODEBOOK_CACHE[key]
    path = os.path.join(_CODEBOOK_DIR, f"codebook_d{d}_b{bits}.json")
    if os.path.exists(path):
        with open(path, "r") as f:
            cb = json.load(f)
    else:
        print(f"[TurboQuant] Computing Lloyd-Max codebook for d={d}, bits={bits}...")
        cb = compute_lloyd_max_codebook(d, bits)
        try:
            os.makedirs(_CODEBOOK_DIR, exist_ok=True)
            with open(path, "w") as f:
                json.dump(cb, f, indent=2)
        except OSError:
            pass   # read-only install: keep the in-memory copy
        print(f"[TurboQuant] MSE per coord = {cb['mse_per_coord']:.6e}, "
              f"total MSE = {cb['mse_total']:.6f}")
    _CODEBOOK_CACHE[key] = cb
    return cb


def get_codebook_tensors(d: int, bits: int, device, dtype: torch.dtype = torch.float32):
    """(centroids [2^bits], boundaries [2^bits + 1]) as tensors on ``device``."""
    cb = get_codebook(d, bits)
    return (torch.tensor(cb["centroids"], device=device, dtype=dtype),
            torch.tensor(cb["boundaries"], device=device, dtype=dtype))
