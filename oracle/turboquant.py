"""Reference arithmetic of the TurboQuant path on CPU tensors (test infrastructure).

* codebook      — leankv/turboquant/codebook.py:62-131 (Lloyd-Max on the Beta marginal)
* rotation      — leankv/turboquant/rotation.py:12-29
* quantize      — leankv/turboquant/quantizer.py:119-129 (+ _pack_indices :38-62)
* dequantize    — leankv/turboquant/quantizer.py:131-137 (+ _unpack_indices :65-85)
* kv_attention  — what a decode step computes from the cache: cache.py:169-189 builds
                  fp16 K_hat / V_hat from the cold store, then HF attention takes
                  softmax(q K^T * scale) V with GQA head sharing (repeat_kv)
"""

from __future__ import annotations

import numpy as np
import torch


# ── codebook ────────────────────────────────────────────────────────────────
def beta_pdf(x, d):
    from scipy import special

    logc = special.gammaln(d / 2.0) - 0.5 * np.log(np.pi) - special.gammaln((d - 1) / 2.0)
    x = np.clip(x, -1 + 1e-15, 1 - 1e-15)
    return np.exp(logc + (d - 3) / 2.0 * np.log(1 - x**2))


def lloyd_max(d: int, bits: int, max_iter: int = 200, tol: float = 1e-12) -> dict:
    from scipy import integrate

    n = 2**bits
    f = lambda x: beta_pdf(np.array([x]), d)[0]

    def edges_of(c):
        e = np.zeros(n + 1)
        e[0], e[-1] = -1.0, 1.0
        for i in range(n - 1):
            e[i + 1] = (c[i] + c[i + 1]) / 2.0
        return e

    grid = np.linspace(-1 + 1e-10, 1 - 1e-10, 10000)
    cdf = np.cumsum(beta_pdf(grid, d)) * (grid[1] - grid[0])
    cdf /= cdf[-1]
    qe = np.linspace(0, 1, n + 1)
    c = np.zeros(n)
    for i in range(n):
        c[i] = grid[min(np.searchsorted(cdf, (qe[i] + qe[i + 1]) / 2.0), len(grid) - 1)]
    prev = float("inf")
    cost = prev
    for _ in range(max_iter):
        e = edges_of(c)
        new = np.zeros(n)
        for i in range(n):
            num, _ = integrate.quad(lambda x: x * f(x), e[i], e[i + 1])
            den, _ = integrate.quad(f, e[i], e[i + 1])
            new[i] = (e[i] + e[i + 1]) / 2.0 if den < 1e-30 else num / den
        e2 = edges_of(new)
        cost = 0.0
        for i in range(n):
            val, _ = integrate.quad(lambda x, ci=new[i]: (x - ci) ** 2 * f(x), e2[i], e2[i + 1])
            cost += val
        c = new
        if abs(prev - cost) < tol:
            break
        prev = cost
    return {"centroids": c.tolist(), "boundaries": edges_of(c).tolist(),
            "mse_per_coord": float(cost), "mse_total": float(cost * d), "d": d, "bits": bits}


# ── rotation ────────────────────────────────────────────────────────────────
def rotation_matrix(d: int, seed: int) -> torch.Tensor:
    g = torch.Generator(device="cpu")
    g.manual_seed(seed)
    G = torch.randn(d, d, generator=g, dtype=torch.float32)
    Q, R = torch.linalg.qr(G)
    return Q * torch.sign(torch.diag(R)).unsqueeze(0)


# ── packing ─────────────────────────────────────────────────────────────────
def _layout(bits):
    return (8, 1) if bits == 1 else (4, 2) if bits == 2 else (2, 4) if bits <= 4 else (1, 8)


def pack(codes: torch.Tensor, bits: int) -> torch.Tensor:
    per, width = _layout(bits)
    if per == 1:
        return codes.to(torch.uint8)
    c = codes.to(torch.int64)
    pad = (-c.shape[-1]) % per
    if pad:
        c = torch.nn.functional.pad(c, (0, pad))
    c = c.reshape(*c.shape[:-1], -1, per)
    out = torch.zeros(c.shape[:-1], dtype=torch.int64, device=c.device)
    for i in range(per):
        out |= c[..., i] << (width * i)
    return out.to(torch.uint8)


def unpack(packed: torch.Tensor, bits: int, d: int) -> torch.Tensor:
    per, width = _layout(bits)
    if per == 1:
        return packed.long()
    p = packed.to(torch.int64)
    parts = [(p >> (width * i)) & ((1 << width) - 1) for i in range(per)]
    return torch.stack(parts, dim=-1).reshape(*packed.shape[:-1], -1)[..., :d]


# ── quantize / dequantize ───────────────────────────────────────────────────
def quantize(x: torch.Tensor, Pi: torch.Tensor, decision_boundaries: torch.Tensor, bits: int):
    """Returns (packed indices uint8, norms in x.dtype, unpacked codes int64, rotated y fp32)."""
    norms = x.norm(dim=-1)
    unit = x / (norms.unsqueeze(-1) + 1e-10)
    y = torch.matmul(unit.float(), Pi.T)
    codes = torch.searchsorted(decision_boundaries, y.contiguous())
    return pack(codes, bits), norms, codes, y


def dequantize(packed: torch.Tensor, norms: torch.Tensor, Pi: torch.Tensor,
               centroids: torch.Tensor, bits: int, d: int) -> torch.Tensor:
    y_hat = centroids[unpack(packed, bits, d)]
    return torch.matmul(y_hat, Pi) * norms.unsqueeze(-1)


def kv_attention(q: torch.Tensor, k_hat: torch.Tensor, v_hat: torch.Tensor, scale: float,
                 lengths=None) -> torch.Tensor:
    """q [B,Hq,D]; k_hat/v_hat [B,Hkv,T,D] (already rounded to the cache dtype).
    fp32 scores, fp32 softmax over the first lengths[b] tokens, fp32 value sum."""
    B, Hq, D = q.shape
    Hkv, T = k_hat.shape[1], k_hat.shape[2]
    rep = Hq // Hkv
    k = k_hat.float().repeat_interleave(rep, dim=1)
    v = v_hat.float().repeat_interleave(rep, dim=1)
    s = torch.einsum("bhd,bhtd->bht", q.float(), k) * scale
    if lengths is not None:
        mask = (torch.arange(T, device=q.device).unsqueeze(0)
                >= torch.as_tensor(lengths, device=q.device).unsqueeze(1))
        s = s.masked_fill(mask.unsqueeze(1), float("-inf"))
    p = torch.softmax(s, dim=-1)
    return torch.einsum("bht,bhtd->bhd", p, v)
