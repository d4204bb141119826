"""Seeded synthetic inputs with the shapes and value distributions of the benchmark configurations.

The reference measures on real Mistral-7B weights and prompts; none of that is available
offline, so these generators stand in: N(0, 0.02) weights, Laplace(0, 1) activations
thresholded at their own 40th-percentile magnitude, N(0, 1) keys/values with a few outlier
channels. All draws use torch's CPU generator so the same seed gives the same tensors on
every machine; tensors are moved to ``device`` afterwards.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

from .teal.sparse_fns import compute_threshold_for_sparsity


@dataclass
class GemvCase:
    weight: torch.Tensor      # [N, Z] fp16, row-major (as nn.Linear stores it)
    x: torch.Tensor           # [1, Z] fp16
    threshold: float
    n_active: int


def sparse_gemv_case(n_out: int = 4096, n_in: int = 14336, sparsity: float = 0.4, seed: int = 0,
                     device="cpu") -> GemvCase:
    """Config 1: W ~ N(0, 0.02) [n_out, n_in]; x ~ Laplace(0, 1); threshold = 40th percentile |x|."""
    gen = torch.Generator(device="cpu").manual_seed(seed)
    w = (torch.randn(n_out, n_in, generator=gen) * 0.02).half()
    u = torch.rand(1, n_in, generator=gen) - 0.5                 # inverse-CDF Laplace(0, 1)
    x = (-torch.sign(u) * torch.log1p(-2 * u.abs().clamp(max=0.4999999))).half()
    t = compute_threshold_for_sparsity(x, sparsity)
    n_act = int((x.abs() > t).sum()) if t > 0 else n_in
    return GemvCase(w.to(device), x.to(device), t, n_act)


@dataclass
class SwigluCase:
    w_gate: torch.Tensor      # [N, Z] fp16
    w_up: torch.Tensor
    x: torch.Tensor           # [1, Z] fp16
    threshold: float
    n_active: int


def swiglu_case(n_out: int = 14336, n_in: int = 4096, sparsity: float = 0.4, seed: int = 1,
                device="cpu") -> SwigluCase:
    """Config 2: gate/up ~ N(0, 0.02) [n_out, n_in]; x ~ Laplace(0, 1) thresholded to 40 % zeros."""
    gen = torch.Generator(device="cpu").manual_seed(seed)
    u = torch.rand(1, n_in, generator=gen) - 0.5
    x = (-torch.sign(u) * torch.log1p(-2 * u.abs().clamp(max=0.4999999))).half()
    wg = (torch.randn(n_out, n_in, generator=gen) * 0.02).half()
    wu = (torch.randn(n_out, n_in, generator=gen) * 0.02).half()
    t = compute_threshold_for_sparsity(x, sparsity)
    n_act = int((x.abs() > t).sum()) if t > 0 else n_in
    return SwigluCase(wg.to(device), wu.to(device), x.to(device), t, n_act)


@dataclass
class KvCase:
    k: torch.Tensor           # [B, Hkv, T, 128] fp16
    v: torch.Tensor
    q: torch.Tensor           # [B, Hq, 128] fp16
    page_ids: torch.Tensor    # [B, ceil(T/16)] int32, a permutation of the pool's pages
    n_pages: int


def kv_case(batch: int = 16, n_q_heads: int = 32, n_kv_heads: int = 8, context: int = 4096,
            head_dim: int = 128, n_outliers: int = 4, outlier_scale: float = 8.0, seed: int = 3,
            device="cpu") -> KvCase:
    """Config 3: K, V ~ N(0, 1) with ``n_outliers`` channels per head scaled by ``outlier_scale``;
    one query token per sequence; page ids shuffled over the pool."""
    gen = torch.Generator(device="cpu").manual_seed(seed)
    k = torch.randn(batch, n_kv_heads, context, head_dim, generator=gen)
    v = torch.randn(batch, n_kv_heads, context, head_dim, generator=gen)
    for h in range(n_kv_heads):
        ck = torch.randperm(head_dim, generator=gen)[:n_outliers]
        cv = torch.randperm(head_dim, generator=gen)[:n_outliers]
        k[:, h, :, ck] *= outlier_scale
        v[:, h, :, cv] *= outlier_scale
    q = torch.randn(batch, n_q_heads, head_dim, generator=gen)
    pages_per_seq = (context + 15) // 16
    n_pages = batch * pages_per_seq
    page_ids = torch.randperm(n_pages, generator=gen).to(torch.int32).reshape(batch, pages_per_seq)
    return KvCase(k.half().to(device), v.half().to(device), q.half().to(device),
                  page_ids.to(device), n_pages)
