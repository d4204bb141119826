"""Reference arithmetic of the TEAL path on CPU tensors (test infrastructure).

Follows leankv/teal/sparse_fns.py:32-39 (mask), :47-69 (threshold) and the B=1 branch of
leankv/teal/patching.py:169-177, whose result equals ``F.linear`` on the masked input.
"""

from __future__ import annotations

import torch
import torch.nn.functional as F


def sparsify(x: torch.Tensor, threshold: float) -> torch.Tensor:
    """x * (|x| > threshold); identity when threshold <= 0 (sparse_fns.py:34-39)."""
    if threshold <= 0:
        return x
    return x * (x.abs() > threshold)


def threshold_for_sparsity(acts: torch.Tensor, target: float) -> float:
    """k-th smallest magnitude, k = int(target * numel) (sparse_fns.py:47-69)."""
    mags = acts.abs().flatten()
    k = int(target * mags.numel())
    if k <= 0:
        return 0.0
    if k >= mags.numel():
        return mags.max().item()
    return torch.kthvalue(mags, k).values.item()


def threshold_from_histogram(counts: torch.Tensor, edges: torch.Tensor, target: float) -> float:
    """sparse_fns.py:72-103."""
    cdf = counts.cumsum(0).float()
    cdf = cdf / cdf[-1]
    idx = min(torch.searchsorted(cdf, target).item(), len(edges) - 2)
    if idx > 0:
        frac = (target - cdf[idx - 1]) / (cdf[idx] - cdf[idx - 1] + 1e-10)
        return (edges[idx] + frac * (edges[idx + 1] - edges[idx])).item()
    return edges[idx].item()


def n_active(x: torch.Tensor, threshold: float) -> int:
    return int((x.abs() > threshold).sum().item()) if threshold > 0 else x.numel()


def sparse_linear(x: torch.Tensor, weight: torch.Tensor, threshold: float,
                  accumulate: str = "native") -> torch.Tensor:
    """F.linear(sparsify(x), weight). accumulate: 'native' = the tensors' own dtype (the
    reference hook path), 'fp32' / 'fp64' = widened operands (tighter secondary oracle)."""
    xs = sparsify(x, threshold)
    if accumulate == "native":
        return F.linear(xs, weight)
    dt = torch.float32 if accumulate == "fp32" else torch.float64
    return F.linear(xs.to(dt), weight.to(dt))


def swiglu(x: torch.Tensor, w_gate: torch.Tensor, w_up: torch.Tensor, t_gate: float,
           t_up: float, accumulate: str = "native") -> torch.Tensor:
    """act_fn(gate_proj(x_g)) * up_proj(x_u) as the HF MLP computes it around the hooks
    (fp16 gate, fp16 up, SiLU and product in the activation dtype)."""
    g = sparse_linear(x, w_gate, t_gate, accumulate).to(x.dtype)
    u = sparse_linear(x, w_up, t_up, accumulate).to(x.dtype)
    return F.silu(g) * u
