"""Magnitude thresholding of activations (API of ``leankv/teal/sparse_fns.py``).

``SparsifyFn`` is the hook-mode primitive: it zeroes activations with ``|x| <= t`` using
ordinary tensor ops and leaves the matmul dense, exactly like the reference's
"correctness only" mode. The speed path does not call it: the CUDA sparse GEMV applies
the same test (strict ``>``, threshold rounded to the activation dtype) inside the kernel.
"""

from __future__ import annotations

import torch


class SparsifyFn:
    """Zero every activation whose magnitude does not exceed ``threshold``."""

    def __init__(self, threshold: float = 0.0, enabled: bool = True):
        self.threshold = threshold
        self.enabled = enabled
        self._kept_fraction = None   # 0-dim tensor from the last call; read lazily

    def __call__(self, x: torch.Tensor) -> torch.Tensor:
        if not self.enabled or self.threshold <= 0:
            return x
        keep = x.abs() > self.threshold
        # The reference calls .item() here, which stalls the stream on every projection;
        # the statistic is kept on the device and only read when someone asks for it.
        self._kept_fraction = keep.float().mean()
        return x * keep

    @property
    def _last_sparsity(self) -> float:
        return 0.0 if self._kept_fraction is None else 1.0 - float(self._kept_fraction.item())

    @property
    def last_sparsity(self) -> float:
        """Fraction of activations zeroed by the most recent call."""
        return self._last_sparsity


def compute_threshold_for_sparsity(activations: torch.Tensor, target_sparsity: float) -> float:
    """Magnitude of the k-th smallest |activation|, k = int(target_sparsity * numel).

    Same order statistic as ``sparse_fns.py:47-69`` (``torch.kthvalue``), so thresholds
    and therefore masks are identical to the reference's for the same activations.
    """
    mags = activations.abs().flatten()
    k = int(target_sparsity * mags.numel())
    if k <= 0:
        return 0.0
    if k >= mags.numel():
        return mags.max().item()
    return torch.kthvalue(mags, k).values.item()


def compute_threshold_from_histogram(hist_counts: torch.Tensor, hist_edges: torch.Tensor,
                                     target_sparsity: float) -> float:
    """Threshold at which the histogram's CDF reaches ``target_sparsity`` (``sparse_fns.py:72-103``).

    Linear interpolation inside the crossing bin; the first bin returns its left edge.
    """
    cdf = hist_counts.cumsum(0).float()
    cdf = cdf / cdf[-1]
    b = min(int(torch.searchsorted(cdf, target_sparsity).item()), len(hist_edges) - 2)
    if b == 0:
        return hist_edges[0].item()
    below = cdf[b - 1]
    frac = (target_sparsity - below) / (cdf[b] - below + 1e-10)
    return (hist_edges[b] + frac * (hist_edges[b + 1] - hist_edges[b])).item()
