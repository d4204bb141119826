"""Random rotations for TurboQuant.

The rotation is generated on the host exactly as ``leankv/turboquant/rotation.py:12-29``
does (torch CPU generator -> Gaussian matrix -> QR -> sign fix), because it must be the
same matrix the reference would use for a given seed. It is a one-time 128x128 set-up
step; the per-vector rotations themselves run inside the CUDA kernels.
"""

from __future__ import annotations

import torch


def generate_rotation_matrix(d: int, device, dtype: torch.dtype = torch.float32,
                             seed: int = 42) -> torch.Tensor:
    """Orthogonal Pi in R^{d x d}: Q of a seeded Gaussian matrix, columns signed so R's diagonal is positive."""
    gen = torch.Generator(device="cpu").manual_seed(seed)
    gauss = torch.randn(d, d, generator=gen, dtype=torch.float32)
    q, r = torch.linalg.qr(gauss)
    q = q * torch.sign(torch.diagonal(r)).unsqueeze(0)
    # LAPACK hands Q back column-major; the kernels read Pi row-major, so fix the layout once here
    return q.contiguous().to(device=device, dtype=dtype)


def generate_qjl_matrix(d: int, device, dtype: torch.dtype = torch.float32,
                        seed: int = 12345) -> torch.Tensor:
    """i.i.d. N(0,1) projection used by the inner-product variant (rotation.py:32-42)."""
    gen = torch.Generator(device="cpu").manual_seed(seed)
    return torch.randn(d, d, generator=gen, dtype=torch.float32).to(device=device, dtype=dtype)


def rotate_forward(x: torch.Tensor, Pi: torch.Tensor) -> torch.Tensor:
    """y = x @ Pi^T (plain torch; the kernels fuse this step)."""
    return torch.matmul(x, Pi.T)


def rotate_backward(y: torch.Tensor, Pi: torch.Tensor) -> torch.Tensor:
    """x = y @ Pi."""
    return torch.matmul(y, Pi)
