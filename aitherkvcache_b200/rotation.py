"""Seeded orthogonal transforms used by the quantisers.

Same functions as the reference's ``aither_kvcache/rotation.py``
(``random_orthogonal`` :20-35, ``hadamard_matrix`` :38-50, ``random_signs``
:53-57, ``randomized_hadamard_matrix`` :60-81, ``fast_hadamard_transform``
:84-108).  The matrices are built once at construction time on the host with
torch's CPU generator - that is what fixes their values for a given seed - and
then live on the device as kernel operands.
"""
from __future__ import annotations

import math

import torch


def random_orthogonal(d: int, seed: int = 42, device: str = "cuda",
                      dtype: torch.dtype = torch.float32) -> torch.Tensor:
    """Haar-distributed orthogonal matrix: QR of a seeded Gaussian matrix with
    the column signs fixed so that diag(R) > 0 (Mezzadri 2007)."""
    g = torch.Generator(device="cpu")
    g.manual_seed(seed)
    gauss = torch.randn(d, d, generator=g, dtype=dtype)
    q, r = torch.linalg.qr(gauss)
    s = torch.sign(torch.diagonal(r))
    s = torch.where(s == 0, torch.ones_like(s), s)
    return (q * s[None, :]).to(device=device)


def hadamard_matrix(d: int, dtype: torch.dtype = torch.float32) -> torch.Tensor:
    """Orthonormal Walsh-Hadamard matrix (Sylvester construction), d a power of two."""
    assert d > 0 and d & (d - 1) == 0, f"d must be power of 2, got {d}"
    h = torch.ones(1, 1, dtype=dtype)
    while h.shape[0] < d:
        h = torch.cat([torch.cat([h, h], 1), torch.cat([h, -h], 1)], 0)
    return h / math.sqrt(d)


def random_signs(d: int, seed: int = 42, device: str = "cuda") -> torch.Tensor:
    """Seeded +-1 vector."""
    g = torch.Generator(device="cpu")
    g.manual_seed(seed)
    b = torch.randint(0, 2, (d,), generator=g, dtype=torch.float32)
    return (b * 2 - 1).to(device)


def randomized_hadamard_matrix(d: int, seed: int = 42, device: str = "cuda",
                               dtype: torch.dtype = torch.float32,
                               num_rounds: int = 3) -> torch.Tensor:
    """H D_k ... H D_1 as a dense matrix (the kernels treat it like any rotation)."""
    h = hadamard_matrix(d, dtype=dtype).to(device)
    out = torch.eye(d, dtype=dtype, device=device)
    for r in range(num_rounds):
        signs = random_signs(d, seed=seed + r, device=device).to(dtype)
        out = h @ (signs[:, None] * out)
    return out


def fast_hadamard_transform(x: torch.Tensor) -> torch.Tensor:
    """Un-normalised Walsh-Hadamard transform of the last dimension (butterflies)."""
    d = x.shape[-1]
    assert d > 0 and d & (d - 1) == 0, f"last dim must be power of 2, got {d}"
    lead = x.shape[:-1]
    y = x.clone()
    h = 1
    while h < d:
        v = y.reshape(*lead, d // (2 * h), 2, h)
        y = torch.stack([v[..., 0, :] + v[..., 1, :], v[..., 0, :] - v[..., 1, :]], dim=-2).reshape(*lead, d)
        h *= 2
    return y
