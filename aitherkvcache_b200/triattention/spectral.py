"""RoPE-pair primitives (interface of the reference's ``triattention/spectral.py:34-110``)."""
import torch


def rope_frequencies(head_dim: int, base: float = 1_000_000.0, device: str = "cpu",
                     dtype: torch.dtype = torch.float32) -> torch.Tensor:
    """theta_i = base^(-2i/d), i = 0 .. d/2-1, evaluated in ``dtype`` like the reference."""
    i = torch.arange(head_dim // 2, device=device, dtype=dtype)
    return base ** (-2.0 * i / head_dim)


def pair_energies(x: torch.Tensor) -> torch.Tensor:
    """E_i = x[2i]^2 + x[2i+1]^2."""
    p = x.reshape(*x.shape[:-1], x.shape[-1] // 2, 2)
    return (p ** 2).sum(dim=-1)


def spectral_concentration(x: torch.Tensor, k: int) -> torch.Tensor:
    """Share of the energy held by the k strongest pairs."""
    e = pair_energies(x.float())
    return e.topk(k, dim=-1).values.sum(-1) / (e.sum(-1) + 1e-12)
