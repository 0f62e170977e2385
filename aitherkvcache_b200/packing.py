"""MSB-first packing of 2/3/4-bit codes into bytes: the on-cache byte format.

Interface of the reference's ``aither_kvcache/packing.py`` (:13-131).  The
kernels pack and unpack in registers; these tensor helpers exist for callers
that hold raw codes.
  4-bit: byte = c[2k] << 4 | c[2k+1]
  2-bit: byte = c[4k] << 6 | c[4k+1] << 4 | c[4k+2] << 2 | c[4k+3]
  3-bit: eight codes form a 24-bit big-endian word (c[0] in bits 23..21) -> 3 bytes
"""
from __future__ import annotations

import torch


def packed_size(dim: int, bits: int) -> int:
    if bits == 4:
        return dim // 2
    if bits == 3:
        assert dim % 8 == 0
        return dim * 3 // 8
    if bits == 2:
        return dim // 4
    raise ValueError(f"Unsupported bit-width: {bits}")


def _fields(indices: torch.Tensor, per: int) -> torch.Tensor:
    d = indices.shape[-1]
    assert d % per == 0, f"Dimension must be divisible by {per}, got {d}"
    return indices.to(torch.int32).reshape(*indices.shape[:-1], d // per, per)


def pack_4bit(indices: torch.Tensor) -> torch.Tensor:
    f = _fields(indices, 2)
    return ((f[..., 0] << 4) | f[..., 1]).to(torch.uint8)


def pack_2bit(indices: torch.Tensor) -> torch.Tensor:
    f = _fields(indices, 4)
    return ((f[..., 0] << 6) | (f[..., 1] << 4) | (f[..., 2] << 2) | f[..., 3]).to(torch.uint8)


def pack_3bit(indices: torch.Tensor) -> torch.Tensor:
    f = _fields(indices, 8) & 7
    shifts = torch.arange(21, -1, -3, device=indices.device, dtype=torch.int32)
    word = (f << shifts).sum(-1)
    out = torch.stack([(word >> 16) & 255, (word >> 8) & 255, word & 255], dim=-1)
    return out.reshape(*indices.shape[:-1], -1).to(torch.uint8)


def unpack_4bit(packed: torch.Tensor, dim: int) -> torch.Tensor:
    p = packed.to(torch.int32)
    return torch.stack([p >> 4, p & 15], dim=-1).reshape(*packed.shape[:-1], dim).to(torch.uint8)


def unpack_2bit(packed: torch.Tensor, dim: int) -> torch.Tensor:
    p = packed.to(torch.int32)
    return torch.stack([p >> 6, (p >> 4) & 3, (p >> 2) & 3, p & 3], dim=-1).reshape(
        *packed.shape[:-1], dim).to(torch.uint8)


def unpack_3bit(packed: torch.Tensor, dim: int) -> torch.Tensor:
    g = packed.to(torch.int32).reshape(*packed.shape[:-1], dim // 8, 3)
    word = (g[..., 0] << 16) | (g[..., 1] << 8) | g[..., 2]
    shifts = torch.arange(21, -1, -3, device=packed.device, dtype=torch.int32)
    return ((word[..., None] >> shifts) & 7).reshape(*packed.shape[:-1], dim).to(torch.uint8)
