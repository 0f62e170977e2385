"""Fused "reshape_and_cache" for a TurboQuant-packed paged KV cache.

Interface of the reference's ``aither_kvcache/fused_kv_update.py``
(``fused_tq4_kv_update`` :300-405, ``fused_encode_and_store`` :412-468): one
kernel launch per cache tensor reads raw K or V vectors, encodes them and
scatter-writes packed codes and norms to ``slot_mapping`` positions.  Unlike the
reference this also covers 3- and 2-bit codebooks (the bit width is inferred
from the number of boundaries).
"""
from __future__ import annotations

import torch

from . import _lib

_BITS_FROM_BOUNDARIES = {15: 4, 7: 3, 3: 2}
_rot_t_cache: dict = {}


def _transposed(rotation: torch.Tensor) -> torch.Tensor:
    """R^T, contiguous, cached per rotation tensor (the kernel reads columns of R)."""
    key = (rotation.data_ptr(), rotation._version, tuple(rotation.shape), str(rotation.device))
    hit = _rot_t_cache.get(key)
    if hit is None:
        if len(_rot_t_cache) > 64:
            _rot_t_cache.clear()
        hit = rotation.to(torch.float32).t().contiguous()
        _rot_t_cache[key] = hit
    return hit


def fused_tq4_kv_update(
    x: torch.Tensor,
    slot_mapping: torch.Tensor,
    out_packed: torch.Tensor,
    out_norms: torch.Tensor,
    rotation: torch.Tensor,
    boundaries: torch.Tensor,
    block_size: int = 16,
    max_blocks: int = 0,
    rotation_t: torch.Tensor = None,
) -> None:
    """Encode ``x`` [tokens, kv_heads, head_dim] into ``out_packed``
    [blocks, block_size, kv_heads, packed_dim] / ``out_norms`` [blocks, block_size, kv_heads]
    in place.  Tokens whose slot is negative or falls outside ``max_blocks`` are skipped."""
    if max_blocks == 0:
        max_blocks = out_packed.shape[0]
    num_tokens, num_kv_heads, head_dim = x.shape
    if num_tokens == 0:
        return
    if head_dim <= 0 or head_dim & (head_dim - 1):
        raise ValueError(f"head_dim must be a power of 2, got {head_dim}")
    bits = _BITS_FROM_BOUNDARIES.get(boundaries.numel())
    if bits is None:
        raise ValueError(f"expected 15, 7 or 3 boundaries, got {boundaries.numel()}")
    dev = _lib.require_cuda(x, slot_mapping, out_packed, out_norms, rotation, boundaries)
    if x.dtype not in _lib._FLOAT_CODES:
        x = x.float()
    if x.stride(-1) != 1:
        x = x.contiguous()
    if out_packed.stride(-1) != 1:
        raise ValueError("out_packed must be contiguous in its last dimension")
    if out_norms.dtype != torch.float32 or out_packed.dtype != torch.uint8:
        raise TypeError("out_packed must be uint8 and out_norms float32")
    slots = slot_mapping.to(torch.int64).contiguous()
    rt = rotation_t if rotation_t is not None else _transposed(rotation)
    bnd = boundaries.to(torch.float32).contiguous()
    with torch.cuda.device(dev):
        rc = _lib.lib().akv_tq_kv_update(
            x.data_ptr(), _lib.float_code(x), num_tokens, num_kv_heads, head_dim, x.stride(0), x.stride(1),
            slots.data_ptr(), out_packed.data_ptr(), out_packed.stride(0), out_packed.stride(1),
            out_packed.stride(2), out_norms.data_ptr(), out_norms.stride(0), out_norms.stride(1),
            out_norms.stride(2), bits, rt.data_ptr(), bnd.data_ptr(), block_size, max_blocks,
            _lib.stream_ptr(dev))
    _lib.check(rc, "akv_tq_kv_update")


def fused_encode_and_store(tq_cache, layer_idx: int, key: torch.Tensor, value: torch.Tensor,
                           slot_mapping: torch.Tensor) -> None:
    """K and V of one layer into a cache object with ``tq``, ``k_packed``, ``k_norms``,
    ``v_packed``, ``v_norms`` (each indexed by layer), ``block_size`` and ``max_blocks``."""
    tq = tq_cache.tq
    for x, packed, norms in ((key, tq_cache.k_packed, tq_cache.k_norms),
                             (value, tq_cache.v_packed, tq_cache.v_norms)):
        fused_tq4_kv_update(x=x, slot_mapping=slot_mapping, out_packed=packed[layer_idx],
                            out_norms=norms[layer_idx], rotation=tq.rotation,
                            boundaries=tq.boundaries_inner, block_size=tq_cache.block_size,
                            max_blocks=tq_cache.max_blocks, rotation_t=getattr(tq, "rotation_T", None))
