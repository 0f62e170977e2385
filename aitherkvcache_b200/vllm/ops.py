"""``tq::decode_step`` / ``tq::hybrid_decode_step``: encode the new token's K/V into the packed cache, then paged
decode attention over it - one call, no host synchronisation.

Same schema as the reference's op (``aither_kvcache/vllm/hooks.py:129-205``):

    tq::decode_step(query, key, value, kv_cache, output, k_norms, v_norms, slot_mapping,
                    block_table, seq_lens, int layer_idx, int num_heads, int num_kv_heads,
                    int head_size, float scale, int num_actual) -> Tensor
    mutates kv_cache, output, k_norms, v_norms; returns output.clone()

    kv_cache  uint8 [num_blocks, 2, block_size, num_kv_heads, >= packed_dim]
    k_norms   float32 [layers, num_blocks, block_size, num_kv_heads]

Differences from the reference body: tokens with a negative slot are skipped instead of
wrapping to the last block, and ``scale`` is honoured (the reference ignores it and always
uses 1/sqrt(head_size)).
"""
from __future__ import annotations

from typing import Dict, Tuple

import torch

from ..fused_attention import TQPagedAttention
from ..fused_kv_update import fused_tq4_kv_update
from ..quantizer import TurboQuant

_quantizers: Dict[int, TurboQuant] = {}        # head_size -> quantiser
_attn: Dict[Tuple[int, int, int], TQPagedAttention] = {}   # (head_size, layer, num_heads) -> attention
_registered = False


def init_quantizer(head_size: int, bits: int = 4, device: str = "cuda", **kw) -> TurboQuant:
    """Create (or replace) the process-wide quantiser for one head size."""
    tq = TurboQuant(head_dim=head_size, bits=bits, device=device, **kw)
    _quantizers[head_size] = tq
    for key in [k for k in _attn if k[0] == head_size]:
        del _attn[key]
    return tq


def _get_tq(head_size: int) -> Tuple[TurboQuant, int]:
    tq = _quantizers.get(head_size)
    if tq is None:
        raise RuntimeError(f"no quantiser for head_size {head_size}: call init_quantizer() first")
    return tq, tq._packed_dim


def decode_step(query, key, value, kv_cache, output, k_norms, v_norms, slot_mapping, block_table,
                seq_lens, layer_idx: int, num_heads: int, num_kv_heads: int, head_size: int,
                scale: float, num_actual: int) -> torch.Tensor:
    tq, pd = _get_tq(head_size)
    key_cache, value_cache = kv_cache[:, 0], kv_cache[:, 1]
    block_size = key_cache.shape[1]
    kc, vc = key_cache[..., :pd], value_cache[..., :pd]
    kn, vn = k_norms[layer_idx], v_norms[layer_idx]
    for x, cache, norms in ((key, kc, kn), (value, vc, vn)):
        fused_tq4_kv_update(x, slot_mapping, cache, norms, tq.rotation, tq.boundaries_inner,
                            block_size, cache.shape[0], rotation_t=tq.rotation_T)
    attn = _attn.get((head_size, layer_idx, num_heads))
    if attn is None:
        attn = TQPagedAttention(tq, num_heads)
        _attn[(head_size, layer_idx, num_heads)] = attn
    attn.forward(query[:num_actual], kc, kn, vc, vn, block_table, seq_lens, block_size=block_size,
                 num_kv_heads=num_kv_heads, out=output[:num_actual], scale=scale)
    return output.clone()


_hybrid: Dict[int, object] = {}                # head_size -> HybridTurboQuant
_hybrid_attn: Dict[Tuple[int, int], object] = {}


def init_hybrid_quantizer(head_size: int, mode: str = "tq35", device: str = "cuda", **kw):
    """Create (or replace) the process-wide hybrid quantiser for one head size."""
    from ..hybrid_quantizer import HybridTurboQuant
    htq = HybridTurboQuant(head_dim=head_size, mode=mode, device=device, **kw)
    htq.calibrate_uniform()
    _hybrid[head_size] = htq
    for key in [k for k in _hybrid_attn if k[0] == head_size]:
        del _hybrid_attn[key]
    return htq


def hybrid_decode_step(query, key, value, kv_cache, output, slot_mapping, block_table, seq_lens,
                       layer_idx: int, num_heads: int, num_kv_heads: int, head_size: int, scale: float,
                       num_actual: int) -> torch.Tensor:
    """Same schema as the reference's ``tq::hybrid_decode_step`` (``vllm/hooks.py:240-355``):
    encode the new K/V records into ``kv_cache`` (uint8 ``[blocks, 2, block_size, kv_heads, >= packed_dim]``,
    norms embedded), then attend.  Where the reference decompresses every referenced block and runs
    dense SDPA, this attends over the records directly.  Tokens with a negative slot are skipped."""
    from ..hybrid_quantizer import HybridPagedAttention
    htq = _hybrid.get(head_size)
    if htq is None:
        raise RuntimeError(f"no hybrid quantiser for head_size {head_size}: call init_hybrid_quantizer() first")
    pd = htq.packed_dim
    key_cache, value_cache = kv_cache[:, 0], kv_cache[:, 1]
    block_size = key_cache.shape[1]
    n, h, d = key.shape
    valid = (slot_mapping >= 0).view(-1, 1, 1)
    slot = slot_mapping.clamp(min=0)
    bi, oi = slot // block_size, slot % block_size
    for x, cache in ((key, key_cache), (value, value_cache)):
        rec = htq.encode(x.reshape(n * h, d)).reshape(n, h, pd)
        cache[bi, oi, :, :pd] = torch.where(valid, rec, cache[bi, oi, :, :pd])
    attn = _hybrid_attn.get((head_size, num_heads))
    if attn is None:
        attn = HybridPagedAttention(htq, num_heads)
        _hybrid_attn[(head_size, num_heads)] = attn
    attn.forward(query[:num_actual], key_cache[..., :pd], value_cache[..., :pd], block_table, seq_lens,
                 block_size=block_size, num_kv_heads=num_kv_heads, out=output[:num_actual], scale=scale)
    return output.clone()


def register_custom_ops() -> bool:
    """Register ``tq::decode_step`` and ``tq::hybrid_decode_step`` with ``torch.library`` (idempotent)."""
    global _registered
    if _registered:
        return True
    if not hasattr(torch.library, "custom_op"):
        return False

    @torch.library.custom_op("tq::decode_step", mutates_args=("kv_cache", "output", "k_norms", "v_norms"))
    def _op(query: torch.Tensor, key: torch.Tensor, value: torch.Tensor, kv_cache: torch.Tensor,
            output: torch.Tensor, k_norms: torch.Tensor, v_norms: torch.Tensor,
            slot_mapping: torch.Tensor, block_table: torch.Tensor, seq_lens: torch.Tensor,
            layer_idx: int, num_heads: int, num_kv_heads: int, head_size: int, scale: float,
            num_actual: int) -> torch.Tensor:
        return decode_step(query, key, value, kv_cache, output, k_norms, v_norms, slot_mapping,
                           block_table, seq_lens, layer_idx, num_heads, num_kv_heads, head_size, scale,
                           num_actual)

    @_op.register_fake
    def _fake(query, key, value, kv_cache, output, k_norms, v_norms, slot_mapping, block_table, seq_lens,
              layer_idx, num_heads, num_kv_heads, head_size, scale, num_actual):
        return output.clone()

    @torch.library.custom_op("tq::hybrid_decode_step", mutates_args=("kv_cache", "output"))
    def _hop(query: torch.Tensor, key: torch.Tensor, value: torch.Tensor, kv_cache: torch.Tensor,
             output: torch.Tensor, slot_mapping: torch.Tensor, block_table: torch.Tensor,
             seq_lens: torch.Tensor, layer_idx: int, num_heads: int, num_kv_heads: int, head_size: int,
             scale: float, num_actual: int) -> torch.Tensor:
        return hybrid_decode_step(query, key, value, kv_cache, output, slot_mapping, block_table, seq_lens,
                                  layer_idx, num_heads, num_kv_heads, head_size, scale, num_actual)

    @_hop.register_fake
    def _hfake(query, key, value, kv_cache, output, slot_mapping, block_table, seq_lens, layer_idx,
               num_heads, num_kv_heads, head_size, scale, num_actual):
        return output.clone()

    _registered = True
    return True
