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

import ctypes
from typing import Dict, Tuple

import torch

from .. import _lib

from ..fused_attention import TQPagedAttention
from ..fused_kv_update import fused_tq4_kv_update
from ..quantizer import TurboQuant

_quantizers: Dict[int, TurboQuant] = {}        # head_size -> quantiser
_attn: Dict[Tuple[int, int, int], TQPagedAttention] = {}   # (head_size, layer, num_heads) -> attention
_registered = False
_step_state: Dict[tuple, object] = {}            # cached argument blocks of decode_step


def init_quantizer(head_size: int, bits: int = 4, device: str = "cuda", **kw) -> TurboQuant:
    """Create (or replace) the process-wide quantiser for one head size."""
    tq = TurboQuant(head_dim=head_size, bits=bits, device=device, **kw)
    _quantizers[head_size] = tq
    for key in [k for k in _attn if k[0] == head_size]:
        del _attn[key]
    _step_state.clear()
    return tq


def _get_tq(head_size: int) -> Tuple[TurboQuant, int]:
    tq = _quantizers.get(head_size)
    if tq is None:
        raise RuntimeError(f"no quantiser for head_size {head_size}: call init_quantizer() first")
    return tq, tq._packed_dim


def _decode_step_slow(query, key, value, kv_cache, output, k_norms, v_norms, slot_mapping, block_table,
                      seq_lens, layer_idx, num_heads, num_kv_heads, head_size, scale, num_actual):
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


def decode_step(query, key, value, kv_cache, output, k_norms, v_norms, slot_mapping, block_table,
                seq_lens, layer_idx: int, num_heads: int, num_kv_heads: int, head_size: int,
                scale: float, num_actual: int) -> torch.Tensor:
    """Body of ``tq::decode_step``: one call into ``akv_tq_decode_step`` (both cache writes and the
    attention) with an argument block that is reused while the caller keeps its cache, norm and
    output buffers; anything unusual (strided last dimensions, other index dtypes) takes the
    step-by-step path above."""
    fast = (key.dtype == value.dtype and key.dtype in _lib._FLOAT_CODES and query.dtype in _lib._FLOAT_CODES
            and key.stride(-1) == 1 and value.stride(-1) == 1 and query.stride(-1) == 1
            and slot_mapping.dtype == torch.int64 and slot_mapping.is_contiguous()
            and block_table.dim() == 2 and block_table.stride(-1) == 1 and seq_lens.is_contiguous()
            and block_table.dtype in _lib._INDEX_CODES and seq_lens.dtype in _lib._INDEX_CODES
            and output.dtype in _lib._FLOAT_CODES and output.stride(-1) == 1
            and query.is_cuda and kv_cache.is_cuda and key.shape[0] > 0 and num_actual > 0)
    if not fast:
        return _decode_step_slow(query, key, value, kv_cache, output, k_norms, v_norms, slot_mapping,
                                 block_table, seq_lens, layer_idx, num_heads, num_kv_heads, head_size,
                                 scale, num_actual)
    tq, pd = _get_tq(head_size)
    dev = query.device
    # the reference's indexing raises on mismatched sizes; raw pointers would read or write out of bounds
    if slot_mapping.numel() < key.shape[0] or value.shape[0] != key.shape[0]:
        raise ValueError(f"decode_step: {key.shape[0]} key tokens, {value.shape[0]} value tokens, "
                         f"{slot_mapping.numel()} slots")
    if min(query.shape[0], output.shape[0], block_table.shape[0], seq_lens.numel()) < num_actual:
        raise ValueError(f"decode_step: num_actual={num_actual} exceeds query/output/block_table/seq_lens rows "
                         f"({query.shape[0]}, {output.shape[0]}, {block_table.shape[0]}, {seq_lens.numel()})")
    if kv_cache.dim() != 5 or kv_cache.shape[1] != 2 or kv_cache.shape[3] != num_kv_heads or kv_cache.shape[4] < pd:
        raise ValueError(f"decode_step: kv_cache {tuple(kv_cache.shape)} does not hold [blocks, 2, block_size, "
                         f"{num_kv_heads}, >= {pd}]")
    want_norms = (kv_cache.shape[0], kv_cache.shape[2], num_kv_heads)
    if (k_norms.dim() != 4 or v_norms.dim() != 4 or not 0 <= layer_idx < k_norms.shape[0]
            or tuple(k_norms.shape[1:]) != want_norms or tuple(v_norms.shape) != tuple(k_norms.shape)):
        raise ValueError(f"decode_step: norms {tuple(k_norms.shape)} / {tuple(v_norms.shape)} do not match "
                         f"[layers > {layer_idx}, {want_norms[0]}, {want_norms[1]}, {want_norms[2]}]")
    state_key = (kv_cache.data_ptr(), tuple(kv_cache.shape), tuple(kv_cache.stride()), k_norms.data_ptr(),
                 v_norms.data_ptr(), tuple(k_norms.shape), tuple(k_norms.stride()), tuple(v_norms.stride()),
                 dev.index, tq.bits, layer_idx, num_heads, num_kv_heads, head_size,
                 num_actual, block_table.shape[1], tq.rotation.data_ptr(), tq.rotation_T.data_ptr(),
                 tq.centroids.data_ptr(), tq.boundaries_inner.data_ptr())
    st = _step_state.get(state_key)
    if st is None:
        if kv_cache.dtype != torch.uint8 or kv_cache.stride(-1) != 1:
            raise ValueError("kv_cache must be uint8 with a contiguous last dimension")
        if k_norms.dtype != torch.float32 or v_norms.dtype != torch.float32:
            raise TypeError("norm tensors must be float32")
        attn = _attn.get((head_size, layer_idx, num_heads))
        if attn is None:
            attn = TQPagedAttention(tq, num_heads)
            _attn[(head_size, layer_idx, num_heads)] = attn
        kc, vc = kv_cache[:, 0, :, :, :pd], kv_cache[:, 1, :, :, :pd]
        kn, vn = k_norms[layer_idx], v_norms[layer_idx]
        block_size = kv_cache.shape[2]
        L = _lib.lib()
        nbytes = L.akv_tq_paged_attn_workspace_bytes(num_actual, num_heads, num_kv_heads, head_size, tq.bits,
                                                     block_size, block_table.shape[1], attn.SPLITK_BLOCKS)
        ws = attn._get_workspace(nbytes, dev)
        p = _lib.TQDecodeStepParams()
        p.boundaries = tq.boundaries_inner.data_ptr()
        p.max_blocks = kv_cache.shape[0]
        a = p.attn
        a.k_packed, a.v_packed = kc.data_ptr(), vc.data_ptr()
        a.kp_stride_blk, a.kp_stride_pos, a.kp_stride_head = kc.stride(0), kc.stride(1), kc.stride(2)
        a.vp_stride_blk, a.vp_stride_pos, a.vp_stride_head = vc.stride(0), vc.stride(1), vc.stride(2)
        a.k_norms, a.v_norms = kn.data_ptr(), vn.data_ptr()
        a.kn_stride_blk, a.kn_stride_pos, a.kn_stride_head = kn.stride(0), kn.stride(1), kn.stride(2)
        a.vn_stride_blk, a.vn_stride_pos, a.vn_stride_head = vn.stride(0), vn.stride(1), vn.stride(2)
        a.num_seqs, a.num_q_heads, a.num_kv_heads, a.head_dim = num_actual, num_heads, num_kv_heads, head_size
        a.block_size, a.max_blocks_per_seq, a.num_blocks = block_size, block_table.shape[1], kv_cache.shape[0]
        a.bits = tq.bits
        a.rotation, a.rotation_t, a.centroids = (tq.rotation.data_ptr(), tq.rotation_T.data_ptr(),
                                                 tq.centroids.data_ptr())
        a.workspace, a.workspace_bytes = ws.data_ptr(), ws.numel()
        a.blocks_per_split = attn.SPLITK_BLOCKS
        st = (p, ws, (kc, vc, kn, vn))
        _step_state[state_key] = st
    p = st[0]
    a = p.attn
    p.key, p.value, p.kv_dtype = key.data_ptr(), value.data_ptr(), _lib._FLOAT_CODES[key.dtype]
    p.num_tokens = key.shape[0]
    p.k_stride_tok, p.k_stride_head = key.stride(0), key.stride(1)
    p.v_stride_tok, p.v_stride_head = value.stride(0), value.stride(1)
    p.slot_mapping = slot_mapping.data_ptr()
    a.query, a.q_dtype = query.data_ptr(), _lib._FLOAT_CODES[query.dtype]
    a.q_stride_seq, a.q_stride_head = query.stride(0), query.stride(1)
    a.block_tables, a.bt_dtype, a.bt_stride_seq = (block_table.data_ptr(), _lib._INDEX_CODES[block_table.dtype],
                                                   block_table.stride(0))
    a.context_lens, a.cl_dtype = seq_lens.data_ptr(), _lib._INDEX_CODES[seq_lens.dtype]
    a.scale = float(scale)
    a.out, a.out_dtype = output.data_ptr(), _lib._FLOAT_CODES[output.dtype]
    a.out_stride_seq, a.out_stride_head = output.stride(0), output.stride(1)
    a.stream = torch.cuda.current_stream(dev).cuda_stream
    # the op returns a copy of `output`: when every row of `output` is written by this call the merge kernel
    # writes the copy itself (one launch less than a clone)
    res = None
    if num_actual == output.shape[0]:
        res = torch.empty(output.shape, dtype=output.dtype, device=dev)
    a.out_copy = res.data_ptr() if res is not None else None
    if torch.cuda.current_device() == dev.index:
        rc = _lib.lib().akv_tq_decode_step(ctypes.byref(p))
    else:
        with torch.cuda.device(dev):
            rc = _lib.lib().akv_tq_decode_step(ctypes.byref(p))
    _lib.check(rc, "akv_tq_decode_step")
    return res if res is not None else output.clone()


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
    dense SDPA, this attends over the records directly (``akv_hybrid_decode_step``: cache write and
    attention in three kernel launches).  Tokens with a negative slot are skipped."""
    from ..hybrid_quantizer import HybridPagedAttention
    htq = _hybrid.get(head_size)
    if htq is None:
        raise RuntimeError(f"no hybrid quantiser for head_size {head_size}: call init_hybrid_quantizer() first")
    pd = htq.packed_dim
    if kv_cache.dim() != 5 or kv_cache.shape[1] != 2 or kv_cache.shape[3] != num_kv_heads or kv_cache.shape[4] < pd:
        raise ValueError(f"hybrid_decode_step: kv_cache {tuple(kv_cache.shape)} does not hold [blocks, 2, block_size, "
                         f"{num_kv_heads}, >= {pd}]")
    if min(query.shape[0], output.shape[0], block_table.shape[0], seq_lens.numel()) < num_actual:
        raise ValueError(f"hybrid_decode_step: num_actual={num_actual} exceeds query/output/block_table/seq_lens rows")
    key_cache, value_cache = kv_cache[:, 0], kv_cache[:, 1]
    block_size = key_cache.shape[1]
    attn = _hybrid_attn.get((head_size, num_heads))
    if attn is None:
        attn = HybridPagedAttention(htq, num_heads)
        _hybrid_attn[(head_size, num_heads)] = attn
    # one call: the records of the new tokens are written by the attention's first launch
    attn.forward(query[:num_actual], key_cache[..., :pd], value_cache[..., :pd], block_table, seq_lens,
                 block_size=block_size, num_kv_heads=num_kv_heads, out=output[:num_actual], scale=scale,
                 new_kv=(key, value, slot_mapping))
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
