"""Split-K across the GPUs of one node: every rank attends over its contiguous slice of the
key positions and emits an un-normalised partial (m, l, acc) per (sequence, query head);
one all-gather moves the partials (a few hundred KB) over NVLink and a local kernel merges
them by log-sum-exp (``akv_lse_merge``).  The reference has no multi-device path; the merge
arithmetic is that of its intra-GPU split-K reduce (``fused_attention.py:479-531``).

Batched decode needs none of this: sequences are independent, each rank serves its own.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch
import torch.distributed as dist

from . import _lib


def shard_range(total: int, rank: int, world: int, multiple: int = 1) -> Tuple[int, int]:
    """Contiguous [lo, hi) slice of ``total`` positions for ``rank``; boundaries are multiples
    of ``multiple`` (e.g. the KV block size) and trailing ranks may be empty."""
    per = -(-total // world)
    per = -(-per // multiple) * multiple
    lo = min(rank * per, total)
    return lo, min(lo + per, total)


def all_gather_partials(raw: torch.Tensor, group=None) -> torch.Tensor:
    """[rows, D+2] on every rank -> [world, rows, D+2] on every rank (one collective)."""
    world = dist.get_world_size(group)
    out = torch.empty((world,) + tuple(raw.shape), dtype=raw.dtype, device=raw.device)
    if raw.is_cuda:
        dist.all_gather_into_tensor(out, raw.contiguous(), group=group)     # one NCCL all-gather
    else:                                                                   # host tensors (tests on gloo)
        dist.all_gather(list(out.unbind(0)), raw.contiguous(), group=group)
    return out


def merge_partials(parts: torch.Tensor, num_seqs: int, num_q_heads: int, head_dim: int,
                   rotation: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None,
                   out_dtype: torch.dtype = torch.float32) -> torch.Tensor:
    """LSE-merge ``parts`` [P, num_seqs*num_q_heads, head_dim+2] (CUDA, float32).  With ``rotation``
    (the TurboQuant matrix R) the result is rotated back, ``out = R^T (acc / l)``; without, ``acc / l``."""
    dev = _lib.require_cuda(parts, rotation)
    assert parts.dtype == torch.float32 and parts.is_contiguous()
    assert parts.shape[1:] == (num_seqs * num_q_heads, head_dim + 2)
    if out is None:
        out = torch.empty(num_seqs, num_q_heads, head_dim, dtype=out_dtype, device=dev)
    with torch.cuda.device(dev):
        rc = _lib.lib().akv_lse_merge(parts.data_ptr(), parts.shape[0], num_seqs, num_q_heads, head_dim,
                                      _lib.ptr(rotation), out.data_ptr(), _lib.float_code(out), out.stride(0),
                                      out.stride(1), _lib.stream_ptr(dev))
    _lib.check(rc, "akv_lse_merge")
    return out


def tri_decode_step_sharded(tri, query, k_enc_local, v_enc_local, lo: int, total_len: int,
                            query_pos: Optional[torch.Tensor] = None, group=None) -> torch.Tensor:
    """TriAttention decode step with the key positions [lo, lo + S_local) held by this rank.
    Positions default to 0..total_len-1 for keys and total_len for the query."""
    B, QH, D = query.shape
    raw = tri.decode_step_partial(query, k_enc_local, v_enc_local, query_pos=query_pos, key_pos_start=lo,
                                  query_pos_default=total_len)
    parts = all_gather_partials(raw, group)
    return merge_partials(parts, B, QH, D)


def tq_paged_attention_sharded(attn, query, k_packed, k_norms, v_packed, v_norms, block_tables_local,
                               context_lens_local, group=None, block_size: int = 16) -> torch.Tensor:
    """TurboQuant paged decode attention where each rank's block table / context length describe
    only the slice of every sequence that this rank stores."""
    S, QH, D = query.shape
    raw = torch.empty(S * QH, D + 2, dtype=torch.float32, device=query.device)
    attn.forward(query, k_packed, k_norms, v_packed, v_norms, block_tables_local, context_lens_local,
                 block_size=block_size, raw_out=raw)
    parts = all_gather_partials(raw, group)
    return merge_partials(parts, S, QH, D, rotation=attn.rotation, out_dtype=query.dtype)
