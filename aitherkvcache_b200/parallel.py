"""Split-K across the GPUs of one node: every rank attends over its contiguous slice of the
key positions and emits an un-normalised partial (m, l, acc) per (sequence, query head);
one all-gather moves the partials (a few hundred KB) over NVLink and a local kernel merges
them by log-sum-exp (``akv_lse_merge``).  The reference has no multi-device path; the merge
arithmetic is that of its intra-GPU split-K reduce (``fused_attention.py:479-531``).

Batched decode needs none of this: sequences are independent, each rank serves its own.
"""
from __future__ import annotations

import ctypes
import os
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


class PeerExchange:
    """Exchange buffers for ``p2p_merge_partials``: one symmetric-memory allocation per rank that every
    peer of the node can write over NVLink (``torch.distributed._symmetric_memory``; no multicast object
    is requested), holding the double-buffered partial slots of all ranks followed by one flag word per
    rank, plus two local state words (step counter, current half).  Collective: every rank of ``group``
    constructs it with the same sizes, in the same order."""

    def __init__(self, num_seqs: int, num_q_heads: int, head_dim: int, device, group=None):
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")      # plain peer stores only
        import torch.distributed._symmetric_memory as symm_mem
        self.group = group if group is not None else dist.group.WORLD
        self.world, self.rank = dist.get_world_size(self.group), dist.get_rank(self.group)
        self.num_seqs, self.num_q_heads, self.head_dim = num_seqs, num_q_heads, head_dim
        self.device = torch.device(device)
        nbytes = _lib.lib().akv_p2p_exchange_bytes(self.world, num_seqs, num_q_heads, head_dim)
        assert nbytes % 16 == 0
        with torch.cuda.device(self.device):
            self.buf = symm_mem.empty(nbytes // 4 + 64, dtype=torch.float32, device=self.device)
            self.buf.zero_()
            self.handle = symm_mem.rendezvous(self.buf, self.group)
            ptrs = [int(p) for p in self.handle.buffer_ptrs]
            self.peer_buffers = (ctypes.c_void_p * self.world)(*ptrs)
            self.peer_flags = (ctypes.c_void_p * self.world)(*[p + nbytes for p in ptrs])
            self.state = torch.zeros(2, dtype=torch.int32, device=self.device)
            torch.cuda.synchronize(self.device)
        dist.barrier(self.group)          # every rank's zeroes are in place before anyone pushes


def p2p_merge_partials(exchange: PeerExchange, raw: torch.Tensor, rotation: Optional[torch.Tensor] = None,
                       out: Optional[torch.Tensor] = None, out_dtype: torch.dtype = torch.float32) -> torch.Tensor:
    """The all-gather + merge of ``all_gather_partials`` / ``merge_partials`` as three small kernels over
    peer memory (``akv_p2p_lse_merge``): every rank stores its partial ``raw`` [rows, D+2] into all ranks'
    exchange buffers, waits (bounded) for the others' partials of the same step, and merges locally.
    Every rank of the group must call it the same number of times."""
    dev = _lib.require_cuda(raw, rotation)
    S, QH, D = exchange.num_seqs, exchange.num_q_heads, exchange.head_dim
    assert raw.dtype == torch.float32 and raw.is_contiguous() and raw.shape == (S * QH, D + 2)
    if out is None:
        out = torch.empty(S, QH, D, dtype=out_dtype, device=dev)
    p = _lib.P2PMergeParams()
    p.local_raw = raw.data_ptr()
    p.num_seqs, p.num_q_heads, p.head_dim = S, QH, D
    p.world, p.rank = exchange.world, exchange.rank
    p.peer_buffers = ctypes.cast(exchange.peer_buffers, ctypes.POINTER(ctypes.c_void_p))
    p.peer_flags = ctypes.cast(exchange.peer_flags, ctypes.POINTER(ctypes.c_void_p))
    p.state = exchange.state.data_ptr()
    p.rotation = _lib.ptr(rotation)
    p.out, p.out_dtype, p.out_stride_seq, p.out_stride_head = out.data_ptr(), _lib.float_code(out), out.stride(0), out.stride(1)
    p.stream = _lib.stream_ptr(dev)
    with torch.cuda.device(dev):
        rc = _lib.lib().akv_p2p_lse_merge(ctypes.byref(p))
    _lib.check(rc, "akv_p2p_lse_merge")
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
