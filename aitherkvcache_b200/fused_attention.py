"""Paged decode attention that reads the TurboQuant-packed cache directly.

Interface of the reference's ``TQPagedAttention`` (``aither_kvcache/fused_attention.py``
:538-748).  The query is rotated once, scores and the value sum are formed in the
rotated domain from the packed codes, and the result is rotated back; no fp16 K/V is
materialised.  All of it - rotation, split-K partials, log-sum-exp merge, inverse
rotation - runs in the kernels behind ``akv_tq_paged_attn``.
"""
from __future__ import annotations

import ctypes
import math
import os
from typing import Optional

import torch

from . import _lib


class TQPagedAttention:
    """``attn = TQPagedAttention(tq, num_query_heads); out = attn.forward(...)``."""

    # Kept for interface compatibility.  The reference switches to split-K above
    # SPLITK_THRESHOLD blocks; here every call is split-K and only the split size
    # is tunable (AITHER_TQ_SPLITK_BLOCKS = KV blocks per work item, 0 = default).
    SPLITK_THRESHOLD = int(os.environ.get("AITHER_TQ_SPLITK_THRESHOLD", "64"))
    SPLITK_NUM_SPLITS = int(os.environ.get("AITHER_TQ_SPLITK_SPLITS", "16"))
    SPLITK_BLOCKS = int(os.environ.get("AITHER_TQ_SPLITK_BLOCKS", "0"))

    # bytes of scratch the staged prefill kernel may ask for (AITHER_TQ_PREFILL_SCRATCH_MB overrides; 0 = never staged)
    STAGED_WORKSPACE_LIMIT = int(os.environ.get("AITHER_TQ_PREFILL_SCRATCH_MB", "2048")) << 20

    def __init__(self, tq, num_query_heads: int, block_selector=None):
        # optional BlockSelector (block_selector.py): filters block_tables / context_lens per query on the
        # device before the attention kernels run (hook of the reference: fused_attention.py:664-668)
        self._block_selector = block_selector
        self.rotation = tq.rotation
        self.rotation_T = getattr(tq, "rotation_T", None)
        if self.rotation_T is None:
            self.rotation_T = tq.rotation.t().contiguous()
        self.centroids = tq.centroids
        self.scale = 1.0 / math.sqrt(tq.head_dim)
        self.head_dim = tq.head_dim
        self.num_levels = tq.num_levels
        self.bits = tq.bits
        self.packed_dim = tq._packed_dim
        self.num_query_heads = num_query_heads
        self._workspace: Optional[torch.Tensor] = None
        self._prefill_ws: Optional[torch.Tensor] = None
        self._params = None
        self._params_key = None

    def _build_params(self, dev, query, k_packed, k_norms, v_packed, v_norms, block_tables, context_lens,
                      block_size, num_kv_heads, out, raw_out, scale) -> "_lib.TQAttnParams":
        num_seqs, num_q_heads, head_dim = query.shape
        for name, t in (("k_packed", k_packed), ("v_packed", v_packed)):
            if t.dtype != torch.uint8 or t.stride(-1) != 1:
                raise ValueError(f"{name} must be uint8 with a contiguous last dimension")
        if k_norms.dtype != torch.float32 or v_norms.dtype != torch.float32:
            raise TypeError("norm tensors must be float32")
        max_blocks = block_tables.shape[1] if block_tables.dim() == 2 else 0
        L = _lib.lib()
        nbytes = L.akv_tq_paged_attn_workspace_bytes(num_seqs, num_q_heads, num_kv_heads, head_dim,
                                                     self.bits, block_size, max_blocks, self.SPLITK_BLOCKS)
        ws = self._get_workspace(nbytes, dev)
        p = _lib.TQAttnParams()
        p.query, p.q_dtype = query.data_ptr(), _lib.float_code(query)
        p.q_stride_seq, p.q_stride_head = query.stride(0), query.stride(1)
        p.k_packed = k_packed.data_ptr()
        p.kp_stride_blk, p.kp_stride_pos, p.kp_stride_head = k_packed.stride(0), k_packed.stride(1), k_packed.stride(2)
        p.k_norms = k_norms.data_ptr()
        p.kn_stride_blk, p.kn_stride_pos, p.kn_stride_head = k_norms.stride(0), k_norms.stride(1), k_norms.stride(2)
        p.v_packed = v_packed.data_ptr()
        p.vp_stride_blk, p.vp_stride_pos, p.vp_stride_head = v_packed.stride(0), v_packed.stride(1), v_packed.stride(2)
        p.v_norms = v_norms.data_ptr()
        p.vn_stride_blk, p.vn_stride_pos, p.vn_stride_head = v_norms.stride(0), v_norms.stride(1), v_norms.stride(2)
        p.block_tables, p.bt_dtype = block_tables.data_ptr(), _lib.index_code(block_tables)
        p.bt_stride_seq = block_tables.stride(0) if block_tables.dim() == 2 else 0
        p.context_lens, p.cl_dtype = context_lens.data_ptr(), _lib.index_code(context_lens)
        p.num_seqs, p.num_q_heads, p.num_kv_heads, p.head_dim = num_seqs, num_q_heads, num_kv_heads, head_dim
        p.block_size, p.max_blocks_per_seq, p.num_blocks = block_size, max_blocks, k_packed.shape[0]
        p.bits = self.bits
        p.rotation, p.rotation_t, p.centroids = (self.rotation.data_ptr(), self.rotation_T.data_ptr(),
                                                 self.centroids.data_ptr())
        p.scale = self.scale if scale is None else float(scale)
        if raw_out is not None:
            assert raw_out.dtype == torch.float32 and raw_out.is_contiguous()
            assert raw_out.numel() == num_seqs * num_q_heads * (head_dim + 2)
            p.raw_out = raw_out.data_ptr()
        else:
            p.out, p.out_dtype = out.data_ptr(), _lib.float_code(out)
            p.out_stride_seq, p.out_stride_head = out.stride(0), out.stride(1)
        p.workspace, p.workspace_bytes = ws.data_ptr(), ws.numel()
        p.blocks_per_split = self.SPLITK_BLOCKS
        return p

    # Split-K scratch is shared by all instances on a device (one per layer would multiply it);
    # calls are stream-ordered, so instances used on one stream can safely take turns.
    _shared_workspace: dict = {}

    def _get_workspace(self, nbytes: int, device) -> torch.Tensor:
        ws = TQPagedAttention._shared_workspace.get(device)
        if ws is None or ws.numel() < nbytes:
            ws = torch.empty(max(nbytes, 256), dtype=torch.uint8, device=device)
            TQPagedAttention._shared_workspace[device] = ws
            self._params_key = None
        self._workspace = ws
        return ws

    def prefill(self, query, k_packed, k_norms, v_packed, v_norms, block_tables, seq_lens, query_start_loc,
                block_size: int = 16, num_kv_heads: Optional[int] = None, out: Optional[torch.Tensor] = None,
                scale: Optional[float] = None, max_seq_len: Optional[int] = None) -> Optional[torch.Tensor]:
        """Chunked-prefill attention: ``query`` [tokens, query_heads, head_dim] holds the last
        ``query_start_loc[s+1] - query_start_loc[s]`` tokens of every sequence s; token i of a sequence attends
        causally over the cached tokens up to its own position (``seq_lens`` counts the chunk's tokens, whose K/V
        are already in the cache).  The query tokens of a sequence share one pass over its packed blocks
        (``akv_tq_prefill_attn``); the reference decompresses the blocks and calls vLLM's unified attention
        (``vllm/backend.py:1093-1244``).  Returns None when the kernel is not built for the shapes (the caller
        then attends row by row with ``forward``).

        ``max_seq_len``: the longest entry of ``seq_lens`` when the host knows it (vLLM's metadata carries it; it is
        never read back from the device here).  With it, large chunks take the staged tensor-core kernel: the codes of
        every key tile become fp16 operand images once, in a scratch buffer of 512 bytes per (token, KV head) of
        ``num_seqs x max_seq_len`` (up to ``STAGED_WORKSPACE_LIMIT`` bytes), instead of once per 128 query rows."""
        if num_kv_heads is None:
            num_kv_heads = k_packed.shape[2]
        dev = _lib.require_cuda(query, k_packed, k_norms, v_packed, v_norms, block_tables, seq_lens, query_start_loc)
        n_tok, num_q_heads, head_dim = query.shape
        G = num_q_heads // num_kv_heads
        aligned = all((t.data_ptr() | t.stride(0) | t.stride(1) | t.stride(2)) % 16 == 0 for t in (k_packed, v_packed))
        if (head_dim != 128 or G not in (1, 2, 4, 8) or block_size % 16
                or k_norms.dtype != torch.float32 or v_norms.dtype != torch.float32):
            return None
        if (self.bits != 4 or not aligned) and not max_seq_len:
            return None      # 3- / 2-bit codes and rows that are not readable in 16-byte pieces: staged tensor-core kernel only
        assert num_q_heads == self.num_query_heads and k_packed.shape[1] == block_size
        num_seqs = query_start_loc.numel() - 1
        if block_tables.dim() != 2 or block_tables.shape[0] < num_seqs or seq_lens.numel() < num_seqs:
            raise ValueError(f"block_tables {tuple(block_tables.shape)} / seq_lens {tuple(seq_lens.shape)} do not cover "
                             f"{num_seqs} sequences")
        if query.dtype not in _lib._FLOAT_CODES:
            query = query.float()
        if query.stride(-1) != 1:
            query = query.contiguous()
        if block_tables.stride(-1) != 1:
            block_tables = block_tables.contiguous()
        seq_lens, query_start_loc = seq_lens.contiguous(), query_start_loc.contiguous()
        if out is None:
            out = torch.empty(n_tok, num_q_heads, head_dim, dtype=query.dtype, device=dev)
        L = _lib.lib()
        nbytes = L.akv_tq_prefill_attn_workspace_bytes(n_tok, num_q_heads)
        if max_seq_len is not None and max_seq_len > 0:
            staged = L.akv_tq_prefill_attn_workspace_bytes_staged(n_tok, num_q_heads, num_kv_heads, num_seqs, int(max_seq_len))
            if staged <= self.STAGED_WORKSPACE_LIMIT:
                nbytes = staged
        if self._prefill_ws is None or self._prefill_ws.numel() < nbytes or self._prefill_ws.device != dev:
            self._prefill_ws = torch.empty(max(nbytes, 256), dtype=torch.uint8, device=dev)
        p = _lib.TQPrefillParams()
        p.query, p.q_dtype, p.q_stride_tok, p.q_stride_head = query.data_ptr(), _lib.float_code(query), query.stride(0), query.stride(1)
        p.k_packed, p.kp_stride_blk, p.kp_stride_pos, p.kp_stride_head = k_packed.data_ptr(), k_packed.stride(0), k_packed.stride(1), k_packed.stride(2)
        p.k_norms, p.kn_stride_blk, p.kn_stride_pos, p.kn_stride_head = k_norms.data_ptr(), k_norms.stride(0), k_norms.stride(1), k_norms.stride(2)
        p.v_packed, p.vp_stride_blk, p.vp_stride_pos, p.vp_stride_head = v_packed.data_ptr(), v_packed.stride(0), v_packed.stride(1), v_packed.stride(2)
        p.v_norms, p.vn_stride_blk, p.vn_stride_pos, p.vn_stride_head = v_norms.data_ptr(), v_norms.stride(0), v_norms.stride(1), v_norms.stride(2)
        p.block_tables, p.bt_dtype, p.bt_stride_seq = block_tables.data_ptr(), _lib.index_code(block_tables), block_tables.stride(0)
        p.seq_lens, p.sl_dtype = seq_lens.data_ptr(), _lib.index_code(seq_lens)
        p.query_start_loc, p.qs_dtype = query_start_loc.data_ptr(), _lib.index_code(query_start_loc)
        p.num_seqs, p.num_tokens, p.num_q_heads, p.num_kv_heads = num_seqs, n_tok, num_q_heads, num_kv_heads
        p.head_dim, p.block_size, p.max_blocks_per_seq, p.num_blocks = head_dim, block_size, block_tables.shape[1], k_packed.shape[0]
        p.bits = self.bits
        p.rotation, p.rotation_t, p.centroids = self.rotation.data_ptr(), self.rotation_T.data_ptr(), self.centroids.data_ptr()
        p.scale = self.scale if scale is None else float(scale)
        p.out, p.out_dtype, p.out_stride_tok, p.out_stride_head = out.data_ptr(), _lib.float_code(out), out.stride(0), out.stride(1)
        p.workspace, p.workspace_bytes = self._prefill_ws.data_ptr(), self._prefill_ws.numel()
        p.stream = _lib.stream_ptr(dev)
        p.max_seq_len = int(max_seq_len) if max_seq_len else 0
        with torch.cuda.device(dev):
            rc = L.akv_tq_prefill_attn(ctypes.byref(p))
        if rc == _lib.AKV_ERR_UNSUPPORTED:          # e.g. a ragged batch of 3-bit sequences: nothing was launched
            return None
        _lib.check(rc, "akv_tq_prefill_attn")
        return out

    def forward(
        self,
        query: torch.Tensor,           # [num_seqs, num_query_heads, head_dim]
        k_packed: torch.Tensor,        # [num_blocks, block_size, num_kv_heads, packed_dim] uint8
        k_norms: torch.Tensor,         # [num_blocks, block_size, num_kv_heads] float32
        v_packed: torch.Tensor,
        v_norms: torch.Tensor,
        block_tables: torch.Tensor,    # [num_seqs, max_blocks_per_seq] int32/int64
        context_lens: torch.Tensor,    # [num_seqs] int32/int64
        block_size: int = 16,
        num_kv_heads: Optional[int] = None,
        out: Optional[torch.Tensor] = None,
        raw_out: Optional[torch.Tensor] = None,
        scale: Optional[float] = None,
        kernel_events=None,
    ) -> torch.Tensor:
        """Returns [num_seqs, num_query_heads, head_dim] in ``query.dtype``.

        With ``raw_out`` (float32 [num_seqs*num_query_heads, head_dim+2]) the call writes the
        un-normalised partial (m, l, acc) instead, for merging across devices.
        ``scale`` defaults to 1/sqrt(head_dim).  ``kernel_events`` is an optional pair of
        ``torch.cuda.Event(enable_timing=True)`` recorded around the split-K kernel alone.
        """
        if num_kv_heads is None:
            num_kv_heads = k_packed.shape[2]
        dev = _lib.require_cuda(query, k_packed, k_norms, v_packed, v_norms, block_tables, context_lens)
        num_seqs, num_q_heads, head_dim = query.shape
        assert head_dim == self.head_dim and num_q_heads == self.num_query_heads
        assert k_packed.shape[1] == block_size, "block_size does not match the cache"
        if block_tables.dim() != 2 or block_tables.shape[0] < num_seqs or context_lens.numel() < num_seqs:
            raise ValueError(f"block_tables {tuple(block_tables.shape)} / context_lens {tuple(context_lens.shape)} "
                             f"do not cover {num_seqs} sequences")
        if (k_packed.shape[-1] < self.packed_dim or v_packed.shape[-1] < self.packed_dim
                or k_packed.shape[2] != num_kv_heads or tuple(k_norms.shape) != tuple(k_packed.shape[:3])
                or tuple(v_norms.shape) != tuple(v_packed.shape[:3]) or v_packed.shape[:3] != k_packed.shape[:3]):
            raise ValueError(f"packed cache {tuple(k_packed.shape)} / {tuple(v_packed.shape)} and norms "
                             f"{tuple(k_norms.shape)} / {tuple(v_norms.shape)} do not match "
                             f"[blocks, {block_size}, {num_kv_heads}, >= {self.packed_dim}]")
        if query.dtype not in _lib._FLOAT_CODES:
            query = query.float()
        if query.stride(-1) != 1:
            query = query.contiguous()
        if block_tables.stride(-1) != 1:
            block_tables = block_tables.contiguous()
        context_lens = context_lens.contiguous()
        if self._block_selector is not None:
            block_tables, context_lens = self._block_selector.select_for_query(
                query, block_tables, context_lens, block_size, rotation_T=self.rotation_T)
        if out is None and raw_out is None:
            out = torch.empty(num_seqs, num_q_heads, head_dim, dtype=query.dtype, device=dev)
        target = raw_out if raw_out is not None else out

        # The argument block only depends on pointers, shapes and strides: reuse it while
        # the caller keeps passing the same buffers (the steady state of a decode loop).
        tensors = (query, k_packed, k_norms, v_packed, v_norms, block_tables, context_lens, target)
        key = tuple((t.data_ptr(), t.shape, t.stride(), t.dtype) for t in tensors) + (
            block_size, num_kv_heads, raw_out is not None, scale, self.SPLITK_BLOCKS)
        p = self._params if key == self._params_key else None
        if p is None:
            p = self._build_params(dev, query, k_packed, k_norms, v_packed, v_norms, block_tables,
                                   context_lens, block_size, num_kv_heads, out, raw_out, scale)
            self._params, self._params_key = p, key
        p.stream = _lib.stream_ptr(dev)
        if kernel_events is not None:
            for ev in kernel_events:      # torch creates the CUDA event on first record
                if not ev.cuda_event:
                    ev.record(torch.cuda.current_stream(dev))
            p.ev_kernel_start, p.ev_kernel_stop = kernel_events[0].cuda_event, kernel_events[1].cuda_event
        else:
            p.ev_kernel_start = p.ev_kernel_stop = None
        with torch.cuda.device(dev):
            rc = _lib.lib().akv_tq_paged_attn(ctypes.byref(p))
        _lib.check(rc, "akv_tq_paged_attn")
        return raw_out if raw_out is not None else out
