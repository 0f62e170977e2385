"""Query-aware block selection for sparse paged decode attention.

Interface of the reference's ``aither_kvcache/block_selector.py`` (``BlockSelector`` :231-340,
``BlockRepresentativeCache`` :29-126, ``score_blocks`` :128-172, ``select_blocks`` :175-228): per
physical block and KV head the mean of the norm-weighted rotated-domain keys is kept up to date as
tokens are written; at decode time every block of a sequence is scored against the GQA-averaged
rotated query, the first / last few blocks are always kept, the ``max_selected`` best are gathered
in logical order into a shorter block table.  Output shapes are fixed, nothing synchronises the host.

All of it runs in the kernels behind ``akv_block_select_update`` / ``akv_block_select``
(csrc/block_select.cu); the representative store lives in three device tensors owned by this object.

One deliberate difference: when a sequence has more blocks than are kept, the reference counts the
(always kept, possibly partial) last block as full, ``min(ctx, k * block_size)``, which lets the
attention read slots that were never written; here the adjusted context length counts only the real
tokens of that block (``exact_tail=False`` restores the reference's arithmetic).
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch

from . import _lib


class BlockSelector:
    def __init__(self, max_blocks: int, num_kv_heads: int, half_d: int, device, centroids: torch.Tensor,
                 select_ratio: float = 1.0, num_sink_blocks: int = 2, num_recent_blocks: int = 2,
                 min_blocks_for_selection: int = 64, rotation: Optional[torch.Tensor] = None, bits: int = 4,
                 exact_tail: bool = True):
        self.max_blocks, self.num_kv_heads, self.head_dim = max_blocks, num_kv_heads, 2 * half_d
        if self.head_dim != 128:
            raise NotImplementedError("block selection is built for head_dim 128")
        self.device = torch.device(device)
        self.centroids = centroids.to(self.device, torch.float32).contiguous()
        self.bits = bits
        self.select_ratio = select_ratio
        self.num_sink_blocks, self.num_recent_blocks = num_sink_blocks, num_recent_blocks
        self.min_blocks = min_blocks_for_selection
        self.enabled = select_ratio < 1.0
        self.exact_tail = exact_tail
        self._max_selected = max(num_sink_blocks + num_recent_blocks + 1,
                                 math.ceil(max_blocks * select_ratio)) if self.enabled else 0
        self.rotation_T = None if rotation is None else rotation.to(self.device, torch.float32).t().contiguous()
        if self.enabled:
            self._acc = torch.zeros(max_blocks, num_kv_heads, self.head_dim, dtype=torch.float32, device=self.device)
            self.rep = torch.zeros_like(self._acc)
            self._counts = torch.zeros(max_blocks, num_kv_heads, dtype=torch.int32, device=self.device)
        self._workspace: Optional[torch.Tensor] = None
        self._out_bt: Optional[torch.Tensor] = None
        self._out_cl: Optional[torch.Tensor] = None

    @property
    def max_selected(self) -> int:
        return self._max_selected

    def update_reps(self, block_indices: torch.Tensor, positions: torch.Tensor, k_packed: torch.Tensor,
                    k_norms: torch.Tensor) -> None:
        """``block_indices`` [N] int64 physical blocks of the newly written tokens, ``k_packed``
        [N, kv_heads, packed_dim] uint8, ``k_norms`` [N, kv_heads] float32.  (``positions`` is unused, as
        in the reference.)"""
        if not self.enabled:
            return
        _lib.require_cuda(block_indices, k_packed, k_norms)
        n = block_indices.numel()
        if n == 0:
            return
        if k_packed.dtype != torch.uint8 or k_packed.stride(-1) != 1 or k_norms.dtype != torch.float32:
            raise ValueError("k_packed must be uint8 with a contiguous last dimension, k_norms float32")
        if k_packed.shape[0] != n or k_norms.shape[0] != n or k_packed.shape[1] != self.num_kv_heads:
            raise ValueError(f"update_reps: {n} tokens, k_packed {tuple(k_packed.shape)}, k_norms {tuple(k_norms.shape)}")
        bi = block_indices.to(torch.int64).contiguous()
        with torch.cuda.device(self.device):
            rc = _lib.lib().akv_block_select_update(
                bi.data_ptr(), n, k_packed.data_ptr(), k_packed.stride(0), k_packed.stride(1), k_norms.data_ptr(),
                k_norms.stride(0), k_norms.stride(1), self.centroids.data_ptr(), self.bits, self.num_kv_heads,
                self.head_dim, self.max_blocks, self._acc.data_ptr(), self._counts.data_ptr(), self.rep.data_ptr(),
                _lib.stream_ptr(self.device))
        _lib.check(rc, "akv_block_select_update")

    def clear_blocks(self, block_indices: torch.Tensor) -> None:
        if not self.enabled or block_indices.numel() == 0:
            return
        bi = block_indices.to(torch.int64).contiguous()
        with torch.cuda.device(self.device):
            rc = _lib.lib().akv_block_select_clear(bi.data_ptr(), bi.numel(), self.num_kv_heads, self.max_blocks,
                                                   self._acc.data_ptr(), self._counts.data_ptr(), self.rep.data_ptr(),
                                                   _lib.stream_ptr(self.device))
        _lib.check(rc, "akv_block_select_clear")

    def select_for_query(self, query: torch.Tensor, block_tables: torch.Tensor, context_lens: torch.Tensor,
                         block_size: int = 16, rotation_T: Optional[torch.Tensor] = None,
                         scores_out: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, torch.Tensor]:
        """``query`` [num_seqs, q_heads, 128] (not rotated; the kernel rotates the group means).  Returns
        ``(block_tables, context_lens)`` unchanged when selection is off or the table is short, else int32
        ``[num_seqs, max_selected]`` / ``[num_seqs]`` tensors that are reused from call to call."""
        if not self.enabled or block_tables.shape[1] < self.min_blocks:
            return block_tables, context_lens
        rt = rotation_T if rotation_T is not None else self.rotation_T
        if rt is None:
            raise ValueError("the selector needs the rotation (pass rotation= at construction or rotation_T= here)")
        dev = _lib.require_cuda(query, block_tables, context_lens, rt)
        S, QH, D = query.shape
        if query.dtype not in _lib._FLOAT_CODES:
            query = query.float()
        if query.stride(-1) != 1:
            query = query.contiguous()
        if block_tables.stride(-1) != 1:
            block_tables = block_tables.contiguous()
        context_lens = context_lens.contiguous()
        max_bps = block_tables.shape[1]
        L = _lib.lib()
        nbytes = L.akv_block_select_workspace_bytes(S, self.num_kv_heads, max_bps)
        if self._workspace is None or self._workspace.numel() < nbytes:
            self._workspace = torch.empty(max(nbytes, 256), dtype=torch.uint8, device=dev)
        if self._out_bt is None or self._out_bt.shape != (S, self._max_selected):
            self._out_bt = torch.zeros(S, self._max_selected, dtype=torch.int32, device=dev)
            self._out_cl = torch.zeros(S, dtype=torch.int32, device=dev)
        with torch.cuda.device(dev):
            rc = L.akv_block_select(query.data_ptr(), _lib.float_code(query), query.stride(0), query.stride(1), S, QH,
                                    self.num_kv_heads, D, rt.data_ptr(), self.rep.data_ptr(), self.max_blocks,
                                    block_tables.data_ptr(), _lib.index_code(block_tables), block_tables.stride(0),
                                    context_lens.data_ptr(), _lib.index_code(context_lens), block_size, max_bps,
                                    self._max_selected, self.num_sink_blocks, self.num_recent_blocks,
                                    1 if self.exact_tail else 0, self._out_bt.data_ptr(), self._out_cl.data_ptr(),
                                    _lib.ptr(scores_out), self._workspace.data_ptr(), self._workspace.numel(),
                                    _lib.stream_ptr(dev))
        _lib.check(rc, "akv_block_select")
        return self._out_bt, self._out_cl

    def select(self, q_even: torch.Tensor, q_odd: torch.Tensor, block_tables: torch.Tensor,
               context_lens: torch.Tensor, gqa_ratio: int, block_size: int = 16) -> Tuple[torch.Tensor, torch.Tensor]:
        """The reference's signature: ``q_even`` / ``q_odd`` are the even / odd coordinates of the already
        rotated query [num_seqs, q_heads, 64].  The rotated query is re-interleaved and scored with an
        identity rotation."""
        if not self.enabled or block_tables.shape[1] < self.min_blocks:
            return block_tables, context_lens
        q_rot = torch.stack((q_even, q_odd), dim=-1).reshape(q_even.shape[0], q_even.shape[1], self.head_dim)
        eye = getattr(self, "_eye", None)
        if eye is None or eye.device != q_rot.device:
            eye = self._eye = torch.eye(self.head_dim, dtype=torch.float32, device=q_rot.device)
        return self.select_for_query(q_rot, block_tables, context_lens, block_size, rotation_T=eye)
