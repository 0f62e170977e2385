"""Paged storage of TriAttention records: the reference's ``SpectralKVCache``
(triattention/cache.py:37-232) with the same six tensors, methods and statistics.

Per physical block: indices and packed coefficients [block_size, kv_heads, F] uint8 and scales
[block_size, kv_heads] float16, for keys and for values.  ``TriAttention.paged_decode_step`` reads these
tensors through a block table inside the decode kernel; ``fetch_sequence`` is the reference's gather.
Fill counts live on the host: the reference reads them back with ``.item()`` on every store.
"""
import math
from typing import Optional, Tuple

import torch

from .config import TriAttentionConfig
from .encoder import SpectralEncoding


class SpectralKVCache:
    def __init__(self, config: TriAttentionConfig, max_blocks: int = 1024, device: str = "cuda"):
        self.config, self.max_blocks, self.device = config, max_blocks, device
        self.block_size, self.num_kv_heads, self.num_freqs = config.block_size, config.num_kv_heads, config.num_freqs
        shape = (max_blocks, self.block_size, self.num_kv_heads)
        for side in "kv":
            setattr(self, side + "_indices", torch.zeros(*shape, self.num_freqs, dtype=torch.uint8, device=device))
            setattr(self, side + "_packed", torch.zeros(*shape, self.num_freqs, dtype=torch.uint8, device=device))
            setattr(self, side + "_scales", torch.zeros(*shape, dtype=torch.float16, device=device))
        self._block_fill = torch.zeros(max_blocks, dtype=torch.int32)

    @property
    def k_encoding(self) -> SpectralEncoding:
        """The key arrays of all blocks as one encoding [max_blocks, block_size, kv_heads, ...]."""
        return SpectralEncoding(self.k_indices, self.k_packed, self.k_scales)

    @property
    def v_encoding(self) -> SpectralEncoding:
        return SpectralEncoding(self.v_indices, self.v_packed, self.v_scales)

    def _sides(self):
        return ((self.k_indices, self.k_packed, self.k_scales), (self.v_indices, self.v_packed, self.v_scales))

    @property
    def bytes_allocated(self) -> int:
        return sum(t.element_size() * t.numel() for side in self._sides() for t in side)

    @property
    def bytes_per_token(self) -> int:
        return self.config.bytes_per_kv_token * 2

    def store_token(self, block_idx: int, slot_idx: int, k_enc: SpectralEncoding, v_enc: SpectralEncoding) -> None:
        """One token: encodings shaped [kv_heads, F] / [kv_heads]."""
        for dst, enc in zip(self._sides(), (k_enc, v_enc)):
            for d, src in zip(dst, enc):
                d[block_idx, slot_idx] = src
        self._block_fill[block_idx] = max(int(self._block_fill[block_idx]), slot_idx + 1)

    def store_block(self, block_idx: int, k_enc: SpectralEncoding, v_enc: SpectralEncoding,
                    num_tokens: Optional[int] = None) -> None:
        """Up to block_size tokens: encodings shaped [tokens, kv_heads, F] / [tokens, kv_heads]."""
        n = min(k_enc.indices.shape[0] if num_tokens is None else num_tokens, self.block_size)
        for dst, enc in zip(self._sides(), (k_enc, v_enc)):
            for d, src in zip(dst, enc):
                d[block_idx, :n] = src[:n]
        self._block_fill[block_idx] = n

    def store_sequence(self, block_table: torch.Tensor, k_enc: SpectralEncoding, v_enc: SpectralEncoding) -> None:
        """[tokens, kv_heads, ...] encodings of one sequence into the blocks its table names, with one indexed
        copy per tensor (not in the reference, which loops ``store_block``)."""
        n = k_enc.indices.shape[0]
        nb = math.ceil(n / self.block_size)
        blocks = block_table[:nb].long().to(self.k_indices.device)
        slots = (blocks[:, None] * self.block_size
                 + torch.arange(self.block_size, device=blocks.device)[None]).reshape(-1)[:n]
        for dst, enc in zip(self._sides(), (k_enc, v_enc)):
            for d, src in zip(dst, enc):
                d.view(-1, *d.shape[2:])[slots] = src
        fill = torch.full((nb,), self.block_size, dtype=torch.int32)
        fill[-1] = n - (nb - 1) * self.block_size
        self._block_fill[blocks.cpu()] = fill

    def fetch_sequence(self, block_table: torch.Tensor, context_len: int) -> Tuple[SpectralEncoding, SpectralEncoding]:
        """The first ``context_len`` tokens of the blocks in ``block_table``, [context_len, kv_heads, ...]."""
        blocks = block_table[:math.ceil(context_len / self.block_size)].long().to(self.k_indices.device)
        k, v = ([t[blocks].reshape(-1, *t.shape[2:])[:context_len] for t in side] for side in self._sides())
        return SpectralEncoding(*k), SpectralEncoding(*v)

    def copy_block(self, src_block: int, dst_block: int) -> None:
        for side in self._sides():
            for t in side:
                t[dst_block] = t[src_block]
        self._block_fill[dst_block] = self._block_fill[src_block]

    def clear_block(self, block_idx: int) -> None:
        for side in self._sides():
            for t in side:
                t[block_idx].zero_()
        self._block_fill[block_idx] = 0

    def memory_stats(self) -> dict:
        total_tokens = int(self._block_fill.sum())
        return {
            "max_blocks": self.max_blocks,
            "used_blocks": int((self._block_fill > 0).sum()),
            "total_tokens": total_tokens,
            "bytes_allocated": self.bytes_allocated,
            "bytes_per_token": self.bytes_per_token,
            "compression_ratio": self.config.kv_compression_ratio,
            "equivalent_fp16_bytes": total_tokens * self.config.head_dim * 2 * 2,
        }
