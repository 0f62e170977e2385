"""TriAttention: attention over spectrally compressed K/V via the RoPE trig series.

Interface of the reference's ``triattention/attention.py`` (``TriAttention`` :38-450:
``encode_kv`` :96-112, ``decode_step`` :186-215) and ``triattention/scorer.py``
(``TrigSeriesScorer.score`` :115-208).  Scoring, softmax and the scattered value sum are
one kernel (``akv_tri_decode_step``); nothing of size [B, QH, S, F] is materialised.
"""
import ctypes
import math
from typing import Optional, Tuple

import torch

from .. import _lib
from .config import TriAttentionConfig
from .encoder import SpectralEncoding, SpectralKVEncoder
from .spectral import rope_frequencies


class TriAttention:
    def __init__(self, config: TriAttentionConfig, device: str = "cuda"):
        self.config, self.device = config, device
        self.head_dim = config.head_dim
        self.num_query_heads, self.num_kv_heads = config.num_query_heads, config.num_kv_heads
        self.gqa_ratio = config.gqa_ratio
        self.scale = 1.0 / math.sqrt(config.head_dim)
        self.encoder = SpectralKVEncoder(config)
        # the table is evaluated on the host like the reference's default (device="cpu")
        self._theta = rope_frequencies(config.head_dim, config.rope_base, device="cpu").to(device)
        self.tokens_per_split = 0
        self._workspace: Optional[torch.Tensor] = None

    def to(self, device: str) -> "TriAttention":
        self.device = device
        self._theta = self._theta.to(device)
        return self

    def encode_kv(self, keys: torch.Tensor, values: torch.Tensor) -> Tuple[SpectralEncoding, SpectralEncoding]:
        """keys / values [B, S, kv_heads, head_dim] (keys before RoPE) -> two SpectralEncoding."""
        return self.encoder.encode(keys), self.encoder.encode(values)

    def _run(self, query, k_enc, v_enc, query_pos, key_positions, out=None, raw_out=None, scores_out=None,
             key_pos_start: int = 0, query_pos_default: Optional[int] = None, kernel_events=None,
             block_tables: Optional[torch.Tensor] = None, context_lens: Optional[torch.Tensor] = None):
        cb = self.config.coeff_bits
        want = torch.float16 if cb == 16 else torch.uint8
        assert k_enc.packed.dtype == want and v_enc.packed.dtype == want, f"coeff_bits={cb} takes {want} coefficients"
        dev = _lib.require_cuda(query, k_enc.indices, k_enc.packed, k_enc.scales, v_enc.indices, v_enc.packed,
                                v_enc.scales, query_pos, key_positions, self._theta, block_tables, context_lens)
        B, QH, D = query.shape
        S, KVH, F = k_enc.indices.shape[1:]
        paged = block_tables is not None
        if paged:                                  # records are [num_blocks, block_size, KVH, ...]
            num_blocks, block_size = k_enc.indices.shape[:2]
            assert key_positions is None, "paged records take positions from the slot order"
            assert block_tables.dim() == 2 and block_tables.shape[0] == B and block_tables.dtype in _lib._INDEX_CODES
            if block_tables.stride(1) != 1:
                block_tables = block_tables.contiguous()
            S = block_tables.shape[1] * block_size
        if context_lens is not None:
            assert context_lens.dtype in _lib._INDEX_CODES and context_lens.numel() == B
            context_lens = context_lens.reshape(-1).contiguous()
        assert D == self.head_dim and QH == self.num_query_heads and KVH == self.num_kv_heads
        if query.dtype not in _lib._FLOAT_CODES:
            query = query.float()
        if query.stride(-1) != 1:
            query = query.contiguous()
        t = [x.contiguous() for x in (k_enc.indices, k_enc.packed, k_enc.scales, v_enc.indices, v_enc.packed, v_enc.scales)]
        assert t[2].dtype == torch.float16 and t[5].dtype == torch.float16
        if key_positions is not None:
            key_positions = key_positions.to(torch.int64).expand(B, S).contiguous()
        if query_pos is not None:
            query_pos = query_pos.to(torch.int64).reshape(-1).expand(B).contiguous()
        L = _lib.lib()
        nbytes = L.akv_tri_decode_workspace_bytes(B, QH, S, self.tokens_per_split)
        if self._workspace is None or self._workspace.numel() < nbytes or self._workspace.device != dev:
            self._workspace = torch.empty(max(nbytes, 256), dtype=torch.uint8, device=dev)
        p = _lib.TriDecodeParams()
        p.query, p.q_dtype, p.q_stride_batch, p.q_stride_head = query.data_ptr(), _lib.float_code(query), query.stride(0), query.stride(1)
        p.k_indices, p.k_packed, p.k_scales = t[0].data_ptr(), t[1].data_ptr(), t[2].data_ptr()
        p.v_indices, p.v_packed, p.v_scales = t[3].data_ptr(), t[4].data_ptr(), t[5].data_ptr()
        p.batch, p.seq_len, p.num_kv_heads, p.num_q_heads, p.head_dim, p.num_freqs = B, S, KVH, QH, D, F
        p.key_positions, p.key_pos_start = _lib.ptr(key_positions), key_pos_start
        p.query_pos = _lib.ptr(query_pos)
        p.query_pos_default = S if query_pos_default is None else query_pos_default
        p.theta, p.scale = self._theta.data_ptr(), self.scale
        p.out, p.raw_out, p.scores_out = _lib.ptr(out), _lib.ptr(raw_out), _lib.ptr(scores_out)
        p.workspace, p.workspace_bytes = self._workspace.data_ptr(), self._workspace.numel()
        p.tokens_per_split = self.tokens_per_split
        p.coeff_bits, p.post_rope = cb, 0 if self.config.pre_rope else 1
        if paged:
            p.block_tables, p.bt_dtype, p.bt_stride_batch = block_tables.data_ptr(), _lib.index_code(block_tables), block_tables.stride(0)
            p.block_size, p.num_blocks = block_size, num_blocks
        if context_lens is not None:
            p.context_lens, p.cl_dtype = context_lens.data_ptr(), _lib.index_code(context_lens)
        p.stream = _lib.stream_ptr(dev)
        if kernel_events is not None:
            for ev in kernel_events:
                if not ev.cuda_event:
                    ev.record(torch.cuda.current_stream(dev))
            p.ev_kernel_start, p.ev_kernel_stop = kernel_events[0].cuda_event, kernel_events[1].cuda_event
        with torch.cuda.device(dev):
            rc = L.akv_tri_decode_step(ctypes.byref(p))
        _lib.check(rc, "akv_tri_decode_step")

    def decode_step(self, query: torch.Tensor, k_enc: SpectralEncoding, v_enc: SpectralEncoding,
                    query_pos: Optional[torch.Tensor] = None,
                    key_positions: Optional[torch.Tensor] = None, **kw) -> torch.Tensor:
        """query [B, QH, D]; returns float32 [B, QH, D].  Defaults: key positions 0..S-1, query at S."""
        B, QH, D = query.shape
        out = torch.empty(B, QH, D, dtype=torch.float32, device=query.device)
        self._run(query, k_enc, v_enc, query_pos, key_positions, out=out, **kw)
        return out

    def paged_decode_step(self, query: torch.Tensor, cache, block_tables: torch.Tensor, context_lens: torch.Tensor,
                          query_pos: Optional[torch.Tensor] = None, **kw) -> torch.Tensor:
        """One decode step straight off a ``SpectralKVCache``: query [B, QH, D], block_tables [B, max_blocks_per_seq],
        context_lens [B].  Equal to ``decode_step`` on ``cache.fetch_sequence(block_tables[b], context_lens[b])`` for every
        b (the reference's route, triattention/cache.py:157-198 then attention.py:186-215), without the gather.  Keys
        sit at positions 0..len-1; the query position defaults to each sequence's length."""
        B, QH, D = query.shape
        out = torch.empty(B, QH, D, dtype=torch.float32, device=query.device)
        if query_pos is None:
            query_pos = context_lens
        self._run(query, cache.k_encoding, cache.v_encoding, query_pos, None, out=out, block_tables=block_tables,
                  context_lens=context_lens, **kw)
        return out

    def decode_step_partial(self, query, k_enc, v_enc, query_pos=None, key_positions=None,
                            key_pos_start: int = 0, query_pos_default: Optional[int] = None) -> torch.Tensor:
        """Un-normalised (m, l, acc) per (batch, q head) over this device's key range:
        float32 [B*QH, D+2], to be all-gathered and merged (see ``parallel.merge_partials``)."""
        B, QH, D = query.shape
        raw = torch.empty(B * QH, D + 2, dtype=torch.float32, device=query.device)
        self._run(query, k_enc, v_enc, query_pos, key_positions, raw_out=raw, key_pos_start=key_pos_start,
                  query_pos_default=query_pos_default)
        return raw

    def forward(self, query, key, value, positions=None, attention_mask=None) -> torch.Tensor:
        """Encode K/V, then attend.  query [B, QH, D] (one step) or [B, QH, S_q, D] (one decode
        step per query position, query i at position i, as the reference's prefill loop)."""
        if attention_mask is not None:
            raise NotImplementedError("additive masks are not part of the decode kernel")
        k_enc, v_enc = self.encode_kv(key, value)
        if query.dim() == 3:
            q_pos = torch.zeros(query.shape[0], dtype=torch.int64, device=query.device)
            return self.decode_step(query, k_enc, v_enc, q_pos, positions)
        outs = []
        for qi in range(query.shape[2]):
            q_pos = torch.full((query.shape[0],), qi, dtype=torch.int64, device=query.device)
            outs.append(self.decode_step(query[:, :, qi], k_enc, v_enc, q_pos, positions))
        return torch.stack(outs, dim=2)


class TrigSeriesScorer:
    """``score(query, k_enc, query_pos, key_positions)`` -> float32 [B, QH, S] pre-softmax logits."""

    def __init__(self, config: TriAttentionConfig, device: str = "cuda"):
        self.config = config
        self._tri = TriAttention(config, device=device)
        self.scale = self._tri.scale

    def to(self, device: str) -> "TrigSeriesScorer":
        self._tri.to(device)
        return self

    def score(self, query, k_enc, query_pos=None, key_positions=None) -> torch.Tensor:
        B, QH, D = query.shape
        S = k_enc.indices.shape[1]
        scores = torch.empty(B, QH, S, dtype=torch.float32, device=query.device)
        sink = torch.empty(B, QH, D, dtype=torch.float32, device=query.device)
        self._tri._run(query, k_enc, k_enc, query_pos, key_positions, out=sink, scores_out=scores)
        return scores
