"""vLLM v1 ``CUSTOM`` attention backend over a TurboQuant-packed KV cache.

Surface of the reference's ``aither_kvcache/vllm/backend.py`` (``TurboQuantBackend`` :261-311,
``TurboQuantImpl`` :324-1273, ``register_turboquant_backend`` :1280-1295) restricted to what the
hot path needs: the cache is uint8 ``[num_blocks, 2, block_size, kv_heads, head_size]``
(``get_kv_cache_shape`` keeps the reference's 5-D form; the first ``packed_dim`` bytes of a row
hold the codes), ``do_kv_cache_update`` encodes new K/V straight into it (norms in per-layer
float32 tensors for the uniform codec, as the reference's PRIMARY mode; inside the record for the
hybrid codec), and every forward - single-token decode, chunked prefill, or a batch that mixes
the two - attends over the packed cache with the paged kernels: each query token becomes one row
with its own causal context length and its sequence's block-table row, built on the device
without a host synchronisation.  Nothing is decompressed to fp16.  The reference's shadow mode,
cold tier and block selection are not part of this build.

The codec is picked like the reference does (``vllm/backend.py:618-626``): ``AITHER_TQ_MODE=tq35``
selects the hybrid codec, otherwise ``AITHER_TQ_BITS`` (default 4) the uniform one; a
``tq-t4nc`` / ``tq-t3nc`` / ``tq-t2nc`` / ``tq-t35nc`` cache-dtype string overrides both.  The
classes are created on first attribute access so that importing this module does not import vLLM.
"""
from __future__ import annotations

import inspect
import types
import os
from typing import Dict, Optional, Tuple

import torch

KV_DTYPE_BITS = {"tq-t4nc": 4, "tq-t3nc": 3, "tq-t2nc": 2}
KV_DTYPE_HYBRID = {"tq-t35nc": "tq35", "tq-t25nc": "tq25"}


def bits_from_env_or_dtype(cache_dtype_str: Optional[str] = None) -> int:
    if cache_dtype_str in KV_DTYPE_BITS:
        return KV_DTYPE_BITS[cache_dtype_str]
    return int(os.environ.get("AITHER_TQ_BITS", "4"))


def codec_from_env_or_dtype(cache_dtype_str: Optional[str] = None) -> Tuple[str, object]:
    """``("uniform", bits)`` or ``("hybrid", "tq35" | "tq25")``."""
    if cache_dtype_str in KV_DTYPE_HYBRID:
        return "hybrid", KV_DTYPE_HYBRID[cache_dtype_str]
    if cache_dtype_str in KV_DTYPE_BITS:
        return "uniform", KV_DTYPE_BITS[cache_dtype_str]
    mode = os.environ.get("AITHER_TQ_MODE", "").replace("-primary", "")
    if mode in ("tq35", "tq25"):
        return "hybrid", mode
    if mode in ("tq4", "tq3", "tq2"):
        return "uniform", int(mode[2])
    return "uniform", bits_from_env_or_dtype(cache_dtype_str)


class _LayerState:
    """Quantiser, attention object and norm tensors shared by the impl instances of a process."""
    quantizers: Dict[tuple, object] = {}
    attention: Dict[tuple, object] = {}
    k_norms: Dict[str, torch.Tensor] = {}
    v_norms: Dict[str, torch.Tensor] = {}


def _quantizer(head_size: int, bits: int, device):
    from ..quantizer import TurboQuant
    key = (head_size, bits, str(device))
    tq = _LayerState.quantizers.get(key)
    if tq is None:
        tq = TurboQuant(head_dim=head_size, bits=bits, device=str(device))
        _LayerState.quantizers[key] = tq
    return tq


def _hybrid_quantizer(head_size: int, mode: str, device):
    from ..hybrid_quantizer import HybridTurboQuant
    key = (head_size, mode, str(device))
    htq = _LayerState.quantizers.get(key)
    if htq is None:
        htq = HybridTurboQuant(head_dim=head_size, mode=mode, device=str(device))
        htq.calibrate_uniform()
        _LayerState.quantizers[key] = htq
    return htq


def token_rows(query_start_loc: torch.Tensor, seq_lens: torch.Tensor, block_table: torch.Tensor,
               num_tokens: int):
    """One attention row per query token of a (chunked-prefill or mixed) batch, computed on the device:
    token t of sequence s, the i-th of its n_s query tokens, attends causally over the first
    ``seq_lens[s] - (n_s - 1 - i)`` cached tokens through sequence s's block-table row.
    Returns (block_tables [num_tokens, max_blocks], context_lens int32 [num_tokens])."""
    dev = block_table.device
    tok = torch.arange(num_tokens, device=dev, dtype=query_start_loc.dtype)
    ends = query_start_loc[1:]
    seq = torch.bucketize(tok, ends, right=True).clamp_(max=ends.numel() - 1)
    ctx = seq_lens.index_select(0, seq) - (ends.index_select(0, seq) - 1 - tok).to(seq_lens.dtype)
    return block_table.index_select(0, seq), ctx.clamp_(min=0).to(torch.int32)


class TurboQuantImplBase:
    """Backend-independent part of the impl (usable and testable without vLLM)."""

    PREFILL_ROWS = 64        # query tokens per attention call of a prefill chunk

    def _tq_setup(self, num_heads: int, head_size: int, scale: float, num_kv_heads: int,
                  kv_cache_dtype: str = "auto") -> None:
        self.num_heads, self.head_size, self.scale = num_heads, head_size, float(scale)
        self.num_kv_heads = num_kv_heads
        self.tq_codec, what = codec_from_env_or_dtype(kv_cache_dtype)
        if self.tq_codec == "hybrid":
            from ..hybrid_quantizer import HybridTurboQuant
            self.tq_mode, self.tq_bits = what, 0
            self.packed_dim = HybridTurboQuant.packed_dim_for_mode(head_size, what)
        else:
            self.tq_mode, self.tq_bits = "", int(what)
            self.packed_dim = head_size * self.tq_bits // 8

    def _planar(self, kv_cache: torch.Tensor) -> bool:
        """Pages of the uniform codecs are laid out in planes unless ``AITHER_TQ_RECORD_PAGES`` is set: in each of a
        block's K and V halves first the codes of all (position, head) rows back to back, then their float32 norms
        (the rest of a page that vLLM sized for fp16 K/V stays unused).  The bytes per block are those of the
        reference's pages - ``vllm/engine.py:125-133`` puts the norm behind the codes of the same row (68-byte rows at
        4 bits) in primary mode, ``vllm/backend.py:440-454`` keeps the codes at the start of head_size-byte rows and the
        norms in side tensors otherwise - but code rows are dense and start on 16-byte boundaries, which the TMA-fed
        decode kernel and the vectorised prefill pre-pass need: attention over strided or 68-byte rows runs at half
        the speed."""
        pd = self.packed_dim
        return (self.tq_codec == "uniform" and kv_cache.dim() == 5 and kv_cache.shape[-1] >= pd + 4 and pd % 4 == 0
                and kv_cache.is_contiguous() and (kv_cache.shape[2] * kv_cache.shape[3] * pd) % 16 == 0
                and not os.environ.get("AITHER_TQ_RECORD_PAGES"))

    def _planes(self, kv_cache: torch.Tensor):
        """(codes [blocks, 2, block_size, heads, packed_dim] uint8, norms [blocks, 2, block_size, heads] float32): views
        of a planar primary-mode cache, nothing is copied."""
        nb, _, bs, H, W = kv_cache.shape
        pd = self.packed_dim
        flat = kv_cache.view(nb, 2, bs * H * W)
        codes = flat[:, :, :bs * H * pd].view(nb, 2, bs, H, pd)
        norms = flat[:, :, bs * H * pd:bs * H * (pd + 4)].view(torch.float32).view(nb, 2, bs, H)
        return codes, norms

    def _codes(self, kv_cache: torch.Tensor):
        """The K and V code (or record) rows [blocks, block_size, heads, packed_dim] of a cache in any layout."""
        if self._planar(kv_cache):
            codes, _ = self._planes(kv_cache)
            return codes[:, 0], codes[:, 1]
        pd = self.packed_dim
        return kv_cache[:, 0, :, :, :pd], kv_cache[:, 1, :, :, :pd]

    def _norms(self, layer_name: str, kv_cache: torch.Tensor):
        pd = self.packed_dim
        if self._planar(kv_cache):
            _, norms = self._planes(kv_cache)
            return norms[:, 0], norms[:, 1]
        if kv_cache.shape[-1] == pd + 4 and pd % 4 == 0:
            # primary-mode records: the norm is the float32 behind the codes of the same row
            # (reference page layout, vllm/engine.py:125-133); strided views, nothing is copied
            try:
                n = kv_cache[..., pd:pd + 4].view(torch.float32).squeeze(-1)   # [blocks, 2, block_size, kv_heads]
                return n[:, 0], n[:, 1]
            except RuntimeError:       # rows that are not 4-byte aligned views: side tensors below
                pass
        kn = _LayerState.k_norms.get(layer_name)
        shape = (kv_cache.shape[0], kv_cache.shape[2], kv_cache.shape[3])
        if kn is None or kn.shape != shape or kn.device != kv_cache.device:
            kn = torch.zeros(shape, dtype=torch.float32, device=kv_cache.device)
            _LayerState.k_norms[layer_name] = kn
            _LayerState.v_norms[layer_name] = torch.zeros_like(kn)
        return kn, _LayerState.v_norms[layer_name]

    def do_kv_cache_update(self, layer, key, value, kv_cache, slot_mapping) -> None:
        """Encode ``key`` / ``value`` [tokens, kv_heads, head_size] into the packed cache in place."""
        pd, bs = self.packed_dim, kv_cache.shape[2]
        if self.tq_codec == "hybrid":
            from ..hybrid_quantizer import hybrid_kv_update
            htq = _hybrid_quantizer(self.head_size, self.tq_mode, kv_cache.device)
            for x, rows in zip((key, value), self._codes(kv_cache)):
                hybrid_kv_update(htq, x, slot_mapping, rows, bs, kv_cache.shape[0])
            return
        from ..fused_kv_update import fused_tq4_kv_update
        tq = _quantizer(self.head_size, self.tq_bits, kv_cache.device)
        kn, vn = self._norms(getattr(layer, "layer_name", "layer"), kv_cache)
        for x, rows, norms in zip((key, value), self._codes(kv_cache), (kn, vn)):
            fused_tq4_kv_update(x, slot_mapping, rows, norms, tq.rotation,
                                tq.boundaries_inner, bs, kv_cache.shape[0], rotation_t=tq.rotation_T)

    def _attend(self, layer, q, out, kv_cache, block_table, context_lens) -> None:
        pd, bs = self.packed_dim, kv_cache.shape[2]
        kc, vc = self._codes(kv_cache)
        key_ = (self.head_size, self.tq_codec, self.tq_mode or self.tq_bits, self.num_heads, str(kv_cache.device))
        attn = _LayerState.attention.get(key_)
        if self.tq_codec == "hybrid":
            if attn is None:
                from ..hybrid_quantizer import HybridPagedAttention
                attn = HybridPagedAttention(_hybrid_quantizer(self.head_size, self.tq_mode, kv_cache.device),
                                            self.num_heads)
                _LayerState.attention[key_] = attn
            attn.forward(q, kc, vc, block_table, context_lens, block_size=bs, num_kv_heads=self.num_kv_heads,
                         out=out, scale=self.scale)
            return
        if attn is None:
            from ..fused_attention import TQPagedAttention
            attn = TQPagedAttention(_quantizer(self.head_size, self.tq_bits, kv_cache.device), self.num_heads)
            _LayerState.attention[key_] = attn
        kn, vn = self._norms(getattr(layer, "layer_name", "layer"), kv_cache)
        attn.forward(q, kc, kn, vc, vn, block_table, context_lens, block_size=bs, num_kv_heads=self.num_kv_heads,
                     out=out, scale=self.scale)

    def _prefill(self, layer, q, out, kv_cache, md) -> bool:
        """Prefill chunks and mixed batches through the chunked-prefill kernels (the query tokens of a sequence share
        one pass over its packed blocks); False when they are not built for the case (3- / 2-bit codes in a batch too
        ragged for the staged tensor-core kernel, rows that are not readable in 16-byte pieces), in which case every
        token becomes a row of the decode kernels."""
        pd, bs = self.packed_dim, kv_cache.shape[2]
        if self.tq_codec == "hybrid":      # tq35 records: staged tensor-core kernel over decoded operand images
            key_ = (self.head_size, self.tq_codec, self.tq_mode or self.tq_bits, self.num_heads, str(kv_cache.device))
            attn = _LayerState.attention.get(key_)
            if attn is None:
                from ..hybrid_quantizer import HybridPagedAttention
                attn = HybridPagedAttention(_hybrid_quantizer(self.head_size, self.tq_mode, kv_cache.device), self.num_heads)
                _LayerState.attention[key_] = attn
            res = attn.prefill(q, *self._codes(kv_cache), md.block_table, md.seq_lens,
                               md.query_start_loc, block_size=bs, num_kv_heads=self.num_kv_heads, out=out, scale=self.scale,
                               max_seq_len=getattr(md, "max_seq_len", None))
            return res is not None
        key_ = (self.head_size, self.tq_codec, self.tq_bits, self.num_heads, str(kv_cache.device))
        attn = _LayerState.attention.get(key_)
        if attn is None:
            from ..fused_attention import TQPagedAttention
            attn = TQPagedAttention(_quantizer(self.head_size, self.tq_bits, kv_cache.device), self.num_heads)
            _LayerState.attention[key_] = attn
        kn, vn = self._norms(getattr(layer, "layer_name", "layer"), kv_cache)
        kc, vc = self._codes(kv_cache)
        res = attn.prefill(q, kc, kn, vc, vn, md.block_table, md.seq_lens,
                           md.query_start_loc, block_size=bs, num_kv_heads=self.num_kv_heads, out=out, scale=self.scale,
                           max_seq_len=getattr(md, "max_seq_len", None))      # host-side bound from vLLM's metadata: staged kernel
        return res is not None

    def _mixed(self, layer, q, out, kv_cache, md, n) -> bool:
        """A batch with chunks: the sequences that contribute more than one token go through the chunked-prefill kernels,
        the single-token ones through the decode kernels, which stream a context once per sequence instead of once per
        mostly empty row tile.  The split is made on the device (no host copy of ``query_start_loc``): each side sees a
        length of zero for the other side's sequences and returns at once for them."""
        qsl, seq_lens = md.query_start_loc, md.seq_lens
        num_seqs = qsl.numel() - 1
        if n == num_seqs * md.max_query_len:       # every sequence brings max_query_len > 1 tokens: no decode side
            return self._prefill(layer, q, out, kv_cache, md)
        qlen = qsl[1:] - qsl[:-1]
        single = qlen == 1
        zero = torch.zeros_like(seq_lens[:num_seqs])
        chunk_md = types.SimpleNamespace(block_table=md.block_table, query_start_loc=qsl,
                                         seq_lens=torch.where(single, zero, seq_lens[:num_seqs]),
                                         max_seq_len=getattr(md, "max_seq_len", None))
        if not self._prefill(layer, q, out, kv_cache, chunk_md):
            return False
        rows = qsl[:-1].long().clamp_(max=n - 1)                      # the one query row of a single-token sequence
        dec_out = torch.empty(num_seqs, self.num_heads, self.head_size, dtype=out.dtype, device=out.device)
        self._attend(layer, q.index_select(0, rows), dec_out, kv_cache, md.block_table,
                     torch.where(single, seq_lens[:num_seqs], zero))
        # rows of the other sequences are written back unchanged (a sequence without tokens would share its row index
        # with its neighbour; vLLM schedules no such sequence)
        out.index_copy_(0, rows, torch.where(single[:, None, None], dec_out, out.index_select(0, rows)))
        return True

    def forward(self, layer, query, key, value, kv_cache, attn_metadata, output=None, output_scale=None,
                output_block_scale=None):
        if output is None:
            output = torch.empty_like(query)
        if attn_metadata is None:       # profiling run
            return output.fill_(0)
        n = attn_metadata.num_actual_tokens
        q = query[:n].view(n, self.num_heads, self.head_size)
        out = output[:n].view(n, self.num_heads, self.head_size)
        if attn_metadata.max_query_len == 1:      # one token per sequence: rows are the sequences
            self._attend(layer, q, out, kv_cache, attn_metadata.block_table, attn_metadata.seq_lens)
            return output
        if self._mixed(layer, q, out, kv_cache, attn_metadata, n):
            return output
        bt, ctx = token_rows(attn_metadata.query_start_loc, attn_metadata.seq_lens, attn_metadata.block_table, n)
        # the split-K workspace grows with the number of rows of a call: a chunk goes through in slices
        for lo in range(0, n, self.PREFILL_ROWS):
            hi = min(n, lo + self.PREFILL_ROWS)
            self._attend(layer, q[lo:hi], out[lo:hi], kv_cache, bt[lo:hi], ctx[lo:hi])
        return output


_backend_cls = None
_impl_cls = None


def _make_impl_class():
    from vllm.v1.attention.backends.triton_attn import TritonAttentionImpl

    base_params = list(inspect.signature(TritonAttentionImpl.__init__).parameters)[1:]

    class TurboQuantImpl(TurboQuantImplBase, TritonAttentionImpl):
        def __init__(self, *args, **kwargs):
            # vLLM passes kv_cache_dtype by position or by name depending on its version: find it by the
            # base class's own signature, keep it for the codec choice and give the base class "auto"
            # (it would reject the tq-* names)
            bound = dict(zip(base_params, args))
            bound.update(kwargs)
            kv_cache_dtype = bound.get("kv_cache_dtype", "auto")
            bound["kv_cache_dtype"] = "auto"
            TritonAttentionImpl.__init__(self, **bound)
            self._tq_setup(bound["num_heads"], bound["head_size"], bound["scale"],
                           bound.get("num_kv_heads") or bound["num_heads"], kv_cache_dtype)

    return TurboQuantImpl


def _make_backend_class():
    from vllm.v1.attention.backend import AttentionBackend

    class TurboQuantBackend(AttentionBackend):
        supported_kv_cache_dtypes = ["auto", "bfloat16", "fp8", "fp8_e4m3", "fp8_e5m2", *KV_DTYPE_BITS,
                                     *KV_DTYPE_HYBRID]
        accept_output_buffer = True
        forward_includes_kv_cache_update = False

        @staticmethod
        def get_name() -> str:
            return "CUSTOM"

        @staticmethod
        def get_impl_cls():
            global _impl_cls
            if _impl_cls is None:
                _impl_cls = _make_impl_class()
            return _impl_cls

        @staticmethod
        def get_builder_cls():
            from vllm.v1.attention.backend import AttentionCGSupport
            from vllm.v1.attention.backends.triton_attn import TritonAttentionMetadataBuilder

            class TQMetadataBuilder(TritonAttentionMetadataBuilder):
                # The single-token decode step is a fixed sequence of kernel launches on raw device
                # pointers (no host synchronisation, no allocation once the shared workspace exists), so
                # it can be captured; prefill and mixed batches build per-token rows whose shapes
                # follow the batch and stay eager.  (The reference declares NEVER.)
                _cudagraph_support = AttentionCGSupport.UNIFORM_SINGLE_TOKEN_DECODE

            return TQMetadataBuilder

        @staticmethod
        def get_kv_cache_shape(num_blocks, block_size, num_kv_heads, head_size, cache_dtype_str="auto"):
            from .engine import is_primary_mode, tq_dim_for_head
            if is_primary_mode():      # the cache is the packed cache: one record per (token, KV head)
                return (num_blocks, 2, block_size, num_kv_heads, tq_dim_for_head(head_size))
            return (num_blocks, 2, block_size, num_kv_heads, head_size)

        @staticmethod
        def get_supported_head_sizes():
            return [64, 128, 256]

    return TurboQuantBackend


def __getattr__(name):
    global _backend_cls, _impl_cls
    if name == "TurboQuantBackend":
        if _backend_cls is None:
            _backend_cls = _make_backend_class()
        return _backend_cls
    if name == "TurboQuantImpl":
        if _impl_cls is None:
            _impl_cls = _make_impl_class()
        return _impl_cls
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")


def register_turboquant_backend() -> bool:
    """Register the backend with vLLM; False when vLLM is not importable."""
    try:
        from vllm.v1.attention.backends.registry import AttentionBackendEnum, register_backend
    except ImportError:
        return False
    register_backend(AttentionBackendEnum.CUSTOM, "aitherkvcache_b200.vllm.backend.TurboQuantBackend")
    return True
