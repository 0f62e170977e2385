"""vLLM v1 ``CUSTOM`` attention backend over a TurboQuant-packed KV cache.

Surface of the reference's ``aither_kvcache/vllm/backend.py`` (``TurboQuantBackend`` :261-311,
``TurboQuantImpl`` :324-1273, ``register_turboquant_backend`` :1280-1295) restricted to what the
hot path needs: the cache is uint8 ``[num_blocks, 2, block_size, kv_heads, packed_dim + 4]``
(``get_kv_cache_shape`` keeps the reference's 5-D form), ``do_kv_cache_update`` encodes new
K/V straight into it (norms in per-layer float32 tensors, as the reference's PRIMARY mode),
and decode steps call the paged attention kernel on strided views of it.  Prefill chunks
(more than one query token per sequence) decode the needed blocks and use dense attention;
the reference's shadow mode, cold tier and block selection are not part of this build.

The codec is picked like the reference does (``AITHER_TQ_BITS``, default 4) or from a
``tq-t4nc`` / ``tq-t3nc`` / ``tq-t2nc`` cache-dtype string.  The classes are created on first
attribute access so that importing this module does not import vLLM.
"""
from __future__ import annotations

import math
import os
from typing import Dict, Optional

import torch

KV_DTYPE_BITS = {"tq-t4nc": 4, "tq-t3nc": 3, "tq-t2nc": 2}


def bits_from_env_or_dtype(cache_dtype_str: Optional[str] = None) -> int:
    if cache_dtype_str in KV_DTYPE_BITS:
        return KV_DTYPE_BITS[cache_dtype_str]
    return int(os.environ.get("AITHER_TQ_BITS", "4"))


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


class TurboQuantImplBase:
    """Backend-independent part of the impl (usable and testable without vLLM)."""

    def _tq_setup(self, num_heads: int, head_size: int, scale: float, num_kv_heads: int,
                  kv_cache_dtype: str = "auto") -> None:
        self.num_heads, self.head_size, self.scale = num_heads, head_size, float(scale)
        self.num_kv_heads = num_kv_heads
        self.tq_bits = bits_from_env_or_dtype(kv_cache_dtype)
        self.packed_dim = head_size * self.tq_bits // 8

    def _norms(self, layer_name: str, kv_cache: torch.Tensor):
        kn = _LayerState.k_norms.get(layer_name)
        shape = (kv_cache.shape[0], kv_cache.shape[2], kv_cache.shape[3])
        if kn is None or kn.shape != shape or kn.device != kv_cache.device:
            kn = torch.zeros(shape, dtype=torch.float32, device=kv_cache.device)
            _LayerState.k_norms[layer_name] = kn
            _LayerState.v_norms[layer_name] = torch.zeros_like(kn)
        return kn, _LayerState.v_norms[layer_name]

    def do_kv_cache_update(self, layer, key, value, kv_cache, slot_mapping) -> None:
        """Encode ``key`` / ``value`` [tokens, kv_heads, head_size] into the packed cache in place."""
        from ..fused_kv_update import fused_tq4_kv_update
        tq = _quantizer(self.head_size, self.tq_bits, kv_cache.device)
        kn, vn = self._norms(getattr(layer, "layer_name", "layer"), kv_cache)
        pd, bs = self.packed_dim, kv_cache.shape[2]
        for x, side, norms in ((key, 0, kn), (value, 1, vn)):
            fused_tq4_kv_update(x, slot_mapping, kv_cache[:, side, :, :, :pd], norms, tq.rotation,
                                tq.boundaries_inner, bs, kv_cache.shape[0], rotation_t=tq.rotation_T)

    def forward(self, layer, query, key, value, kv_cache, attn_metadata, output=None, output_scale=None,
                output_block_scale=None):
        if output is None:
            output = torch.empty_like(query)
        if attn_metadata is None:       # profiling run
            return output.fill_(0)
        n = attn_metadata.num_actual_tokens
        q = query[:n].view(n, self.num_heads, self.head_size)
        out = output[:n].view(n, self.num_heads, self.head_size)
        tq = _quantizer(self.head_size, self.tq_bits, kv_cache.device)
        kn, vn = self._norms(getattr(layer, "layer_name", "layer"), kv_cache)
        pd, bs = self.packed_dim, kv_cache.shape[2]
        kc, vc = kv_cache[:, 0, :, :, :pd], kv_cache[:, 1, :, :, :pd]
        if attn_metadata.max_query_len == 1:
            from ..fused_attention import TQPagedAttention
            key_ = (self.head_size, self.tq_bits, self.num_heads, str(kv_cache.device))
            attn = _LayerState.attention.get(key_)
            if attn is None:
                attn = TQPagedAttention(tq, self.num_heads)
                _LayerState.attention[key_] = attn
            attn.forward(q, kc, kn, vc, vn, attn_metadata.block_table, attn_metadata.seq_lens, block_size=bs,
                         num_kv_heads=self.num_kv_heads, out=out, scale=self.scale)
            return output
        self._prefill(q, out, tq, kc, kn, vc, vn, attn_metadata, bs)
        return output

    def _prefill(self, q, out, tq, kc, kn, vc, vn, md, bs) -> None:
        """Chunked prefill: decode each sequence's context to fp16 and run causal dense attention."""
        starts = md.query_start_loc.tolist()
        lens = md.seq_lens.tolist()
        gqa = self.num_heads // self.num_kv_heads
        for s in range(len(lens)):
            q0, q1 = starts[s], starts[s + 1]
            if q1 <= q0:
                continue
            ctx = lens[s]
            blocks = md.block_table[s, :(ctx + bs - 1) // bs].long()
            k = tq.decode(kc[blocks].reshape(-1, self.num_kv_heads, kc.shape[-1])[:ctx],
                          kn[blocks].reshape(-1, self.num_kv_heads)[:ctx])
            v = tq.decode(vc[blocks].reshape(-1, self.num_kv_heads, vc.shape[-1])[:ctx],
                          vn[blocks].reshape(-1, self.num_kv_heads)[:ctx])
            kh = k.permute(1, 0, 2).repeat_interleave(gqa, dim=0).to(q.dtype)
            vh = v.permute(1, 0, 2).repeat_interleave(gqa, dim=0).to(q.dtype)
            nq = q1 - q0
            pos_q = torch.arange(ctx - nq, ctx, device=q.device)[:, None]
            mask = torch.arange(ctx, device=q.device)[None, :] <= pos_q
            o = torch.nn.functional.scaled_dot_product_attention(q[q0:q1].transpose(0, 1), kh, vh, attn_mask=mask,
                                                                 scale=self.scale)
            out[q0:q1] = o.transpose(0, 1)


_backend_cls = None
_impl_cls = None


def _make_impl_class():
    from vllm.v1.attention.backends.triton_attn import TritonAttentionImpl

    class TurboQuantImpl(TurboQuantImplBase, TritonAttentionImpl):
        def __init__(self, num_heads, head_size, scale, num_kv_heads=None, *args, kv_cache_dtype="auto", **kwargs):
            TritonAttentionImpl.__init__(self, num_heads, head_size, scale, num_kv_heads, *args,
                                         kv_cache_dtype="auto", **kwargs)
            self._tq_setup(num_heads, head_size, scale, num_kv_heads or num_heads, kv_cache_dtype)

    return TurboQuantImpl


def _make_backend_class():
    from vllm.v1.attention.backend import AttentionBackend

    class TurboQuantBackend(AttentionBackend):
        supported_kv_cache_dtypes = ["auto", "bfloat16", "fp8", "fp8_e4m3", "fp8_e5m2", *KV_DTYPE_BITS]
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
                _cudagraph_support = AttentionCGSupport.NEVER

            return TQMetadataBuilder

        @staticmethod
        def get_kv_cache_shape(num_blocks, block_size, num_kv_heads, head_size, cache_dtype_str="auto"):
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
