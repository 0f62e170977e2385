"""PRIMARY-mode page sizing: vLLM allocates blocks of the compressed size, and the cache IS the packed cache.

Interface of the reference's ``vllm/engine.py`` (``apply_tq_patches`` :52-107, ``_tq_page_size_bytes`` :110-123,
``_tq_dim_for_head`` :126-135, ``_align_page_size`` :138-154, ``_patch_page_size`` :157-193, ``_patch_max_memory``
:196-220).  A row of the primary cache is one record of ``tq_dim`` bytes per (token, KV head):

* uniform codecs: ``packed_dim + 4`` bytes per (token, KV head) as in the reference, which leaves four of them
  unused and keeps norms in separate tensors (``vllm/backend.py:440-454``); here they hold the float32 norm.  Inside
  a block's K half and V half the bytes are laid out in planes - all code rows, then all norms - so that code rows
  start on 16-byte boundaries (TMA copies, 16-byte loads); ``AITHER_TQ_RECORD_PAGES=1`` keeps the norm behind the codes
  of its own row (68-byte records), which the general kernels read through strided pointers at half the speed;
* hybrid codecs: the 64 / 44-byte record, norms inside.

With the installed vLLM the cache tensor is shaped by the backend's own ``get_kv_cache_shape`` (which returns the
record layout in primary mode, see ``backend.py``), so no reshape patch is needed; the reference's block-manager / free
hook (cold tier) is not part of this build.
"""
from __future__ import annotations

import logging
import os

logger = logging.getLogger("aitherkvcache_b200.engine")

_ORIGINALS: dict = {}


def tq_mode_from_env() -> str:
    """``AITHER_TQ_MODE`` without the ``-primary`` suffix ("" when unset)."""
    return os.environ.get("AITHER_TQ_MODE", "").replace("-primary", "")


def is_primary_mode() -> bool:
    mode = os.environ.get("AITHER_TQ_MODE", "")
    if mode:
        return mode.endswith("-primary")
    return os.environ.get("AITHER_TQ_PRIMARY", "0") == "1"


def _bits(bits=None) -> int:
    mode = tq_mode_from_env()
    if bits is None and mode in ("tq4", "tq3", "tq2"):
        return int(mode[2])
    return int(bits if bits is not None else os.environ.get("AITHER_TQ_BITS", "4"))


def tq_dim_for_head(head_size: int, bits=None) -> int:
    """Bytes of one record (last axis of the primary cache)."""
    mode = tq_mode_from_env()
    if mode in ("tq35", "tq25"):
        from ..hybrid_quantizer import HybridTurboQuant
        return HybridTurboQuant.packed_dim_for_mode(head_size, mode)
    from ..packing import packed_size
    return packed_size(head_size, _bits(bits)) + 4


def tq_page_size_bytes(block_size: int, num_kv_heads: int, head_size: int, bits=None) -> int:
    """Bytes of one block of the primary cache (K and V)."""
    return 2 * block_size * num_kv_heads * tq_dim_for_head(head_size, bits)


def align_page_size(raw_bytes: int) -> int:
    """Next power of two: page sizes of layers with different head sizes then divide one another."""
    if raw_bytes <= 0:
        return raw_bytes
    return 1 << (raw_bytes - 1).bit_length()


def apply_tq_patches(bits: int = 4) -> bool:
    """Make vLLM size its KV-cache blocks for the packed records (primary mode only; call before the
    engine starts).  Returns True when every patch that the mode needs is in place."""
    if bits == 0:
        return True
    if not is_primary_mode():
        logger.info("AITHER_TQ_MODE is not a -primary mode: vLLM keeps its own page size")
        return True
    os.environ.setdefault("AITHER_TQ_BITS", str(bits))
    try:
        from vllm.v1.kv_cache_interface import AttentionSpec, FullAttentionSpec
    except ImportError:
        logger.warning("vLLM v1 KV-cache specs not found: page-size patch skipped")
        return False

    # The installed vLLM views a layer's raw bytes with the backend's own cache shape, so a page must be exactly
    # block_size x heads x 2 records; the reference's power-of-two rounding (for models whose layers differ in head
    # size) is kept behind AITHER_TQ_ALIGN_PAGES=1, for a runner that strides over padded pages.
    pad = os.environ.get("AITHER_TQ_ALIGN_PAGES", "0") == "1"

    def _real_page_size_bytes(self):
        raw = tq_page_size_bytes(self.block_size, self.num_kv_heads, self.head_size)
        return align_page_size(raw) if pad else raw

    def _max_memory_usage_bytes(self, vllm_config):
        max_model_len = vllm_config.model_config.max_model_len
        try:
            pc = vllm_config.parallel_config
            ways = pc.decode_context_parallel_size * pc.prefill_context_parallel_size
            if ways > 1:
                max_model_len = -(-max_model_len // ways)
        except AttributeError:
            pass
        return -(-max_model_len // self.block_size) * self.page_size_bytes

    for cls in (AttentionSpec, FullAttentionSpec):
        _ORIGINALS.setdefault((cls, "real_page_size_bytes"), cls.__dict__.get("real_page_size_bytes"))
        cls.real_page_size_bytes = property(_real_page_size_bytes)
    _ORIGINALS.setdefault((FullAttentionSpec, "max_memory_usage_bytes"), FullAttentionSpec.__dict__.get("max_memory_usage_bytes"))
    FullAttentionSpec.max_memory_usage_bytes = _max_memory_usage_bytes
    logger.info("page size patched: %d bytes per block of 16 x 8 heads x 128 (fp16: %d)",
                tq_page_size_bytes(16, 8, 128), 2 * 16 * 8 * 128 * 2)
    return True


def remove_tq_patches() -> None:
    """Put back what ``apply_tq_patches`` replaced (tests)."""
    for (cls, name), orig in list(_ORIGINALS.items()):
        if orig is None:
            try:
                delattr(cls, name)
            except AttributeError:
                pass
        else:
            setattr(cls, name, orig)
    _ORIGINALS.clear()
