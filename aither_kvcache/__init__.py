"""Import-path alias: ``import aither_kvcache`` (the reference's package name) resolves to the
sm_100a implementation in ``aitherkvcache_b200``, so code written against the reference's module
paths - ``aither_kvcache.quantizer``, ``aither_kvcache.fused_attention``,
``aither_kvcache.hybrid_quantizer``, ``aither_kvcache.triattention``, ``aither_kvcache.vllm.ops`` ... -
runs unchanged.  Do not install next to the reference itself: both would claim the same name."""
import importlib
import sys

import aitherkvcache_b200 as _impl
from aitherkvcache_b200 import *  # noqa: F401,F403
from aitherkvcache_b200 import __all__, __version__  # noqa: F401

_SUBMODULES = ("quantizer", "codebook", "rotation", "packing", "fused_attention", "fused_kv_update",
               "hybrid_quantizer", "parallel", "triattention", "triattention.config", "triattention.encoder",
               "triattention.attention", "triattention.spectral", "vllm", "vllm.ops", "vllm.backend", "vllm.plugin")
for _name in _SUBMODULES:
    sys.modules[f"{__name__}.{_name}"] = importlib.import_module(f"aitherkvcache_b200.{_name}")
for _name in ("quantizer", "codebook", "rotation", "packing", "fused_attention", "fused_kv_update",
              "hybrid_quantizer", "parallel", "triattention", "vllm"):
    setattr(sys.modules[__name__], _name, sys.modules[f"{__name__}.{_name}"])
