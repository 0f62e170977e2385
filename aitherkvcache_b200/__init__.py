"""B200-native kernels behind the aither-kvcache compressed-KV API.

    from aitherkvcache_b200 import TurboQuant, TQPagedAttention
    tq = TurboQuant(head_dim=128, bits=4)        # device="cuda"
    packed, norms = tq.encode(kv)
    kv_hat = tq.decode(packed, norms)

Everything numeric runs in hand-written sm_100a CUDA kernels loaded from
``libakv_b200.so`` (see include/akv_b200.h); there is no Triton and no CPU path.
"""
from .quantizer import TurboQuant, TurboQuantConfig
from .fused_attention import TQPagedAttention
from .fused_kv_update import fused_tq4_kv_update, fused_encode_and_store

# kv-cache dtype names of the serving integration -> codec selection
KV_CACHE_DTYPES = {
    "tq-t4nc": {"kind": "uniform", "bits": 4},
    "tq-t3nc": {"kind": "uniform", "bits": 3},
    "tq-t2nc": {"kind": "uniform", "bits": 2},
    "tq-t35nc": {"kind": "hybrid", "mode": "tq35"},
}

__all__ = [
    "TurboQuant", "TurboQuantConfig", "TQPagedAttention",
    "fused_tq4_kv_update", "fused_encode_and_store", "KV_CACHE_DTYPES",
]
__version__ = "0.1.0"
