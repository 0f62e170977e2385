"""vLLM plugin entry point (``vllm.general_plugins``): registers the TurboQuant attention
backend under ``AttentionBackendEnum.CUSTOM`` (``--attention-backend CUSTOM``), as the
reference's ``aither_kvcache/vllm/plugin.py:18-33`` does.  The eviction plugin the reference
installs next to it is not part of this package."""
import sys


def register() -> None:
    try:
        from vllm.v1.attention.backends.registry import AttentionBackendEnum, register_backend
    except ImportError:
        return          # vLLM (v1) is not installed
    try:
        register_backend(AttentionBackendEnum.CUSTOM, "aitherkvcache_b200.vllm.backend.TurboQuantBackend")
        print("[aitherkvcache_b200] registered TurboQuant CUSTOM attention backend", file=sys.stderr, flush=True)
    except Exception as exc:        # never take the server down from a plugin hook
        print(f"[aitherkvcache_b200] backend registration failed: {exc}", file=sys.stderr, flush=True)
