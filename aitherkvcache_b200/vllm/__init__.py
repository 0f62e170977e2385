"""Serving-side surface: the ``tq::decode_step`` / ``tq::hybrid_decode_step`` custom ops
and the vLLM ``CUSTOM`` attention backend, wired to the sm_100a kernels."""
from .ops import (decode_step, hybrid_decode_step, init_hybrid_quantizer, init_quantizer,  # noqa: F401
                  register_custom_ops)
