"""ctypes binding of libakv_b200.so (the C ABI declared in include/akv_b200.h).

There is no fallback: if the shared library is missing or a call fails, an
exception is raised.
"""
from __future__ import annotations

import ctypes as C
import os

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libakv_b200.so")

AKV_F16, AKV_BF16, AKV_F32 = 0, 1, 2
AKV_I32, AKV_I64 = 0, 1

_FLOAT_CODES = {torch.float16: AKV_F16, torch.bfloat16: AKV_BF16, torch.float32: AKV_F32}
_INDEX_CODES = {torch.int32: AKV_I32, torch.int64: AKV_I64}

c_i64, c_int, c_vp, c_f = C.c_int64, C.c_int, C.c_void_p, C.c_float


class TQAttnParams(C.Structure):
    """Mirror of ``akv_tq_attn_params``."""
    _fields_ = [
        ("query", c_vp), ("q_dtype", c_int), ("q_stride_seq", c_i64), ("q_stride_head", c_i64),
        ("k_packed", c_vp), ("kp_stride_blk", c_i64), ("kp_stride_pos", c_i64), ("kp_stride_head", c_i64),
        ("k_norms", c_vp), ("kn_stride_blk", c_i64), ("kn_stride_pos", c_i64), ("kn_stride_head", c_i64),
        ("v_packed", c_vp), ("vp_stride_blk", c_i64), ("vp_stride_pos", c_i64), ("vp_stride_head", c_i64),
        ("v_norms", c_vp), ("vn_stride_blk", c_i64), ("vn_stride_pos", c_i64), ("vn_stride_head", c_i64),
        ("block_tables", c_vp), ("bt_dtype", c_int), ("bt_stride_seq", c_i64),
        ("context_lens", c_vp), ("cl_dtype", c_int),
        ("num_seqs", c_int), ("num_q_heads", c_int), ("num_kv_heads", c_int), ("head_dim", c_int),
        ("block_size", c_int), ("max_blocks_per_seq", c_int),
        ("num_blocks", c_i64),
        ("bits", c_int),
        ("rotation", c_vp), ("rotation_t", c_vp), ("centroids", c_vp),
        ("scale", c_f),
        ("out", c_vp), ("out_dtype", c_int), ("out_stride_seq", c_i64), ("out_stride_head", c_i64),
        ("raw_out", c_vp),
        ("workspace", c_vp), ("workspace_bytes", C.c_size_t),
        ("blocks_per_split", c_int),
        ("stream", c_vp),
        ("ev_kernel_start", c_vp), ("ev_kernel_stop", c_vp),
        ("out_copy", c_vp),
    ]


class TQPrefillParams(C.Structure):
    """Mirror of ``akv_tq_prefill_params``."""
    _fields_ = [
        ("query", c_vp), ("q_dtype", c_int), ("q_stride_tok", c_i64), ("q_stride_head", c_i64),
        ("k_packed", c_vp), ("kp_stride_blk", c_i64), ("kp_stride_pos", c_i64), ("kp_stride_head", c_i64),
        ("k_norms", c_vp), ("kn_stride_blk", c_i64), ("kn_stride_pos", c_i64), ("kn_stride_head", c_i64),
        ("v_packed", c_vp), ("vp_stride_blk", c_i64), ("vp_stride_pos", c_i64), ("vp_stride_head", c_i64),
        ("v_norms", c_vp), ("vn_stride_blk", c_i64), ("vn_stride_pos", c_i64), ("vn_stride_head", c_i64),
        ("block_tables", c_vp), ("bt_dtype", c_int), ("bt_stride_seq", c_i64),
        ("seq_lens", c_vp), ("sl_dtype", c_int),
        ("query_start_loc", c_vp), ("qs_dtype", c_int),
        ("num_seqs", c_int), ("num_tokens", c_int), ("num_q_heads", c_int), ("num_kv_heads", c_int),
        ("head_dim", c_int), ("block_size", c_int), ("max_blocks_per_seq", c_int),
        ("num_blocks", c_i64),
        ("bits", c_int),
        ("rotation", c_vp), ("rotation_t", c_vp), ("centroids", c_vp),
        ("scale", c_f),
        ("out", c_vp), ("out_dtype", c_int), ("out_stride_tok", c_i64), ("out_stride_head", c_i64),
        ("workspace", c_vp), ("workspace_bytes", C.c_size_t),
        ("stream", c_vp),
        ("max_seq_len", c_int),
        ("hybrid_tables", c_vp),
    ]


class TQDecodeStepParams(C.Structure):
    """Mirror of ``akv_tq_decode_step_params``."""
    _fields_ = [
        ("key", c_vp), ("value", c_vp), ("kv_dtype", c_int),
        ("num_tokens", c_i64),
        ("k_stride_tok", c_i64), ("k_stride_head", c_i64), ("v_stride_tok", c_i64), ("v_stride_head", c_i64),
        ("slot_mapping", c_vp),
        ("boundaries", c_vp),
        ("max_blocks", c_i64),
        ("attn", TQAttnParams),
    ]


class HybridTables(C.Structure):
    """Mirror of ``akv_hybrid_tables``."""
    _fields_ = [
        ("head_dim", c_int), ("packed_dim", c_int),
        ("group_index", c_vp), ("num_index_heads", c_int),
        ("had_signs", c_vp), ("qjl_signs", c_vp), ("centroids", c_vp), ("boundaries", c_vp),
        ("qjl_scale0", c_f), ("qjl_scale1", c_f),
    ]


class HybridAttnParams(C.Structure):
    """Mirror of ``akv_hybrid_attn_params``."""
    _fields_ = [
        ("query", c_vp), ("q_dtype", c_int), ("q_stride_seq", c_i64), ("q_stride_head", c_i64),
        ("k_cache", c_vp), ("k_stride_blk", c_i64), ("k_stride_pos", c_i64), ("k_stride_head", c_i64),
        ("v_cache", c_vp), ("v_stride_blk", c_i64), ("v_stride_pos", c_i64), ("v_stride_head", c_i64),
        ("block_tables", c_vp), ("bt_dtype", c_int), ("bt_stride_seq", c_i64),
        ("context_lens", c_vp), ("cl_dtype", c_int),
        ("num_seqs", c_int), ("num_q_heads", c_int), ("num_kv_heads", c_int), ("block_size", c_int),
        ("max_blocks_per_seq", c_int),
        ("num_blocks", c_i64),
        ("tables", C.POINTER(HybridTables)),
        ("scale", c_f),
        ("out", c_vp), ("out_dtype", c_int), ("out_stride_seq", c_i64), ("out_stride_head", c_i64),
        ("workspace", c_vp), ("workspace_bytes", C.c_size_t),
        ("blocks_per_split", c_int),
        ("stream", c_vp),
    ]


class HybridDecodeStepParams(C.Structure):
    """Mirror of ``akv_hybrid_decode_step_params``."""
    _fields_ = [
        ("key", c_vp), ("value", c_vp), ("kv_dtype", c_int),
        ("num_tokens", c_i64),
        ("k_stride_tok", c_i64), ("k_stride_head", c_i64), ("v_stride_tok", c_i64), ("v_stride_head", c_i64),
        ("slot_mapping", c_vp),
        ("max_blocks", c_i64),
        ("attn", HybridAttnParams),
    ]


class P2PMergeParams(C.Structure):
    """Mirror of ``akv_p2p_merge_params``."""
    _fields_ = [
        ("local_raw", c_vp),
        ("num_seqs", c_int), ("num_q_heads", c_int), ("head_dim", c_int),
        ("world", c_int), ("rank", c_int),
        ("peer_buffers", C.POINTER(c_vp)), ("peer_flags", C.POINTER(c_vp)),
        ("state", c_vp),
        ("rotation", c_vp),
        ("out", c_vp), ("out_dtype", c_int), ("out_stride_seq", c_i64), ("out_stride_head", c_i64),
        ("stream", c_vp),
    ]


class TriDecodeParams(C.Structure):
    """Mirror of ``akv_tri_decode_params``."""
    _fields_ = [
        ("query", c_vp), ("q_dtype", c_int), ("q_stride_batch", c_i64), ("q_stride_head", c_i64),
        ("k_indices", c_vp), ("k_packed", c_vp), ("k_scales", c_vp),
        ("v_indices", c_vp), ("v_packed", c_vp), ("v_scales", c_vp),
        ("batch", c_int), ("seq_len", c_int), ("num_kv_heads", c_int), ("num_q_heads", c_int),
        ("head_dim", c_int), ("num_freqs", c_int),
        ("key_positions", c_vp), ("key_pos_start", c_i64),
        ("query_pos", c_vp), ("query_pos_default", c_i64),
        ("theta", c_vp),
        ("scale", c_f),
        ("out", c_vp), ("raw_out", c_vp),
        ("workspace", c_vp), ("workspace_bytes", C.c_size_t),
        ("tokens_per_split", c_int),
        ("stream", c_vp),
        ("ev_kernel_start", c_vp), ("ev_kernel_stop", c_vp),
        ("scores_out", c_vp),
        ("block_tables", c_vp), ("bt_dtype", c_int), ("bt_stride_batch", c_i64),
        ("block_size", c_int), ("num_blocks", c_i64),
        ("context_lens", c_vp), ("cl_dtype", c_int),
        ("coeff_bits", c_int), ("post_rope", c_int),
    ]


_SIGNATURES = {
    "akv_version": (c_int, []),
    "akv_last_error": (C.c_char_p, []),
    "akv_device_arch": (c_int, []),
    "akv_launch_count": (C.c_longlong, []),
    "akv_last_split_kernel": (C.c_char_p, []),
    "akv_device_status": (c_int, [C.POINTER(c_int), c_int]),
    "akv_debug_tc_withhold": (c_int, [c_int, c_int]),
    "akv_tq_encode": (c_int, [c_vp, c_int, c_i64, c_i64, c_int, c_int, c_vp, c_vp, c_vp, c_i64, c_vp, c_vp]),
    "akv_tq_decode": (c_int, [c_vp, c_i64, c_vp, c_i64, c_int, c_int, c_vp, c_vp, c_vp, c_int, c_vp]),
    "akv_tq_kv_update": (c_int, [c_vp, c_int, c_i64, c_int, c_int, c_i64, c_i64, c_vp, c_vp, c_i64, c_i64,
                                 c_i64, c_vp, c_i64, c_i64, c_i64, c_int, c_vp, c_vp, c_int, c_i64, c_vp]),
    "akv_tq_paged_attn_workspace_bytes": (C.c_size_t, [c_int] * 8),
    "akv_tq_paged_attn": (c_int, [C.POINTER(TQAttnParams)]),
    "akv_tq_prefill_attn_workspace_bytes": (C.c_size_t, [c_int, c_int]),
    "akv_tq_prefill_attn_workspace_bytes_staged": (C.c_size_t, [c_int] * 5),
    "akv_tq_prefill_attn": (c_int, [C.POINTER(TQPrefillParams)]),
    "akv_tq_decode_step": (c_int, [C.POINTER(TQDecodeStepParams)]),
    "akv_tq_paged_attn_static_scratch_bytes": (C.c_size_t, []),
    "akv_tq_paged_attn_static": (c_int, [C.POINTER(TQAttnParams)]),
    "akv_block_select_update": (c_int, [c_vp, c_i64, c_vp, c_i64, c_i64, c_vp, c_i64, c_i64, c_vp, c_int, c_int, c_int,
                                        c_i64, c_vp, c_vp, c_vp, c_vp]),
    "akv_block_select_clear": (c_int, [c_vp, c_i64, c_int, c_i64, c_vp, c_vp, c_vp, c_vp]),
    "akv_block_select_workspace_bytes": (C.c_size_t, [c_int] * 3),
    "akv_block_select": (c_int, [c_vp, c_int, c_i64, c_i64, c_int, c_int, c_int, c_int, c_vp, c_vp, c_i64, c_vp, c_int,
                                 c_i64, c_vp, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_vp, c_vp, c_vp, c_vp,
                                 C.c_size_t, c_vp]),
    "akv_hybrid_encode": (c_int, [c_vp, c_int, c_i64, c_i64, C.POINTER(HybridTables), c_vp, c_i64, c_vp]),
    "akv_hybrid_decode": (c_int, [c_vp, c_i64, c_i64, C.POINTER(HybridTables), c_vp, c_int, c_vp]),
    "akv_hybrid_paged_attn_workspace_bytes": (C.c_size_t, [c_int] * 5),
    "akv_hybrid_paged_attn": (c_int, [C.POINTER(HybridAttnParams)]),
    "akv_hybrid_kv_update": (c_int, [c_vp, c_int, c_i64, c_int, c_i64, c_i64, c_vp, C.POINTER(HybridTables), c_vp,
                                     c_i64, c_i64, c_i64, c_int, c_i64, c_vp]),
    "akv_hybrid_decode_step": (c_int, [C.POINTER(HybridDecodeStepParams)]),
    "akv_tri_encode": (c_int, [c_vp, c_int, c_i64, c_i64, c_int, c_int, c_vp, c_vp, c_vp, c_vp]),
    "akv_tri_encode_bits": (c_int, [c_vp, c_int, c_i64, c_i64, c_int, c_int, c_int, c_vp, c_vp, c_vp, c_vp]),
    "akv_tri_decode_workspace_bytes": (C.c_size_t, [c_int] * 4),
    "akv_tri_decode_step": (c_int, [C.POINTER(TriDecodeParams)]),
    "akv_p2p_exchange_bytes": (C.c_size_t, [c_int] * 4),
    "akv_p2p_lse_merge": (c_int, [C.POINTER(P2PMergeParams)]),
    "akv_lse_merge": (c_int, [c_vp, c_int, c_int, c_int, c_int, c_vp, c_vp, c_int, c_i64, c_i64, c_vp]),
}

_lib = None


def exported_symbols():
    """Names every build of the library must export."""
    return sorted(_SIGNATURES)


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m aitherkvcache_b200._build` "
                "(there is no CPU or Triton fallback)")
        handle = C.CDLL(LIB_PATH)
        for name, (res, args) in _SIGNATURES.items():
            fn = getattr(handle, name)
            fn.restype, fn.argtypes = res, args
        _lib = handle
    return _lib


AKV_ERR_ARG, AKV_ERR_UNSUPPORTED, AKV_ERR_WORKSPACE = -1, -2, -3


class AkvError(RuntimeError):
    pass


def check(rc: int, what: str) -> None:
    if rc != 0:
        msg = lib().akv_last_error().decode("utf-8", "replace")
        if rc == -1:
            raise ValueError(f"{what}: {msg}")
        raise AkvError(f"{what} failed (code {rc}): {msg}")


def device_status(reset: bool = False) -> dict:
    """Device-side status words of the current device (synchronises): all zero unless a bounded
    wait gave up or a fixed-address kernel found its shared-memory window taken."""
    out = (c_int * 5)()
    check(lib().akv_device_status(out, 1 if reset else 0), "akv_device_status")
    return {"tc_encode": out[0], "tc_decode": out[1], "attn_window": out[2], "hybrid_window": out[3], "p2p": out[4]}


def float_code(t: torch.Tensor) -> int:
    try:
        return _FLOAT_CODES[t.dtype]
    except KeyError:
        raise TypeError(f"unsupported floating dtype {t.dtype}") from None


def index_code(t: torch.Tensor) -> int:
    try:
        return _INDEX_CODES[t.dtype]
    except KeyError:
        raise TypeError(f"index tensors must be int32 or int64, got {t.dtype}") from None


def require_cuda(*tensors: torch.Tensor) -> torch.device:
    dev = None
    for t in tensors:
        if t is None:
            continue
        if not t.is_cuda:
            raise RuntimeError(
                "aitherkvcache_b200 runs on CUDA tensors only (no CPU fallback); got a tensor on "
                f"{t.device}")
        if dev is None:
            dev = t.device
        elif t.device != dev:
            raise RuntimeError(f"tensors on different devices: {dev} and {t.device}")
    return dev


def stream_ptr(device: torch.device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def ptr(t) -> int:
    return 0 if t is None else t.data_ptr()
