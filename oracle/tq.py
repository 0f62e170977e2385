"""numpy restatement of the uniform TurboQuant codec and its paged attention.

TEST INFRASTRUCTURE ONLY (see oracle/__init__.py).

Reference files followed (paths inside the reference project):
  aither_kvcache/codebook.py:28-82      Lloyd-Max tables, 1/sqrt(d) scaling
  aither_kvcache/packing.py:13-131      MSB-first 4/3/2-bit packing
  aither_kvcache/quantizer.py:122-212   encode / decode
  aither_kvcache/fused_kv_update.py:220-293   paged write (torch fallback)
  aither_kvcache/fused_attention.py:91-185    rotated-domain paged attention
  aither_kvcache/vllm/hooks.py:303-345        decode -> fp16 -> SDPA attention
"""
from __future__ import annotations

import math
import numpy as np

# Standard-normal Lloyd-Max centroids (Max 1960), as tabulated by the
# reference in codebook.py:28-53.  Positive halves only; the tables are odd.
_HALF = {
    1: [0.798284],
    2: [0.452781, 1.510469],
    3: [0.245104, 0.756031, 1.344134, 2.152090],
    4: [0.128350, 0.388089, 0.656804, 0.942391,
        1.256233, 1.618002, 2.069016, 2.733266],
}


def codebook(d: int, bits: int):
    """(centroids f32[2^bits], inner boundaries f32[2^bits-1]).

    codebook.py:62-82 scales by 1/sqrt(d) and takes midpoints in float64;
    quantizer.py:95-99 then stores both as float32.
    """
    if bits not in _HALF:
        raise ValueError(f"Supported bit-widths: {sorted(_HALF)}. Got {bits}")
    pos = np.asarray(_HALF[bits], dtype=np.float64)
    std = np.concatenate([-pos[::-1], pos])
    c64 = std * (1.0 / math.sqrt(d))
    b64 = (c64[:-1] + c64[1:]) / 2
    return c64.astype(np.float32), b64.astype(np.float32)


def packed_size(dim: int, bits: int) -> int:
    """packing.py:121-131."""
    if bits == 4:
        return dim // 2
    if bits == 3:
        assert dim % 8 == 0
        return dim * 3 // 8
    if bits == 2:
        return dim // 4
    raise ValueError(f"Unsupported bit-width: {bits}")


def pack(idx: np.ndarray, bits: int) -> np.ndarray:
    """MSB-first packing of [..., D] codes (packing.py:13-98)."""
    idx = np.asarray(idx).astype(np.uint32)
    lead = idx.shape[:-1]
    D = idx.shape[-1]
    if bits == 4:
        return ((idx[..., 0::2] << 4) | idx[..., 1::2]).astype(np.uint8)
    if bits == 2:
        return ((idx[..., 0::4] << 6) | (idx[..., 1::4] << 4)
                | (idx[..., 2::4] << 2) | idx[..., 3::4]).astype(np.uint8)
    if bits == 3:
        g = idx.reshape(*lead, D // 8, 8)
        word = np.zeros(g.shape[:-1], dtype=np.uint32)
        for i in range(8):
            word |= (g[..., i] & 7) << (21 - 3 * i)
        out = np.stack([(word >> 16) & 0xFF, (word >> 8) & 0xFF, word & 0xFF], axis=-1)
        return out.reshape(*lead, (D // 8) * 3).astype(np.uint8)
    raise ValueError(bits)


def unpack(packed: np.ndarray, dim: int, bits: int) -> np.ndarray:
    """Inverse of :func:`pack` -> uint8 [..., dim]."""
    p = np.asarray(packed).astype(np.uint32)
    lead = p.shape[:-1]
    out = np.empty((*lead, dim), dtype=np.uint8)
    if bits == 4:
        out[..., 0::2] = (p >> 4) & 15
        out[..., 1::2] = p & 15
    elif bits == 2:
        out[..., 0::4] = (p >> 6) & 3
        out[..., 1::4] = (p >> 4) & 3
        out[..., 2::4] = (p >> 2) & 3
        out[..., 3::4] = p & 3
    elif bits == 3:
        g = p.reshape(*lead, dim // 8, 3)
        word = (g[..., 0] << 16) | (g[..., 1] << 8) | g[..., 2]
        o = out.reshape(*lead, dim // 8, 8)
        for i in range(8):
            o[..., i] = (word >> (21 - 3 * i)) & 7
    else:
        raise ValueError(bits)
    return out


def l2norm_f32(x: np.ndarray) -> np.ndarray:
    """Row L2 norm with the rounding order of torch's CPU ``x.norm(dim=-1)``.

    quantizer.py:144 calls ``x_flat.norm(dim=-1)`` on float32 rows.  That
    reduction keeps eight strided float32 partial sums (element i goes to lane
    i mod 8), squares and adds with separate roundings, folds the lanes
    0..7 in order and takes sqrtf.  The recipe was found by probing torch
    2.11 CPU and reproduces it bit for bit for row lengths 32..256.
    """
    x = np.ascontiguousarray(x, dtype=np.float32)
    n, d = x.shape
    sq = x * x
    if d % 8:
        padded = np.zeros((n, (d + 7) // 8 * 8), np.float32)
        padded[:, :d] = sq
        sq = padded
        d = sq.shape[1]
    lanes = np.zeros((n, 8), np.float32)
    for i in range(d // 8):
        lanes += sq[:, 8 * i:8 * i + 8]
    s = lanes[:, 0].copy()
    for j in range(1, 8):
        s += lanes[:, j]
    return np.sqrt(s)


def encode(x: np.ndarray, R: np.ndarray, boundaries: np.ndarray, bits: int,
           return_margin: bool = False):
    """quantizer.py:122-166 + 203-207.

    x: [..., D] float16/float32.  Returns (packed u8 [..., pd], norms f32 [...]).
    The rotation product is formed in float64 and rounded to float32; the
    reference's sgemm differs from that by a few 1e-8, which matters only for
    coordinates closer than ~1e-6 to a boundary.  With ``return_margin`` the
    per-coordinate distance to the nearest boundary is returned as well so a
    caller can exempt those coordinates.
    """
    x = np.asarray(x)
    lead = x.shape[:-1]
    D = x.shape[-1]
    xf = np.ascontiguousarray(x.reshape(-1, D), dtype=np.float32)
    norms = l2norm_f32(xf)
    u = xf / (norms[:, None] + np.float32(1e-10))
    y64 = u.astype(np.float64) @ R.astype(np.float64).T
    y = y64.astype(np.float32)
    # searchsorted(left): number of boundaries strictly below y.
    idx = np.searchsorted(boundaries.astype(np.float32), y, side="left")
    idx = np.clip(idx, 0, (1 << bits) - 1)
    packed = pack(idx, bits).reshape(*lead, packed_size(D, bits))
    norms = norms.reshape(lead)
    if return_margin:
        margin = np.abs(y64[..., None] - boundaries.astype(np.float64)).min(-1)
        return packed, norms, margin.reshape(*lead, D)
    return packed, norms


def decode_f32(packed, norms, R, centroids, bits):
    """quantizer.py:168-197 up to (not including) the final dtype cast."""
    packed = np.asarray(packed)
    lead = packed.shape[:-1]
    D = R.shape[0]
    idx = unpack(packed.reshape(-1, packed.shape[-1]), D, bits)
    yhat = centroids.astype(np.float32)[idx]
    xhat = (yhat.astype(np.float64) @ R.astype(np.float64)).astype(np.float32)
    xhat = xhat * np.asarray(norms, np.float32).reshape(-1, 1)
    return xhat.reshape(*lead, D)


def decode(packed, norms, R, centroids, bits, dtype=np.float16):
    return decode_f32(packed, norms, R, centroids, bits).astype(dtype)


def paged_kv_update(x, slot_mapping, out_packed, out_norms, R, boundaries,
                    bits, block_size, max_blocks=0):
    """fused_kv_update.py:220-293 (4-bit) and vllm/hooks.py:487-497 (3/2-bit).

    Tokens whose slot is negative, or whose block index is >= max_blocks, are
    skipped.  Writes in place.
    """
    if max_blocks == 0:
        max_blocks = out_packed.shape[0]
    slot = np.asarray(slot_mapping).astype(np.int64)
    keep = slot >= 0
    blk = np.where(keep, slot // block_size, 0)
    keep &= blk < max_blocks
    if not keep.any():
        return
    packed, norms = encode(np.asarray(x)[keep], R, boundaries, bits)
    out_packed[blk[keep], (slot % block_size)[keep]] = packed
    out_norms[blk[keep], (slot % block_size)[keep]] = norms


def _gather_ctx(arr, block_table_row, ctx, block_size):
    nb = (ctx + block_size - 1) // block_size
    blocks = np.asarray(block_table_row[:nb]).astype(np.int64)
    g = arr[blocks]                         # [nb, bs, H, ...]
    return g.reshape(nb * block_size, *arr.shape[2:])[:ctx]


def paged_attention_rotated(query, k_packed, k_norms, v_packed, v_norms,
                            block_tables, context_lens, R, centroids, bits,
                            scale, block_size=16, out_dtype=None):
    """fused_attention.py:91-185 computed in float64 (no fp16 round trip).

    score_t = n^K_t * (R q . c[idxK_t]) * scale ; softmax over t ;
    out = R^T ( sum_t w_t n^V_t c[idxV_t] ).  ctx == 0 gives zeros.
    Returns float64 unless out_dtype is given.
    """
    q = np.asarray(query)
    S, QH, D = q.shape
    H = k_packed.shape[2]
    gqa = QH // H
    R64 = R.astype(np.float64)
    c64 = centroids.astype(np.float64)
    out = np.zeros((S, QH, D), np.float64)
    for s in range(S):
        ctx = int(context_lens[s])
        if ctx == 0:
            continue
        kc = c64[unpack(_gather_ctx(k_packed, block_tables[s], ctx, block_size), D, bits)]
        vc = c64[unpack(_gather_ctx(v_packed, block_tables[s], ctx, block_size), D, bits)]
        kn = _gather_ctx(k_norms, block_tables[s], ctx, block_size).astype(np.float64)
        vn = _gather_ctx(v_norms, block_tables[s], ctx, block_size).astype(np.float64)
        qrot = q[s].astype(np.float32).astype(np.float64) @ R64.T     # [QH, D]
        for qh in range(QH):
            h = qh // gqa
            sc = (kc[:, h] @ qrot[qh]) * kn[:, h] * scale
            w = np.exp(sc - sc.max())
            w /= w.sum()
            acc = (w * vn[:, h]) @ vc[:, h]
            out[s, qh] = R64.T @ acc
    return out if out_dtype is None else out.astype(out_dtype)


def paged_attention_decode_sdpa(query, k_packed, k_norms, v_packed, v_norms,
                                block_tables, context_lens, R, centroids, bits,
                                scale, block_size=16):
    """Decode the gathered blocks to fp16, then dense attention per sequence.

    This is the comparison the decode-attention benchmark configuration names
    ("fp16 SDPA on reference-decoded K/V") and what vllm/hooks.py:303-345 does
    for the hybrid codec.  K/V are rounded to fp16 exactly as
    TurboQuant.decode does; the attention itself accumulates in float32.
    Returns float16 [S, QH, D].
    """
    q = np.asarray(query)
    S, QH, D = q.shape
    H = k_packed.shape[2]
    gqa = QH // H
    out = np.zeros((S, QH, D), np.float16)
    for s in range(S):
        ctx = int(context_lens[s])
        if ctx == 0:
            continue
        kp = _gather_ctx(k_packed, block_tables[s], ctx, block_size)
        vp = _gather_ctx(v_packed, block_tables[s], ctx, block_size)
        kn = _gather_ctx(k_norms, block_tables[s], ctx, block_size)
        vn = _gather_ctx(v_norms, block_tables[s], ctx, block_size)
        K = decode(kp, kn, R, centroids, bits).astype(np.float32)   # [ctx,H,D]
        V = decode(vp, vn, R, centroids, bits).astype(np.float32)
        qf = q[s].astype(np.float16).astype(np.float32).reshape(H, gqa, D)
        sc = np.einsum("hgd,thd->hgt", qf, K, optimize=True) * np.float32(scale)
        sc -= sc.max(-1, keepdims=True)
        w = np.exp(sc)
        w /= w.sum(-1, keepdims=True)
        o = np.einsum("hgt,thd->hgd", w, V, optimize=True)
        out[s] = o.reshape(QH, D).astype(np.float16)
    return out
