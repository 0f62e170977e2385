"""numpy restatement of the hybrid (tq35 / tq25) codec.

TEST INFRASTRUCTURE ONLY (see oracle/__init__.py).

Reference: aither_kvcache/hybrid_quantizer.py
  :52-123   mode table and byte layout
  :130-234  fast Walsh-Hadamard transform, signed + normalised
  :241-303  Lloyd iteration on the Beta((d-1)/2) grid
  :310-410  MSB-first multi-bit and sign packing
  :616-779  encode ; :785-933 decode

Every step of the reference encode is element-wise float32 (no BLAS), so this
restatement is expected to reproduce its bytes exactly.
"""
from __future__ import annotations

import math
import numpy as np

from .tq import l2norm_f32

MODES = {"tq35": (0.50, (4, 3)), "tq25": (0.25, (3, 2))}


def group_layout(dim, mse_bits):
    mse = math.ceil(dim * mse_bits / 8)
    qjl = math.ceil(dim / 8)
    return dict(dim=dim, mse_bits=mse_bits, mse=mse, qjl=qjl, total=mse + qjl + 4)


def layout(head_dim, mode):
    ratio, (b0, b1) = MODES[mode]
    g0 = round(head_dim * ratio)
    l0 = group_layout(g0, b0 - 1)
    l1 = group_layout(head_dim - g0, b1 - 1)
    return l0, l1, l0["total"] + l1["total"]


def beta_codebook(dim, bits):
    """hybrid_quantizer.py:241-303 in float64 numpy -> (centroids, boundaries) f32."""
    L = 1 << bits
    grid = np.linspace(-0.999, 0.999, 10000, dtype=np.float64)
    expo = (dim - 3) / 2.0
    base = 1.0 - grid * grid
    w = base ** expo if expo >= 0 else np.maximum(base, 1e-30) ** expo
    w = w / w.sum()
    c = np.linspace(grid[0], grid[-1], L, dtype=np.float64)
    for _ in range(200):
        b = (c[:-1] + c[1:]) / 2.0
        a = np.clip(np.searchsorted(b, grid, side="left"), 0, L - 1)
        new = c.copy()
        for k in range(L):
            m = a == k
            ws = w[m].sum()
            if ws > 1e-30:
                new[k] = (grid[m] * w[m]).sum() / ws
        done = np.abs(c - new).max() < 1e-10
        c = new
        if done:
            break
    b = (c[:-1] + c[1:]) / 2.0
    return c.astype(np.float32), b.astype(np.float32)


def _pow2_parts(n):
    parts = []
    while n > 0:
        p = 1 << (n.bit_length() - 1)
        parts.append(p)
        n -= p
    return parts


def fwht(x):
    """Un-normalised FWHT on the last axis, stages h = 1, 2, 4, ... in float32
    (hybrid_quantizer.py:130-193; non-power-of-two sizes are block diagonal)."""
    x = np.array(x, dtype=np.float32, copy=True)
    n = x.shape[-1]
    off = 0
    for p in _pow2_parts(n):
        blk = x[..., off:off + p]
        h = 1
        while h < p:
            v = blk.reshape(*blk.shape[:-1], -1, 2 * h)
            l = v[..., :h].copy()
            r = v[..., h:].copy()
            v[..., :h] = l + r
            v[..., h:] = l - r
            h *= 2
        off += p
    return x


def had(x, signs, inverse=False):
    """structured_hadamard(..., normalized=True) (:200-234)."""
    dim = x.shape[-1]
    y = fwht(x) * signs if inverse else fwht(x * signs)
    return (y / np.float32(math.sqrt(dim))).astype(np.float32)


def pack_bits(idx, bits):
    """pack_multibit (:310-353): MSB-first bit stream."""
    idx = np.asarray(idx).astype(np.uint8)
    lead, dim = idx.shape[:-1], idx.shape[-1]
    shifts = np.arange(bits - 1, -1, -1, dtype=np.uint8)
    stream = ((idx[..., None] >> shifts) & 1).reshape(*lead, dim * bits)
    return np.packbits(stream, axis=-1, bitorder="big")


def unpack_bits(packed, dim, bits):
    stream = np.unpackbits(np.asarray(packed, np.uint8), axis=-1, bitorder="big")
    stream = stream[..., :dim * bits].reshape(*packed.shape[:-1], dim, bits)
    w = (1 << np.arange(bits - 1, -1, -1)).astype(np.uint8)
    return (stream * w).sum(-1).astype(np.uint8)


def _fp16_bytes(v):
    return np.asarray(v, np.float32).astype(np.float16).view(np.uint8).reshape(*v.shape, 2)


def _bytes_fp16(b):
    return np.ascontiguousarray(b).view(np.float16).reshape(b.shape[:-1]).astype(np.float32)


class Tables:
    """Sign vectors and codebooks of one HybridTurboQuant instance.  The sign
    vectors come from torch's CPU generator (:514-523) and are therefore passed
    in; the codebooks are recomputed here."""

    def __init__(self, head_dim, mode, had0, had1, qjl0, qjl1, codebooks=None):
        self.head_dim, self.mode = head_dim, mode
        self.l0, self.l1, self.packed_dim = layout(head_dim, mode)
        self.signs = [(np.asarray(had0, np.float32), np.asarray(qjl0, np.float32)),
                      (np.asarray(had1, np.float32), np.asarray(qjl1, np.float32))]
        # The Lloyd iteration sums 10 000 float64 terms; its result depends on
        # the summation order at the 1e-17 level, which decides on which side of
        # an exact 0.0 the middle boundary lands.  Pass the instance's own
        # tables when bytes for all-zero inputs must match.
        self.cb = codebooks or [beta_codebook(self.l0["dim"], self.l0["mse_bits"]),
                                beta_codebook(self.l1["dim"], self.l1["mse_bits"])]
        self.cb = [(np.asarray(c, np.float32), np.asarray(b, np.float32)) for c, b in self.cb]
        self.qjl_scale = [math.sqrt(math.pi / 2.0) / self.l0["dim"],
                          math.sqrt(math.pi / 2.0) / self.l1["dim"]]


def _encode_group(xg, lay, had_s, qjl_s, cent, bnd):
    """_encode_single_group (:712-779)."""
    n = l2norm_f32(xg)
    u = xg / (n[:, None] + np.float32(1e-10))
    r = had(u, had_s)
    idx = np.clip(np.searchsorted(bnd, r, side="left"), 0, (1 << lay["mse_bits"]) - 1)
    uhat = had(cent[idx], had_s, inverse=True)
    res = (u - uhat).astype(np.float32)
    rho = l2norm_f32(res)
    p = had(res, qjl_s)
    return np.concatenate([pack_bits(idx, lay["mse_bits"]),
                           pack_bits((p >= 0).astype(np.uint8), 1),
                           _fp16_bytes(n), _fp16_bytes(rho)], axis=-1)


def encode(x, t: Tables, g0_idx=None, g1_idx=None):
    """HybridTurboQuant.encode with one shared dim split (:616-710)."""
    x = np.asarray(x)
    lead = x.shape[:-1]
    xf = np.ascontiguousarray(x.reshape(-1, t.head_dim), dtype=np.float32)
    if g0_idx is None:
        g0_idx = np.arange(t.l0["dim"])
        g1_idx = np.arange(t.l0["dim"], t.head_dim)
    parts = []
    for g, (lay, gi) in enumerate(((t.l0, g0_idx), (t.l1, g1_idx))):
        parts.append(_encode_group(np.ascontiguousarray(xf[:, gi]), lay,
                                   t.signs[g][0], t.signs[g][1], *t.cb[g]))
    return np.concatenate(parts, axis=-1).reshape(*lead, t.packed_dim)


def _decode_group(pg, lay, had_s, qjl_s, cent, qjl_scale):
    """_decode_single_group (:878-933)."""
    G = lay["dim"]
    a, b = lay["mse"], lay["mse"] + lay["qjl"]
    idx = unpack_bits(pg[:, :a], G, lay["mse_bits"])
    mse_hat = had(cent[idx], had_s, inverse=True)
    sg = 2.0 * unpack_bits(pg[:, a:b], G, 1).astype(np.float32) - 1.0
    qjl_hat = had((sg * np.float32(qjl_scale)).astype(np.float32), qjl_s, inverse=True)
    n = _bytes_fp16(pg[:, b:b + 2])
    rho = _bytes_fp16(pg[:, b + 2:b + 4])
    return ((mse_hat + qjl_hat * rho[:, None]) * n[:, None]).astype(np.float32)


def decode(packed, t: Tables, g0_idx=None, g1_idx=None):
    """HybridTurboQuant.decode (:785-876) -> float32 [..., head_dim]."""
    packed = np.asarray(packed, np.uint8)
    lead = packed.shape[:-1]
    pf = packed.reshape(-1, t.packed_dim)
    if g0_idx is None:
        g0_idx = np.arange(t.l0["dim"])
        g1_idx = np.arange(t.l0["dim"], t.head_dim)
    out = np.zeros((pf.shape[0], t.head_dim), np.float32)
    b0 = t.l0["total"]
    out[:, g0_idx] = _decode_group(pf[:, :b0], t.l0, *t.signs[0], t.cb[0][0], t.qjl_scale[0])
    out[:, g1_idx] = _decode_group(pf[:, b0:], t.l1, *t.signs[1], t.cb[1][0], t.qjl_scale[1])
    return out.reshape(*lead, t.head_dim)


def paged_attention_decode_sdpa(query, k_cache, v_cache, block_tables, context_lens,
                                t: Tables, scale, block_size=16, kv_dtype=np.float16):
    """Body of tq::hybrid_decode_step (vllm/hooks.py:297-345): decode every
    context token, round K/V to a 16-bit float, dense attention with GQA.
    The reference rounds to bf16; numpy has no bf16, fp16 is used here and the
    tolerance of the comparison covers both."""
    q = np.asarray(query)
    S, QH, D = q.shape
    H = k_cache.shape[2]
    gqa = QH // H
    out = np.zeros((S, QH, D), np.float32)
    for s in range(S):
        ctx = int(context_lens[s])
        if ctx == 0:
            continue
        nb = (ctx + block_size - 1) // block_size
        blocks = np.asarray(block_tables[s][:nb]).astype(np.int64)
        K = decode(k_cache[blocks].reshape(nb * block_size, H, -1)[:ctx], t).astype(kv_dtype).astype(np.float32)
        V = decode(v_cache[blocks].reshape(nb * block_size, H, -1)[:ctx], t).astype(kv_dtype).astype(np.float32)
        qf = q[s].astype(np.float32).reshape(H, gqa, D)
        sc = np.einsum("hgd,thd->hgt", qf, K, optimize=True) * np.float32(scale)
        sc -= sc.max(-1, keepdims=True)
        w = np.exp(sc)
        w /= w.sum(-1, keepdims=True)
        out[s] = np.einsum("hgt,thd->hgd", w, V, optimize=True).reshape(QH, D)
    return out
