"""numpy restatement of TriAttention's spectral codec and decode step.

TEST INFRASTRUCTURE ONLY (see oracle/__init__.py).

Reference:
  aither_kvcache/triattention/spectral.py:34-51    RoPE frequencies
  aither_kvcache/triattention/encoder.py:73-149    top-F pair selection, 4-bit / 8-bit / fp16 coefficients
  aither_kvcache/triattention/scorer.py:84-208     trig-series scores (pre-RoPE) or sparse dot product (post-RoPE)
  aither_kvcache/triattention/attention.py:186-280 softmax + scattered value sum
"""
from __future__ import annotations

import math
import numpy as np


def rope_frequencies(head_dim, base=1_000_000.0):
    """spectral.py:34-51: float32 pow of a float32 exponent.  torch evaluates
    ``base ** t`` with powf; numpy's float32 power agrees to 1 ulp, and the
    fixtures carry the reference's own table for exact work."""
    i = np.arange(head_dim // 2, dtype=np.float32)
    e = (np.float32(-2.0) * i) / np.float32(head_dim)
    return np.power(np.float32(base), e).astype(np.float32)


def encode(x, num_freqs=12, coeff_bits=4):
    """encoder.py:73-149.

    Returns (indices u8[...,F] ascending, packed, scales f16[...]); packed is u8[...,F] for
    coeff_bits 4, u8[...,2F] for 8 and f16[...,F,2] (scales all 1) for 16.
    Ties between equal pair energies at rank F are broken towards the lower
    pair id here; torch.topk does not promise an order, so callers compare
    index sets only where the F-th and (F+1)-th energies differ.
    """
    x = np.asarray(x)
    lead, D = x.shape[:-1], x.shape[-1]
    P = D // 2
    pairs = x.reshape(-1, P, 2).astype(np.float32)
    sq = pairs * pairs
    energy = sq[..., 0] + sq[..., 1]
    order = np.argsort(-energy, axis=-1, kind="stable")[:, :num_freqs]
    top = np.sort(order, axis=-1)
    tp = np.take_along_axis(pairs, top[..., None], axis=1)          # [N,F,2]
    idx = top.astype(np.uint8).reshape(*lead, num_freqs)
    if coeff_bits == 16:
        return idx, tp.astype(np.float16).reshape(*lead, num_freqs, 2), np.ones(lead, np.float16)
    scales = np.maximum(np.abs(tp).reshape(len(tp), -1).max(-1), np.float32(1e-8))
    normed = tp / scales[:, None, None]
    half, top_code = (np.float32(7.5), 15) if coeff_bits == 4 else (np.float32(127.5), 255)
    q = np.clip(np.rint((normed + np.float32(1.0)) * half), 0, top_code).astype(np.uint8)
    packed = ((q[..., 0] << 4) | q[..., 1]).reshape(*lead, num_freqs) if coeff_bits == 4 \
        else q.reshape(*lead, 2 * num_freqs)
    return idx, packed, scales.astype(np.float16).reshape(lead)


def rank_gap(x, num_freqs=12):
    """Difference between the F-th and (F+1)-th largest pair energy per vector
    (0 means the top-F set is ambiguous)."""
    x = np.asarray(x)
    pairs = x.reshape(-1, x.shape[-1] // 2, 2).astype(np.float32)
    sq = pairs * pairs
    e = np.sort(sq[..., 0] + sq[..., 1], axis=-1)[:, ::-1]
    return (e[:, num_freqs - 1] - e[:, num_freqs]).reshape(x.shape[:-1])


def unpack_coeffs(packed, scales, coeff_bits=4):
    """scorer.py:84-113."""
    p = np.asarray(packed)
    if coeff_bits == 16:
        return p[..., 0].astype(np.float32), p[..., 1].astype(np.float32)
    s = np.asarray(scales).astype(np.float32)[..., None]
    if coeff_bits == 8:
        raw = p.astype(np.float32).reshape(*p.shape[:-1], p.shape[-1] // 2, 2)
        return ((raw[..., 0] / np.float32(127.5) - np.float32(1.0)) * s,
                (raw[..., 1] / np.float32(127.5) - np.float32(1.0)) * s)
    k0 = ((p >> 4).astype(np.float32) / np.float32(7.5) - np.float32(1.0)) * s
    k1 = ((p & 15).astype(np.float32) / np.float32(7.5) - np.float32(1.0)) * s
    return k0, k1


def scores(query, k_idx, k_packed, k_scales, theta, query_pos=None, key_positions=None, coeff_bits=4, pre_rope=True):
    """scorer.py:115-208.  query [B,QH,D]; k_* [B,S,KVH,F] / [B,S,KVH].  Post-RoPE is the
    same sum with every phase zero (scorer.py:201-203).

    The phase is the float32 product float32(pos_k - pos_q) * theta, exactly as
    the reference forms it; everything after that is float64 here.
    Returns float64 [B,QH,S].
    """
    q = np.asarray(query).astype(np.float32)
    B, QH, D = q.shape
    S, KVH, F = k_idx.shape[1:]
    gqa = QH // KVH
    if key_positions is None:
        key_positions = np.broadcast_to(np.arange(S), (B, S))
    if query_pos is None:
        query_pos = np.full((B,), S)
    k0, k1 = unpack_coeffs(k_packed, k_scales, coeff_bits)
    delta = (np.asarray(key_positions).astype(np.float32)
             - np.asarray(query_pos).astype(np.float32)[:, None])            # [B,S]
    if not pre_rope:
        delta = np.zeros_like(delta)
    idx = np.asarray(k_idx).astype(np.int64)
    phase = (delta[:, :, None, None] * theta.astype(np.float32)[idx]).astype(np.float32)
    cos, sin = np.cos(phase.astype(np.float64)), np.sin(phase.astype(np.float64))
    k0r = k0 * cos - k1 * sin        # key pair rotated by the relative phase
    k1r = k1 * cos + k0 * sin
    out = np.zeros((B, QH, S), np.float64)
    qe, qo = q[..., 0::2].astype(np.float64), q[..., 1::2].astype(np.float64)
    for b in range(B):
        for qh in range(QH):
            h = qh // gqa
            ge = qe[b, qh][idx[b, :, h]]          # [S,F]
            go = qo[b, qh][idx[b, :, h]]
            out[b, qh] = (ge * k0r[b, :, h] + go * k1r[b, :, h]).sum(-1)
    return out * (1.0 / math.sqrt(D))


def decode_step(query, k_enc, v_enc, theta, query_pos=None, key_positions=None, coeff_bits=4, pre_rope=True):
    """attention.py:186-280 -> float32 [B,QH,D]."""
    sc = scores(query, *k_enc, theta, query_pos, key_positions, coeff_bits, pre_rope)
    B, QH, S = sc.shape
    v_idx, v_packed, v_scales = v_enc
    KVH, F = v_idx.shape[2:]
    gqa = QH // KVH
    D = np.asarray(query).shape[-1]
    w = np.exp(sc - sc.max(-1, keepdims=True))
    w /= w.sum(-1, keepdims=True)
    v0, v1 = unpack_coeffs(v_packed, v_scales, coeff_bits)
    out = np.zeros((B, QH, D), np.float64)
    for b in range(B):
        for qh in range(QH):
            h = qh // gqa
            ii = np.asarray(v_idx[b, :, h]).astype(np.int64).reshape(-1)
            # scatter-add of the weighted coefficients into their pair slots (bincount = add.at, faster)
            out[b, qh, 0::2] = np.bincount(ii, (w[b, qh][:, None] * v0[b, :, h]).reshape(-1), minlength=D // 2)
            out[b, qh, 1::2] = np.bincount(ii, (w[b, qh][:, None] * v1[b, :, h]).reshape(-1), minlength=D // 2)
    return out.astype(np.float32)
