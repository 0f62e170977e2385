"""Builders shared by the GPU parity tests (inputs on CPU via numpy/torch, seeded)."""
import math

import numpy as np
import torch

from oracle import tq as otq


def ordered_fp16(h):
    i = np.asarray(h).view(np.int16).astype(np.int32)
    return np.where(i < 0, -(i & 0x7FFF), i)


def make_paged_cache(seed, ctx_lens, num_kv_heads, head_dim, bits, R, boundaries, block_size=16,
                     extra_blocks=2, k_scale=1.0):
    """Random K/V (fp16 N(0,1)), encoded by the oracle into randomly placed blocks.

    Returns dict of numpy arrays: k_packed, k_norms, v_packed, v_norms, block_tables(int32),
    context_lens(int64), plus the raw fp16 k, v per physical block."""
    g = torch.Generator().manual_seed(seed)
    nblk = [(int(c) + block_size - 1) // block_size for c in ctx_lens]
    total = sum(nblk) + extra_blocks
    perm = torch.randperm(total, generator=g).numpy()
    maxb = max(max(nblk), 1)
    bt = np.zeros((len(ctx_lens), maxb), np.int32)
    p = 0
    for s, n in enumerate(nblk):
        bt[s, :n] = perm[p:p + n]
        p += n
    k = (torch.randn(total, block_size, num_kv_heads, head_dim, generator=g) * k_scale).half().numpy()
    v = torch.randn(total, block_size, num_kv_heads, head_dim, generator=g).half().numpy()
    kp, kn = otq.encode(k, R, boundaries, bits)
    vp, vn = otq.encode(v, R, boundaries, bits)
    return dict(k_packed=kp, k_norms=kn, v_packed=vp, v_norms=vn, block_tables=bt,
                context_lens=np.asarray(ctx_lens, np.int64), k=k, v=v)


def to_cuda(d, keys):
    return {k: torch.from_numpy(np.ascontiguousarray(d[k])).cuda() for k in keys}
