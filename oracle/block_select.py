"""TEST INFRASTRUCTURE - not part of the product path.

Numpy restatement of the reference's block selection (aither_kvcache/block_selector.py):
  * ``representatives``  BlockRepresentativeCache.update + finalize, :65-113
  * ``score_blocks``     :128-172
  * ``select_blocks``    :175-228

Pinned against the reference in this container by ``tests/golden/make_golden.py`` (fixture
``block_select.npz``: the reference's own scores, filtered tables and context lengths for a seeded
case); ``tests/test_oracle_golden.py`` checks this file against that fixture.
"""
from __future__ import annotations

import numpy as np


def representatives(block_idx, codes, k_norms, centroids, max_blocks):
    """codes [N, H, D] int (unpacked), k_norms [N, H] -> rep [max_blocks, H, D] float64 (natural dim order)."""
    N, H, D = codes.shape
    acc = np.zeros((max_blocks, H, D), np.float64)
    cnt = np.zeros((max_blocks, H), np.int64)
    w = centroids.astype(np.float64)[codes] * np.asarray(k_norms, np.float64)[..., None]
    np.add.at(acc, np.asarray(block_idx), w)
    np.add.at(cnt, np.asarray(block_idx), 1)
    return acc / np.maximum(cnt, 1)[..., None]


def score_blocks(q_rot, rep, block_tables, context_lens, gqa_ratio, block_size):
    """q_rot [S, QH, D] rotated queries -> scores [S, max_bps] float64, -inf past the context."""
    S, QH, D = q_rot.shape
    H = QH // gqa_ratio
    qm = q_rot.astype(np.float64).reshape(S, H, gqa_ratio, D).mean(2)
    bt = np.clip(np.asarray(block_tables), 0, None)
    g = rep[bt]                                            # [S, B, H, D]
    sc = (qm[:, None] * g).sum((-1, -2))
    nb = (np.asarray(context_lens) + block_size - 1) // block_size
    sc[np.arange(bt.shape[1])[None, :] >= nb[:, None]] = -np.inf
    return sc


def select_blocks(scores, block_tables, context_lens, block_size, max_selected, num_sink_blocks=2,
                  num_recent_blocks=2, exact_tail=False):
    """Returns (filtered block tables [S, max_selected], filtered context lengths [S]).  Ties go to the
    lower logical index (torch.topk leaves them unspecified)."""
    scores = np.asarray(scores, np.float64)
    S, B = scores.shape
    ctx = np.asarray(context_lens).astype(np.int64)
    nb = (ctx + block_size - 1) // block_size
    idx = np.arange(B)[None, :]
    valid = idx < nb[:, None]
    mandatory = ((idx < num_sink_blocks) | (idx >= nb[:, None] - num_recent_blocks)) & valid
    sel = scores.copy()
    sel[mandatory] = np.inf
    sel[~valid] = -np.inf
    k = min(max_selected, B)
    out_bt = np.zeros((S, max_selected), np.int64)
    out_cl = np.minimum(ctx, k * block_size)
    for s in range(S):
        order = np.lexsort((np.arange(B), -sel[s]))       # by descending score, then ascending index
        chosen = np.sort(order[:k])
        out_bt[s, :k] = np.asarray(block_tables)[s, chosen]
        if exact_tail and nb[s] > k and num_recent_blocks > 0:
            out_cl[s] = (k - 1) * block_size + (ctx[s] - (nb[s] - 1) * block_size)
    return out_bt, out_cl
