"""Host logic of the multi-GPU split-K path on CPU ranks (gloo, world size 2 and 3):
range partition, the all-gather of partials and the log-sum-exp merge rule (restated in
torch here, as the checker).  One rank contributes an empty range (l = 0)."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from aitherkvcache_b200.parallel import all_gather_partials, shard_range


def merge_rule(parts):
    """[P, rows, D+2] (m in log2 units, l, acc) -> acc / l, the rule akv_lse_merge implements."""
    m, l, acc = parts[..., 0], parts[..., 1], parts[..., 2:]
    live = l > 0
    M = torch.where(live, m, torch.full_like(m, -float("inf"))).max(0).values
    w = torch.where(live, torch.exp2(m - M), torch.zeros_like(m))
    L = (l * w).sum(0)
    out = (acc * w[..., None]).sum(0)
    return torch.where(L[:, None] > 0, out / L[:, None], torch.zeros_like(out))


def partial_of(scores, values):
    """Un-normalised partial of softmax(scores) @ values for one slice ([rows, n], [n, D])."""
    rows = scores.shape[0]
    if scores.shape[1] == 0:
        return torch.cat([torch.full((rows, 1), -float("inf")), torch.zeros(rows, 1 + values.shape[1])], 1)
    s2 = scores * 1.4426950408889634
    m = s2.max(1, keepdim=True).values
    p = torch.exp2(s2 - m)
    return torch.cat([m, p.sum(1, keepdim=True), p @ values], 1)


def test_shard_range_covers_everything():
    for total, world, mult in [(131072, 8, 16), (100, 3, 16), (5, 4, 1), (0, 2, 16), (33, 2, 16)]:
        spans = [shard_range(total, r, world, mult) for r in range(world)]
        assert spans[0][0] == 0 and spans[-1][1] == total
        for (a, b), (c, d) in zip(spans, spans[1:]):
            assert b == c and a <= b
        assert all(lo % mult == 0 for lo, _ in spans)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, total, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        g = torch.Generator().manual_seed(0)
        rows, D = 6, 16
        scores = torch.randn(rows, total, generator=g) * 3
        values = torch.randn(total, D, generator=g)
        lo, hi = shard_range(total, rank, world, 16)
        raw = partial_of(scores[:, lo:hi], values[lo:hi]).float().contiguous()
        parts = all_gather_partials(raw)
        assert parts.shape == (world, rows, D + 2)
        out = merge_rule(parts)
        ref = torch.softmax(scores, 1) @ values
        results[rank] = float((out - ref).abs().max())
        if hi == lo:
            assert parts[rank, :, 1].abs().max() == 0
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,total", [(2, 100), (3, 33), (2, 10)])
def test_gloo_ranks_merge_to_the_full_softmax(world, total):
    results = mp.Manager().dict()
    mp.spawn(_worker, args=(world, _free_port(), total, results), nprocs=world, join=True)
    assert len(results) == world
    assert max(results.values()) < 1e-5
