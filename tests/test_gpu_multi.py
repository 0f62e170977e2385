"""Two-GPU split-K over NCCL (skipped on a single-GPU box): every rank attends over its own key
range, partials are all-gathered and merged; the result must equal the single-GPU call."""
import math
import os
import socket

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, results):
    import torch.distributed as dist
    from aitherkvcache_b200 import TQPagedAttention, TurboQuant
    from aitherkvcache_b200.parallel import shard_range, tq_paged_attention_sharded, tri_decode_step_sharded
    from aitherkvcache_b200.triattention import SpectralEncoding, TriAttention, TriAttentionConfig
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        dev = f"cuda:{rank}"
        # --- TriAttention, key range split ---
        B, S, H, QH = 2, 3000, 8, 32
        tri = TriAttention(TriAttentionConfig(num_kv_heads=H, num_query_heads=QH), device=dev)
        g = torch.Generator().manual_seed(1)
        keys = torch.randn(B, S, H, 128, generator=g).half().to(dev)
        vals = torch.randn(B, S, H, 128, generator=g).half().to(dev)
        q = torch.randn(B, QH, 128, generator=g).half().to(dev)
        k_enc, v_enc = tri.encode_kv(keys, vals)
        full = tri.decode_step(q, k_enc, v_enc)
        lo, hi = shard_range(S, rank, world, 32)
        sl = lambda e: SpectralEncoding(*[t[:, lo:hi].contiguous() for t in e])   # noqa: E731
        out = tri_decode_step_sharded(tri, q, sl(k_enc), sl(v_enc), lo, S)
        err_tri = float((out - full).abs().max())
        # --- TurboQuant paged attention, each rank holds a block range of every sequence ---
        tq = TurboQuant(head_dim=128, bits=4, device=dev)
        ctx = [640, 50]
        nblk = [(c + 15) // 16 for c in ctx]
        total = sum(nblk)
        k = torch.randn(total * 16, H, 128, generator=g).half().to(dev)
        v = torch.randn(total * 16, H, 128, generator=g).half().to(dev)
        kp, kn = tq.encode(k.reshape(total, 16, H, 128))
        vp, vn = tq.encode(v.reshape(total, 16, H, 128))
        bt = torch.zeros(2, max(nblk), dtype=torch.int32)
        bt[0, :nblk[0]] = torch.arange(nblk[0])
        bt[1, :nblk[1]] = torch.arange(nblk[0], total)
        q2 = torch.randn(2, QH, 128, generator=g).half().to(dev)
        attn = TQPagedAttention(tq, QH)
        full2 = attn.forward(q2, kp, kn, vp, vn, bt.to(dev), torch.tensor(ctx, dtype=torch.int32, device=dev))
        bt_l = torch.zeros_like(bt)
        cl_l = []
        for s, c in enumerate(ctx):
            a, b = shard_range(c, rank, world, 16)
            nb = (b - a + 15) // 16
            bt_l[s, :nb] = bt[s, a // 16:a // 16 + nb]
            cl_l.append(b - a)
        out2 = tq_paged_attention_sharded(attn, q2, kp, kn, vp, vn, bt_l.to(dev),
                                          torch.tensor(cl_l, dtype=torch.int32, device=dev))
        # --- the same merges over peer memory instead of NCCL: three steps (both buffer halves), then the
        #     step captured in a CUDA graph and replayed; equal to the NCCL route bit for bit ---
        from aitherkvcache_b200 import _lib
        from aitherkvcache_b200.parallel import PeerExchange, p2p_merge_partials
        ex = PeerExchange(2, QH, 128, dev)
        raw = torch.empty(2 * QH, 130, dtype=torch.float32, device=dev)
        p2p_out = torch.empty_like(full2)
        err_p2p = 0.0
        for step in range(3):
            attn.forward(q2 * (1.0 + 0.25 * step), kp, kn, vp, vn, bt_l.to(dev),
                         torch.tensor(cl_l, dtype=torch.int32, device=dev), raw_out=raw)
            p2p_merge_partials(ex, raw, rotation=attn.rotation, out=p2p_out)
            want = tq_paged_attention_sharded(attn, q2 * (1.0 + 0.25 * step), kp, kn, vp, vn, bt_l.to(dev),
                                              torch.tensor(cl_l, dtype=torch.int32, device=dev))
            err_p2p = max(err_p2p, float((p2p_out.float() - want.float()).abs().max()))
        bt_dev, cl_dev = bt_l.to(dev), torch.tensor(cl_l, dtype=torch.int32, device=dev)
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            attn.forward(q2, kp, kn, vp, vn, bt_dev, cl_dev, raw_out=raw)
            p2p_merge_partials(ex, raw, rotation=attn.rotation, out=p2p_out)
        torch.cuda.current_stream().wait_stream(side)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            attn.forward(q2, kp, kn, vp, vn, bt_dev, cl_dev, raw_out=raw)
            p2p_merge_partials(ex, raw, rotation=attn.rotation, out=p2p_out)
        for _ in range(3):
            graph.replay()
        torch.cuda.synchronize()
        err_p2p = max(err_p2p, float((p2p_out.float() - out2.float()).abs().max()))
        status = _lib.device_status()
        results[rank] = (err_tri, float((out2.float() - full2.float()).abs().max()), err_p2p, status["p2p"])
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_gpu_split_k_matches_single_gpu():
    import torch.multiprocessing as mp
    results = mp.Manager().dict()
    mp.spawn(_worker, args=(2, _free_port(), results), nprocs=2, join=True)
    assert len(results) == 2
    for err_tri, err_tq, err_p2p, p2p_status in results.values():
        assert err_tri < 1e-4 and err_tq < 2e-3
        assert err_p2p == 0.0 and p2p_status == 0
