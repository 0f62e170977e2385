"""The serving ops (tq::decode_step, tq::hybrid_decode_step) and the backend impl on a GPU."""
import math
import types

import numpy as np
import pytest
import torch

from conftest import load_golden
from helpers import make_paged_cache
from oracle import tq as otq
from oracle import hybrid as ohy

pytestmark = pytest.mark.gpu


def _setup_decode(bits, H, QH, ctx, seed):
    """A packed cache holding ctx-1 tokens per sequence; the op appends token ctx-1."""
    t = load_golden(f"tq_d128_b{bits}.npz")
    d = make_paged_cache(seed, ctx, H, 128, bits, t["rotation"], t["boundaries"])
    pd = 128 * bits // 8
    nb = d["k_packed"].shape[0]
    kv = torch.zeros(nb, 2, 16, H, pd + 4, dtype=torch.uint8, device="cuda")
    kv[:, 0, :, :, :pd] = torch.from_numpy(d["k_packed"]).cuda()
    kv[:, 1, :, :, :pd] = torch.from_numpy(d["v_packed"]).cuda()
    kn = torch.from_numpy(d["k_norms"]).cuda().unsqueeze(0).repeat(2, 1, 1, 1).contiguous()
    vn = torch.from_numpy(d["v_norms"]).cuda().unsqueeze(0).repeat(2, 1, 1, 1).contiguous()
    g = torch.Generator().manual_seed(seed)
    S = len(ctx)
    q = torch.randn(S + 2, QH, 128, generator=g).half()          # two padding rows beyond num_actual
    key = torch.randn(S, H, 128, generator=g).half()
    val = torch.randn(S, H, 128, generator=g).half()
    slots = torch.tensor([int(d["block_tables"][s, (c - 1) // 16]) * 16 + (c - 1) % 16 for s, c in enumerate(ctx)])
    return t, d, kv, kn, vn, q, key, val, slots


@pytest.mark.parametrize("bits", (4, 3, 2))
def test_decode_step_op(bits):
    from aitherkvcache_b200.vllm import ops
    H, QH, ctx = 8, 32, [300, 17, 64]
    t, d, kv, kn, vn, q, key, val, slots = _setup_decode(bits, H, QH, ctx, 31 + bits)
    tq = ops.init_quantizer(128, bits=bits)
    tq.rotation = torch.from_numpy(t["rotation"]).cuda()
    assert ops.register_custom_ops()
    S = len(ctx)
    out = torch.zeros(S + 2, QH, 128, dtype=torch.float16, device="cuda")
    layer = 1
    res = torch.ops.tq.decode_step(q.cuda(), key.cuda(), val.cuda(), kv, out, kn, vn, slots.cuda(),
                                   torch.from_numpy(d["block_tables"]).cuda(),
                                   torch.tensor(ctx, dtype=torch.int32, device="cuda"),
                                   layer, QH, H, 128, 1.0 / math.sqrt(128), S)
    assert res.data_ptr() != out.data_ptr() and torch.equal(res, out)
    assert (out[S:] == 0).all()
    # oracle: write the new token into a copy of the cache, then attend
    pd = 128 * bits // 8
    kp, vp = d["k_packed"].copy(), d["v_packed"].copy()
    knr, vnr = d["k_norms"].copy(), d["v_norms"].copy()
    otq.paged_kv_update(key.numpy(), slots.numpy(), kp, knr, t["rotation"], t["boundaries"], bits, 16)
    otq.paged_kv_update(val.numpy(), slots.numpy(), vp, vnr, t["rotation"], t["boundaries"], bits, 16)
    assert np.array_equal(kn[layer].cpu().numpy().view(np.uint32), knr.view(np.uint32))
    assert (kv[:, 0, :, :, :pd].cpu().numpy() != kp).mean() < 1e-4
    assert np.array_equal(kn[0].cpu().numpy(), d["k_norms"]), "other layers' norms untouched"
    ref = otq.paged_attention_rotated(q[:S].numpy(), kp, knr, vp, vnr, d["block_tables"], np.asarray(ctx),
                                      t["rotation"], t["centroids"], bits, 1.0 / math.sqrt(128))
    assert np.abs(out[:S].float().cpu().numpy() - ref).max() < 2e-3


def test_decode_step_single_call_matches_stepwise_path():
    """The one-call entry point and the step-by-step path (taken here through an int32 slot mapping)
    write the same cache bytes and return the same output; the cached argument block survives a
    second step with different inputs."""
    from aitherkvcache_b200.vllm import ops
    H, QH, ctx = 8, 32, [300, 17, 64]
    outs, caches = [], []
    for slot_dtype in (torch.int64, torch.int32):
        t, d, kv, kn, vn, q, key, val, slots = _setup_decode(4, H, QH, ctx, 77)
        tq = ops.init_quantizer(128, bits=4)
        tq.rotation = torch.from_numpy(t["rotation"]).cuda()
        assert ops.register_custom_ops()
        S = len(ctx)
        out = torch.zeros(S + 2, QH, 128, dtype=torch.float16, device="cuda")
        bt = torch.from_numpy(d["block_tables"]).cuda()
        sl = torch.tensor(ctx, dtype=torch.int32, device="cuda")
        res = []
        for step in range(2):
            g = torch.Generator().manual_seed(500 + step)
            qq = torch.randn(S + 2, QH, 128, generator=g).half().cuda()
            kk = torch.randn(S, H, 128, generator=g).half().cuda()
            vv = torch.randn(S, H, 128, generator=g).half().cuda()
            res.append(torch.ops.tq.decode_step(qq, kk, vv, kv, out, kn, vn, slots.to(slot_dtype).cuda(), bt, sl,
                                                0, QH, H, 128, 1.0 / math.sqrt(128), S).clone())
        outs.append(res)
        caches.append((kv.clone(), kn.clone(), vn.clone()))
    for a, b in zip(outs[0], outs[1]):
        assert torch.equal(a, b)
    for a, b in zip(caches[0], caches[1]):
        assert torch.equal(a, b)
    assert not torch.equal(outs[0][0], outs[0][1])


def test_hybrid_decode_step_op():
    from aitherkvcache_b200.vllm import ops
    g = load_golden("hybrid_tq35.npz")
    htq = ops.init_hybrid_quantizer(128, "tq35")
    t = ohy.Tables(128, "tq35", g["had0"], g["had1"], g["qjl0"], g["qjl1"],
                   codebooks=[(g["cent0"], g["bnd0"]), (g["cent1"], g["bnd1"])])
    H, QH, ctx, bs = 8, 32, [200, 33], 16
    gen = torch.Generator().manual_seed(8)
    nblk = [(c + bs - 1) // bs for c in ctx]
    total = sum(nblk)
    bt = torch.zeros(2, max(nblk), dtype=torch.int32)
    perm = torch.randperm(total, generator=gen)
    p = 0
    for s, n in enumerate(nblk):
        bt[s, :n] = perm[p:p + n].to(torch.int32)
        p += n
    k = torch.randn(total, bs, H, 128, generator=gen).half()
    v = torch.randn(total, bs, H, 128, generator=gen).half()
    kv = torch.zeros(total, 2, bs, H, 64, dtype=torch.uint8, device="cuda")
    kv[:, 0] = htq.encode(k.cuda())
    kv[:, 1] = htq.encode(v.cuda())
    q = torch.randn(2, QH, 128, generator=gen).half()
    key = torch.randn(2, H, 128, generator=gen).half()
    val = torch.randn(2, H, 128, generator=gen).half()
    slots = torch.tensor([int(bt[s, (c - 1) // bs]) * bs + (c - 1) % bs for s, c in enumerate(ctx)])
    ops.register_custom_ops()
    out = torch.zeros(2, QH, 128, dtype=torch.float16, device="cuda")
    res = torch.ops.tq.hybrid_decode_step(q.cuda(), key.cuda(), val.cuda(), kv, out, slots.cuda(), bt.cuda(),
                                          torch.tensor(ctx, dtype=torch.int32, device="cuda"), 0, QH, H, 128,
                                          1.0 / math.sqrt(128), 2)
    assert torch.equal(res, out)
    kc, vc = ohy.encode(k.numpy(), t), ohy.encode(v.numpy(), t)
    for s, c in enumerate(ctx):
        kc[int(bt[s, (c - 1) // bs]), (c - 1) % bs] = ohy.encode(key[s].numpy(), t)
        vc[int(bt[s, (c - 1) // bs]), (c - 1) % bs] = ohy.encode(val[s].numpy(), t)
    assert np.array_equal(kv[:, 0].cpu().numpy(), kc)
    ref = ohy.paged_attention_decode_sdpa(q.numpy(), kc, vc, bt.numpy(), np.asarray(ctx), t, 1.0 / math.sqrt(128), bs)
    assert np.abs(out.float().cpu().numpy() - ref).max() < 2e-3


def test_backend_impl_cache_update_decode_and_prefill():
    """TurboQuantImplBase (the vLLM-independent part of the CUSTOM backend impl)."""
    from aitherkvcache_b200.vllm.backend import TurboQuantImplBase, _LayerState
    H, QH, bs, bits = 8, 32, 16, 4
    impl = TurboQuantImplBase()
    impl._tq_setup(QH, 128, 1.0 / math.sqrt(128), H, "tq-t4nc")
    assert impl.tq_bits == 4 and impl.packed_dim == 64
    layer = types.SimpleNamespace(layer_name="model.layers.0.attn")
    nb = 12
    kv = torch.zeros(nb, 2, bs, H, 68, dtype=torch.uint8, device="cuda")
    gen = torch.Generator().manual_seed(4)
    lens = [40, 100]
    bt = torch.tensor([[3, 7, 1, 0, 0, 0, 0], [2, 4, 5, 6, 8, 9, 10]], dtype=torch.int32)
    # prefill both sequences in one chunk
    T = sum(lens)
    key = torch.randn(T, H, 128, generator=gen).half().cuda()
    val = torch.randn(T, H, 128, generator=gen).half().cuda()
    qry = torch.randn(T, QH * 128, generator=gen).half().cuda()
    slots = torch.cat([(bt[s, :(n + bs - 1) // bs].long()[:, None] * bs + torch.arange(bs)[None]).reshape(-1)[:n]
                       for s, n in enumerate(lens)])
    impl.do_kv_cache_update(layer, key, val, kv, slots.cuda())
    md = types.SimpleNamespace(num_actual_tokens=T, max_query_len=max(lens), block_table=bt.cuda(),
                               seq_lens=torch.tensor(lens, dtype=torch.int32, device="cuda"),
                               query_start_loc=torch.tensor([0, lens[0], T], dtype=torch.int32, device="cuda"))
    out = torch.zeros(T, QH * 128, dtype=torch.float16, device="cuda")
    impl.forward(layer, qry, key, val, kv, md, output=out)
    # decode step for the last token of each sequence must agree with its prefill row
    last = [lens[0] - 1, T - 1]
    md1 = types.SimpleNamespace(num_actual_tokens=2, max_query_len=1, block_table=bt.cuda(),
                                seq_lens=torch.tensor(lens, dtype=torch.int32, device="cuda"))
    out1 = torch.zeros(2, QH * 128, dtype=torch.float16, device="cuda")
    impl.forward(layer, qry[last], None, None, kv, md1, output=out1)
    assert (out1.float() - out[last].float()).abs().max().item() < 2e-3
    tq = next(iter(_LayerState.quantizers.values()))
    kn = _LayerState.k_norms[layer.layer_name]
    op, on = otq.encode(key.cpu().numpy(), tq.rotation.cpu().numpy(), tq.boundaries_inner.cpu().numpy(), bits)
    got_n = kn.reshape(-1, H)[slots.cuda()].cpu().numpy()
    assert np.array_equal(got_n.view(np.uint32), on.view(np.uint32))
