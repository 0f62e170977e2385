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


@pytest.mark.parametrize("nseq", (3, 72))
def test_decode_step_single_call_matches_stepwise_path(nseq):
    """The one-call entry point and the step-by-step path (taken here through an int32 slot mapping)
    write the same cache bytes and return the same output; the cached argument block survives a
    second step with different inputs.  72 sequences x 32 heads = 2304 rows: both rotations run as
    tensor-core products while the new token's vectors keep their blocks of the plan launch."""
    from aitherkvcache_b200.vllm import ops
    H, QH = 8, 32
    ctx = [300, 17, 64] + [int(v) for v in np.random.default_rng(5).integers(1, 120, nseq - 3)]
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


@pytest.mark.parametrize("dense", (True, False))
@pytest.mark.parametrize("nseq", (3, 72))
def test_decode_step_returned_copy_is_written_by_the_merge(nseq, dense):
    """With num_actual == output rows the op's return value is a second destination of the merge kernel (no clone
    launch): it must be a dense tensor of its own holding exactly `output`, for a dense and a strided `output`, on
    the per-row merge (96 rows) and on the tensor-core rotation (2304 rows; dense: device copy, strided: the
    product once more), and equal to what the clone path (padding rows in `output`) returns."""
    from aitherkvcache_b200 import _lib
    from aitherkvcache_b200.vllm import ops
    H, QH = 8, 32
    ctx = [300, 17, 64] + [int(v) for v in np.random.default_rng(6).integers(1, 120, nseq - 3)]
    S = len(ctx)
    results = []
    for pad in (0, 2):
        t, d, kv, kn, vn, q, key, val, slots = _setup_decode(4, H, QH, ctx, 78)
        tq = ops.init_quantizer(128, bits=4)
        tq.rotation = torch.from_numpy(t["rotation"]).cuda()
        assert ops.register_custom_ops()
        big = torch.zeros(S + pad, QH + (0 if dense else 1), 128, dtype=torch.float16, device="cuda")
        out = big[:, :QH]
        n0 = _lib.lib().akv_launch_count()
        res = torch.ops.tq.decode_step(q.cuda()[:S + pad], key.cuda(), val.cuda(), kv, out, kn, vn, slots.cuda(),
                                       torch.from_numpy(d["block_tables"]).cuda(),
                                       torch.tensor(ctx, dtype=torch.int32, device="cuda"),
                                       0, QH, H, 128, 1.0 / math.sqrt(128), S)
        assert res.is_contiguous() and res.shape == out.shape and res.data_ptr() != out.data_ptr()
        assert torch.equal(res, out)
        results.append(res[:S].clone())
        if not dense:
            assert (big[:, QH] == 0).all(), "the strided output's gaps stay untouched"
    assert torch.equal(results[0], results[1])
    assert results[0].abs().max() > 0


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
    kn = impl._norms(layer.layer_name, kv)[0]          # 68-byte rows: the norms live behind the codes
    op, on = otq.encode(key.cpu().numpy(), tq.rotation.cpu().numpy(), tq.boundaries_inner.cpu().numpy(), bits)
    got_n = kn.reshape(-1, H)[slots.cuda()].cpu().numpy()
    assert np.array_equal(got_n.view(np.uint32), on.view(np.uint32))


def test_hybrid_decode_step_is_three_launches_and_skips_negative_slots():
    """tq::hybrid_decode_step writes the new records and attends in three kernel launches; a token with a
    negative slot is skipped even when another token of the batch writes block 0, offset 0."""
    from aitherkvcache_b200 import _lib
    from aitherkvcache_b200.vllm import ops
    g = load_golden("hybrid_tq35.npz")
    htq = ops.init_hybrid_quantizer(128, "tq35")
    t = ohy.Tables(128, "tq35", g["had0"], g["had1"], g["qjl0"], g["qjl1"],
                   codebooks=[(g["cent0"], g["bnd0"]), (g["cent1"], g["bnd1"])])
    H, QH, bs, total = 8, 32, 16, 6
    gen = torch.Generator().manual_seed(18)
    kv = torch.zeros(total, 2, bs, H, 64, dtype=torch.uint8, device="cuda")
    kv[:, 0] = htq.encode(torch.randn(total, bs, H, 128, generator=gen).half().cuda())
    kv[:, 1] = htq.encode(torch.randn(total, bs, H, 128, generator=gen).half().cuda())
    before = kv.clone()
    bt = torch.tensor([[0, 3], [2, 5], [4, 1]], dtype=torch.int32, device="cuda")
    ctx = torch.tensor([1, 20, 7], dtype=torch.int32, device="cuda")
    q = torch.randn(3, QH, 128, generator=gen).half().cuda()
    key = torch.randn(3, H, 128, generator=gen).bfloat16()
    val = torch.randn(3, H, 128, generator=gen).bfloat16()
    slots = torch.tensor([0, -1, 4 * bs + 6], dtype=torch.int64)     # seq 0 -> block 0 offset 0; seq 1 skipped
    ops.register_custom_ops()
    out = torch.zeros(3, QH, 128, dtype=torch.float16, device="cuda")
    L = _lib.lib()
    args = (q, key.cuda(), val.cuda(), kv, out, slots.cuda(), bt, ctx, 0, QH, H, 128, 1.0 / math.sqrt(128), 3)
    torch.ops.tq.hybrid_decode_step(*args)          # first call sets function attributes
    kv.copy_(before)
    n0 = L.akv_launch_count()
    torch.ops.tq.hybrid_decode_step(*args)
    assert L.akv_launch_count() - n0 == 3
    kc, vc = before[:, 0].cpu().numpy().copy(), before[:, 1].cpu().numpy().copy()
    kc[0, 0] = ohy.encode(key[0].float().numpy(), t)
    vc[0, 0] = ohy.encode(val[0].float().numpy(), t)
    kc[4, 6] = ohy.encode(key[2].float().numpy(), t)
    vc[4, 6] = ohy.encode(val[2].float().numpy(), t)
    assert np.array_equal(kv[:, 0].cpu().numpy(), kc) and np.array_equal(kv[:, 1].cpu().numpy(), vc)
    ref = ohy.paged_attention_decode_sdpa(q.cpu().numpy(), kc, vc, bt.cpu().numpy(), ctx.cpu().numpy(), t,
                                          1.0 / math.sqrt(128), bs)
    assert np.abs(out.float().cpu().numpy() - ref).max() < 2e-3


@pytest.mark.parametrize("dtype", (torch.float16, torch.bfloat16, torch.float32))
def test_hybrid_kv_update_paged_write(dtype):
    """akv_hybrid_kv_update: records land at their slots byte for byte (oracle encoder), skipped and
    out-of-range slots leave the cache alone, a strided cache view (the K half of a [blocks, 2, ...] tensor)
    is addressed through its strides."""
    from aitherkvcache_b200.hybrid_quantizer import HybridTurboQuant, hybrid_kv_update
    g = load_golden("hybrid_tq35.npz")
    htq = HybridTurboQuant(128, "tq35", device="cuda")
    htq.calibrate_uniform()
    t = ohy.Tables(128, "tq35", g["had0"], g["had1"], g["qjl0"], g["qjl1"],
                   codebooks=[(g["cent0"], g["bnd0"]), (g["cent1"], g["bnd1"])])
    H, bs, blocks, T = 8, 16, 9, 70
    gen = torch.Generator().manual_seed(4)
    x = torch.randn(T, H, 128, generator=gen).to(dtype)
    slots = torch.randperm(blocks * bs, generator=gen)[:T].to(torch.int64)
    slots[5] = -1
    slots[9] = blocks * bs + 3            # beyond the cache
    kv = torch.full((blocks, 2, bs, H, 64), 0xAB, dtype=torch.uint8, device="cuda")
    hybrid_kv_update(htq, x.cuda(), slots.cuda(), kv[:, 0])
    want = np.full((blocks, bs, H, 64), 0xAB, np.uint8)
    rec = ohy.encode(x.float().numpy(), t)
    for i, s in enumerate(slots.tolist()):
        if 0 <= s < blocks * bs:
            want[s // bs, s % bs] = rec[i]
    assert np.array_equal(kv[:, 0].cpu().numpy(), want)
    assert (kv[:, 1] == 0xAB).all()


def _causal_oracle(q, kp, kn, vp, vn, bt, lens, qlens, R, cent, bits):
    """Oracle for a chunked-prefill batch: query token i of a sequence's n query tokens sees the first
    len - (n - 1 - i) cached tokens (decode -> fp16 -> dense attention per token)."""
    outs = []
    p = 0
    for s, (ln, n) in enumerate(zip(lens, qlens)):
        for i in range(n):
            c = ln - (n - 1 - i)
            outs.append(otq.paged_attention_decode_sdpa(q[p:p + 1], kp, kn, vp, vn, bt[s:s + 1], np.asarray([c]), R, cent,
                                                        bits, 1.0 / math.sqrt(128))[0])
            p += 1
    return np.stack(outs).astype(np.float32)


def test_backend_mixed_batch_attends_over_the_packed_cache():
    """A batch that mixes a prefill chunk in the middle of a sequence, a decode token and a full prefill:
    every query token is a row of the paged kernel with its causal context; compared token by token with
    the oracle.  More rows than one slice holds, so the slicing is exercised too."""
    from aitherkvcache_b200.vllm.backend import TurboQuantImplBase, _LayerState
    H, QH, bs, bits = 8, 32, 16, 4
    impl = TurboQuantImplBase()
    impl._tq_setup(QH, 128, 1.0 / math.sqrt(128), H, "tq-t4nc")
    impl.PREFILL_ROWS = 32
    layer = types.SimpleNamespace(layer_name="mixed.layers.0.attn")
    lens, qlens = [150, 77, 60], [50, 1, 60]          # cached tokens incl. this step's, query tokens of this step
    nb = sum((n + bs - 1) // bs for n in lens) + 1
    gen = torch.Generator().manual_seed(14)
    perm = torch.randperm(nb, generator=gen)
    bt = torch.zeros(3, 10, dtype=torch.int32)
    p = 0
    for s, n in enumerate(lens):
        k = (n + bs - 1) // bs
        bt[s, :k] = perm[p:p + k].to(torch.int32)
        p += k
    kv = torch.zeros(nb, 2, bs, H, 128, dtype=torch.uint8, device="cuda")
    # the whole context of every sequence goes through the cache update (earlier steps + this one)
    T = sum(lens)
    key = torch.randn(T, H, 128, generator=gen).half().cuda()
    val = torch.randn(T, H, 128, generator=gen).half().cuda()
    slots = torch.cat([(bt[s, :(n + bs - 1) // bs].long()[:, None] * bs + torch.arange(bs)[None]).reshape(-1)[:n]
                       for s, n in enumerate(lens)])
    impl.do_kv_cache_update(layer, key, val, kv, slots.cuda())
    nq = sum(qlens)
    qry = torch.randn(nq, QH * 128, generator=gen).half()
    qsl = torch.tensor([0, 50, 51, 111], dtype=torch.int32, device="cuda")
    # max_seq_len as vLLM's metadata carries it: the prefill kernel may then stage its operand images
    md = types.SimpleNamespace(num_actual_tokens=nq, max_query_len=max(qlens), block_table=bt.cuda(), max_seq_len=max(lens),
                               seq_lens=torch.tensor(lens, dtype=torch.int32, device="cuda"), query_start_loc=qsl)
    out = torch.zeros(nq, QH * 128, dtype=torch.float16, device="cuda")
    impl.forward(layer, qry.cuda(), None, None, kv, md, output=out)
    tq = _LayerState.quantizers[(128, 4, "cuda:0")]
    kn, vn = impl._norms(layer.layer_name, kv)
    kc_, vc_ = impl._codes(kv)
    ref = _causal_oracle(qry.reshape(nq, QH, 128).numpy(), kc_.cpu().numpy(), kn.cpu().numpy(),
                         vc_.cpu().numpy(), vn.cpu().numpy(), bt.numpy(), lens, qlens,
                         tq.rotation.cpu().numpy(), tq.centroids.cpu().numpy(), bits)
    got = out.float().cpu().numpy().reshape(nq, QH, 128)
    assert (np.abs(got - ref) <= 2e-3 * np.maximum(1.0, np.abs(ref))).all()


@pytest.mark.parametrize("mode,PD", (("tq35", 64), ("tq25", 44)))
def test_backend_hybrid_mode_from_environment(monkeypatch, mode, PD):
    """AITHER_TQ_MODE=tq35 / tq25 selects the hybrid codec in the backend impl: records (norms inside) written by
    do_kv_cache_update equal the oracle's, decode and prefill rows match the oracle's decode -> attention."""
    from aitherkvcache_b200.vllm.backend import TurboQuantImplBase
    monkeypatch.setenv("AITHER_TQ_MODE", mode)
    g = load_golden(f"hybrid_{mode}.npz")
    t = ohy.Tables(128, mode, g["had0"], g["had1"], g["qjl0"], g["qjl1"],
                   codebooks=[(g["cent0"], g["bnd0"]), (g["cent1"], g["bnd1"])])
    H, QH, bs = 8, 32, 16
    impl = TurboQuantImplBase()
    impl._tq_setup(QH, 128, 1.0 / math.sqrt(128), H, "auto")
    assert impl.tq_codec == "hybrid" and impl.packed_dim == PD
    layer = types.SimpleNamespace(layer_name=f"hy{PD}.layers.0.attn")
    lens = [45, 130]
    bt = torch.tensor([[3, 7, 1, 0, 0, 0, 0, 0, 0], [2, 4, 5, 6, 8, 9, 10, 11, 12]], dtype=torch.int32)
    kv = torch.zeros(14, 2, bs, H, 128, dtype=torch.uint8, device="cuda")
    gen = torch.Generator().manual_seed(24)
    T = sum(lens)
    key = torch.randn(T, H, 128, generator=gen).half()
    val = torch.randn(T, H, 128, generator=gen).half()
    slots = torch.cat([(bt[s, :(n + bs - 1) // bs].long()[:, None] * bs + torch.arange(bs)[None]).reshape(-1)[:n]
                       for s, n in enumerate(lens)])
    impl.do_kv_cache_update(layer, key.cuda(), val.cuda(), kv, slots.cuda())
    kc = kv[:, 0, ..., :PD].cpu().numpy()
    vc = kv[:, 1, ..., :PD].cpu().numpy()
    assert np.array_equal(kc.reshape(-1, H, PD)[slots.numpy()], ohy.encode(key.numpy(), t))
    q = torch.randn(2, QH * 128, generator=gen).half()
    md1 = types.SimpleNamespace(num_actual_tokens=2, max_query_len=1, block_table=bt.cuda(),
                                seq_lens=torch.tensor(lens, dtype=torch.int32, device="cuda"))
    out1 = torch.zeros(2, QH * 128, dtype=torch.float16, device="cuda")
    impl.forward(layer, q.cuda(), None, None, kv, md1, output=out1)
    ref = ohy.paged_attention_decode_sdpa(q.reshape(2, QH, 128).numpy(), kc, vc, bt.numpy(), np.asarray(lens), t,
                                          1.0 / math.sqrt(128), bs)
    assert np.abs(out1.float().cpu().numpy().reshape(2, QH, 128) - ref).max() < 2e-3
    # the last three tokens of sequence 1 as a prefill chunk: the last row equals the decode row
    q3 = torch.cat([torch.randn(2, QH * 128, generator=gen).half(), q[1:2]])
    md3 = types.SimpleNamespace(num_actual_tokens=3, max_query_len=3, block_table=bt[1:2].cuda(),
                                seq_lens=torch.tensor(lens[1:], dtype=torch.int32, device="cuda"),
                                query_start_loc=torch.tensor([0, 3], dtype=torch.int32, device="cuda"))
    out3 = torch.zeros(3, QH * 128, dtype=torch.float16, device="cuda")
    impl.forward(layer, q3.cuda(), None, None, kv, md3, output=out3)
    assert (out3[2].float() - out1[1].float()).abs().max().item() < 1e-3
    ref0 = ohy.paged_attention_decode_sdpa(q3[:1].reshape(1, QH, 128).numpy(), kc, vc, bt.numpy()[1:2],
                                           np.asarray([lens[1] - 2]), t, 1.0 / math.sqrt(128), bs)
    assert np.abs(out3[0].float().cpu().numpy().reshape(QH, 128) - ref0[0]).max() < 2e-3
    # a mixed batch with the host-side length bound of vLLM's metadata: sequence 0 brings one token (decode kernel),
    # sequence 1 its last 64 (tq35: staged tensor-core prefill over decoded operand images; tq25: rows)
    qm = torch.cat([q[0:1], torch.randn(63, QH * 128, generator=gen).half(), q[1:2]])
    mdm = types.SimpleNamespace(num_actual_tokens=65, max_query_len=64, block_table=bt.cuda(), max_seq_len=max(lens),
                                seq_lens=torch.tensor(lens, dtype=torch.int32, device="cuda"),
                                query_start_loc=torch.tensor([0, 1, 65], dtype=torch.int32, device="cuda"))
    outm = torch.zeros(65, QH * 128, dtype=torch.float16, device="cuda")
    impl.forward(layer, qm.cuda(), None, None, kv, mdm, output=outm)
    if mode == "tq35":
        from aitherkvcache_b200 import _lib
        assert _lib.lib().akv_last_split_kernel() != b"tq_prefill_attn_tc_staged_kernel"      # the decode side ran last ...
    assert (outm[0].float() - out1[0].float()).abs().max().item() < 1e-3
    assert (outm[64].float() - out1[1].float()).abs().max().item() < 2e-3
    refm = ohy.paged_attention_decode_sdpa(qm[1:2].reshape(1, QH, 128).numpy(), kc, vc, bt.numpy()[1:2],
                                           np.asarray([lens[1] - 63]), t, 1.0 / math.sqrt(128), bs, kv_dtype=np.float16)
    assert np.abs(outm[1].float().cpu().numpy().reshape(QH, 128) - refm[0]).max() < 2e-3


def test_backend_decode_step_replays_from_a_cuda_graph():
    """The single-token decode forward of the backend impl (what the metadata builder declares
    graph-capturable): captured once, replayed with new query / sequence-length contents in the same
    buffers, equal to the eager result."""
    from aitherkvcache_b200.vllm.backend import TurboQuantImplBase
    H, QH, bs = 8, 32, 16
    impl = TurboQuantImplBase()
    impl._tq_setup(QH, 128, 1.0 / math.sqrt(128), H, "tq-t4nc")
    layer = types.SimpleNamespace(layer_name="graph.layers.0.attn")
    lens = [300, 41, 1000, 7]
    nblk = [(n + bs - 1) // bs for n in lens]
    gen = torch.Generator().manual_seed(31)
    perm = torch.randperm(sum(nblk), generator=gen)
    bt = torch.zeros(4, max(nblk), dtype=torch.int32)
    p = 0
    for s, k in enumerate(nblk):
        bt[s, :k] = perm[p:p + k].to(torch.int32)
        p += k
    kv = torch.zeros(sum(nblk), 2, bs, H, 128, dtype=torch.uint8, device="cuda")
    T = sum(lens)
    slots = torch.cat([(bt[s, :nblk[s]].long()[:, None] * bs + torch.arange(bs)[None]).reshape(-1)[:n]
                       for s, n in enumerate(lens)])
    impl.do_kv_cache_update(layer, torch.randn(T, H, 128, generator=gen).half().cuda(),
                            torch.randn(T, H, 128, generator=gen).half().cuda(), kv, slots.cuda())
    q = torch.randn(4, QH * 128, generator=gen).half().cuda()
    seq_lens = torch.tensor(lens, dtype=torch.int32, device="cuda")
    md = types.SimpleNamespace(num_actual_tokens=4, max_query_len=1, block_table=bt.cuda(), seq_lens=seq_lens)
    out = torch.zeros(4, QH * 128, dtype=torch.float16, device="cuda")
    impl.forward(layer, q, None, None, kv, md, output=out)            # warm-up: workspace, argument block
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        impl.forward(layer, q, None, None, kv, md, output=out)
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        impl.forward(layer, q, None, None, kv, md, output=out)
    for trial in range(2):
        q.copy_(torch.randn(4, QH * 128, generator=gen).half())
        seq_lens.copy_(torch.tensor([n - trial * 5 for n in lens], dtype=torch.int32).clamp(min=1))
        graph.replay()
        got = out.clone()
        impl.forward(layer, q, None, None, kv, md, output=out)
        torch.cuda.synchronize()
        assert torch.equal(got, out)


@pytest.mark.parametrize("bits", (4, 3))
@pytest.mark.parametrize("layout", ("planes", "records"))
def test_backend_primary_records_keep_norms_in_the_row(monkeypatch, bits, layout):
    """Primary-mode cache [blocks, 2, block_size, heads, packed_dim + 4] bytes per block as in the reference.  "records"
    (AITHER_TQ_RECORD_PAGES): the float32 norm of a vector sits behind its codes in the same row, the reference's page
    format.  "planes" (default): in each K / V half of a block first all code rows, then all norms, so that code rows
    stay 16-byte aligned.  Writes and attention over either layout equal the separate-norm layout bit for bit."""
    from aitherkvcache_b200 import _lib
    from aitherkvcache_b200.vllm.backend import TurboQuantBackend, TurboQuantImplBase, _LayerState
    monkeypatch.setenv("AITHER_TQ_MODE", f"tq{bits}-primary")
    if layout == "records":
        monkeypatch.setenv("AITHER_TQ_RECORD_PAGES", "1")
    else:
        monkeypatch.delenv("AITHER_TQ_RECORD_PAGES", raising=False)
    H, QH, bs, pd = 8, 32, 16, 128 * bits // 8
    assert TurboQuantBackend.get_kv_cache_shape(14, bs, H, 128) == (14, 2, bs, H, pd + 4)
    impl = TurboQuantImplBase()
    impl._tq_setup(QH, 128, 1.0 / math.sqrt(128), H, "auto")
    assert impl.tq_codec == "uniform" and impl.tq_bits == bits and impl.packed_dim == pd
    lens = [45, 130]
    bt = torch.tensor([[3, 7, 1, 0, 0, 0, 0, 0, 0], [2, 4, 5, 6, 8, 9, 10, 11, 12]], dtype=torch.int32)
    gen = torch.Generator().manual_seed(31)
    T = sum(lens)
    key = torch.randn(T, H, 128, generator=gen).half().cuda()
    val = torch.randn(T, H, 128, generator=gen).half().cuda()
    slots = torch.cat([(bt[s, :(n + bs - 1) // bs].long()[:, None] * bs + torch.arange(bs)[None]).reshape(-1)[:n]
                       for s, n in enumerate(lens)]).cuda()
    q = torch.randn(2, QH * 128, generator=gen).half().cuda()
    md = types.SimpleNamespace(num_actual_tokens=2, max_query_len=1, block_table=bt.cuda(),
                               seq_lens=torch.tensor(lens, dtype=torch.int32, device="cuda"))
    outs, caches, kernels = [], [], []
    for width, name in ((pd + 4, "prim.layers.0.attn"), (128, "sep.layers.0.attn")):
        layer = types.SimpleNamespace(layer_name=name)
        kv = torch.zeros(14, 2, bs, H, width, dtype=torch.uint8, device="cuda")
        if width == 128:       # a strided view: codes at the start of 128-byte rows, norms in side tensors
            kv = torch.zeros(14, 2, bs, H, 256, dtype=torch.uint8, device="cuda")[..., :128]
        impl.do_kv_cache_update(layer, key, val, kv, slots)
        out = torch.zeros(2, QH * 128, dtype=torch.float16, device="cuda")
        impl.forward(layer, q, None, None, kv, md, output=out)
        outs.append(out)
        caches.append(kv)
        kernels.append(_lib.lib().akv_last_split_kernel())
    prim, sep = caches
    assert "prim.layers.0.attn" not in _LayerState.k_norms            # no side tensors for the primary layouts
    if layout == "records":
        assert torch.equal(prim[..., :pd], sep[..., :pd])
        kn = prim[:, 0, :, :, pd:].contiguous().view(torch.float32).squeeze(-1)
    else:
        flat = prim.view(14, 2, -1)
        assert torch.equal(flat[:, :, :bs * H * pd].reshape(14, 2, bs, H, pd), sep[..., :pd])
        kn = flat[:, 0, bs * H * pd:].contiguous().view(torch.float32).view(14, bs, H)
        assert kernels[0] != b"tq_attn_mma_kernel"      # 16-byte aligned code rows: a TMA-fed kernel serves the primary cache
    assert torch.equal(kn, _LayerState.k_norms["sep.layers.0.attn"])
    if kernels[0] == kernels[1]:
        assert torch.equal(outs[0], outs[1])
    else:       # another kernel over the same bytes: equal up to the order of the float32 sums
        assert (outs[0].float() - outs[1].float()).abs().max().item() < 1e-3


@pytest.mark.parametrize("layout", ("planes", "records"))
@pytest.mark.parametrize("bits", (4, 3))
def test_backend_primary_records_chunked_prefill(monkeypatch, bits, layout):
    """A prefill chunk over the primary-mode record layout (68- / 52-byte rows, norm inside, not readable in 16-byte
    pieces) with vLLM's host-side length bound: the staged tensor-core kernel serves it (pre-pass by byte loads); rows
    equal the decode kernels run token by token over the same cache."""
    from aitherkvcache_b200 import _lib
    from aitherkvcache_b200.vllm.backend import TurboQuantImplBase
    monkeypatch.setenv("AITHER_TQ_MODE", f"tq{bits}-primary")
    if layout == "records":
        monkeypatch.setenv("AITHER_TQ_RECORD_PAGES", "1")
    else:
        monkeypatch.delenv("AITHER_TQ_RECORD_PAGES", raising=False)
    H, QH, bs, pd = 8, 32, 16, 128 * bits // 8
    impl = TurboQuantImplBase()
    impl._tq_setup(QH, 128, 1.0 / math.sqrt(128), H, "auto")
    layer = types.SimpleNamespace(layer_name=f"primchunk{bits}{layout}.layers.0.attn")
    n, chunk = 330, 96
    nb = (n + bs - 1) // bs
    gen = torch.Generator().manual_seed(9)
    bt = torch.randperm(nb + 2, generator=gen)[:nb].to(torch.int32).reshape(1, nb)
    kv = torch.zeros(nb + 2, 2, bs, H, pd + 4, dtype=torch.uint8, device="cuda")
    key = torch.randn(n, H, 128, generator=gen).half().cuda()
    val = torch.randn(n, H, 128, generator=gen).half().cuda()
    slots = (bt[0].long()[:, None] * bs + torch.arange(bs)[None]).reshape(-1)[:n].cuda()
    impl.do_kv_cache_update(layer, key, val, kv, slots)
    q = torch.randn(chunk, QH * 128, generator=gen).half().cuda()
    md = types.SimpleNamespace(num_actual_tokens=chunk, max_query_len=chunk, block_table=bt.cuda(), max_seq_len=n,
                               seq_lens=torch.tensor([n], dtype=torch.int32, device="cuda"),
                               query_start_loc=torch.tensor([0, chunk], dtype=torch.int32, device="cuda"))
    out = torch.zeros(chunk, QH * 128, dtype=torch.float16, device="cuda")
    impl.forward(layer, q, None, None, kv, md, output=out)
    assert _lib.lib().akv_last_split_kernel() == b"tq_prefill_attn_tc_staged_kernel"
    # token by token: every query token as its own single-token sequence
    md1 = types.SimpleNamespace(num_actual_tokens=chunk, max_query_len=1, block_table=bt.expand(chunk, -1).contiguous().cuda(),
                                seq_lens=torch.arange(n - chunk + 1, n + 1, dtype=torch.int32, device="cuda"))
    ref = torch.zeros_like(out)
    impl.forward(layer, q, None, None, kv, md1, output=ref)
    assert ((out.float() - ref.float()).abs() <= 2e-3 * ref.float().abs().clamp(min=1.0)).all()
