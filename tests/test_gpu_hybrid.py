"""GPU parity of the hybrid (tq35 / tq25) kernels against reference fixtures and the oracle."""
import math

import numpy as np
import pytest
import torch

from conftest import load_golden
from oracle import hybrid as ohy

pytestmark = pytest.mark.gpu


def _htq(mode, g=None, heads=1):
    from aitherkvcache_b200.hybrid_quantizer import HybridTurboQuant
    h = HybridTurboQuant(head_dim=128, mode=mode, device="cuda")
    h.calibrate_uniform(num_kv_heads=heads)
    if g is not None:   # tables are bit-identical to the reference's on this torch build; use the fixture's anyway
        for name, key in (("_g0_had_signs", "had0"), ("_g1_had_signs", "had1"), ("_g0_qjl_signs", "qjl0"),
                          ("_g1_qjl_signs", "qjl1"), ("_g0_centroids", "cent0"), ("_g0_boundaries", "bnd0"),
                          ("_g1_centroids", "cent1"), ("_g1_boundaries", "bnd1")):
            assert np.abs(getattr(h, name).cpu().numpy() - g[key]).max() < 1e-7
            setattr(h, name, torch.from_numpy(g[key]).cuda())
        h._tables = None
    return h


def _oracle_tables(g, mode):
    return ohy.Tables(128, mode, g["had0"], g["had1"], g["qjl0"], g["qjl1"],
                      codebooks=[(g["cent0"], g["bnd0"]), (g["cent1"], g["bnd1"])])


@pytest.mark.parametrize("mode", ("tq35", "tq25"))
def test_encode_bytes_equal_reference(mode):
    g = load_golden(f"hybrid_{mode}.npz")
    h = _htq(mode, g)
    packed = h.encode(torch.from_numpy(g["x"]).cuda())
    assert packed.dtype == torch.uint8 and packed.shape == g["packed"].shape
    got, ref = packed.cpu().numpy(), g["packed"]
    lay = h.layout
    a0 = lay.group0.mse_packed_bytes
    fields = {"g0 codes": slice(0, a0), "g0 qjl bits": slice(a0, a0 + lay.group0.qjl_packed_bytes),
              "g0 norms": slice(lay.group0.total_bytes - 4, lay.group0.total_bytes),
              "g1 codes": slice(lay.group0.total_bytes, lay.group0.total_bytes + lay.group1.mse_packed_bytes),
              "g1 norms": slice(lay.packed_dim - 4, lay.packed_dim)}
    for name, sl in fields.items():
        assert np.array_equal(got[:, sl], ref[:, sl]), f"{name} differ in {(got[:, sl] != ref[:, sl]).any(1).sum()} rows"
    assert np.array_equal(got, ref)


@pytest.mark.parametrize("mode", ("tq35", "tq25"))
def test_decode_bit_equal_reference(mode):
    g = load_golden(f"hybrid_{mode}.npz")
    h = _htq(mode, g)
    dec = h.decode(torch.from_numpy(g["packed"]).cuda())
    assert dec.dtype == torch.float32 and dec.shape == g["decoded"].shape
    fin = np.isfinite(g["decoded"])
    assert np.array_equal(dec.cpu().numpy()[fin].view(np.uint32), g["decoded"][fin].view(np.uint32))


def test_config3_shape_vs_oracle_and_quality():
    """[8, 4096, 8, 128] fp16 N(0,1), seed 0 (first 64 K vectors compared byte for byte)."""
    g = load_golden("hybrid_tq35.npz")
    h = _htq("tq35", g)
    x = torch.randn(8, 4096, 8, 128, generator=torch.Generator().manual_seed(0)).half()
    packed = h.encode(x.cuda())
    assert packed.shape == (8, 4096, 8, 64)
    ref = ohy.encode(x[:2].numpy(), _oracle_tables(g, "tq35"))
    assert np.array_equal(packed[:2].cpu().numpy(), ref)
    assert np.array_equal(packed.reshape(-1, 64)[:768].cpu().numpy(), g["packed"][:768])
    dec = h.decode(packed[:2])
    cos = torch.nn.functional.cosine_similarity(dec.reshape(-1, 128).cpu(), x[:2].float().reshape(-1, 128), dim=-1)
    assert cos.mean().item() > 0.97


def test_per_head_calibration_and_errors():
    from aitherkvcache_b200.hybrid_quantizer import HybridTurboQuant
    h = HybridTurboQuant(128, "tq35", device="cuda")
    with pytest.raises(RuntimeError):
        h.encode(torch.randn(4, 128, device="cuda"))
    with pytest.raises(ValueError):
        HybridTurboQuant(128, "tq45", device="cuda")
    gen = torch.Generator().manual_seed(3)
    sample = torch.randn(512, 4, 128, generator=gen) * torch.rand(1, 4, 128, generator=gen) * 3
    h.calibrate(sample.cuda())
    x = torch.randn(6, 4, 128, generator=gen).half()
    packed = h.encode(x.cuda())                       # 24 rows cycle over the 4 heads
    assert packed.shape == (6, 4, 64)
    g0, g1 = h._group0_indices.cpu().numpy(), h._group1_indices.cpu().numpy()
    t = ohy.Tables(128, "tq35", h._g0_had_signs.cpu().numpy(), h._g1_had_signs.cpu().numpy(),
                   h._g0_qjl_signs.cpu().numpy(), h._g1_qjl_signs.cpu().numpy(),
                   codebooks=[(h._g0_centroids.cpu().numpy(), h._g0_boundaries.cpu().numpy()),
                              (h._g1_centroids.cpu().numpy(), h._g1_boundaries.cpu().numpy())])
    for hd in range(4):
        ref = ohy.encode(x[:, hd].numpy(), t, g0[hd], g1[hd])
        assert np.array_equal(packed[:, hd].cpu().numpy(), ref)
        dec = h.decode(packed)[:, hd].cpu().numpy()
        assert np.array_equal(dec.view(np.uint32), ohy.decode(ref, t, g0[hd], g1[hd]).view(np.uint32))
    assert h.decode(packed).shape == (6, 4, 128)
    r = h.validate(2000)
    assert r["cosine_similarity"] > 0.9


@pytest.mark.parametrize("mode", ("tq35", "tq25"))
@pytest.mark.parametrize("H,QH,ctx", [(8, 32, [700, 33, 1, 0]), (2, 4, [100, 48]), (2, 16, [257])])
def test_paged_attention_vs_oracle(H, QH, ctx, mode):
    from aitherkvcache_b200.hybrid_quantizer import HybridPagedAttention
    g = load_golden(f"hybrid_{mode}.npz")
    h = _htq(mode, g, heads=1)
    t = _oracle_tables(g, mode)
    gen = torch.Generator().manual_seed(12)
    bs = 16
    nblk = [(c + bs - 1) // bs for c in ctx]
    total = sum(nblk) + 2
    perm = torch.randperm(total, generator=gen)
    bt = torch.zeros(len(ctx), max(nblk), dtype=torch.int32)
    p = 0
    for s, n in enumerate(nblk):
        bt[s, :n] = perm[p:p + n].to(torch.int32)
        p += n
    k = torch.randn(total, bs, H, 128, generator=gen).half()
    v = torch.randn(total, bs, H, 128, generator=gen).half()
    q = torch.randn(len(ctx), QH, 128, generator=gen).half()
    kc, vc = h.encode(k.cuda()), h.encode(v.cuda())
    assert np.array_equal(kc.cpu().numpy(), ohy.encode(k.numpy(), t))
    out = HybridPagedAttention(h, QH).forward(q.cuda(), kc, vc, bt.cuda(), torch.tensor(ctx, dtype=torch.int32).cuda())
    assert out.dtype == torch.float16 and out.shape == (len(ctx), QH, 128)
    out = out.float().cpu().numpy()
    for kv_dtype in (np.float32, np.float16):
        ref = ohy.paged_attention_decode_sdpa(q.numpy(), kc.cpu().numpy(), vc.cpu().numpy(), bt.numpy(),
                                              np.asarray(ctx), t, 1.0 / math.sqrt(128), bs, kv_dtype=kv_dtype)
        assert np.abs(out - ref).max() < 2e-3
    for s, c in enumerate(ctx):
        if c == 0:
            assert (out[s] == 0).all()


def test_paged_attention_full_size_properties():
    """tq35 attention at the headline shapes (16 sequences of 4096..32768 tokens, 32 query / 8 KV heads,
    permuted block tables): with one value record per (sequence, KV head) repeated over all tokens the
    output must be that record's decoded vector whatever the scores are; the shortest sequence is also
    compared with the oracle."""
    from aitherkvcache_b200.hybrid_quantizer import HybridPagedAttention
    g = load_golden("hybrid_tq35.npz")
    h = _htq("tq35", g, heads=1)
    t = _oracle_tables(g, "tq35")
    H, QH, D, BS, S = 8, 32, 128, 16, 16
    gen = torch.Generator().manual_seed(1)
    ctx = torch.randint(4096, 32769, (S,), generator=gen)
    nblk = [(int(c) + BS - 1) // BS for c in ctx]
    total = sum(nblk)
    perm = torch.randperm(total, generator=gen)
    bt = torch.zeros(S, max(nblk), dtype=torch.int32)
    p = 0
    for s, n in enumerate(nblk):
        bt[s, :n] = perm[p:p + n].to(torch.int32)
        p += n
    gg = torch.Generator(device="cuda").manual_seed(2)
    kc = h.encode(torch.randn(total, BS, H, D, generator=gg, device="cuda").half())
    v_rec = h.encode(torch.randn(S, H, D, generator=gg, device="cuda").half())        # [S, H, packed_dim]
    vc = torch.empty_like(kc)
    for s, n in enumerate(nblk):
        vc[bt[s, :n].cuda().long()] = v_rec[s][None, None].expand(n, BS, H, v_rec.shape[-1])
    q = torch.randn(S, QH, D, generator=torch.Generator().manual_seed(5)).half().cuda()
    out = HybridPagedAttention(h, QH).forward(q, kc, vc, bt.cuda(), ctx.to(torch.int32).cuda()).float().cpu().numpy()
    want = np.repeat(h.decode(v_rec).float().cpu().numpy(), QH // H, axis=1)
    assert np.abs(out - want).max() <= 2e-3 * max(1.0, float(np.abs(want).max()))

    pick = np.argsort(ctx.numpy())[:1]
    ref = ohy.paged_attention_decode_sdpa(q.cpu().numpy()[pick], kc.cpu().numpy(), vc.cpu().numpy(), bt.numpy()[pick],
                                          ctx.numpy()[pick], t, 1.0 / math.sqrt(D), BS, kv_dtype=np.float32)
    assert (np.abs(out[pick] - ref) <= 2e-3 * np.maximum(1.0, np.abs(ref))).all()


def test_paged_attention_full_size_random_values_vs_oracle():
    """tq35 attention at the headline shapes with random K and random V: the shortest and the longest
    (about 31 K tokens) sequence against the oracle's decode -> dense attention, element by element."""
    from aitherkvcache_b200.hybrid_quantizer import HybridPagedAttention
    g = load_golden("hybrid_tq35.npz")
    h = _htq("tq35", g, heads=1)
    t = _oracle_tables(g, "tq35")
    H, QH, D, BS, S = 8, 32, 128, 16, 16
    gen = torch.Generator().manual_seed(1)
    ctx = torch.randint(4096, 32769, (S,), generator=gen)
    nblk = [(int(c) + BS - 1) // BS for c in ctx]
    total = sum(nblk)
    perm = torch.randperm(total, generator=gen)
    bt = torch.zeros(S, max(nblk), dtype=torch.int32)
    p = 0
    for s, n in enumerate(nblk):
        bt[s, :n] = perm[p:p + n].to(torch.int32)
        p += n
    gg = torch.Generator(device="cuda").manual_seed(2)
    kc = h.encode(torch.randn(total, BS, H, D, generator=gg, device="cuda").half())
    vc = h.encode(torch.randn(total, BS, H, D, generator=gg, device="cuda").half())
    q = torch.randn(S, QH, D, generator=torch.Generator().manual_seed(5)).half().cuda()
    out = HybridPagedAttention(h, QH).forward(q, kc, vc, bt.cuda(), ctx.to(torch.int32).cuda()).float().cpu().numpy()
    order = np.argsort(ctx.numpy())
    pick = np.array([order[0], order[-1]])
    assert int(ctx[pick[1]]) > 30000
    ref = ohy.paged_attention_decode_sdpa(q.cpu().numpy()[pick], kc.cpu().numpy(), vc.cpu().numpy(), bt.numpy()[pick],
                                          ctx.numpy()[pick], t, 1.0 / math.sqrt(D), BS, kv_dtype=np.float32)
    assert np.abs(out[pick] - ref).max() < 2e-3


@pytest.mark.parametrize("mode", ("tq35", "tq25"))
@pytest.mark.parametrize("H,QH", [(8, 32), (2, 16), (2, 2)])
def test_chunked_prefill_over_hybrid_records(H, QH, mode):
    """Chunked prefill over a tq35 / tq25 cache: the pre-pass decodes every 128-key tile of records into fp16 operand
    images, the tensor-core attention kernel runs over them in the original domain.  Against the record-domain decode
    kernel row by row (all rows) and the oracle (decode -> fp16 -> attention) on the last row of each chunk."""
    from aitherkvcache_b200 import _lib
    from aitherkvcache_b200.hybrid_quantizer import HybridPagedAttention
    g = load_golden(f"hybrid_{mode}.npz")
    h = _htq(mode, g, heads=1)
    t = _oracle_tables(g, mode)
    gen = torch.Generator().manual_seed(21 + H)
    bs = 16
    seqs = [(500, 140), (0, 200), (130, 128)]          # (cached before the chunk, chunk length)
    lens = [p + q for p, q in seqs]
    nblk = [(n + bs - 1) // bs for n in lens]
    total = sum(nblk) + 2
    perm = torch.randperm(total, generator=gen)
    bt = torch.zeros(len(seqs), max(nblk), dtype=torch.int32)
    o = 0
    for s, n in enumerate(nblk):
        bt[s, :n] = perm[o:o + n].to(torch.int32)
        o += n
    kc = h.encode(torch.randn(total, bs, H, 128, generator=gen).half().cuda())
    vc = h.encode(torch.randn(total, bs, H, 128, generator=gen).half().cuda())
    nq = sum(q for _, q in seqs)
    qsl = torch.tensor([0] + list(np.cumsum([q for _, q in seqs])), dtype=torch.int32)
    query = torch.randn(nq, QH, 128, generator=gen).half().cuda()
    attn = HybridPagedAttention(h, QH)
    sl = torch.tensor(lens, dtype=torch.int32).cuda()
    assert attn.prefill(query, kc, vc, bt.cuda(), sl, qsl.cuda(), block_size=bs) is None          # no host-side bound
    out = attn.prefill(query, kc, vc, bt.cuda(), sl, qsl.cuda(), block_size=bs, max_seq_len=max(lens))
    assert out is not None and out.dtype == torch.float16
    assert _lib.lib().akv_last_split_kernel() == b"tq_prefill_attn_tc_staged_kernel"
    rows_bt = torch.cat([bt[s:s + 1].expand(q, -1) for s, (_, q) in enumerate(seqs)])
    rows_ctx = torch.cat([torch.arange(p + 1, p + q + 1) for p, q in seqs]).to(torch.int32)
    ref = torch.cat([attn.forward(query[lo:lo + 64], kc, vc, rows_bt[lo:lo + 64].contiguous().cuda(), rows_ctx[lo:lo + 64].cuda())
                     for lo in range(0, nq, 64)])
    # rows with a handful of keys return value vectors of magnitude 2..4, where one fp16 step (the staged values are
    # fp16) is 2e-3 already: the tolerance scales with the magnitude
    assert ((out.float() - ref.float()).abs() <= 2e-3 * ref.float().abs().clamp(min=1.0)).all()
    for s in range(len(seqs)):
        row = int(qsl[s + 1]) - 1
        want = ohy.paged_attention_decode_sdpa(query[row:row + 1].cpu().numpy(), kc.cpu().numpy(), vc.cpu().numpy(),
                                               bt[s:s + 1].numpy(), np.asarray([lens[s]]), t, 1.0 / math.sqrt(128), bs,
                                               kv_dtype=np.float16)
        assert np.abs(out[row].float().cpu().numpy() - want[0]).max() < 2e-3
    assert not any(_lib.device_status().values())
