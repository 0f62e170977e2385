"""GPU parity of the TriAttention kernels against reference fixtures and the oracle."""
import numpy as np
import pytest
import torch

from conftest import load_golden
from oracle import tri as otri

pytestmark = pytest.mark.gpu


def _tri(kvh=2, qh=8, f=12):
    from aitherkvcache_b200.triattention import TriAttention, TriAttentionConfig
    cfg = TriAttentionConfig(head_dim=128, num_freqs=f, coeff_bits=4, num_kv_heads=kvh, num_query_heads=qh,
                             rope_base=1_000_000.0)
    return TriAttention(cfg, device="cuda")


def _enc_to_cuda(g, side):
    from aitherkvcache_b200.triattention import SpectralEncoding
    return SpectralEncoding(torch.from_numpy(g[f"{side}_indices"]).cuda(), torch.from_numpy(g[f"{side}_packed"]).cuda(),
                            torch.from_numpy(g[f"{side}_scales"]).cuda())


def test_encode_matches_reference():
    g = load_golden("tri_f12_int4.npz")
    tri = _tri()
    assert np.array_equal(tri._theta.cpu().numpy().view(np.uint32), g["theta"].view(np.uint32))
    k_enc, v_enc = tri.encode_kv(torch.from_numpy(g["keys"]).cuda(), torch.from_numpy(g["values"]).cuda())
    for side, enc, x in (("k", k_enc, g["keys"]), ("v", v_enc, g["values"])):
        assert enc.indices.dtype == torch.uint8 and enc.packed.dtype == torch.uint8 and enc.scales.dtype == torch.float16
        assert enc.indices.shape == (2, 200, 2, 12) and enc.scales.shape == (2, 200, 2)
        clear = otri.rank_gap(x, 12) > 0        # top-F set unambiguous
        assert clear.mean() > 0.999
        assert np.array_equal(enc.indices.cpu().numpy()[clear], g[f"{side}_indices"][clear])
        assert np.array_equal(enc.packed.cpu().numpy()[clear], g[f"{side}_packed"][clear])
        assert np.array_equal(enc.scales.cpu().numpy()[clear].view(np.uint16), g[f"{side}_scales"][clear].view(np.uint16))


def test_decode_step_matches_reference():
    g = load_golden("tri_f12_int4.npz")
    tri = _tri()
    k_enc, v_enc = _enc_to_cuda(g, "k"), _enc_to_cuda(g, "v")
    q = torch.from_numpy(g["query"]).cuda()
    out = tri.decode_step(q, k_enc, v_enc)
    assert out.dtype == torch.float32 and out.shape == (2, 8, 128)
    assert np.abs(out.cpu().numpy() - g["out_default"]).max() < 2e-3
    qpos, kpos = torch.from_numpy(g["query_pos"]).cuda(), torch.from_numpy(g["key_positions"]).cuda()
    out = tri.decode_step(q, k_enc, v_enc, qpos, kpos)
    assert np.abs(out.cpu().numpy() - g["out_far"]).max() < 2e-3
    from aitherkvcache_b200.triattention import TrigSeriesScorer
    sc = TrigSeriesScorer(tri.config, device="cuda").score(q, k_enc, qpos, kpos)
    assert sc.shape == (2, 8, 200)
    assert np.abs(sc.cpu().numpy() - g["scores_far"]).max() < 5e-3     # fp16 operands of the score product


def _synthetic(B, S, H, seed=2):
    g = torch.Generator().manual_seed(seed)
    s_i = torch.exp(-torch.arange(64, dtype=torch.float32) / 16.0)
    scale = torch.stack([s_i[torch.randperm(64, generator=g)] for _ in range(H)])
    keys = (torch.randn(B, S, H, 64, 2, generator=g) * scale[None, None, :, :, None]).reshape(B, S, H, 128).half()
    values = torch.randn(B, S, H, 128, generator=g).half()
    return keys, values, g


@pytest.mark.parametrize("S", (1, 31, 32, 33, 2500))
def test_decode_step_vs_oracle_long_positions(S):
    """Benchmark head layout (32Q/8KV), keys at the far end of a 128K context."""
    B, H, QH = 2, 8, 32
    tri = _tri(H, QH)
    keys, values, g = _synthetic(B, S, H)
    q = torch.randn(B, QH, 128, generator=g).half()
    k_enc, v_enc = tri.encode_kv(keys.cuda(), values.cuda())
    kpos = torch.arange(131072 - S, 131072).unsqueeze(0).expand(B, -1).contiguous()
    qpos = torch.full((B,), 131072)
    out = tri.decode_step(q.cuda(), k_enc, v_enc, qpos.cuda(), kpos.cuda()).cpu().numpy()
    k_np = tuple(t.cpu().numpy() for t in k_enc)
    v_np = tuple(t.cpu().numpy() for t in v_enc)
    ref = otri.decode_step(q.numpy(), k_np, v_np, tri._theta.cpu().numpy(), qpos.numpy(), kpos.numpy())
    assert np.abs(out - ref).max() < 2e-3
    # the encoder against the oracle on the same data
    oi, op, osc = otri.encode(keys.numpy(), 12)
    clear = otri.rank_gap(keys.numpy(), 12) > 0
    assert np.array_equal(k_np[0][clear], oi[clear]) and np.array_equal(k_np[1][clear], op[clear])
    assert np.array_equal(k_np[2][clear].view(np.uint16), osc[clear].view(np.uint16))


def test_split_ranges_merge_like_devices():
    """Key range split in contiguous parts, raw partials merged by akv_lse_merge (one part empty)."""
    from aitherkvcache_b200 import _lib
    from aitherkvcache_b200.triattention import SpectralEncoding
    B, S, H, QH = 2, 1000, 8, 32
    tri = _tri(H, QH)
    keys, values, g = _synthetic(B, S, H, seed=5)
    q = torch.randn(B, QH, 128, generator=g).half().cuda()
    k_enc, v_enc = tri.encode_kv(keys.cuda(), values.cuda())
    full = tri.decode_step(q, k_enc, v_enc)
    bounds = [0, 400, 400, 1000]            # rank 1 holds nothing
    parts = []
    for r in range(3):
        lo, hi = bounds[r], bounds[r + 1]
        sl = lambda e: SpectralEncoding(e.indices[:, lo:hi].contiguous(), e.packed[:, lo:hi].contiguous(),   # noqa: E731
                                        e.scales[:, lo:hi].contiguous())
        parts.append(tri.decode_step_partial(q, sl(k_enc), sl(v_enc), key_pos_start=lo, query_pos_default=S))
    stacked = torch.stack(parts).contiguous()
    assert stacked[1, :, 1].abs().max().item() == 0.0
    out = torch.empty(B, QH, 128, dtype=torch.float32, device="cuda")
    rc = _lib.lib().akv_lse_merge(stacked.data_ptr(), 3, B, QH, 128, None, out.data_ptr(), _lib.AKV_F32,
                                  out.stride(0), out.stride(1), torch.cuda.current_stream().cuda_stream)
    _lib.check(rc, "akv_lse_merge")
    assert (out - full).abs().max().item() < 1e-4


def test_decode_step_full_size_properties():
    """The 128K-token workload (1 x 131072 keys, 32 query / 8 KV heads): with the same value vector at
    every position of a KV head the output must be that vector's spectral reconstruction whatever the
    scores are, and splitting the key range in uneven parts and merging the raw partials must give
    the same result as the single call."""
    from aitherkvcache_b200 import _lib
    from aitherkvcache_b200.triattention import SpectralEncoding
    B, S, H, QH = 1, 131072, 8, 32
    tri = _tri(H, QH)
    keys, _, g = _synthetic(B, S, H, seed=9)
    v_one = torch.randn(B, 1, H, 128, generator=g).half()
    q = torch.randn(B, QH, 128, generator=g).half().cuda()
    k_enc, v_enc = tri.encode_kv(keys.cuda(), v_one.expand(B, S, H, 128).contiguous().cuda())
    out = tri.decode_step(q, k_enc, v_enc)
    first = SpectralEncoding(v_enc.indices[:, :1], v_enc.packed[:, :1], v_enc.scales[:, :1])
    want = tri.encoder.decode(first)[:, 0].repeat_interleave(QH // H, dim=1)          # [B, QH, 128]
    assert (out.float() - want).abs().max().item() <= 2e-3 * max(1.0, want.abs().max().item())

    bounds = [0, 1, 40000, 40000, 131071, 131072]
    parts = []
    for r in range(len(bounds) - 1):
        lo, hi = bounds[r], bounds[r + 1]
        sl = lambda e: SpectralEncoding(e.indices[:, lo:hi].contiguous(), e.packed[:, lo:hi].contiguous(),   # noqa: E731
                                        e.scales[:, lo:hi].contiguous())
        parts.append(tri.decode_step_partial(q, sl(k_enc), sl(v_enc), key_pos_start=lo, query_pos_default=S))
    stacked = torch.stack(parts).contiguous()
    merged = torch.empty(B, QH, 128, dtype=torch.float32, device="cuda")
    rc = _lib.lib().akv_lse_merge(stacked.data_ptr(), len(parts), B, QH, 128, None, merged.data_ptr(), _lib.AKV_F32,
                                  merged.stride(0), merged.stride(1), torch.cuda.current_stream().cuda_stream)
    _lib.check(rc, "akv_lse_merge")
    assert (merged - out.float()).abs().max().item() < 1e-3


def test_decode_step_full_context_random_values_vs_oracle():
    """One batch element of the 128K-token workload (131072 keys at positions 0..131071, query at 131072,
    32 query / 8 KV heads) with random keys AND random values, element by element against the oracle:
    covers relative positions from -1 down to -131072."""
    B, S, H, QH = 1, 131072, 8, 32
    tri = _tri(H, QH)
    keys, values, g = _synthetic(B, S, H, seed=11)
    q = torch.randn(B, QH, 128, generator=g).half()
    k_enc, v_enc = tri.encode_kv(keys.cuda(), values.cuda())
    out = tri.decode_step(q.cuda(), k_enc, v_enc).cpu().numpy()
    k_np = tuple(t.cpu().numpy() for t in k_enc)
    v_np = tuple(t.cpu().numpy() for t in v_enc)
    ref = otri.decode_step(q.numpy(), k_np, v_np, tri._theta.cpu().numpy())
    assert np.abs(out - ref).max() < 2e-3


def _paged_case(ctx, H=8, QH=32, seed=11, bt_dtype=torch.int32):
    """Sequences of the given lengths encoded and stored into a SpectralKVCache through shuffled block tables."""
    from aitherkvcache_b200.triattention import SpectralEncoding, SpectralKVCache
    tri = _tri(H, QH)
    B, S_max = len(ctx), max(max(ctx), 1)
    keys, values, g = _synthetic(B, S_max, H, seed=seed)
    q = torch.randn(B, QH, 128, generator=g).half().cuda()
    k_enc, v_enc = tri.encode_kv(keys.cuda(), values.cuda())
    nblk = [(c + 15) // 16 for c in ctx]
    cache = SpectralKVCache(tri.config, max_blocks=sum(nblk) + 3, device="cuda")
    # every block starts as junk that an over-read would pick up
    cache.k_indices.random_(0, 64), cache.v_indices.random_(0, 64)
    cache.k_packed.random_(0, 256), cache.v_packed.random_(0, 256)
    cache.k_scales.fill_(3.0), cache.v_scales.fill_(3.0)
    perm = torch.randperm(sum(nblk) + 3, generator=g)
    bt = torch.zeros(B, max(max(nblk), 1) + 2, dtype=bt_dtype)
    used = 0
    for b, c in enumerate(ctx):
        bt[b, :nblk[b]] = perm[used:used + nblk[b]].to(bt_dtype)
        used += nblk[b]
        if c:
            cache.store_sequence(bt[b], SpectralEncoding(*[t[b, :c] for t in k_enc]), SpectralEncoding(*[t[b, :c] for t in v_enc]))
    return tri, cache, q, bt.cuda(), torch.tensor(ctx, dtype=bt_dtype).cuda(), k_enc, v_enc


@pytest.mark.parametrize("ctx,bt_dtype", (((700, 33, 16, 1), torch.int32), ((2100, 0, 517), torch.int64)))
def test_paged_decode_equals_gather_then_decode(ctx, bt_dtype):
    """Block-table addressing inside the kernel = the reference's fetch_sequence + decode_step per sequence
    (ragged lengths, a partial last block, an empty sequence), and both agree with the oracle."""
    tri, cache, q, bt, cl, k_enc, v_enc = _paged_case(ctx, bt_dtype=bt_dtype)
    out = tri.paged_decode_step(q, cache, bt, cl)
    assert out.shape == (len(ctx), 32, 128) and out.dtype == torch.float32
    for b, c in enumerate(ctx):
        if c == 0:
            assert out[b].abs().max().item() == 0.0
            continue
        kf, vf = cache.fetch_sequence(bt[b], c)
        for got, want in zip(kf + vf, [t[b, :c] for t in k_enc] + [t[b, :c] for t in v_enc]):
            assert torch.equal(got, want)
        dense = tri.decode_step(q[b:b + 1], type(kf)(*[t[None] for t in kf]), type(vf)(*[t[None] for t in vf]))
        assert (out[b] - dense[0]).abs().max().item() < 1e-5
        ref = otri.decode_step(q[b:b + 1].cpu().numpy(), tuple(t[None].cpu().numpy() for t in kf),
                               tuple(t[None].cpu().numpy() for t in vf), tri._theta.cpu().numpy())
        assert np.abs(out[b].cpu().numpy() - ref[0]).max() < 2e-3


def test_paged_decode_query_positions_and_block_ops():
    """Explicit query positions; copy_block / clear_block act on what the kernel reads."""
    ctx = (300, 64)
    tri, cache, q, bt, cl, k_enc, v_enc = _paged_case(ctx, seed=12)
    qpos = torch.tensor([5000, 64], dtype=torch.int64).cuda()
    out = tri.paged_decode_step(q, cache, bt, cl, query_pos=qpos)
    for b, c in enumerate(ctx):
        kf, vf = cache.fetch_sequence(bt[b], c)
        dense = tri.decode_step(q[b:b + 1], type(kf)(*[t[None] for t in kf]), type(vf)(*[t[None] for t in vf]), qpos[b:b + 1])
        assert (out[b] - dense[0]).abs().max().item() < 1e-5
    # fork sequence 1's first block into a spare block and point the table at the copy: same result
    spare = int(set(range(cache.max_blocks)).difference(bt.cpu().flatten().tolist()).pop())
    cache.copy_block(int(bt[1, 0]), spare)
    bt2 = bt.clone()
    bt2[1, 0] = spare
    assert torch.equal(tri.paged_decode_step(q, cache, bt2, cl, query_pos=qpos), out)
    # a cleared block holds zero scales: its 16 tokens score 0 and add nothing to the values
    cache.clear_block(spare)
    out3 = tri.paged_decode_step(q, cache, bt2, cl, query_pos=qpos)
    assert torch.equal(out3[0], out[0]) and not torch.equal(out3[1], out[1])
    stats = cache.memory_stats()
    assert stats["total_tokens"] == 364 and stats["used_blocks"] == 19 + 4


@pytest.mark.parametrize("name,bits,pre", (("c8", 8, True), ("c16", 16, True), ("post4", 4, False), ("post8", 8, False)))
def test_coefficient_modes_and_post_rope_match_reference(name, bits, pre):
    """8-bit and fp16 coefficients, post-RoPE scoring: encoder, decode step and scorer against reference fixtures."""
    from aitherkvcache_b200.triattention import SpectralEncoding, TriAttention, TriAttentionConfig, TrigSeriesScorer
    base, g = load_golden("tri_f12_int4.npz"), load_golden("tri_f12_modes.npz")
    cfg = TriAttentionConfig(head_dim=128, num_freqs=12, coeff_bits=bits, num_kv_heads=2, num_query_heads=8,
                             rope_base=1_000_000.0, pre_rope=pre)
    tri = TriAttention(cfg, device="cuda")
    k_enc, v_enc = tri.encode_kv(torch.from_numpy(base["keys"]).cuda(), torch.from_numpy(base["values"]).cuda())
    for side, enc, x in (("k", k_enc, base["keys"]), ("v", v_enc, base["values"])):
        clear = otri.rank_gap(x, 12) > 0
        assert enc.packed.shape == g[f"{name}_{side}_packed"].shape
        assert np.array_equal(enc.indices.cpu().numpy()[clear], g[f"{name}_{side}_indices"][clear])
        assert np.array_equal(enc.packed.cpu().numpy()[clear].view(np.uint8), g[f"{name}_{side}_packed"][clear].view(np.uint8))
        assert np.array_equal(enc.scales.cpu().numpy()[clear].view(np.uint16), g[f"{name}_{side}_scales"][clear].view(np.uint16))
    gk = SpectralEncoding(*[torch.from_numpy(g[f"{name}_k_{f}"]).cuda() for f in ("indices", "packed", "scales")])
    gv = SpectralEncoding(*[torch.from_numpy(g[f"{name}_v_{f}"]).cuda() for f in ("indices", "packed", "scales")])
    q = torch.from_numpy(base["query"]).cuda()
    qpos, kpos = torch.from_numpy(base["query_pos"]).cuda(), torch.from_numpy(base["key_positions"]).cuda()
    assert np.abs(tri.decode_step(q, gk, gv).cpu().numpy() - g[f"{name}_out_default"]).max() < 2e-3
    assert np.abs(tri.decode_step(q, gk, gv, qpos, kpos).cpu().numpy() - g[f"{name}_out_far"]).max() < 2e-3
    sc = TrigSeriesScorer(cfg, device="cuda").score(q, gk, qpos, kpos)
    assert np.abs(sc.cpu().numpy() - g[f"{name}_scores_far"]).max() < 5e-3
    # the dense reconstruction of the encoder agrees with the oracle's coefficients
    dense = tri.encoder.decode(gk).cpu().numpy()
    k0, k1 = otri.unpack_coeffs(g[f"{name}_k_packed"], g[f"{name}_k_scales"], bits)
    ids = g[f"{name}_k_indices"].astype(np.int64)
    assert np.allclose(np.take_along_axis(dense[..., 0::2], ids, -1), k0, rtol=1e-6, atol=1e-6)     # torch's device division is 1 ulp off before the subtraction
    assert np.allclose(np.take_along_axis(dense[..., 1::2], ids, -1), k1, rtol=1e-6, atol=1e-6)


@pytest.mark.parametrize("bits,pre", ((8, True), (16, True), (4, False), (16, False)))
def test_coefficient_modes_benchmark_heads_vs_oracle(bits, pre):
    """32Q/8KV heads, 1500 keys at the far end of a 128K context, every coefficient format, against the oracle
    (4-bit post-RoPE goes through the record-lane kernel, the others through the dense-tile kernel)."""
    from aitherkvcache_b200.triattention import TriAttention, TriAttentionConfig
    B, S, H, QH = 2, 1500, 8, 32
    cfg = TriAttentionConfig(head_dim=128, num_freqs=12, coeff_bits=bits, num_kv_heads=H, num_query_heads=QH,
                             rope_base=1_000_000.0, pre_rope=pre)
    tri = TriAttention(cfg, device="cuda")
    keys, values, g = _synthetic(B, S, H, seed=21)
    q = torch.randn(B, QH, 128, generator=g).half()
    k_enc, v_enc = tri.encode_kv(keys.cuda(), values.cuda())
    kpos = torch.arange(131072 - S, 131072).unsqueeze(0).expand(B, -1).contiguous()
    qpos = torch.full((B,), 131072)
    out = tri.decode_step(q.cuda(), k_enc, v_enc, qpos.cuda(), kpos.cuda()).cpu().numpy()
    k_np, v_np = tuple(t.cpu().numpy() for t in k_enc), tuple(t.cpu().numpy() for t in v_enc)
    ref = otri.decode_step(q.numpy(), k_np, v_np, tri._theta.cpu().numpy(), qpos.numpy(), kpos.numpy(), bits, pre)
    assert np.abs(out - ref).max() < 2e-3
    oi, op, osc = otri.encode(keys.numpy(), 12, bits)
    clear = otri.rank_gap(keys.numpy(), 12) > 0
    assert np.array_equal(k_np[0][clear], oi[clear]) and np.array_equal(k_np[1][clear].view(np.uint8), op[clear].view(np.uint8))
