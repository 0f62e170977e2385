"""Pin the numpy oracle against fixtures produced by the unmodified reference."""
import math

import numpy as np
import pytest

from oracle import tq as otq
from oracle import hybrid as ohy
from oracle import tri as otri
from conftest import load_golden

BITS = (4, 3, 2)


@pytest.mark.parametrize("d", (128, 64))
@pytest.mark.parametrize("bits", BITS)
def test_codebook_matches_reference(d, bits):
    g = load_golden(f"tq_d{d}_b{bits}.npz")
    c, b = otq.codebook(d, bits)
    assert np.array_equal(c.view(np.uint32), g["centroids"].view(np.uint32))
    assert np.array_equal(b.view(np.uint32), g["boundaries"].view(np.uint32))


@pytest.mark.parametrize("bits", BITS)
def test_pack_roundtrip(bits):
    rng = np.random.default_rng(bits)
    idx = rng.integers(0, 1 << bits, size=(5, 7, 128), dtype=np.uint8)
    p = otq.pack(idx, bits)
    assert p.shape[-1] == otq.packed_size(128, bits) == {4: 64, 3: 48, 2: 32}[bits]
    assert np.array_equal(otq.unpack(p, 128, bits), idx)


def _ordered(h):
    """fp16 bit patterns mapped to integers that are monotone in the value."""
    i = h.view(np.int16).astype(np.int32)
    return np.where(i < 0, -(i & 0x7FFF), i)


def _codes_equal_outside_margin(packed, ref_packed, margin, d, bits):
    a = otq.unpack(packed, d, bits)
    b = otq.unpack(ref_packed, d, bits)
    diff = a != b
    near = margin < 1e-6
    assert not (diff & ~near).any(), "code differs away from any boundary"
    return diff.mean(), near.mean()


@pytest.mark.parametrize("d", (128, 64))
@pytest.mark.parametrize("bits", BITS)
@pytest.mark.parametrize("which", ("", "_bf16", "_f32"))
def test_encode_matches_reference(d, bits, which):
    g = load_golden(f"tq_d{d}_b{bits}.npz")
    x = g["x"] if which == "" else g["x_bf16_as_f32"] if which == "_bf16" else g["x_f32"]
    packed, norms, margin = otq.encode(x, g["rotation"], g["boundaries"], bits, return_margin=True)
    ref_p, ref_n = (g["packed"], g["norms"]) if which == "" else (g[f"packed{which}"], g[f"norms{which}"])
    assert np.array_equal(norms.view(np.uint32), ref_n.view(np.uint32)), "norms must be bit-equal"
    mism, near = _codes_equal_outside_margin(packed, ref_p, margin, d, bits)
    assert mism <= near
    if which == "":
        # the last 7 rows are hand-made (zero vector, one-hot, ...): their rotated
        # coordinates can sit exactly on the 0.0 boundary.  The random rows must not.
        assert (margin[:-7] < 1e-6).mean() <= 2e-4
        zero_row = otq.unpack(packed[-7], d, bits)
        assert (zero_row == (1 << bits) // 2 - 1).all(), "y == boundary goes to the lower code"
        assert np.array_equal(packed[-7:], ref_p[-7:])


@pytest.mark.parametrize("d", (128, 64))
@pytest.mark.parametrize("bits", BITS)
def test_decode_matches_reference(d, bits):
    g = load_golden(f"tq_d{d}_b{bits}.npz")
    dec = otq.decode(g["packed"], g["norms"], g["rotation"], g["centroids"], bits)
    ref = g["decoded"]
    fin = np.isfinite(ref.astype(np.float32))
    assert np.array_equal(np.isfinite(dec.astype(np.float32)), fin)
    # the reference's sgemm and the float64 product may round differently to fp16: allow 1 fp16 ulp
    # (near a zero crossing the float32 sum itself carries ~1e-7 * norm of noise, which is many
    # fp16 ulps of a tiny value, so those are judged on absolute error instead)
    ulp = np.abs(_ordered(dec[fin]) - _ordered(ref[fin]))
    abs_err = np.abs(dec.astype(np.float32) - ref.astype(np.float32))[fin]
    noise = (1e-6 * np.broadcast_to(g["norms"][:, None], ref.shape))[fin]
    assert ((ulp <= 1) | (abs_err <= noise)).all()
    assert (ulp != 0).mean() < 2e-3


def test_paged_write_matches_reference():
    g = load_golden("paged_write_b4.npz")
    t = load_golden("tq_d128_b4.npz")
    outp = np.full_like(g["out_packed"], 0xAB)
    outn = np.full_like(g["out_norms"], -7.0)
    otq.paged_kv_update(g["x"], g["slot_mapping"], outp, outn, t["rotation"], t["boundaries"], 4,
                        int(g["block_size"]), int(g["max_blocks"]))
    assert np.array_equal(outn.view(np.uint32), g["out_norms"].view(np.uint32))
    assert (outp != g["out_packed"]).mean() < 1e-4
    untouched = g["out_norms"] == -7.0
    assert untouched.any() and (outp[untouched] == 0xAB).all()


@pytest.mark.parametrize("bits", BITS)
def test_paged_attention_matches_reference(bits):
    g = load_golden(f"paged_attn_b{bits}.npz")
    t = load_golden(f"tq_d128_b{bits}.npz")
    args = (g["query"], g["k_packed"], g["k_norms"], g["v_packed"], g["v_norms"],
            g["block_tables"], g["context_lens"], t["rotation"], t["centroids"], bits, 1.0 / math.sqrt(128))
    rot = otq.paged_attention_rotated(*args)
    assert np.abs(rot - g["out_rotated_domain"].astype(np.float64)).max() < 2e-3
    assert (rot[0] == 0).all(), "zero context gives zeros"
    sdpa = otq.paged_attention_decode_sdpa(*args)
    assert np.abs(sdpa.astype(np.float64) - g["out_decode_sdpa"].astype(np.float64)).max() < 2e-3
    assert np.abs(rot - g["out_decode_sdpa"].astype(np.float64)).max() < 2e-3


def _hybrid_tables(g, mode):
    own = ohy.Tables(128, mode, g["had0"], g["had1"], g["qjl0"], g["qjl1"])
    for k, (c, b) in enumerate(own.cb):
        # the restated Lloyd iteration agrees to float32 rounding; the middle boundary is a
        # float64 sum that cancels to ~1e-17, whose sign depends on the summation order
        assert np.abs(c - g[f"cent{k}"]).max() < 1e-7
        assert np.abs(b - g[f"bnd{k}"]).max() < 1e-7
    t = ohy.Tables(128, mode, g["had0"], g["had1"], g["qjl0"], g["qjl1"],
                   codebooks=[(g["cent0"], g["bnd0"]), (g["cent1"], g["bnd1"])])
    assert np.allclose(t.qjl_scale, g["qjl_scale"], rtol=0, atol=0)
    return t


@pytest.mark.parametrize("mode", ("tq35", "tq25"))
def test_hybrid_encode_bytes_equal(mode):
    g = load_golden(f"hybrid_{mode}.npz")
    t = _hybrid_tables(g, mode)
    assert t.packed_dim == g["packed"].shape[-1] == {"tq35": 64, "tq25": 44}[mode]
    packed = ohy.encode(g["x"], t)
    assert np.array_equal(packed, g["packed"])


@pytest.mark.parametrize("mode", ("tq35", "tq25"))
def test_hybrid_decode_matches(mode):
    g = load_golden(f"hybrid_{mode}.npz")
    t = _hybrid_tables(g, mode)
    dec = ohy.decode(g["packed"], t)
    ref = g["decoded"]
    fin = np.isfinite(ref)
    assert np.array_equal(dec[fin].view(np.uint32), ref[fin].view(np.uint32))


def test_tri_encode_matches():
    g = load_golden("tri_f12_int4.npz")
    assert np.abs(otri.rope_frequencies(128) / g["theta"] - 1).max() < 2e-7
    for side, x in (("k", g["keys"]), ("v", g["values"])):
        idx, packed, scales = otri.encode(x, 12)
        clear = otri.rank_gap(x, 12) > 0
        assert clear.mean() > 0.999
        assert np.array_equal(idx[clear], g[f"{side}_indices"][clear])
        assert np.array_equal(packed[clear], g[f"{side}_packed"][clear])
        assert np.array_equal(scales[clear].view(np.uint16), g[f"{side}_scales"][clear].view(np.uint16))


def test_tri_decode_step_matches():
    g = load_golden("tri_f12_int4.npz")
    k_enc = (g["k_indices"], g["k_packed"], g["k_scales"])
    v_enc = (g["v_indices"], g["v_packed"], g["v_scales"])
    out = otri.decode_step(g["query"], k_enc, v_enc, g["theta"])
    assert np.abs(out - g["out_default"]).max() < 1e-4
    sc = otri.scores(g["query"], *k_enc, g["theta"], g["query_pos"], g["key_positions"])
    assert np.abs(sc - g["scores_far"]).max() < 1e-4
    out = otri.decode_step(g["query"], k_enc, v_enc, g["theta"], g["query_pos"], g["key_positions"])
    assert np.abs(out - g["out_far"]).max() < 1e-4


def test_torch_cpu_baseline_matches_the_oracle():
    """oracle/tq_torch.py (the timed CPU baseline: float32 torch ops like the reference) against the
    float64 numpy oracle: codes equal outside the boundary window, decode within one fp16 ulp, attention
    within the benchmark tolerance."""
    import math
    import torch
    from helpers import make_paged_cache
    from oracle import tq_torch as ott
    t = load_golden("tq_d128_b4.npz")
    R, cent, bnd = t["rotation"], t["centroids"], t["boundaries"]
    T = lambda a: torch.from_numpy(np.ascontiguousarray(a))     # noqa: E731
    x = torch.randn(300, 8, 128, generator=torch.Generator().manual_seed(0)).half()
    p_np, n_np, margin = otq.encode(x.numpy(), R, bnd, 4, return_margin=True)
    p_t, n_t = ott.encode4(x, T(R), T(bnd))
    diff = otq.unpack(p_t.numpy(), 128, 4) != otq.unpack(p_np, 128, 4)
    assert not (diff & ~(margin.reshape(diff.shape) < 1e-6)).any()
    assert np.abs(n_t.numpy() - n_np).max() <= 1e-6 * np.abs(n_np).max()
    d_np = otq.decode(p_np, n_np, R, cent, 4).astype(np.float32)
    d_t = ott.decode4(T(p_np), T(n_np), T(R), T(cent)).float().numpy()
    assert (np.abs(d_t - d_np) <= np.maximum(np.abs(d_np) * 2.0 ** -10, 1e-5)).all()
    ctx = [700, 33, 0, 90]
    d = make_paged_cache(3, ctx, 8, 128, 4, R, bnd)
    q = torch.randn(len(ctx), 32, 128, generator=torch.Generator().manual_seed(1)).half()
    ref = otq.paged_attention_decode_sdpa(q.numpy(), d["k_packed"], d["k_norms"], d["v_packed"], d["v_norms"],
                                          d["block_tables"], d["context_lens"], R, cent, 4, 1 / math.sqrt(128))
    out = ott.paged_decode_attention(q, T(d["k_packed"]), T(d["k_norms"]), T(d["v_packed"]), T(d["v_norms"]),
                                     T(d["block_tables"]), T(d["context_lens"]), T(R), T(cent))
    assert np.abs(out.float().numpy() - ref.astype(np.float32)).max() < 2e-3


def test_block_select_oracle_matches_the_reference():
    """oracle/block_select.py against the reference's own representatives, scores and filtered tables."""
    from oracle import block_select as obs
    g = load_golden("block_select.npz")
    codes = otq.unpack(g["k_packed"], 128, 4)
    rep = obs.representatives(g["token_blocks"], codes, g["k_norms"], g["centroids"], int(g["num_blocks"]))
    assert np.abs(rep - g["rep"]).max() < 1e-4
    q_rot = g["query"].astype(np.float32) @ g["rotation"].T
    sc = obs.score_blocks(q_rot, rep, g["block_tables"], g["context_lens"], 4, 16)
    fin = np.isfinite(g["scores"])
    assert np.array_equal(np.isfinite(sc), fin)
    assert np.abs(sc[fin] - g["scores"][fin]).max() < 1e-2 * max(1.0, np.abs(g["scores"][fin]).max())
    fbt, fcl = obs.select_blocks(g["scores"], g["block_tables"], g["context_lens"], 16, int(g["max_selected"]))
    assert np.array_equal(fcl, g["filtered_cl"])
    # rows are compared as far as the filtered context reaches (beyond it torch.topk's choice among
    # equal -inf entries is unspecified)
    for s in range(fbt.shape[0]):
        n = (int(fcl[s]) + 15) // 16
        assert np.array_equal(fbt[s, :n], g["filtered_bt"][s, :n])


@pytest.mark.parametrize("name,bits,pre", (("c8", 8, True), ("c16", 16, True), ("post4", 4, False), ("post8", 8, False)))
def test_tri_oracle_coefficient_modes_and_post_rope(name, bits, pre):
    """oracle/tri.py against the reference's 8-bit / fp16 coefficient formats and post-RoPE scoring."""
    from oracle import tri as otri
    base, g = load_golden("tri_f12_int4.npz"), load_golden("tri_f12_modes.npz")
    for side, x in (("k", base["keys"]), ("v", base["values"])):
        idx, packed, scales = otri.encode(x, 12, bits)
        clear = otri.rank_gap(x, 12) > 0
        assert np.array_equal(idx[clear], g[f"{name}_{side}_indices"][clear])
        assert np.array_equal(packed[clear].view(np.uint8), g[f"{name}_{side}_packed"][clear].view(np.uint8))
        assert np.array_equal(scales[clear].view(np.uint16), g[f"{name}_{side}_scales"][clear].view(np.uint16))
    k_enc = tuple(g[f"{name}_k_{f}"] for f in ("indices", "packed", "scales"))
    v_enc = tuple(g[f"{name}_v_{f}"] for f in ("indices", "packed", "scales"))
    theta = base["theta"]
    sc = otri.scores(base["query"], *k_enc, theta, base["query_pos"], base["key_positions"], bits, pre)
    assert np.abs(sc - g[f"{name}_scores_far"]).max() < 2e-4
    out = otri.decode_step(base["query"], k_enc, v_enc, theta, base["query_pos"], base["key_positions"], bits, pre)
    assert np.abs(out - g[f"{name}_out_far"]).max() < 2e-5
    out = otri.decode_step(base["query"], k_enc, v_enc, theta, coeff_bits=bits, pre_rope=pre)
    assert np.abs(out - g[f"{name}_out_default"]).max() < 2e-5
