"""Generate the golden fixtures in this directory from the unmodified reference.

Run once, in a container that has the reference checked out:

    AKV_REFERENCE=/path/to/aitherkvcache python tests/golden/make_golden.py

It imports ``aither_kvcache`` from that path, runs its CPU torch code on small
seeded inputs and stores inputs, tables and outputs as compressed .npz files.
The test-suite and the GPU box only ever read the .npz files.
"""
import math
import os
import sys

import numpy as np
import torch

REF = os.environ.get("AKV_REFERENCE")
if not REF:
    sys.exit("set AKV_REFERENCE to a checkout of the reference (Aitherium/aitherkvcache)")
sys.path.insert(0, REF)
HERE = os.path.dirname(os.path.abspath(__file__))

from aither_kvcache.quantizer import TurboQuant                      # noqa: E402
from aither_kvcache.fused_attention import TQPagedAttentionRef       # noqa: E402
from aither_kvcache.fused_kv_update import _pytorch_tq4_kv_update    # noqa: E402
from aither_kvcache.hybrid_quantizer import HybridTurboQuant         # noqa: E402
from aither_kvcache.triattention.config import TriAttentionConfig    # noqa: E402
from aither_kvcache.triattention.attention import TriAttention       # noqa: E402

torch.set_num_threads(8)


def save(name, **arrs):
    out = {k: (v.numpy() if isinstance(v, torch.Tensor) else np.asarray(v)) for k, v in arrs.items()}
    np.savez_compressed(os.path.join(HERE, name), **out)
    print(name, {k: (v.shape, str(v.dtype)) for k, v in out.items()})


def special_vectors(d):
    g = torch.Generator().manual_seed(7)
    rows = [torch.zeros(d), torch.ones(d) * 1e-4, torch.ones(d) * 200.0]
    e = torch.zeros(d); e[3] = 1.0; rows.append(e)
    e = torch.zeros(d); e[d - 1] = -5.0; rows.append(e)
    rows.append(torch.randn(d, generator=g) * 1e-3)
    rows.append(torch.randn(d, generator=g) * 50.0)
    return torch.stack(rows).half()


def uniform_codec():
    for d in (128, 64):
        for bits in (4, 3, 2):
            tq = TurboQuant(head_dim=d, bits=bits, device="cpu")
            torch.manual_seed(0)
            n = 1024 if d == 128 else 256
            x = torch.cat([torch.randn(4, 1024, 8, d).half().reshape(-1, d)[:n], special_vectors(d)])
            packed, norms = tq.encode(x)
            dec = tq.decode(packed, norms)
            xb = torch.randn(257, d, generator=torch.Generator().manual_seed(3)).bfloat16()
            pb, nb = tq.encode(xb)
            xf = torch.randn(129, d, generator=torch.Generator().manual_seed(4)) * 3.0
            pf, nf = tq.encode(xf)
            save(f"tq_d{d}_b{bits}.npz", x=x, packed=packed, norms=norms, decoded=dec,
                 rotation=tq.rotation, centroids=tq.centroids, boundaries=tq.boundaries_inner,
                 x_bf16_as_f32=xb.float(), packed_bf16=pb, norms_bf16=nb,
                 x_f32=xf, packed_f32=pf, norms_f32=nf)


def paged_write():
    tq = TurboQuant(head_dim=128, bits=4, device="cpu")
    g = torch.Generator().manual_seed(11)
    T, H, bs, nblk = 70, 2, 16, 6
    x = torch.randn(T, H, 128, generator=g).half()
    slots = torch.randperm(nblk * bs + 24, generator=g)[:T].to(torch.int64)   # some beyond the cache
    slots[5] = -1
    slots[33] = -1
    outp = torch.full((nblk, bs, H, 64), 0xAB, dtype=torch.uint8)
    outn = torch.full((nblk, bs, H), -7.0)
    _pytorch_tq4_kv_update(x, slots, outp, outn, tq.rotation, tq.boundaries_inner, bs, nblk)
    save("paged_write_b4.npz", x=x, slot_mapping=slots, out_packed=outp, out_norms=outn,
         block_size=bs, max_blocks=nblk)


def paged_attention():
    for bits in (4, 3, 2):
        tq = TurboQuant(head_dim=128, bits=bits, device="cpu")
        g = torch.Generator().manual_seed(20 + bits)
        H, QH, bs = 2, 8, 16
        ctx = torch.tensor([0, 1, 15, 16, 17, 48, 100], dtype=torch.int64)
        nblk_seq = [(int(c) + bs - 1) // bs for c in ctx]
        total = sum(nblk_seq) + 3
        perm = torch.randperm(total, generator=g)
        maxb = max(nblk_seq) + 1
        bt = torch.zeros(len(ctx), maxb, dtype=torch.int32)
        p = 0
        for s, n in enumerate(nblk_seq):
            bt[s, :n] = perm[p:p + n].to(torch.int32)
            p += n
        k = torch.randn(total, bs, H, 128, generator=g).half() * 1.5
        v = torch.randn(total, bs, H, 128, generator=g).half()
        kp, kn = tq.encode(k)
        vp, vn = tq.encode(v)
        q = torch.randn(len(ctx), QH, 128, generator=g).half()
        ref = TQPagedAttentionRef(tq.rotation, tq.centroids, 1.0 / math.sqrt(128), H, QH, 128, bs, bits=bits)
        out = ref.forward(q, kp, kn, vp, vn, bt, ctx)
        # decode -> fp16 -> SDPA, per sequence
        out2 = torch.zeros_like(out)
        for s in range(len(ctx)):
            c = int(ctx[s])
            if c == 0:
                continue
            blocks = bt[s, :nblk_seq[s]].long()
            K = tq.decode(kp[blocks].reshape(-1, H, kp.shape[-1])[:c], kn[blocks].reshape(-1, H)[:c])
            V = tq.decode(vp[blocks].reshape(-1, H, vp.shape[-1])[:c], vn[blocks].reshape(-1, H)[:c])
            Kh = K.permute(1, 0, 2).repeat_interleave(QH // H, dim=0)
            Vh = V.permute(1, 0, 2).repeat_interleave(QH // H, dim=0)
            o = torch.nn.functional.scaled_dot_product_attention(
                q[s].unsqueeze(1).float(), Kh.float(), Vh.float(), scale=1.0 / math.sqrt(128))
            out2[s] = o.squeeze(1).half()
        save(f"paged_attn_b{bits}.npz", query=q, k_packed=kp, k_norms=kn, v_packed=vp, v_norms=vn,
             block_tables=bt, context_lens=ctx, out_rotated_domain=out, out_decode_sdpa=out2)


def hybrid():
    for mode in ("tq35", "tq25"):
        h = HybridTurboQuant(head_dim=128, mode=mode, device="cpu")
        h.calibrate_uniform()
        g = torch.Generator().manual_seed(0)
        x = torch.cat([torch.randn(8, 4096, 8, 128, generator=g).half().reshape(-1, 128)[:768],
                       special_vectors(128)])
        packed = h.encode(x)
        dec = h.decode(packed)
        save(f"hybrid_{mode}.npz", x=x, packed=packed, decoded=dec,
             had0=h._g0_had_signs, had1=h._g1_had_signs, qjl0=h._g0_qjl_signs, qjl1=h._g1_qjl_signs,
             cent0=h._g0_centroids, bnd0=h._g0_boundaries, cent1=h._g1_centroids, bnd1=h._g1_boundaries,
             qjl_scale=np.array([h._g0_qjl_scale, h._g1_qjl_scale]))


def tri():
    cfg = TriAttentionConfig(head_dim=128, num_freqs=12, coeff_bits=4, num_kv_heads=2,
                             num_query_heads=8, rope_base=1_000_000.0)
    tri = TriAttention(cfg, device="cpu")
    g = torch.Generator().manual_seed(2)
    B, S, H = 2, 200, 2
    s_i = torch.exp(-torch.arange(64, dtype=torch.float32) / 16.0)
    scale = torch.stack([s_i[torch.randperm(64, generator=g)] for _ in range(H)])      # [H,64]
    keys = (torch.randn(B, S, H, 64, 2, generator=g) * scale[None, None, :, :, None]).reshape(B, S, H, 128).half()
    values = torch.randn(B, S, H, 128, generator=g).half()
    q = torch.randn(B, 8, 128, generator=g).half()
    k_enc, v_enc = tri.encode_kv(keys, values)
    out_default = tri.decode_step(q, k_enc, v_enc)
    qpos = torch.tensor([131072, 70000])
    kpos = torch.stack([torch.arange(131072 - S, 131072), torch.arange(0, 3 * S, 3)])
    out_far = tri.decode_step(q, k_enc, v_enc, qpos, kpos)
    sc_far = tri.scorer.score(q, k_enc, qpos, kpos)
    save("tri_f12_int4.npz", keys=keys, values=values, query=q,
         k_indices=k_enc.indices, k_packed=k_enc.packed, k_scales=k_enc.scales,
         v_indices=v_enc.indices, v_packed=v_enc.packed, v_scales=v_enc.scales,
         theta=tri._theta, out_default=out_default, query_pos=qpos, key_positions=kpos,
         out_far=out_far, scores_far=sc_far)


def tri_modes():
    """The encoder's other coefficient formats (8-bit codes, plain fp16) and post-RoPE scoring, on the
    inputs of tri_f12_int4.npz (keys, values, query and positions are read from there): encodings, one decode step far from the keys, and the pre-softmax scores."""
    g = torch.Generator().manual_seed(2)
    B, S, H = 2, 200, 2
    s_i = torch.exp(-torch.arange(64, dtype=torch.float32) / 16.0)
    scale = torch.stack([s_i[torch.randperm(64, generator=g)] for _ in range(H)])
    keys = (torch.randn(B, S, H, 64, 2, generator=g) * scale[None, None, :, :, None]).reshape(B, S, H, 128).half()
    values = torch.randn(B, S, H, 128, generator=g).half()
    q = torch.randn(B, 8, 128, generator=g).half()
    qpos = torch.tensor([131072, 70000])
    kpos = torch.stack([torch.arange(131072 - S, 131072), torch.arange(0, 3 * S, 3)])
    out = {}
    for name, bits, pre in (("c8", 8, True), ("c16", 16, True), ("post4", 4, False), ("post8", 8, False)):
        cfg = TriAttentionConfig(head_dim=128, num_freqs=12, coeff_bits=bits, num_kv_heads=2,
                                 num_query_heads=8, rope_base=1_000_000.0, pre_rope=pre)
        tri = TriAttention(cfg, device="cpu")
        k_enc, v_enc = tri.encode_kv(keys, values)
        out.update({f"{name}_k_indices": k_enc.indices, f"{name}_k_packed": k_enc.packed, f"{name}_k_scales": k_enc.scales,
                    f"{name}_v_indices": v_enc.indices, f"{name}_v_packed": v_enc.packed, f"{name}_v_scales": v_enc.scales,
                    f"{name}_out_far": tri.decode_step(q, k_enc, v_enc, qpos, kpos),
                    f"{name}_out_default": tri.decode_step(q, k_enc, v_enc),
                    f"{name}_scores_far": tri.scorer.score(q, k_enc, qpos, kpos)})
    base = np.load(os.path.join(HERE, "tri_f12_int4.npz"))      # same seeded inputs: stored once, there
    assert np.array_equal(base["keys"], keys.numpy()) and np.array_equal(base["query"], q.numpy())
    save("tri_f12_modes.npz", **out)


def block_select():
    """The reference's BlockSelector on a seeded paged cache: representatives from the packed keys,
    scores, filtered tables (ties are improbable with random data)."""
    from aither_kvcache.block_selector import BlockSelector
    H, QH, D, bs = 2, 8, 128, 16
    tq = TurboQuant(head_dim=D, bits=4, device="cpu")
    g = torch.Generator().manual_seed(5)
    ctx = [1500, 1043, 70, 2000]
    nblk = [(c + bs - 1) // bs for c in ctx]
    total = sum(nblk) + 3
    perm = torch.randperm(total, generator=g)
    bt = torch.zeros(len(ctx), max(nblk), dtype=torch.int64)
    p = 0
    tok_blocks = []
    for s, n in enumerate(nblk):
        bt[s, :n] = perm[p:p + n]
        p += n
        tok_blocks.append(bt[s, :n].repeat_interleave(bs)[:ctx[s]])
    tok_blocks = torch.cat(tok_blocks)
    N = tok_blocks.numel()
    # keys with a per-block drift so that block means differ
    drift = torch.randn(total, H, D, generator=g)
    k = (torch.randn(N, H, D, generator=g) + 1.5 * drift[tok_blocks]).half()
    kp, kn = tq.encode(k)
    sel = BlockSelector(total, H, D // 2, torch.device("cpu"), tq.centroids, select_ratio=0.25,
                        num_sink_blocks=2, num_recent_blocks=2, min_blocks_for_selection=8)
    sel.update_reps(tok_blocks, torch.zeros(N, dtype=torch.int64), kp, kn)
    q = torch.randn(len(ctx), QH, D, generator=g).half()
    q_rot = torch.matmul(q.float(), tq.rotation.T)
    from aither_kvcache.block_selector import score_blocks
    cl = torch.tensor(ctx, dtype=torch.int64)
    scores = score_blocks(q_rot[..., 0::2].contiguous(), q_rot[..., 1::2].contiguous(), sel._rep_cache.rep_even,
                          sel._rep_cache.rep_odd, bt, cl, QH // H, bs)
    fbt, fcl = sel.select(q_rot[..., 0::2].contiguous(), q_rot[..., 1::2].contiguous(), bt, cl, QH // H, bs)
    rep = torch.stack((sel._rep_cache.rep_even, sel._rep_cache.rep_odd), dim=-1).reshape(total, H, D)
    save("block_select.npz", k_packed=kp, k_norms=kn, token_blocks=tok_blocks, block_tables=bt, context_lens=cl,
         query=q, rotation=tq.rotation, centroids=tq.centroids, rep=rep, scores=scores, filtered_bt=fbt,
         filtered_cl=fcl, max_selected=np.array(sel.max_selected), num_blocks=np.array(total))


if __name__ == "__main__":
    if len(sys.argv) > 1:          # regenerate only the named fixtures, e.g. `make_golden.py block_select`
        for name in sys.argv[1:]:
            globals()[name]()
        sys.exit(0)
    block_select()
    uniform_codec()
    paged_write()
    paged_attention()
    hybrid()
    tri()
    tri_modes()
