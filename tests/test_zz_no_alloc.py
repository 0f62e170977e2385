"""The allocation-free attention entry point (akv_tq_paged_attn_static).

A serving engine that has committed all device memory to its KV-cache pool, or a plugin that
must not call into the host program's allocator, cannot provide (or let the library allocate)
the split-K workspace.  This entry point keeps that scratch in a fixed array inside the
library.  The test drives it through the C ABI and compares it with akv_tq_paged_attn on the
same inputs and with the oracle, twice in a row because the array keeps the previous call's
contents.

Collected last on purpose (file name): a run that stops at the first failure has then already
executed every other test.
"""
import ctypes
import math

import numpy as np
import pytest
import torch

from conftest import load_golden
from helpers import make_paged_cache, to_cuda
from oracle import tq as otq

pytestmark = pytest.mark.gpu


def _params(_lib, tq, q, c, out, bits, workspace=None):
    p = _lib.TQAttnParams()
    kp, kn, vp, vn, bt, cl = (c[k] for k in ("k_packed", "k_norms", "v_packed", "v_norms", "block_tables",
                                             "context_lens"))
    p.query, p.q_dtype, p.q_stride_seq, p.q_stride_head = q.data_ptr(), _lib.float_code(q), q.stride(0), q.stride(1)
    p.k_packed, p.kp_stride_blk, p.kp_stride_pos, p.kp_stride_head = kp.data_ptr(), *kp.stride()[:3]
    p.k_norms, p.kn_stride_blk, p.kn_stride_pos, p.kn_stride_head = kn.data_ptr(), *kn.stride()
    p.v_packed, p.vp_stride_blk, p.vp_stride_pos, p.vp_stride_head = vp.data_ptr(), *vp.stride()[:3]
    p.v_norms, p.vn_stride_blk, p.vn_stride_pos, p.vn_stride_head = vn.data_ptr(), *vn.stride()
    p.block_tables, p.bt_dtype, p.bt_stride_seq = bt.data_ptr(), _lib.index_code(bt), bt.stride(0)
    p.context_lens, p.cl_dtype = cl.data_ptr(), _lib.index_code(cl)
    p.num_seqs, p.num_q_heads, p.num_kv_heads, p.head_dim = q.shape[0], q.shape[1], kp.shape[2], q.shape[2]
    p.block_size, p.max_blocks_per_seq, p.num_blocks, p.bits = kp.shape[1], bt.shape[1], kp.shape[0], bits
    p.rotation, p.rotation_t, p.centroids = tq.rotation.data_ptr(), tq.rotation_T.data_ptr(), tq.centroids.data_ptr()
    p.scale = 1.0 / math.sqrt(q.shape[2])
    p.out, p.out_dtype, p.out_stride_seq, p.out_stride_head = out.data_ptr(), _lib.float_code(out), out.stride(0), out.stride(1)
    if workspace is not None:
        p.workspace, p.workspace_bytes = workspace.data_ptr(), workspace.numel()
    p.stream = torch.cuda.current_stream().cuda_stream
    return p


def test_static_scratch_entry_point_matches_workspace_entry_point():
    from aitherkvcache_b200 import TurboQuant, _lib
    L = _lib.lib()
    assert L.akv_tq_paged_attn_static_scratch_bytes() == 8 << 20
    bits, H, QH = 4, 8, 32
    t = load_golden("tq_d128_b4.npz")
    tq = TurboQuant(head_dim=128, bits=bits, device="cuda")
    tq.rotation = torch.from_numpy(t["rotation"]).cuda()
    for call, ctx in enumerate(([900, 17, 2048, 333], [64, 1500, 0, 5])):      # two calls in a row
        d = make_paged_cache(40 + call, ctx, H, 128, bits, t["rotation"], t["boundaries"])
        c = to_cuda(d, ["k_packed", "k_norms", "v_packed", "v_norms", "block_tables", "context_lens"])
        q = torch.randn(len(ctx), QH, 128, generator=torch.Generator().manual_seed(call)).half().cuda()
        ref = torch.full((len(ctx), QH, 128), float("nan"), dtype=torch.float16, device="cuda")
        got = torch.full_like(ref, float("nan"))
        nbytes = L.akv_tq_paged_attn_workspace_bytes(len(ctx), QH, H, 128, bits, 16, c["block_tables"].shape[1], 0)
        ws = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
        _lib.check(L.akv_tq_paged_attn(ctypes.byref(_params(_lib, tq, q, c, ref, bits, ws))), "akv_tq_paged_attn")
        _lib.check(L.akv_tq_paged_attn_static(ctypes.byref(_params(_lib, tq, q, c, got, bits))),
                   "akv_tq_paged_attn_static")
        torch.cuda.synchronize()
        assert torch.isfinite(got).all()
        # the two entry points may pick different split-K kernels; the tolerance is the suite's fp16 one
        assert (got.float() - ref.float()).abs().max().item() <= 2e-3
        want = otq.paged_attention_decode_sdpa(q.cpu().numpy(), d["k_packed"], d["k_norms"], d["v_packed"],
                                               d["v_norms"], d["block_tables"], d["context_lens"], t["rotation"],
                                               t["centroids"], bits, 1.0 / math.sqrt(128))
        assert np.abs(got.float().cpu().numpy() - want.astype(np.float32)).max() <= 2e-3


def test_static_scratch_rejects_oversized_problems():
    from aitherkvcache_b200 import TurboQuant, _lib
    L = _lib.lib()
    tq = TurboQuant(head_dim=128, bits=4, device="cuda")
    S, QH, H = 600, 32, 8          # 19200 rows: even one partial per row exceeds 8 MiB
    kp = torch.zeros(4, 16, H, 64, dtype=torch.uint8, device="cuda")
    kn = torch.zeros(4, 16, H, device="cuda")
    c = {"k_packed": kp, "k_norms": kn, "v_packed": kp, "v_norms": kn,
         "block_tables": torch.zeros(S, 2, dtype=torch.int32, device="cuda"),
         "context_lens": torch.zeros(S, dtype=torch.int32, device="cuda")}
    q = torch.zeros(S, QH, 128, dtype=torch.float16, device="cuda")
    out = torch.zeros_like(q)
    rc = L.akv_tq_paged_attn_static(ctypes.byref(_params(_lib, tq, q, c, out, 4)))
    assert rc == -3
    msg = L.akv_last_error().decode()
    assert "scratch" in msg and "akv_tq_paged_attn" in msg
    # explicit split size that needs more than the array holds is rejected too
    S2 = 64
    c2 = dict(c, block_tables=torch.zeros(S2, 4096, dtype=torch.int32, device="cuda"),
              context_lens=torch.zeros(S2, dtype=torch.int32, device="cuda"))
    q2 = torch.zeros(S2, QH, 128, dtype=torch.float16, device="cuda")
    p = _params(_lib, tq, q2, c2, torch.zeros_like(q2), 4)
    p.blocks_per_split = 8
    assert L.akv_tq_paged_attn_static(ctypes.byref(p)) == -3
    p.blocks_per_split = 0          # automatic: grows the split until it fits
    assert L.akv_tq_paged_attn_static(ctypes.byref(p)) == 0
    torch.cuda.synchronize()
