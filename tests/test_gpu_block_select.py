"""Block selection on the GPU (akv_block_select_update / akv_block_select) against the reference's
fixture and the oracle, and as the block_selector hook of TQPagedAttention."""
import math

import numpy as np
import pytest
import torch

from conftest import load_golden
from helpers import make_paged_cache, to_cuda
from oracle import block_select as obs
from oracle import tq as otq

pytestmark = pytest.mark.gpu


def _selector(g, ratio=0.25, **kw):
    from aitherkvcache_b200.block_selector import BlockSelector
    return BlockSelector(int(g["num_blocks"]), 2, 64, "cuda", torch.from_numpy(g["centroids"]), select_ratio=ratio,
                         num_sink_blocks=2, num_recent_blocks=2, min_blocks_for_selection=8,
                         rotation=torch.from_numpy(g["rotation"]), **kw)


@pytest.mark.parametrize("idx_dtype", (torch.int32, torch.int64))
def test_representatives_scores_and_selection_match_the_reference(idx_dtype):
    g = load_golden("block_select.npz")
    sel = _selector(g, exact_tail=False)
    assert sel.max_selected == int(g["max_selected"])
    tb = torch.from_numpy(g["token_blocks"]).cuda()
    kp, kn = torch.from_numpy(g["k_packed"]).cuda(), torch.from_numpy(g["k_norms"]).cuda()
    # in two instalments, as prefill then decode would
    half = tb.numel() // 2
    sel.update_reps(tb[:half], None, kp[:half], kn[:half])
    sel.update_reps(tb[half:], None, kp[half:], kn[half:])
    assert np.abs(sel.rep.cpu().numpy() - g["rep"]).max() < 1e-3
    q = torch.from_numpy(g["query"]).cuda()
    bt = torch.from_numpy(g["block_tables"]).to(idx_dtype).cuda()
    cl = torch.from_numpy(g["context_lens"]).to(idx_dtype).cuda()
    scores = torch.empty(bt.shape, dtype=torch.float32, device="cuda")
    fbt, fcl = sel.select_for_query(q, bt, cl, 16, scores_out=scores)
    torch.cuda.synchronize()
    sc = scores.cpu().numpy()
    fin = np.isfinite(g["scores"])
    assert np.array_equal(np.isfinite(sc), fin)
    assert np.abs(sc[fin] - g["scores"][fin]).max() < 2e-2 * max(1.0, np.abs(g["scores"][fin]).max())
    assert fbt.shape == (4, sel.max_selected) and fbt.dtype == torch.int32
    assert np.array_equal(fcl.cpu().numpy(), g["filtered_cl"])
    # selection from the GPU's own scores must equal the oracle's selection from the same scores
    want_bt, want_cl = obs.select_blocks(sc, g["block_tables"], g["context_lens"], 16, sel.max_selected)
    got = fbt.cpu().numpy()
    for s in range(4):
        n = (int(want_cl[s]) + 15) // 16
        assert np.array_equal(got[s, :n], want_bt[s, :n])
    # and the reference's selection wherever the score gap at the cut is clear of the summation-order noise
    for s in range(4):
        n = (int(g["filtered_cl"][s]) + 15) // 16
        same = np.array_equal(got[s, :n], g["filtered_bt"][s, :n])
        if not same:
            srt = np.sort(g["scores"][s][np.isfinite(g["scores"][s])])[::-1]
            k = sel.max_selected
            assert k < len(srt) and abs(srt[k - 5] - srt[min(k + 4, len(srt) - 1)]) < 0.5, "selection differs from the reference"
    # the reference's entry point (already rotated, even / odd halves) gives the same table
    q_rot = torch.matmul(q.float(), torch.from_numpy(g["rotation"]).cuda().T)
    fbt2, fcl2 = sel.select(q_rot[..., 0::2].contiguous(), q_rot[..., 1::2].contiguous(), bt, cl, 4, 16)
    assert torch.equal(fcl2, fcl)


def test_selection_edge_cases_and_clear():
    """Ties (all scores equal: lowest indices win), fewer blocks than kept, exact tail length, clear_blocks."""
    g = load_golden("block_select.npz")
    sel = _selector(g)
    S, B, bs = 3, 40, 16
    bt = torch.arange(S * B, dtype=torch.int32).reshape(S, B).cuda() % int(g["num_blocks"])
    cl = torch.tensor([B * bs - 5, 5 * bs, 0], dtype=torch.int32).cuda()
    q = torch.randn(S, 8, 128, generator=torch.Generator().manual_seed(0)).half().cuda()
    sel._max_selected = 12
    fbt, fcl = sel.select_for_query(q, bt, cl, bs)       # representatives are all zero: every score ties at 0
    torch.cuda.synchronize()
    got, gcl = fbt.cpu().numpy(), fcl.cpu().numpy()
    want_bt, want_cl = obs.select_blocks(np.zeros((S, B)), bt.cpu().numpy(), cl.cpu().numpy(), bs, 12, exact_tail=True)
    assert np.array_equal(gcl, want_cl) and gcl[0] == 11 * bs + 11 and gcl[1] == 5 * bs and gcl[2] == 0
    assert np.array_equal(got[0], want_bt[0])            # sinks 0,1; recents 38,39; then 2..9 by index
    assert np.array_equal(got[1, :5], want_bt[1, :5])
    # clear: write something, clear it, the store is zero again
    tb = torch.from_numpy(g["token_blocks"][:200]).cuda()
    sel.update_reps(tb, None, torch.from_numpy(g["k_packed"][:200]).cuda(), torch.from_numpy(g["k_norms"][:200]).cuda())
    assert sel.rep.abs().max().item() > 0
    sel.clear_blocks(torch.unique(tb))
    assert sel.rep.abs().max().item() == 0 and sel._acc.abs().max().item() == 0 and sel._counts.max().item() == 0


def test_paged_attention_with_block_selector_equals_attention_over_the_selected_blocks():
    """TQPagedAttention(block_selector=...): the output equals plain attention over the filtered table the
    selector returns, and keeping every block reproduces the dense result."""
    from aitherkvcache_b200 import TQPagedAttention, TurboQuant
    from aitherkvcache_b200.block_selector import BlockSelector
    t = load_golden("tq_d128_b4.npz")
    tq = TurboQuant(head_dim=128, bits=4, device="cuda")
    tq.rotation = torch.from_numpy(t["rotation"]).cuda()
    H, QH, bs = 8, 32, 16
    ctx = [2100, 1500]
    d = make_paged_cache(61, ctx, H, 128, 4, t["rotation"], t["boundaries"])
    c = to_cuda(d, ["k_packed", "k_norms", "v_packed", "v_norms", "block_tables", "context_lens"])
    nb = c["k_packed"].shape[0]
    sel = BlockSelector(nb, H, 64, "cuda", tq.centroids, select_ratio=0.3, min_blocks_for_selection=8, rotation=tq.rotation)
    blocks = torch.arange(nb, device="cuda").repeat_interleave(bs)
    sel.update_reps(blocks, None, c["k_packed"].reshape(nb * bs, H, 64), c["k_norms"].reshape(nb * bs, H))
    q = torch.randn(len(ctx), QH, 128, generator=torch.Generator().manual_seed(2)).half().cuda()
    sparse = TQPagedAttention(tq, QH, block_selector=sel).forward(q, c["k_packed"], c["k_norms"], c["v_packed"],
                                                                 c["v_norms"], c["block_tables"], c["context_lens"])
    fbt, fcl = sel.select_for_query(q, c["block_tables"], c["context_lens"], bs)
    assert fbt.shape[1] == sel.max_selected < c["block_tables"].shape[1]
    ref = otq.paged_attention_rotated(q.cpu().numpy(), d["k_packed"], d["k_norms"], d["v_packed"], d["v_norms"],
                                      fbt.cpu().numpy(), fcl.cpu().numpy(), t["rotation"], t["centroids"], 4,
                                      1.0 / math.sqrt(128))
    assert np.abs(sparse.float().cpu().numpy() - ref).max() < 2e-3
    dense = TQPagedAttention(tq, QH).forward(q, c["k_packed"], c["k_norms"], c["v_packed"], c["v_norms"],
                                             c["block_tables"], c["context_lens"])
    sel_all = BlockSelector(nb, H, 64, "cuda", tq.centroids, select_ratio=1.0, rotation=tq.rotation)
    same = TQPagedAttention(tq, QH, block_selector=sel_all).forward(q, c["k_packed"], c["k_norms"], c["v_packed"],
                                                                   c["v_norms"], c["block_tables"], c["context_lens"])
    assert torch.equal(same, dense)
