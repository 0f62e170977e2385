"""TEST / BASELINE INFRASTRUCTURE - not part of the product path.

Torch-CPU restatement of the reference's own CPU route for the headline workload, used only as
the timed CPU baseline of ``bench.py`` (``--impl reference`` and the ``cpu_baseline`` leg) and
checked against the float64 numpy oracle in ``tests/test_oracle_golden.py``.  Unlike
``oracle/tq.py`` (the parity checker, float64 accumulation) this file keeps the reference's
arithmetic types, so that its speed is representative of the reference on the same host:
float32 ``torch.matmul`` (sgemm on all host threads), ``torch.searchsorted``, fp16 decode
output, ``F.scaled_dot_product_attention`` (GQA as grouped query rows, the cheaper form on a CPU).

Reference lines followed (paths inside the reference project):
  * ``TurboQuant.encode``  aither_kvcache/quantizer.py:122-166 (+ ``_pytorch_encode`` :203-207)
  * ``TurboQuant.decode``  aither_kvcache/quantizer.py:168-197 (+ ``_pytorch_decode`` :209-212)
  * nibble packing         aither_kvcache/packing.py:13-44 (first code in the high nibble)
  * decompress-then-attend aither_kvcache/vllm/hooks.py:303-345 (gather blocks, decode K and V,
    GQA expansion, SDPA); done one sequence at a time so that ragged contexts need no padding
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F


def encode4(x: torch.Tensor, rotation: torch.Tensor, boundaries: torch.Tensor):
    """x [..., D] -> (packed u8 [..., D/2], norms f32 [...]), 4-bit codes."""
    lead, D = x.shape[:-1], x.shape[-1]
    xf = x.reshape(-1, D).float().contiguous()
    norms = xf.norm(dim=-1)
    y = torch.matmul(xf / (norms.unsqueeze(-1) + 1e-10), rotation.T).contiguous()
    idx = torch.searchsorted(boundaries, y).clamp_(0, 15).to(torch.uint8)
    packed = (idx[:, 0::2] << 4) | idx[:, 1::2]
    return packed.reshape(*lead, D // 2), norms.reshape(lead)


def decode4(packed: torch.Tensor, norms: torch.Tensor, rotation: torch.Tensor, centroids: torch.Tensor,
            dtype=torch.float16) -> torch.Tensor:
    """packed u8 [..., D/2], norms [...] -> [..., D] in ``dtype`` (the reference's cache dtype)."""
    lead = norms.shape
    p = packed.reshape(-1, packed.shape[-1])
    idx = torch.stack(((p >> 4), (p & 15)), dim=-1).reshape(p.shape[0], -1).long()
    x_hat = torch.matmul(centroids[idx], rotation) * norms.reshape(-1, 1).float()
    return x_hat.reshape(*lead, rotation.shape[0]).to(dtype)


def paged_decode_attention(query, k_packed, k_norms, v_packed, v_norms, block_tables, context_lens,
                           rotation, centroids, scale=None, block_size=16, sequences=None):
    """One decode step over a tq-t4nc paged cache on the host: for each sequence gather its blocks,
    decode K and V to fp16, expand the KV heads and run SDPA.  Returns fp16 [S, QH, D]."""
    S, QH, D = query.shape
    H = k_packed.shape[2]
    scale = 1.0 / math.sqrt(D) if scale is None else scale
    out = torch.zeros(S, QH, D, dtype=torch.float16)
    for s in (range(S) if sequences is None else sequences):
        ctx = int(context_lens[s])
        if ctx == 0:
            continue
        nb = (ctx + block_size - 1) // block_size
        blocks = block_tables[s, :nb].long()
        k = decode4(k_packed[blocks].reshape(-1, H, D // 2)[:ctx], k_norms[blocks].reshape(-1, H)[:ctx],
                    rotation, centroids)
        v = decode4(v_packed[blocks].reshape(-1, H, D // 2)[:ctx], v_norms[blocks].reshape(-1, H)[:ctx],
                    rotation, centroids)
        # GQA without materialising the expanded heads (the reference uses repeat_interleave, which
        # costs the CPU two more passes over K and V; this form is the faster one): the g query heads
        # of a KV head are g query rows of one non-causal attention over that head's keys
        g = QH // H
        kk = k.float().permute(1, 0, 2).unsqueeze(0)                      # [1, H, ctx, D]
        vv = v.float().permute(1, 0, 2).unsqueeze(0)
        q = query[s].float().reshape(1, H, g, D)
        o = F.scaled_dot_product_attention(q, kk, vv, scale=scale)        # [1, H, g, D]
        out[s] = o.reshape(QH, D).to(torch.float16)
    return out
