"""Hybrid split-group quantiser (tq35 / tq25) with a 1-bit QJL residual sketch.

Host-side mirror of the reference's ``aither_kvcache/hybrid_quantizer.py``
(``MODE_CONFIGS`` :52-65, ``GroupLayout`` / ``HybridLayout`` :72-123,
``dimension_aware_codebook`` :241-303, ``HybridTurboQuant`` :449-1067): same
constructor, calibration methods, ``encode`` -> one uint8 tensor, ``decode`` ->
float32.  Sign vectors and codebooks are built on the host exactly as the reference
builds them (seeded CPU generator; float64 Lloyd iteration); the per-vector work runs
in ``akv_hybrid_encode`` / ``akv_hybrid_decode`` / ``akv_hybrid_paged_attn``.
The kernels cover head_dim 128.
"""
from __future__ import annotations

import os
import ctypes
import functools
import math
from dataclasses import dataclass
from typing import Dict, Optional, Tuple

import torch

from . import _lib

__all__ = ["HybridTurboQuant", "HybridLayout", "GroupLayout", "HybridPagedAttention"]

# mode -> (share of dims in the outlier group, (outlier bits, regular bits) incl. the QJL bit)
MODE_CONFIGS: Dict[str, dict] = {
    "tq35": {"outlier_ratio": 0.50, "group_bits": (4, 3)},
    "tq25": {"outlier_ratio": 0.25, "group_bits": (3, 2)},
}


@dataclass(frozen=True)
class GroupLayout:
    dim: int
    mse_bits: int
    mse_packed_bytes: int
    qjl_packed_bytes: int
    norm_bytes: int
    residual_norm_bytes: int
    total_bytes: int


@dataclass(frozen=True)
class HybridLayout:
    group0: GroupLayout
    group1: GroupLayout
    packed_dim: int


def _make_group_layout(dim: int, mse_bits: int) -> GroupLayout:
    mse, qjl = math.ceil(dim * mse_bits / 8), math.ceil(dim / 8)
    return GroupLayout(dim, mse_bits, mse, qjl, 2, 2, mse + qjl + 4)


def _make_hybrid_layout(head_dim: int, mode: str) -> HybridLayout:
    cfg = MODE_CONFIGS[mode]
    b0, b1 = cfg["group_bits"]
    g0 = round(head_dim * cfg["outlier_ratio"])
    l0, l1 = _make_group_layout(g0, b0 - 1), _make_group_layout(head_dim - g0, b1 - 1)
    return HybridLayout(l0, l1, l0.total_bytes + l1.total_bytes)


@functools.cache
def dimension_aware_codebook(dim: int, bits: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """Lloyd-Max quantiser for one coordinate of a uniform point on S^{dim-1}
    (density ~ (1-x^2)^((dim-3)/2)), iterated on a 10 000-point float64 grid.
    Returns float32 (centroids[2^bits], boundaries[2^bits-1])."""
    levels = 1 << bits
    grid = torch.linspace(-0.999, 0.999, 10000, dtype=torch.float64)
    expo = (dim - 3) / 2.0
    base = 1.0 - grid * grid
    weights = base.pow(expo) if expo >= 0 else base.clamp(min=1e-30).pow(expo)
    weights = weights / weights.sum()
    cent = torch.linspace(grid[0].item(), grid[-1].item(), levels, dtype=torch.float64)
    for _ in range(200):
        bounds = (cent[:-1] + cent[1:]) / 2.0
        assign = torch.searchsorted(bounds, grid).clamp(0, levels - 1)
        new = torch.zeros_like(cent)
        for k in range(levels):
            sel = assign == k
            w = weights[sel]
            new[k] = (grid[sel] * w).sum() / w.sum() if w.sum() > 1e-30 else cent[k]
        converged = (cent - new).abs().max() < 1e-10
        cent = new
        if converged:
            break
    return cent.float(), ((cent[:-1] + cent[1:]) / 2.0).float()


def pack_multibit(indices: torch.Tensor, bits: int) -> torch.Tensor:
    """MSB-first bit stream of ``bits``-wide codes along the last dim -> uint8."""
    dim = indices.shape[-1]
    shifts = torch.arange(bits - 1, -1, -1, device=indices.device)
    stream = ((indices.to(torch.int32)[..., None] >> shifts) & 1).reshape(*indices.shape[:-1], dim * bits)
    pad = (-stream.shape[-1]) % 8
    if pad:
        stream = torch.nn.functional.pad(stream, (0, pad))
    weights = (1 << torch.arange(7, -1, -1, device=indices.device)).to(torch.int32)
    return (stream.reshape(*indices.shape[:-1], -1, 8) * weights).sum(-1).to(torch.uint8)


def unpack_multibit(packed: torch.Tensor, dim: int, bits: int) -> torch.Tensor:
    shifts = torch.arange(7, -1, -1, device=packed.device)
    stream = ((packed.to(torch.int32)[..., None] >> shifts) & 1).reshape(*packed.shape[:-1], -1)
    stream = stream[..., :dim * bits].reshape(*packed.shape[:-1], dim, bits)
    weights = (1 << torch.arange(bits - 1, -1, -1, device=packed.device)).to(torch.int32)
    return (stream * weights).sum(-1).to(torch.uint8)


class HybridTurboQuant:
    """``htq = HybridTurboQuant(128, "tq35"); htq.calibrate_uniform(); packed = htq.encode(x)``."""

    def __init__(self, head_dim: int = 128, mode: str = "tq35", seed: int = 42, device: str = "cuda") -> None:
        if mode not in MODE_CONFIGS:
            raise ValueError(f"Unsupported mode {mode!r}. Choose from {list(MODE_CONFIGS.keys())}.")
        self.head_dim, self.mode, self.seed, self.device = head_dim, mode, seed, device
        self.layout: HybridLayout = _make_hybrid_layout(head_dim, mode)
        b0, b1 = MODE_CONFIGS[mode]["group_bits"]
        self._g0_mse_bits, self._g1_mse_bits = b0 - 1, b1 - 1
        self._g0_dim, self._g1_dim = self.layout.group0.dim, self.layout.group1.dim

        gen = torch.Generator(device="cpu")
        gen.manual_seed(seed)

        def signs(n: int) -> torch.Tensor:      # drawn in the order had0, had1, qjl0, qjl1
            return (torch.randint(0, 2, (n,), generator=gen, dtype=torch.float32) * 2 - 1).to(device)

        self._g0_had_signs, self._g1_had_signs = signs(self._g0_dim), signs(self._g1_dim)
        self._g0_qjl_signs, self._g1_qjl_signs = signs(self._g0_dim), signs(self._g1_dim)
        c0, b0_ = dimension_aware_codebook(self._g0_dim, self._g0_mse_bits)
        c1, b1_ = dimension_aware_codebook(self._g1_dim, self._g1_mse_bits)
        self._g0_centroids, self._g0_boundaries = c0.to(device), b0_.to(device)
        self._g1_centroids, self._g1_boundaries = c1.to(device), b1_.to(device)
        self._g0_qjl_scale = math.sqrt(math.pi / 2.0) / self._g0_dim
        self._g1_qjl_scale = math.sqrt(math.pi / 2.0) / self._g1_dim
        self._group0_indices: Optional[torch.Tensor] = None
        self._group1_indices: Optional[torch.Tensor] = None
        self._num_kv_heads = 0
        self._calibrated = False
        self._tables = None

    # ---- calibration -------------------------------------------------------------------

    def calibrate(self, sample_vectors: torch.Tensor) -> None:
        """Rank dims per head by mean square over ``[samples, kv_heads, head_dim]`` data."""
        if sample_vectors.dim() != 3:
            raise ValueError(f"Expected [num_samples, num_kv_heads, head_dim], got shape {list(sample_vectors.shape)}")
        _, heads, hdim = sample_vectors.shape
        if hdim != self.head_dim:
            raise ValueError(f"head_dim mismatch: expected {self.head_dim}, got {hdim}")
        order = (sample_vectors.float() ** 2).mean(dim=0).sort(dim=-1, descending=True).indices
        self._num_kv_heads = heads
        self._group0_indices = order[:, :self._g0_dim].to(self.device).contiguous()
        self._group1_indices = order[:, self._g0_dim:].to(self.device).contiguous()
        self._calibrated, self._tables = True, None

    def calibrate_uniform(self, num_kv_heads: int = 1) -> None:
        """First dims -> outlier group, the rest -> regular group, for every head."""
        self._num_kv_heads = num_kv_heads
        idx = torch.arange(self.head_dim, device=self.device)
        self._group0_indices = idx[:self._g0_dim].unsqueeze(0).expand(num_kv_heads, -1).contiguous()
        self._group1_indices = idx[self._g0_dim:].unsqueeze(0).expand(num_kv_heads, -1).contiguous()
        self._calibrated, self._tables = True, None

    def _ensure_calibrated(self) -> None:
        if not self._calibrated:
            raise RuntimeError("HybridTurboQuant: must call calibrate() or calibrate_uniform() before encode/decode.")

    # ---- kernel tables -------------------------------------------------------------------

    def _kernel_tables(self, rows: int):
        """(ctypes struct, tensors kept alive).  Rows cycle over heads when there are several
        index heads and the row count divides evenly; otherwise head 0 is used for all rows."""
        if self.head_dim != 128:
            raise NotImplementedError("the hybrid kernels are built for head_dim 128")
        per_head = self._num_kv_heads > 1 and rows % self._num_kv_heads == 0
        key = per_head
        if self._tables is None or self._tables[0] != key:
            dev = self._g0_had_signs.device
            index = torch.cat([self._group0_indices, self._group1_indices], dim=1).to(torch.int32)
            if not per_head:
                index = index[:1]
            pad = lambda t: torch.nn.functional.pad(t.float(), (0, 8 - t.numel()), value=float("inf"))  # noqa: E731
            keep = dict(
                index=index.contiguous(),
                had=torch.cat([self._g0_had_signs, self._g1_had_signs]).float().contiguous(),
                qjl=torch.cat([self._g0_qjl_signs, self._g1_qjl_signs]).float().contiguous(),
                cent=torch.cat([pad(self._g0_centroids), pad(self._g1_centroids)]).contiguous(),
                bnd=torch.cat([pad(self._g0_boundaries), pad(self._g1_boundaries)]).contiguous(),
            )
            t = _lib.HybridTables()
            t.head_dim, t.packed_dim = self.head_dim, self.layout.packed_dim
            t.group_index, t.num_index_heads = keep["index"].data_ptr(), keep["index"].shape[0]
            t.had_signs, t.qjl_signs = keep["had"].data_ptr(), keep["qjl"].data_ptr()
            t.centroids, t.boundaries = keep["cent"].data_ptr(), keep["bnd"].data_ptr()
            t.qjl_scale0, t.qjl_scale1 = self._g0_qjl_scale, self._g1_qjl_scale
            self._tables = (key, t, keep, dev)
        return self._tables[1]

    # ---- encode / decode -----------------------------------------------------------------

    def encode(self, x: torch.Tensor) -> torch.Tensor:
        """[..., head_dim] -> uint8 [..., packed_dim] (norms embedded as fp16)."""
        self._ensure_calibrated()
        assert x.shape[-1] == self.head_dim, f"Expected last dim {self.head_dim}, got {x.shape[-1]}"
        dev = _lib.require_cuda(x, self._g0_had_signs)
        if x.dtype not in _lib._FLOAT_CODES:
            x = x.float()
        x2 = x.reshape(-1, self.head_dim)
        if x2.stride(-1) != 1:
            x2 = x2.contiguous()
        n = x2.shape[0]
        out = torch.empty(n, self.layout.packed_dim, dtype=torch.uint8, device=dev)
        t = self._kernel_tables(n)
        with torch.cuda.device(dev):
            rc = _lib.lib().akv_hybrid_encode(x2.data_ptr(), _lib.float_code(x2), n,
                                              x2.stride(0) if n > 1 else self.head_dim, ctypes.byref(t),
                                              out.data_ptr(), self.layout.packed_dim, _lib.stream_ptr(dev))
        _lib.check(rc, "akv_hybrid_encode")
        return out.reshape(list(x.shape[:-1]) + [self.layout.packed_dim])

    def decode(self, packed: torch.Tensor) -> torch.Tensor:
        """uint8 [..., packed_dim] -> float32 [..., head_dim]."""
        self._ensure_calibrated()
        pd = self.layout.packed_dim
        assert packed.shape[-1] == pd, f"Expected last dim {pd}, got {packed.shape[-1]}"
        dev = _lib.require_cuda(packed, self._g0_had_signs)
        p2 = packed.reshape(-1, pd)
        if p2.stride(-1) != 1:
            p2 = p2.contiguous()
        n = p2.shape[0]
        out = torch.empty(n, self.head_dim, dtype=torch.float32, device=dev)
        t = self._kernel_tables(n)
        with torch.cuda.device(dev):
            rc = _lib.lib().akv_hybrid_decode(p2.data_ptr(), p2.stride(0) if n > 1 else pd, n, ctypes.byref(t),
                                              out.data_ptr(), _lib.AKV_F32, _lib.stream_ptr(dev))
        _lib.check(rc, "akv_hybrid_decode")
        return out.reshape(list(packed.shape[:-1]) + [self.head_dim])

    # ---- reports ----------------------------------------------------------------------------

    def validate(self, num_vectors: int = 10000) -> dict:
        if not self._calibrated:
            self.calibrate_uniform(num_kv_heads=1)
        x = torch.randn(num_vectors, self.head_dim, device=self.device, dtype=torch.float32)
        x[:, :self._g0_dim] *= 2.0
        x_hat = self.decode(self.encode(x))
        mse = (x - x_hat).pow(2).sum(-1).mean().item()
        energy = x.pow(2).sum(-1).mean().item()
        return {
            "mode": self.mode, "head_dim": self.head_dim, "num_vectors": num_vectors,
            "packed_dim_bytes": self.layout.packed_dim, "mse": mse, "relative_mse": mse / energy,
            "cosine_similarity": torch.nn.functional.cosine_similarity(x, x_hat, dim=-1).mean().item(),
            "max_abs_error": (x - x_hat).abs().max().item(),
            "compression_vs_fp16": self.head_dim * 2 / self.layout.packed_dim,
            "compression_vs_fp8": self.head_dim / self.layout.packed_dim,
            "group0": {"dim": self._g0_dim, "mse_bits": self._g0_mse_bits, "bytes": self.layout.group0.total_bytes},
            "group1": {"dim": self._g1_dim, "mse_bits": self._g1_mse_bits, "bytes": self.layout.group1.total_bytes},
        }

    def compression_ratio(self) -> float:
        return self.head_dim * 2 / self.layout.packed_dim

    def memory_report(self, seq_len: int, num_layers: int = 32, num_kv_heads: int = 8) -> dict:
        vectors = seq_len * num_layers * num_kv_heads * 2
        fp16, fp8, hy = vectors * self.head_dim * 2, vectors * self.head_dim, vectors * self.layout.packed_dim
        return {"config": f"Hybrid-{self.mode.upper()} d={self.head_dim} seq={seq_len} L={num_layers} H={num_kv_heads}",
                "fp16_mb": fp16 / 2 ** 20, "fp8_mb": fp8 / 2 ** 20, f"{self.mode}_mb": hy / 2 ** 20,
                "ratio_vs_fp16": fp16 / hy, "ratio_vs_fp8": fp8 / hy}

    @property
    def packed_dim(self) -> int:
        return self.layout.packed_dim

    @staticmethod
    def packed_dim_for_mode(head_dim: int, mode: str) -> int:
        return _make_hybrid_layout(head_dim, mode).packed_dim

    def __repr__(self) -> str:
        state = "calibrated" if self._calibrated else "uncalibrated"
        return (f"HybridTurboQuant(d={self.head_dim}, mode={self.mode!r}, packed={self.layout.packed_dim}B, "
                f"compress={self.compression_ratio():.1f}x, {state})")


class HybridPagedAttention:
    """Paged decode attention directly over tq35 or tq25 records (no K/V reconstruction).

    Stands in for the decompress-everything + SDPA body of the reference's
    ``tq::hybrid_decode_step`` (``vllm/hooks.py:297-345``).
    ``k_cache`` / ``v_cache``: uint8 ``[num_blocks, block_size, num_kv_heads, 64]`` (tq35; 44 for tq25; views allowed).
    tq35 runs on the tensor-core kernel, tq25 on the scalar one.
    """

    def __init__(self, htq: HybridTurboQuant, num_query_heads: int):
        htq._ensure_calibrated()
        if htq.head_dim != 128:
            raise NotImplementedError("hybrid paged attention is built for head_dim 128")
        self.htq, self.num_query_heads = htq, num_query_heads
        self.scale = 1.0 / math.sqrt(htq.head_dim)
        self._workspace: Optional[torch.Tensor] = None

    # bytes of scratch the staged prefill kernel may ask for (AITHER_TQ_PREFILL_SCRATCH_MB overrides; 0 = never staged)
    STAGED_WORKSPACE_LIMIT = int(os.environ.get("AITHER_TQ_PREFILL_SCRATCH_MB", "2048")) << 20

    def prefill(self, query, k_cache, v_cache, block_tables, seq_lens, query_start_loc, block_size: int = 16,
                num_kv_heads: Optional[int] = None, out: Optional[torch.Tensor] = None, scale: Optional[float] = None,
                max_seq_len: Optional[int] = None) -> Optional[torch.Tensor]:
        """Chunked-prefill attention over tq35 / tq25 records (arguments as ``TQPagedAttention.prefill``): the records of every
        128-key tile are decoded once into fp16 operand images, then the tensor-core attention kernel runs over them
        (``akv_tq_prefill_attn`` with ``hybrid_tables``).  The reference decompresses the active blocks and calls vLLM's
        unified attention (``vllm/hooks.py:726-850``).  Returns None when that kernel does not serve the case (no
        host-side ``max_seq_len``, a batch too ragged for 128-row tiles, scratch beyond ``STAGED_WORKSPACE_LIMIT``): the
        caller then attends row by row with ``forward``."""
        if num_kv_heads is None:
            num_kv_heads = k_cache.shape[2]
        dev = _lib.require_cuda(query, k_cache, v_cache, block_tables, seq_lens, query_start_loc)
        n_tok, num_q_heads, head_dim = query.shape
        G = num_q_heads // num_kv_heads
        aligned = all((t.data_ptr() | t.stride(0) | t.stride(1) | t.stride(2)) % 4 == 0 for t in (k_cache, v_cache))
        pd = self.htq.layout.packed_dim
        if (head_dim != 128 or G not in (1, 2, 4, 8) or block_size % 16 or not aligned
                or not max_seq_len or k_cache.shape[-1] < pd or v_cache.shape[-1] < pd):
            return None
        assert num_q_heads == self.num_query_heads and k_cache.shape[1] == block_size
        num_seqs = query_start_loc.numel() - 1
        if query.dtype not in _lib._FLOAT_CODES:
            query = query.float()
        if query.stride(-1) != 1:
            query = query.contiguous()
        if block_tables.stride(-1) != 1:
            block_tables = block_tables.contiguous()
        seq_lens, query_start_loc = seq_lens.contiguous(), query_start_loc.contiguous()
        if out is None:
            out = torch.empty(n_tok, num_q_heads, head_dim, dtype=query.dtype, device=dev)
        L = _lib.lib()
        nbytes = L.akv_tq_prefill_attn_workspace_bytes_staged(n_tok, num_q_heads, num_kv_heads, num_seqs, int(max_seq_len))
        if nbytes > self.STAGED_WORKSPACE_LIMIT:
            return None
        if getattr(self, "_prefill_ws", None) is None or self._prefill_ws.numel() < nbytes or self._prefill_ws.device != dev:
            self._prefill_ws = torch.empty(max(nbytes, 256), dtype=torch.uint8, device=dev)
        if getattr(self, "_eye", None) is None or self._eye.device != dev:
            self._eye = torch.eye(128, dtype=torch.float32, device=dev)      # the records decode into the original domain
        tables = self.htq._kernel_tables(1)
        p = _lib.TQPrefillParams()
        p.query, p.q_dtype, p.q_stride_tok, p.q_stride_head = query.data_ptr(), _lib.float_code(query), query.stride(0), query.stride(1)
        p.k_packed, p.kp_stride_blk, p.kp_stride_pos, p.kp_stride_head = k_cache.data_ptr(), k_cache.stride(0), k_cache.stride(1), k_cache.stride(2)
        p.v_packed, p.vp_stride_blk, p.vp_stride_pos, p.vp_stride_head = v_cache.data_ptr(), v_cache.stride(0), v_cache.stride(1), v_cache.stride(2)
        p.k_norms = p.v_norms = None
        p.block_tables, p.bt_dtype, p.bt_stride_seq = block_tables.data_ptr(), _lib.index_code(block_tables), block_tables.stride(0)
        p.seq_lens, p.sl_dtype = seq_lens.data_ptr(), _lib.index_code(seq_lens)
        p.query_start_loc, p.qs_dtype = query_start_loc.data_ptr(), _lib.index_code(query_start_loc)
        p.num_seqs, p.num_tokens, p.num_q_heads, p.num_kv_heads = num_seqs, n_tok, num_q_heads, num_kv_heads
        p.head_dim, p.block_size, p.max_blocks_per_seq, p.num_blocks = head_dim, block_size, block_tables.shape[1], k_cache.shape[0]
        p.bits = 4
        p.rotation, p.rotation_t, p.centroids = self._eye.data_ptr(), self._eye.data_ptr(), None
        p.scale = self.scale if scale is None else float(scale)
        p.out, p.out_dtype, p.out_stride_tok, p.out_stride_head = out.data_ptr(), _lib.float_code(out), out.stride(0), out.stride(1)
        p.workspace, p.workspace_bytes = self._prefill_ws.data_ptr(), self._prefill_ws.numel()
        p.stream = _lib.stream_ptr(dev)
        p.max_seq_len = int(max_seq_len)
        p.hybrid_tables = ctypes.cast(ctypes.pointer(tables), ctypes.c_void_p)
        with torch.cuda.device(dev):
            rc = L.akv_tq_prefill_attn(ctypes.byref(p))
        if rc == _lib.AKV_ERR_UNSUPPORTED:
            return None
        _lib.check(rc, "akv_tq_prefill_attn")
        return out

    def forward(self, query, k_cache, v_cache, block_tables, context_lens, block_size: int = 16,
                num_kv_heads: Optional[int] = None, out: Optional[torch.Tensor] = None,
                scale: Optional[float] = None, new_kv=None) -> torch.Tensor:
        """``new_kv = (key, value, slot_mapping)`` (``[tokens, kv_heads, 128]`` each, int64 slots): the
        records of these tokens are written into the caches first, in the same call
        (``akv_hybrid_decode_step``); tokens with a negative slot are skipped."""
        if num_kv_heads is None:
            num_kv_heads = k_cache.shape[2]
        dev = _lib.require_cuda(query, k_cache, v_cache, block_tables, context_lens)
        num_seqs, num_q_heads, head_dim = query.shape
        assert head_dim == 128 and num_q_heads == self.num_query_heads and k_cache.shape[1] == block_size
        if query.dtype not in _lib._FLOAT_CODES:
            query = query.float()
        if query.stride(-1) != 1:
            query = query.contiguous()
        for name, t in (("k_cache", k_cache), ("v_cache", v_cache)):
            if t.dtype != torch.uint8 or t.stride(-1) != 1 or t.shape[-1] < self.htq.layout.packed_dim:
                raise ValueError(f"{name} must be uint8 [..., >={self.htq.layout.packed_dim}] with a contiguous last dimension")
        if block_tables.stride(-1) != 1:
            block_tables = block_tables.contiguous()
        context_lens = context_lens.contiguous()
        max_blocks = block_tables.shape[1]
        if out is None:
            out = torch.empty(num_seqs, num_q_heads, head_dim, dtype=query.dtype, device=dev)
        L = _lib.lib()
        nbytes = L.akv_hybrid_paged_attn_workspace_bytes(num_seqs, num_q_heads, block_size, max_blocks, 0)
        if self._workspace is None or self._workspace.numel() < nbytes or self._workspace.device != dev:
            self._workspace = torch.empty(max(nbytes, 256), dtype=torch.uint8, device=dev)
        tables = self.htq._kernel_tables(1)      # one dim split shared by all heads
        step = _lib.HybridDecodeStepParams() if new_kv is not None else None
        p = step.attn if step is not None else _lib.HybridAttnParams()
        p.query, p.q_dtype, p.q_stride_seq, p.q_stride_head = query.data_ptr(), _lib.float_code(query), query.stride(0), query.stride(1)
        p.k_cache, p.k_stride_blk, p.k_stride_pos, p.k_stride_head = k_cache.data_ptr(), k_cache.stride(0), k_cache.stride(1), k_cache.stride(2)
        p.v_cache, p.v_stride_blk, p.v_stride_pos, p.v_stride_head = v_cache.data_ptr(), v_cache.stride(0), v_cache.stride(1), v_cache.stride(2)
        p.block_tables, p.bt_dtype, p.bt_stride_seq = block_tables.data_ptr(), _lib.index_code(block_tables), block_tables.stride(0)
        p.context_lens, p.cl_dtype = context_lens.data_ptr(), _lib.index_code(context_lens)
        p.num_seqs, p.num_q_heads, p.num_kv_heads = num_seqs, num_q_heads, num_kv_heads
        p.block_size, p.max_blocks_per_seq, p.num_blocks = block_size, max_blocks, k_cache.shape[0]
        p.tables = ctypes.pointer(tables)
        p.scale = self.scale if scale is None else float(scale)
        p.out, p.out_dtype, p.out_stride_seq, p.out_stride_head = out.data_ptr(), _lib.float_code(out), out.stride(0), out.stride(1)
        p.workspace, p.workspace_bytes = self._workspace.data_ptr(), self._workspace.numel()
        p.blocks_per_split = 0
        p.stream = _lib.stream_ptr(dev)
        if step is not None:
            key, value, slots = new_kv
            _lib.require_cuda(key, value, slots)
            if key.shape != value.shape or key.dim() != 3 or key.shape[1] != num_kv_heads or key.shape[2] != 128:
                raise ValueError(f"new K/V must be [tokens, {num_kv_heads}, 128], got {tuple(key.shape)} / {tuple(value.shape)}")
            if key.dtype != value.dtype or key.dtype not in _lib._FLOAT_CODES:
                raise TypeError("new K/V must share one of float16 / bfloat16 / float32")
            if key.stride(-1) != 1:
                key = key.contiguous()
            if value.stride(-1) != 1:
                value = value.contiguous()
            if slots.dtype != torch.int64 or slots.numel() < key.shape[0]:
                raise ValueError("slot_mapping must be int64 with one entry per token")
            slots = slots.contiguous()
            step.key, step.value, step.kv_dtype = key.data_ptr(), value.data_ptr(), _lib.float_code(key)
            step.num_tokens = key.shape[0]
            step.k_stride_tok, step.k_stride_head = key.stride(0), key.stride(1)
            step.v_stride_tok, step.v_stride_head = value.stride(0), value.stride(1)
            step.slot_mapping, step.max_blocks = slots.data_ptr(), k_cache.shape[0]
            with torch.cuda.device(dev):
                rc = L.akv_hybrid_decode_step(ctypes.byref(step))
            _lib.check(rc, "akv_hybrid_decode_step")
            return out
        with torch.cuda.device(dev):
            rc = L.akv_hybrid_paged_attn(ctypes.byref(p))
        _lib.check(rc, "akv_hybrid_paged_attn")
        return out


def hybrid_kv_update(htq: HybridTurboQuant, x: torch.Tensor, slot_mapping: torch.Tensor, cache: torch.Tensor,
                     block_size: Optional[int] = None, max_blocks: int = 0) -> None:
    """Encode ``x`` ``[tokens, kv_heads, 128]`` and store the records at ``cache[slot // block_size,
    slot % block_size, head, :packed_dim]`` (``cache``: uint8 ``[blocks, block_size, kv_heads, >= packed_dim]``,
    views allowed).  The encode + index-put of the reference's ``tq::hybrid_decode_step``
    (``vllm/hooks.py:259-296``) as one kernel; tokens with a negative slot are skipped."""
    htq._ensure_calibrated()
    dev = _lib.require_cuda(x, slot_mapping, cache)
    if x.dim() != 3 or x.shape[2] != htq.head_dim or cache.dim() != 4 or cache.shape[2] != x.shape[1]:
        raise ValueError(f"x {tuple(x.shape)} / cache {tuple(cache.shape)} do not match [tokens, heads, {htq.head_dim}] "
                         "and [blocks, block_size, heads, bytes]")
    if cache.dtype != torch.uint8 or cache.stride(-1) != 1 or cache.shape[-1] < htq.packed_dim:
        raise ValueError(f"cache must be uint8 [..., >= {htq.packed_dim}] with a contiguous last dimension")
    if x.dtype not in _lib._FLOAT_CODES:
        x = x.float()
    if x.stride(-1) != 1:
        x = x.contiguous()
    if slot_mapping.dtype != torch.int64 or slot_mapping.numel() < x.shape[0]:
        raise ValueError("slot_mapping must be int64 with one entry per token")
    slot_mapping = slot_mapping.contiguous()
    bs = cache.shape[1] if block_size is None else block_size
    assert bs == cache.shape[1], "block_size does not match the cache"
    tables = htq._kernel_tables(x.shape[0] * x.shape[1])
    with torch.cuda.device(dev):
        rc = _lib.lib().akv_hybrid_kv_update(x.data_ptr(), _lib.float_code(x), x.shape[0], x.shape[1], x.stride(0),
                                             x.stride(1), slot_mapping.data_ptr(), ctypes.byref(tables),
                                             cache.data_ptr(), cache.stride(0), cache.stride(1), cache.stride(2), bs,
                                             max_blocks or cache.shape[0], _lib.stream_ptr(dev))
    _lib.check(rc, "akv_hybrid_kv_update")
