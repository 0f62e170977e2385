"""TurboQuant: rotate, scalar-quantise with a Lloyd-Max codebook, bit-pack.

Host-side mirror of the reference's ``aither_kvcache/quantizer.py``
(``TurboQuantConfig`` :36-46, ``TurboQuant`` :49-370): same constructor,
attributes (``rotation``, ``centroids``, ``boundaries_inner``, ``head_dim``,
``bits``, ``num_levels``, ``_packed_dim``, ``dtype``) and the same
``encode`` / ``decode`` contracts.  The arithmetic runs in the CUDA kernels
behind ``akv_tq_encode`` / ``akv_tq_decode``; there is no Triton and no CPU path.
"""
from __future__ import annotations

import time
from dataclasses import dataclass
from typing import Optional, Tuple

import torch

from . import _lib
from .codebook import get_codebook, get_theory_bounds
from .packing import packed_size
from .rotation import random_orthogonal, randomized_hadamard_matrix


@dataclass
class TurboQuantConfig:
    head_dim: int = 128
    bits: int = 4                # 2, 3 or 4
    seed: int = 42
    use_hadamard: bool = False   # randomised Hadamard matrix instead of a QR rotation
    hadamard_rounds: int = 3
    device: str = "cuda"
    dtype: torch.dtype = torch.float16   # dtype of decode()'s result
    use_triton: bool = True      # accepted for compatibility; there is only one engine


class TurboQuant:
    """``packed, norms = tq.encode(x)`` / ``x_hat = tq.decode(packed, norms)``.

    Bytes per 128-d vector incl. the float32 norm: 68 / 52 / 36 for 4 / 3 / 2 bits.
    """

    def __init__(self, config: Optional[TurboQuantConfig] = None, **kwargs):
        if config is None:
            config = TurboQuantConfig(**kwargs)
        self.config = config
        self.head_dim = config.head_dim
        self.bits = config.bits
        self.num_levels = 1 << config.bits
        self.device = config.device
        self.dtype = config.dtype
        if config.bits not in (2, 3, 4):
            raise ValueError(f"Supported bit-widths: 2, 3, 4. Got {config.bits}")
        if config.head_dim <= 0 or config.head_dim & (config.head_dim - 1):
            raise ValueError(f"head_dim must be power of 2, got {config.head_dim}")

        if config.use_hadamard:
            rot = randomized_hadamard_matrix(config.head_dim, seed=config.seed, device="cpu",
                                             num_rounds=config.hadamard_rounds)
        else:
            rot = random_orthogonal(config.head_dim, seed=config.seed, device="cpu")
        self.rotation = rot.to(config.device).contiguous()

        cent, bnd, mse = get_codebook(config.head_dim, config.bits)
        self.centroids = torch.tensor(cent, dtype=torch.float32, device=config.device)
        self.boundaries_inner = torch.tensor(bnd, dtype=torch.float32, device=config.device)
        self.mse_total = mse
        self.theory_lower, self.theory_upper = get_theory_bounds(config.bits)
        self._packed_dim = packed_size(config.head_dim, config.bits)
        self._use_triton = False

    # The kernels want R^T for encode (coalesced columns) and R for decode.
    @property
    def rotation(self) -> torch.Tensor:
        return self._rotation

    @rotation.setter
    def rotation(self, value: torch.Tensor) -> None:
        self._rotation = value.to(torch.float32).contiguous()
        self.rotation_T = self._rotation.t().contiguous()

    def encode(self, x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        """x [..., head_dim] (fp16 / bf16 / fp32, CUDA) -> (uint8 [..., packed_dim], float32 [...])."""
        assert x.shape[-1] == self.head_dim, f"Expected last dim {self.head_dim}, got {x.shape[-1]}"
        dev = _lib.require_cuda(x, self.rotation_T)
        if x.dtype not in (torch.float16, torch.bfloat16, torch.float32):
            x = x.float()
        batch = list(x.shape[:-1])
        x2 = x.reshape(-1, self.head_dim)
        if x2.stride(-1) != 1:
            x2 = x2.contiguous()
        n = x2.shape[0]
        packed = torch.empty(n, self._packed_dim, dtype=torch.uint8, device=dev)
        norms = torch.empty(n, dtype=torch.float32, device=dev)
        with torch.cuda.device(dev):
            rc = _lib.lib().akv_tq_encode(
                x2.data_ptr(), _lib.float_code(x2), n, x2.stride(0) if n > 1 else self.head_dim,
                self.head_dim, self.bits, self.rotation_T.data_ptr(), self.boundaries_inner.data_ptr(),
                packed.data_ptr(), self._packed_dim, norms.data_ptr(), _lib.stream_ptr(dev))
        _lib.check(rc, "akv_tq_encode")
        return packed.reshape(batch + [self._packed_dim]), norms.reshape(batch)

    def decode(self, packed: torch.Tensor, norms: torch.Tensor) -> torch.Tensor:
        """(uint8 [..., packed_dim], float32 [...]) -> [..., head_dim] in ``self.dtype``."""
        dev = _lib.require_cuda(packed, norms, self.rotation)
        batch = list(norms.shape)
        p2 = packed.reshape(-1, packed.shape[-1])
        if p2.stride(-1) != 1:
            p2 = p2.contiguous()
        n2 = norms.reshape(-1).float().contiguous()
        n = n2.shape[0]
        out_dtype = self.dtype if self.dtype in _lib._FLOAT_CODES else torch.float32
        out = torch.empty(n, self.head_dim, dtype=out_dtype, device=dev)
        with torch.cuda.device(dev):
            rc = _lib.lib().akv_tq_decode(
                p2.data_ptr(), p2.stride(0) if n > 1 else self._packed_dim, n2.data_ptr(), n,
                self.head_dim, self.bits, self.rotation.data_ptr(), self.centroids.data_ptr(),
                out.data_ptr(), _lib._FLOAT_CODES[out_dtype], _lib.stream_ptr(dev))
        _lib.check(rc, "akv_tq_decode")
        return out.reshape(batch + [self.head_dim]).to(self.dtype)

    # ---- analysis helpers (host arithmetic, same reports as the reference) ----

    def compression_ratio(self) -> float:
        return self.head_dim * 2 / (self._packed_dim + 4)

    def compression_ratio_vs_fp8(self) -> float:
        return self.head_dim / (self._packed_dim + 4)

    def memory_report(self, seq_len: int, num_layers: int = 32, num_kv_heads: int = 8) -> dict:
        vectors = seq_len * num_layers * num_kv_heads * 2
        fp16, fp8, tq = vectors * self.head_dim * 2, vectors * self.head_dim, vectors * (self._packed_dim + 4)
        return {
            "config": f"TQ{self.bits} d={self.head_dim} seq={seq_len} L={num_layers} H={num_kv_heads}",
            "fp16_mb": fp16 / 2 ** 20, "fp8_mb": fp8 / 2 ** 20, f"tq{self.bits}_mb": tq / 2 ** 20,
            "ratio_vs_fp16": fp16 / tq, "ratio_vs_fp8": fp8 / tq,
        }

    def validate(self, num_vectors: int = 10000, device: Optional[str] = None) -> dict:
        dev = device or self.device
        x = torch.randn(num_vectors, self.head_dim, device=dev, dtype=torch.float32)
        x = x / x.norm(dim=-1, keepdim=True)
        x_hat = self.decode(*self.encode(x)).float()
        mse = (x - x_hat).pow(2).sum(-1).mean().item()
        n = min(num_vectors, 5000)
        ia = torch.randint(0, num_vectors, (n,), device=dev)
        ib = torch.randint(0, num_vectors, (n,), device=dev)
        true_ip = (x[ia] * x[ib]).sum(-1)
        est_ip = (x_hat[ia] * x[ib]).sum(-1)
        return {
            "bits": self.bits, "head_dim": self.head_dim, "num_vectors": num_vectors, "mse": mse,
            "mse_theory_lower": self.theory_lower, "mse_theory_upper": self.theory_upper,
            "mse_ratio_to_lower": mse / self.theory_lower,
            "ip_mse": (true_ip - est_ip).pow(2).mean().item(), "ip_bias": (est_ip - true_ip).mean().item(),
            "max_abs_error": (x - x_hat).abs().max().item(),
            "compression_vs_fp16": self.compression_ratio(),
            "compression_vs_fp8": self.compression_ratio_vs_fp8(), "triton_active": False,
        }

    def benchmark(self, num_vectors: int = 32768, warmup: int = 10, iters: int = 100,
                  device: Optional[str] = None) -> dict:
        dev = device or self.device
        x = torch.randn(num_vectors, self.head_dim, device=dev, dtype=torch.float16)
        for _ in range(warmup):
            p, n = self.encode(x)
            self.decode(p, n)
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(iters):
            p, n = self.encode(x)
        torch.cuda.synchronize()
        enc_us = (time.perf_counter() - t0) / iters * 1e6
        t0 = time.perf_counter()
        for _ in range(iters):
            self.decode(p, n)
        torch.cuda.synchronize()
        dec_us = (time.perf_counter() - t0) / iters * 1e6
        return {"bits": self.bits, "num_vectors": num_vectors, "encode_us": enc_us, "decode_us": dec_us,
                "encode_throughput_mvec_s": num_vectors / enc_us,
                "decode_throughput_mvec_s": num_vectors / dec_us, "triton_active": False, "device": dev}

    def __repr__(self) -> str:
        return (f"TurboQuant(d={self.head_dim}, bits={self.bits}, compress={self.compression_ratio():.1f}x, "
                f"mse={self.mse_total:.4f}, engine=CUDA sm_100a)")
