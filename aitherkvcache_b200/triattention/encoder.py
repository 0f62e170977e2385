"""Spectral K/V encoder: keep the F strongest RoPE pairs; coefficients as 4-bit or 8-bit codes against an fp16
scale, or as plain fp16.

Interface of the reference's ``triattention/encoder.py`` (``SpectralEncoding`` :36-43,
``SpectralKVEncoder`` :46-269).  ``encode`` runs in ``akv_tri_encode``; ``decode`` (dense
reconstruction, not on the decode path) is a scatter with tensor ops on the device.
"""
from typing import NamedTuple, Optional

import torch

from .. import _lib
from .config import TriAttentionConfig


class SpectralEncoding(NamedTuple):
    indices: torch.Tensor    # [..., F] uint8, ascending pair ids
    packed: torch.Tensor     # coeff_bits 4: [..., F] uint8, high nibble = even dim, low nibble = odd dim;
                             # 8: [..., 2F] uint8 (even, odd per pair); 16: [..., F, 2] float16
    scales: torch.Tensor     # [...] float16


class SpectralKVEncoder:
    def __init__(self, config: TriAttentionConfig):
        self.config = config
        self.head_dim, self.num_pairs = config.head_dim, config.num_pairs
        self.num_freqs, self.coeff_bits = config.num_freqs, config.coeff_bits
        if self.coeff_bits not in (4, 8, 16):
            raise ValueError(f"Unsupported coeff_bits: {self.coeff_bits}")
        self._half_code = 127.5 if self.coeff_bits == 8 else 7.5

    def encode(self, x: torch.Tensor, num_freqs: Optional[int] = None) -> SpectralEncoding:
        f = num_freqs or self.num_freqs
        dev = _lib.require_cuda(x)
        if x.dtype not in _lib._FLOAT_CODES:
            x = x.float()
        x2 = x.reshape(-1, self.head_dim)
        if x2.stride(-1) != 1:
            x2 = x2.contiguous()
        n = x2.shape[0]
        idx = torch.empty(n, f, dtype=torch.uint8, device=dev)
        cb = self.coeff_bits
        packed = (torch.empty(n, f, 2, dtype=torch.float16, device=dev) if cb == 16
                  else torch.empty(n, f * cb // 4, dtype=torch.uint8, device=dev))
        scales = torch.empty(n, dtype=torch.float16, device=dev)
        with torch.cuda.device(dev):
            rc = _lib.lib().akv_tri_encode_bits(x2.data_ptr(), _lib.float_code(x2), n,
                                                x2.stride(0) if n > 1 else self.head_dim, self.head_dim, f, cb,
                                                idx.data_ptr(), packed.data_ptr(), scales.data_ptr(),
                                                _lib.stream_ptr(dev))
        _lib.check(rc, "akv_tri_encode_bits")
        lead = list(x.shape[:-1])
        return SpectralEncoding(idx.reshape(lead + [f]), packed.reshape(lead + list(packed.shape[1:])), scales.reshape(lead))

    def decode(self, enc: SpectralEncoding) -> torch.Tensor:
        """Dense [..., head_dim] float32 reconstruction (zeros at pairs that were dropped)."""
        s = enc.scales.float().unsqueeze(-1)
        if self.coeff_bits == 16:
            v0, v1 = enc.packed[..., 0].float(), enc.packed[..., 1].float()
        elif self.coeff_bits == 8:
            raw = enc.packed.float().reshape(*enc.indices.shape, 2)
            v0, v1 = (raw[..., 0] / self._half_code - 1.0) * s, (raw[..., 1] / self._half_code - 1.0) * s
        else:
            v0 = ((enc.packed >> 4).float() / self._half_code - 1.0) * s
            v1 = ((enc.packed & 0x0F).float() / self._half_code - 1.0) * s
        out = torch.zeros(*enc.indices.shape[:-1], self.head_dim, dtype=torch.float32, device=enc.indices.device)
        ids = enc.indices.long()
        out.scatter_(-1, ids * 2, v0)
        out.scatter_(-1, ids * 2 + 1, v1)
        return out
