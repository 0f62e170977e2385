"""CPU-side checks: the shared library loads and exports the declared ABI, the host
classes build the same tables as the reference, and product code refuses CPU tensors."""
import ctypes
import os
import re

import numpy as np
import pytest
import torch

from conftest import ROOT, load_golden


def test_library_exports_every_declared_symbol():
    from aitherkvcache_b200 import _build, _lib
    _build.build()
    handle = ctypes.CDLL(_lib.LIB_PATH)
    header = open(os.path.join(ROOT, "include", "akv_b200.h")).read()
    declared = set(re.findall(r"\b(akv_[a-z0-9_]+)\s*\(", header))
    assert declared, "no declarations found"
    for name in declared:
        assert hasattr(handle, name), f"{name} declared in include/akv_b200.h but not exported"
    assert declared == set(_lib.exported_symbols())
    assert _lib.lib().akv_version() >= 100


@pytest.mark.parametrize("d", (128, 64))
@pytest.mark.parametrize("bits", (4, 3, 2))
def test_tables_match_reference(d, bits):
    from aitherkvcache_b200 import TurboQuant
    g = load_golden(f"tq_d{d}_b{bits}.npz")
    tq = TurboQuant(head_dim=d, bits=bits, device="cpu")
    assert np.array_equal(tq.centroids.numpy(), g["centroids"])
    assert np.array_equal(tq.boundaries_inner.numpy(), g["boundaries"])
    assert np.abs(tq.rotation.numpy() - g["rotation"]).max() < 1e-5
    assert torch.allclose(tq.rotation @ tq.rotation.T, torch.eye(d), atol=1e-5)
    assert tq._packed_dim == d * bits // 8 and tq.num_levels == 1 << bits
    assert torch.equal(tq.rotation_T, tq.rotation.t())


def test_config_errors_and_reports():
    from aitherkvcache_b200 import TurboQuant, TurboQuantConfig
    with pytest.raises(ValueError):
        TurboQuant(head_dim=128, bits=1, device="cpu")
    with pytest.raises(ValueError):
        TurboQuant(head_dim=96, bits=4, device="cpu")
    tq = TurboQuant(TurboQuantConfig(head_dim=128, bits=4, device="cpu"))
    assert abs(tq.compression_ratio() - 256 / 68) < 1e-9
    rep = tq.memory_report(seq_len=1024)
    assert rep["ratio_vs_fp16"] == pytest.approx(256 / 68)
    th = TurboQuant(head_dim=128, bits=4, device="cpu", use_hadamard=True)
    assert torch.allclose(th.rotation @ th.rotation.T, torch.eye(128), atol=1e-5)


def test_no_cpu_fallback():
    from aitherkvcache_b200 import TurboQuant
    tq = TurboQuant(head_dim=128, bits=4, device="cpu")
    with pytest.raises(RuntimeError, match="CUDA"):
        tq.encode(torch.randn(4, 128))


@pytest.mark.parametrize("bits", (4, 3, 2))
def test_packing_helpers_match_oracle(bits):
    from aitherkvcache_b200 import packing
    from oracle import tq as otq
    idx = torch.randint(0, 1 << bits, (3, 5, 128), generator=torch.Generator().manual_seed(bits))
    pack = {4: packing.pack_4bit, 3: packing.pack_3bit, 2: packing.pack_2bit}[bits]
    unpack = {4: packing.unpack_4bit, 3: packing.unpack_3bit, 2: packing.unpack_2bit}[bits]
    p = pack(idx)
    assert p.dtype == torch.uint8 and p.shape[-1] == packing.packed_size(128, bits)
    assert np.array_equal(p.numpy(), otq.pack(idx.numpy(), bits))
    assert torch.equal(unpack(p, 128).long(), idx)


def test_vllm_backend_surface():
    """Class attributes and statics of the CUSTOM backend (needs vLLM importable; no GPU)."""
    pytest.importorskip("vllm")
    from aitherkvcache_b200.vllm import backend
    B = backend.TurboQuantBackend
    assert B.get_name() == "CUSTOM"
    assert B.accept_output_buffer is True and B.forward_includes_kv_cache_update is False
    assert B.get_kv_cache_shape(10, 16, 8, 128, "auto") == (10, 2, 16, 8, 128)
    assert {"tq-t4nc", "tq-t3nc", "tq-t2nc"} <= set(B.supported_kv_cache_dtypes)
    assert 128 in B.get_supported_head_sizes()
    impl = B.get_impl_cls()
    assert hasattr(impl, "forward") and hasattr(impl, "do_kv_cache_update")
    assert backend.bits_from_env_or_dtype("tq-t3nc") == 3


def test_kv_cache_dtype_table():
    import aitherkvcache_b200 as a
    assert a.KV_CACHE_DTYPES["tq-t4nc"] == {"kind": "uniform", "bits": 4}
    assert a.KV_CACHE_DTYPES["tq-t35nc"]["mode"] == "tq35"
