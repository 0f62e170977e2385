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


def test_plugin_entry_point_and_backend_construction_under_vllm(monkeypatch):
    """The packaging of the serving boundary: pyproject.toml declares a vllm.general_plugins entry
    point; it resolves to a callable that registers the CUSTOM backend with the installed vLLM, and
    the real TurboQuantImpl (a subclass of vLLM's own impl) constructs with vLLM's argument order."""
    import importlib
    import tomllib
    pytest.importorskip("vllm")
    with open(os.path.join(ROOT, "pyproject.toml"), "rb") as f:
        proj = tomllib.load(f)
    eps = proj["project"]["entry-points"]["vllm.general_plugins"]
    assert eps == {"aitherkvcache_b200": "aitherkvcache_b200.vllm.plugin:register"}
    mod, attr = eps["aitherkvcache_b200"].split(":")
    register = getattr(importlib.import_module(mod), attr)
    register()
    from vllm.v1.attention.backends.registry import AttentionBackendEnum
    cls = AttentionBackendEnum.CUSTOM.get_class()
    assert cls.get_name() == "CUSTOM" and cls.__module__ == "aitherkvcache_b200.vllm.backend"
    assert cls.get_kv_cache_shape(10, 16, 8, 128) == (10, 2, 16, 8, 128)
    from vllm.v1.attention.backend import AttentionCGSupport
    assert cls.get_builder_cls()._cudagraph_support == AttentionCGSupport.UNIFORM_SINGLE_TOKEN_DECODE
    impl_cls = cls.get_impl_cls()
    monkeypatch.delenv("AITHER_TQ_MODE", raising=False)
    monkeypatch.delenv("AITHER_TQ_BITS", raising=False)
    impl = impl_cls(32, 128, 0.0884, 8, None, None, "tq-t3nc")            # positional, as vLLM's layers call it
    assert (impl.tq_codec, impl.tq_bits, impl.packed_dim, impl.num_kv_heads) == ("uniform", 3, 48, 8)
    monkeypatch.setenv("AITHER_TQ_MODE", "tq35")
    impl = impl_cls(num_heads=32, head_size=128, scale=0.0884, num_kv_heads=8, alibi_slopes=None,
                    sliding_window=None, kv_cache_dtype="auto")
    assert (impl.tq_codec, impl.tq_mode, impl.packed_dim) == ("hybrid", "tq35", 64)
    monkeypatch.setenv("AITHER_TQ_MODE", "")
    monkeypatch.setenv("AITHER_TQ_BITS", "2")
    assert impl_cls(32, 128, 0.0884, 8, None, None, "auto").packed_dim == 32


def test_token_rows_of_a_mixed_batch():
    """Per-token attention rows of a chunked-prefill / decode mix: causal context lengths and the
    sequences' block-table rows, against a plain loop."""
    import torch
    from aitherkvcache_b200.vllm.backend import token_rows
    qsl = torch.tensor([0, 5, 6, 6, 14], dtype=torch.int32)        # 5 prefill tokens, 1 decode, an empty one, 8 prefill
    seq_lens = torch.tensor([5, 900, 3, 40], dtype=torch.int32)
    bt = torch.arange(4 * 7, dtype=torch.int32).reshape(4, 7)
    rows_bt, ctx = token_rows(qsl, seq_lens, bt, 14)
    want_ctx, want_seq = [], []
    for s in range(4):
        n = int(qsl[s + 1] - qsl[s])
        for i in range(n):
            want_ctx.append(int(seq_lens[s]) - (n - 1 - i))
            want_seq.append(s)
    assert ctx.tolist() == want_ctx and ctx.dtype == torch.int32
    assert torch.equal(rows_bt, bt[torch.tensor(want_seq)])


def test_spectral_kv_cache_host_semantics():
    """SpectralKVCache on CPU tensors: store / fetch / copy / clear and the statistics of the reference's class."""
    from aitherkvcache_b200.triattention import SpectralEncoding, SpectralKVCache, TriAttentionConfig
    cfg = TriAttentionConfig(head_dim=128, num_freqs=12, coeff_bits=4, num_kv_heads=2, num_query_heads=8)
    cache = SpectralKVCache(cfg, max_blocks=6, device="cpu")
    assert cache.bytes_allocated == 6 * 16 * 2 * (12 + 12 + 2) * 2 and cache.bytes_per_token == 2 * cfg.bytes_per_kv_token
    g = torch.Generator().manual_seed(0)

    def enc(n):
        return SpectralEncoding(torch.randint(0, 64, (n, 2, 12), generator=g, dtype=torch.uint8),
                                torch.randint(0, 256, (n, 2, 12), generator=g, dtype=torch.uint8),
                                torch.rand(n, 2, generator=g).half())
    k, v = enc(37), enc(37)
    table = torch.tensor([4, 1, 5, 0], dtype=torch.int32)
    cache.store_sequence(table, k, v)
    kf, vf = cache.fetch_sequence(table, 37)
    assert all(torch.equal(a, b) for a, b in zip(kf + vf, k + v))
    assert cache.memory_stats()["total_tokens"] == 37 and cache.memory_stats()["used_blocks"] == 3
    # the reference's per-block and per-token stores land in the same places
    other = SpectralKVCache(cfg, max_blocks=6, device="cpu")
    other.store_block(4, SpectralEncoding(*[t[:16] for t in k]), SpectralEncoding(*[t[:16] for t in v]))
    other.store_block(1, SpectralEncoding(*[t[16:32] for t in k]), SpectralEncoding(*[t[16:32] for t in v]))
    for s in range(5):
        other.store_token(5, s, SpectralEncoding(*[t[32 + s] for t in k]), SpectralEncoding(*[t[32 + s] for t in v]))
    for a, b in zip(other._sides(), cache._sides()):
        assert all(torch.equal(x, y) for x, y in zip(a, b))
    assert torch.equal(other._block_fill, cache._block_fill)
    cache.copy_block(5, 2)
    assert torch.equal(cache.k_packed[2], cache.k_packed[5]) and int(cache._block_fill[2]) == 5
    cache.clear_block(5)
    assert cache.k_scales[5].abs().sum() == 0 and cache.memory_stats()["total_tokens"] == 37


def test_primary_mode_page_sizes_and_vllm_patch(monkeypatch):
    """Page sizing of the primary (packed) cache: the reference's formulas (vllm/engine.py:110-154), and the
    page-size patch on the installed vLLM's KV-cache specs."""
    from aitherkvcache_b200.vllm import engine
    monkeypatch.delenv("AITHER_TQ_MODE", raising=False)
    monkeypatch.setenv("AITHER_TQ_BITS", "4")
    assert not engine.is_primary_mode()
    assert engine.tq_dim_for_head(128) == 68 and engine.tq_page_size_bytes(16, 8, 128) == 2 * 16 * 8 * 68
    assert engine.tq_dim_for_head(128, bits=3) == 52 and engine.tq_dim_for_head(128, bits=2) == 36
    assert engine.align_page_size(17408) == 32768 and engine.align_page_size(16384) == 16384 and engine.align_page_size(0) == 0
    monkeypatch.setenv("AITHER_TQ_MODE", "tq35-primary")
    assert engine.is_primary_mode() and engine.tq_dim_for_head(128) == 64
    assert engine.tq_page_size_bytes(16, 8, 128) == 2 * 16 * 8 * 64
    monkeypatch.setenv("AITHER_TQ_MODE", "tq25")
    assert not engine.is_primary_mode() and engine.tq_dim_for_head(128) == 44
    monkeypatch.setenv("AITHER_TQ_MODE", "tq3-primary")
    assert engine.tq_dim_for_head(128) == 52
    vllm_spec = pytest.importorskip("vllm.v1.kv_cache_interface")
    import torch
    monkeypatch.setenv("AITHER_TQ_MODE", "tq4-primary")
    spec = vllm_spec.FullAttentionSpec(block_size=16, num_kv_heads=8, head_size=128, dtype=torch.uint8)
    stock = spec.real_page_size_bytes
    assert stock == 2 * 16 * 8 * 128
    try:
        assert engine.apply_tq_patches(bits=4)
        assert spec.real_page_size_bytes == 17408 and spec.page_size_bytes == 17408        # 16 x 8 x 2 records of 68 bytes
        from aitherkvcache_b200.vllm.backend import TurboQuantBackend
        assert TurboQuantBackend.get_kv_cache_shape(10, 16, 8, 128) == (10, 2, 16, 8, 68)
    finally:
        engine.remove_tq_patches()
    assert spec.real_page_size_bytes == stock
    monkeypatch.delenv("AITHER_TQ_MODE")
    from aitherkvcache_b200.vllm.backend import TurboQuantBackend
    assert TurboQuantBackend.get_kv_cache_shape(10, 16, 8, 128) == (10, 2, 16, 8, 128)


def test_backend_mixed_batch_routing_on_the_host():
    """TurboQuantImplBase.forward on a batch with chunks and single tokens, kernels replaced by recording fakes (no
    GPU): the prefill side sees length zero for the single-token sequences, the decode side for the others, every query
    row is written exactly once and by the right side; a batch of equal chunks skips the decode side."""
    import types
    from aitherkvcache_b200.vllm.backend import TurboQuantImplBase
    impl = TurboQuantImplBase()
    impl._tq_setup(4, 128, 0.1, 2, "auto")
    calls = {}

    def fake_prefill(layer, q, out, kv_cache, md):
        calls["prefill"] = (md.seq_lens.clone(), md.query_start_loc.clone(), getattr(md, "max_seq_len", None))
        qsl = md.query_start_loc.tolist()
        for s, n in enumerate(md.seq_lens.tolist()):
            out[qsl[s]:qsl[s + 1]] = 100.0 + s if n > 0 else 0.0      # the kernels write zeros for rows of empty sequences
        return True

    def fake_attend(layer, q, out, kv_cache, block_table, context_lens):
        calls["attend"] = (context_lens.clone(), q.clone())
        for s, n in enumerate(context_lens.tolist()):
            out[s] = 200.0 + s if n > 0 else 0.0

    impl._prefill, impl._attend = fake_prefill, fake_attend
    qsl = torch.tensor([0, 5, 6, 9, 10], dtype=torch.int32)            # chunk lengths 5, 1, 3, 1
    seq_lens = torch.tensor([50, 7, 3, 90], dtype=torch.int32)
    md = types.SimpleNamespace(num_actual_tokens=10, max_query_len=5, block_table=torch.zeros(4, 8, dtype=torch.int32),
                               seq_lens=seq_lens, query_start_loc=qsl, max_seq_len=90)
    query = torch.arange(10, dtype=torch.float32)[:, None].expand(10, 4 * 128).contiguous()
    out = torch.full((10, 4 * 128), -1.0)
    impl.forward(None, query, None, None, torch.zeros(1), md, output=out)
    assert calls["prefill"][0].tolist() == [50, 0, 3, 0] and calls["prefill"][2] == 90
    assert calls["attend"][0].tolist() == [0, 7, 0, 90]
    assert calls["attend"][1][:, 0, 0].tolist() == [0.0, 5.0, 6.0, 9.0]      # the first query row of every sequence
    rows = out[:, 0].tolist()
    assert rows == [100.0] * 5 + [201.0] + [102.0] * 3 + [203.0]
    # four equal chunks: nothing for the decode kernels to do
    calls.clear()
    md2 = types.SimpleNamespace(num_actual_tokens=8, max_query_len=2, block_table=torch.zeros(4, 8, dtype=torch.int32),
                                seq_lens=seq_lens, query_start_loc=torch.tensor([0, 2, 4, 6, 8], dtype=torch.int32))
    impl.forward(None, query[:8].contiguous(), None, None, torch.zeros(1), md2, output=torch.zeros(8, 4 * 128))
    assert "attend" not in calls and calls["prefill"][0].tolist() == [50, 7, 3, 90]


def test_ctypes_structures_match_the_header_layout(tmp_path):
    """Every parameter struct of include/akv_b200.h against its ctypes mirror: the C compiler's sizeof and the offset
    of every field, in order (gcc on the header itself; no library call)."""
    import ctypes, re, subprocess
    from aitherkvcache_b200 import _lib
    root = os.path.join(os.path.dirname(__file__), "..")
    header = open(os.path.join(root, "include", "akv_b200.h")).read()
    pairs = {"akv_tq_attn_params": _lib.TQAttnParams, "akv_tq_prefill_params": _lib.TQPrefillParams,
             "akv_tq_decode_step_params": _lib.TQDecodeStepParams, "akv_hybrid_tables": _lib.HybridTables,
             "akv_hybrid_attn_params": _lib.HybridAttnParams, "akv_hybrid_decode_step_params": _lib.HybridDecodeStepParams,
             "akv_p2p_merge_params": _lib.P2PMergeParams, "akv_tri_decode_params": _lib.TriDecodeParams}
    lines = ['#include <stdio.h>', '#include <stddef.h>', '#include "akv_b200.h"', 'int main(void) {']
    names = {}
    for cname in pairs:
        body = re.search(r"typedef struct %s \{(.*?)\} %s;" % (cname, cname), header, re.S).group(1)
        body = re.sub(r"/\*.*?\*/", "", body, flags=re.S)
        fields = []
        for decl in body.split(";"):
            decl = decl.strip()
            if not decl:
                continue
            # "const void* a" / "int64_t a, b, c" / "akv_tq_attn_params attn": the names are the last identifier of each part
            first, *rest = decl.split(",")
            fields.append(re.findall(r"[A-Za-z_][A-Za-z_0-9]*", first)[-1])
            fields += [re.findall(r"[A-Za-z_][A-Za-z_0-9]*", part)[-1] for part in rest]
        names[cname] = fields
        lines.append('printf("%s %%zu", sizeof(%s));' % (cname, cname))
        lines += ['printf(" %%zu", offsetof(%s, %s));' % (cname, f) for f in fields]
        lines.append('printf("\\n");')
    lines += ["return 0;", "}"]
    src = tmp_path / "layout.c"
    src.write_text("\n".join(lines))
    exe = tmp_path / "layout"
    subprocess.run(["gcc", "-std=c99", "-I", os.path.join(root, "include"), "-o", str(exe), str(src)], check=True)
    out = subprocess.run([str(exe)], check=True, capture_output=True, text=True).stdout.strip().splitlines()
    for line in out:
        cname, size, *offs = line.split()
        st = pairs[cname]
        assert ctypes.sizeof(st) == int(size), cname
        got = [getattr(st, f).offset for f, _ in st._fields_]
        assert got == [int(o) for o in offs], (cname, names[cname], [f for f, _ in st._fields_])
