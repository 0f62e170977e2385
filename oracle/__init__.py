"""CPU oracle for the compressed-KV hot path.

TEST INFRASTRUCTURE ONLY.  This package restates, in numpy, the arithmetic of
the reference's torch path (aither_kvcache/quantizer.py, packing.py,
fused_kv_update.py, fused_attention.py, hybrid_quantizer.py and
triattention/*).  It exists so the CUDA kernels can be checked on a machine
where the reference itself is not installed.  Only the test-suite, the
smoke check and the CPU-baseline leg of the benchmark may import it; the
product package never does.

Parity status: PINNED.  Every function here is checked in
tests/test_oracle_golden.py against fixtures under tests/golden/ that were
produced by importing the unmodified reference (tests/golden/make_golden.py).
"""
