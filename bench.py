#!/usr/bin/env python
"""Benchmark of the headline path: paged decode attention over a tq-t4nc (4-bit
TurboQuant) KV cache.

Workload (the benchmark specification's paged decode configuration): 16 sequences, context lengths uniform in
[4096, 32768] (torch CPU generator, seed 1), 32 query / 8 KV heads, head_dim 128,
block_size 16, block tables a random permutation of the physical blocks, K and V
N(0,1) fp16 encoded to 4-bit codes + float32 norms, one fp16 query token per sequence.

A step is one decode-attention pass over the whole batch.
  value    : KV-tokens/s with everything resident in HBM (CUDA events around the K timed steps); `timing`
             repeats that region and gives median / min / max
  e2e      : the same through the serving op tq::decode_step with HOST inputs - every step copies
             query, new K/V token, slot mapping, block table and sequence lengths from pinned host
             memory, encodes the new token into the cache, attends, and copies the output back
  roofline : algorithmic packed-KV bytes / duration of the split-K kernel alone (events recorded
             around that launch inside the library)
  parity   : measured in the same run, outside the timed regions: attention output against the CPU
             oracle, packed codes against the oracle's encoder with the fraction of coordinates
             within 1e-6 of a codebook boundary
  splitk   : the long-context configurations, one batch sharded by key range over the N ranks:
             local split-K kernel -> one NCCL all-gather of the (m, l, acc) partials -> LSE merge,
             replayed as a CUDA graph, with the per-phase times of an eager pass beside it
  secondary: (N = 1) the other configured kernels on their shapes
With --gpus N (torchrun) every rank runs its own batch of 16 sequences for the headline value (batched
decode shards by sequence, no collective: weak scaling); the `splitk` entries are strong scaling.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
"""
import argparse
import json
import math
import os
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

import numpy as np  # noqa: E402
import torch  # noqa: E402

H_KV, H_Q, D, BS, BITS = 8, 32, 128, 16, 4
NUM_SEQS = 16
PD = D * BITS // 8
METRIC = "paged TQ4 decode-attn KV-tokens/s"
UNIT = "KV-tokens/s"
WORKLOAD = ("paged decode attention, tq-t4nc cache: 16 seqs, ctx U[4096,32768] seed 1, 32Q/8KV heads, "
            "head_dim 128, block_size 16, permuted block tables")

# dram__bytes_read.sum + dram__bytes_write.sum of ONE launch of the named kernel on the rank-0 headline
# workload, from the ncu capture summarised under profiles/ (the file is named after the kernel).  A kernel
# that is not listed here has no capture and its roofline.traffic is null.
NCU_TRAFFIC_BYTES = {
    "tq4_attn_tma_kernel": 281_556_000,         # 4.362 TB/s x 64.544 us
    "tq4_attn_streamk4_kernel": 281_600_000,
}


def context_lengths(rank=0):
    g = torch.Generator().manual_seed(1 + 1000 * rank)
    return torch.randint(4096, 32769, (NUM_SEQS,), generator=g)


def peak_hbm():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
    except Exception:
        return 6650.0, "fallback (6.65 TB/s)"


def host_threads():
    try:
        return len(os.sched_getaffinity(0))
    except Exception:
        return os.cpu_count() or 1


class ClockSampler:
    """SM clock and throttle reasons sampled while the timed region runs: NVML polled from a thread,
    else nvidia-smi every 200 ms."""
    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    _NVML_REASONS = ((0x8, "hw_slowdown"), (0x40, "hw_thermal_slowdown"), (0x20, "sw_thermal_slowdown"),
                     (0x4, "sw_power_cap"))

    def __init__(self, gpu_index):
        self.gpu, self.proc, self.path = gpu_index, None, None
        self.thread, self.samples, self.halt, self.max_mhz = None, [], False, None

    def _start_nvml(self):
        """Poll NVML from a thread (a timed region of a few milliseconds is over before nvidia-smi's
        first 200 ms tick).  Read-only queries."""
        import threading
        import pynvml
        pynvml.nvmlInit()
        try:
            uuid = str(torch.cuda.get_device_properties(self.gpu).uuid)
            h = pynvml.nvmlDeviceGetHandleByUUID(("GPU-" + uuid) if not uuid.startswith("GPU-") else uuid)
        except Exception:
            h = pynvml.nvmlDeviceGetHandleByIndex(self.gpu)
        self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(h, pynvml.NVML_CLOCK_SM))

        def poll():
            while not self.halt:
                try:
                    self.samples.append((float(pynvml.nvmlDeviceGetClockInfo(h, pynvml.NVML_CLOCK_SM)),
                                         int(pynvml.nvmlDeviceGetCurrentClocksThrottleReasons(h))))
                except Exception:
                    break
                time.sleep(0.0005)

        self.thread = threading.Thread(target=poll, daemon=True)
        self.thread.start()

    def start(self):
        try:
            self._start_nvml()
            return
        except Exception:
            self.thread = None
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "200",
                 "-i", str(self.gpu)], stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        if self.thread is not None:
            self.halt = True
            self.thread.join(timeout=2)
            if self.samples:
                mask = 0
                for _, m in self.samples:
                    mask |= m
                return {"sm_mhz": float(np.median([c for c, _ in self.samples])), "sm_max_mhz": self.max_mhz,
                        "reasons": sorted(n for bit, n in self._NVML_REASONS if mask & bit),
                        "samples": len(self.samples), "source": "nvml, polled during the timed region"}
            return out
        if self.proc is None:
            return out
        time.sleep(0.25)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            pass
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        try:
            for line in open(self.path):
                f = [x.strip() for x in line.split(",")]
                if len(f) < 9:
                    continue
                try:
                    sm.append(float(f[1])); mx.append(float(f[2]))
                except ValueError:
                    continue
                for n, v in zip(names, f[5:9]):
                    if v.lower().startswith("active"):
                        reasons.add(n)
            os.unlink(self.path)
        except Exception:
            pass
        if sm:
            out = {"sm_mhz": float(np.median(sm)), "sm_max_mhz": float(max(mx)), "reasons": sorted(reasons),
                   "samples": len(sm)}
        return out


def block_tables_for(ctx, seed):
    nblk = [(int(c) + BS - 1) // BS for c in ctx]
    total = sum(nblk)
    perm = torch.randperm(total, generator=torch.Generator().manual_seed(seed))
    bt = torch.zeros(len(ctx), max(nblk), dtype=torch.int32)
    p = 0
    for s, n in enumerate(nblk):
        bt[s, :n] = perm[p:p + n].to(torch.int32)
        p += n
    return bt, nblk, total


def build_cache(tq, ctx, device, seed, replicas, keep_sample=0):
    """Encode N(0,1) fp16 K/V into `replicas` paged caches with permuted block tables (on the GPU).
    keep_sample > 0: also return the first `keep_sample` K vectors of sequence 0 (fp16) and their slots."""
    from aitherkvcache_b200 import fused_tq4_kv_update
    bt, nblk, total = block_tables_for(ctx, seed)
    caches, sample = [], None
    gg = torch.Generator(device=device).manual_seed(seed)
    for r in range(replicas):
        kp = torch.zeros(total, BS, H_KV, PD, dtype=torch.uint8, device=device)
        vp = torch.zeros_like(kp)
        kn = torch.zeros(total, BS, H_KV, device=device)
        vn = torch.zeros_like(kn)
        for s, n in enumerate(nblk):
            blocks = bt[s, :n].to(device).long()
            slots = (blocks[:, None] * BS + torch.arange(BS, device=device)[None, :]).reshape(-1)[:int(ctx[s])]
            for packed, norms in ((kp, kn), (vp, vn)):
                x = torch.randn(int(ctx[s]), H_KV, D, generator=gg, device=device, dtype=torch.float32).half()
                fused_tq4_kv_update(x, slots, packed, norms, tq.rotation, tq.boundaries_inner, BS,
                                    rotation_t=tq.rotation_T)
                if keep_sample and sample is None:
                    sample = (x[:keep_sample].cpu(), slots[:keep_sample].cpu())
        caches.append((kp, kn, vp, vn))
    return caches, bt.to(device), total, sample


def parity_report(tq, cache, bt, ctx, q, out, sample):
    """Parity figures of this very run (outside every timed region): the attention output of the
    shortest and the longest sequence against the CPU oracle (decode -> fp16 -> dense attention), and
    a sample of the K vectors the cache was built from against the oracle's encoder."""
    from oracle import tq as otq
    kp, kn, vp, vn = (t.cpu().numpy() for t in cache)
    R, cent = tq.rotation.cpu().numpy(), tq.centroids.cpu().numpy()
    bnd = tq.boundaries_inner.cpu().numpy()
    order = np.argsort(ctx.numpy())
    pick = np.array([order[0], order[-1]])
    ref = otq.paged_attention_decode_sdpa(q.cpu().numpy()[pick], kp, kn, vp, vn, bt.cpu().numpy()[pick],
                                          ctx.numpy()[pick].astype(np.int64), R, cent, BITS, 1.0 / math.sqrt(D), BS)
    err = float(np.abs(out.float().cpu().numpy()[pick] - ref.astype(np.float32)).max())
    x, slots = sample
    ref_p, ref_n, margin = otq.encode(x.numpy(), R, bnd, BITS, return_margin=True)
    got_p = cache[0].reshape(-1, H_KV, PD)[slots.to(cache[0].device)].cpu().numpy()
    got_n = cache[1].reshape(-1, H_KV)[slots.to(cache[1].device)].cpu().numpy()
    a, b = otq.unpack(got_p, D, BITS), otq.unpack(ref_p, D, BITS)
    diff = a != b
    near = margin.reshape(diff.shape) < 1e-6
    return {"max_abs_err": err, "tolerance": 2e-3,
            "attention_checked": f"sequences {int(pick[0])} ({int(ctx[pick[0]])} tokens) and {int(pick[1])} "
                                 f"({int(ctx[pick[1]])} tokens), 32 query heads, vs oracle decode->fp16->attention",
            "boundary_window_frac": float(near.mean()), "code_mismatch_frac": float(diff.mean()),
            "code_mismatch_outside_window": int((diff & ~near).sum()),
            "norms_bit_equal": bool(np.array_equal(got_n.view(np.uint32), ref_n.view(np.uint32))),
            "codes_checked": int(diff.size)}


def cpu_baseline(tq, cache, bt, ctx, q, repeats=2):
    """The reference's CPU route (torch float32: gather -> TurboQuant.decode -> fp16 -> SDPA, all host
    threads; restated in oracle/tq_torch.py) timed on all 16 sequences of the workload."""
    from oracle import tq_torch as ott
    torch.set_num_threads(host_threads())
    kp, kn, vp, vn = (t.cpu() for t in cache)
    R, cent = tq.rotation.cpu(), tq.centroids.cpu()
    btc, qc = bt.cpu(), q.cpu()
    ott.paged_decode_attention(qc, kp, kn, vp, vn, btc, ctx, R, cent, block_size=BS, sequences=[0])   # warm-up
    t0 = time.perf_counter()
    for _ in range(repeats):
        ott.paged_decode_attention(qc, kp, kn, vp, vn, btc, ctx, R, cent, block_size=BS)
    el = (time.perf_counter() - t0) / repeats
    tokens = int(ctx.sum())
    return {"value": tokens / el, "unit": UNIT, "cores": torch.get_num_threads(), "kind": "port",
            "sample": f"all {NUM_SEQS} sequences ({tokens} KV-tokens) x {repeats} passes, {el:.2f} s per pass of torch "
                      "float32 gather -> decode -> fp16 -> SDPA (per-sequence gathers included)"}


def run_reference(args, rank, world):
    """--impl reference: the reference's CPU torch route for the same workload, on the host cores.  The
    reference is Python and does not travel to the GPU box; its route is restated in oracle/tq_torch.py
    (same torch calls, float32 sgemm, all host threads).  The packed cache is built on the host too, so
    nothing of the product library is loaded."""
    if rank != 0:
        return
    from oracle import tq_torch as ott
    threads = host_threads()
    torch.set_num_threads(threads)
    ctx = context_lengths(0)
    bt, nblk, total = block_tables_for(ctx, 1)
    # the reference's own tables (seed-42 rotation, 16-level Lloyd-Max codebook), stored with the fixtures
    with np.load(os.path.join(ROOT, "tests", "golden", "tq_d128_b4.npz")) as z:
        R, cent, bnd = (torch.from_numpy(z[k].astype(np.float32)) for k in ("rotation", "centroids", "boundaries"))
    g = torch.Generator().manual_seed(1)
    kp = torch.zeros(total, BS, H_KV, PD, dtype=torch.uint8)
    vp = torch.zeros_like(kp)
    kn = torch.zeros(total, BS, H_KV)
    vn = torch.zeros_like(kn)
    for s, n in enumerate(nblk):
        c = int(ctx[s])
        slots = (bt[s, :n].long()[:, None] * BS + torch.arange(BS)[None, :]).reshape(-1)[:c]
        for packed, norms in ((kp, kn), (vp, vn)):
            p_, n_ = ott.encode4(torch.randn(c, H_KV, D, generator=g).half(), R, bnd)
            packed.reshape(-1, H_KV, PD)[slots] = p_
            norms.reshape(-1, H_KV)[slots] = n_
    q = torch.randn(NUM_SEQS, H_Q, D, generator=torch.Generator().manual_seed(2)).half()
    tokens = int(ctx.sum())
    times = []
    for i in range(args.warmup + args.steps):
        t0 = time.perf_counter()
        ott.paged_decode_attention(q, kp, kn, vp, vn, bt, ctx, R, cent, block_size=BS)
        if i >= args.warmup:
            times.append(time.perf_counter() - t0)
    el = float(np.sum(times))
    value = tokens * len(times) / el
    sample = (f"all {NUM_SEQS} sequences ({tokens} KV-tokens) every step; torch float32 gather -> decode -> fp16 -> "
              f"SDPA on {threads} host threads")
    line = {"impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * el / len(times),
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
            "data": "synthetic",
            "config": {"workload": WORKLOAD, "kv_tokens_per_gpu": tokens,
                       "packed_kv_bytes_per_step": tokens * H_KV * 2 * (PD + 4)},
            "timing": {"ms_per_step_median": 1e3 * float(np.median(times)), "ms_per_step_min": 1e3 * float(np.min(times)),
                       "ms_per_step_max": 1e3 * float(np.max(times))},
            "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": "port", "sample": sample},
            "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line))


def _event_time(fn, steps, warmup):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / steps


def secondary_kernels(steps, warmup, dev):
    """The other configured kernels on their shapes (configs 0, 2, 3 of the benchmark specification), device-resident,
    CUDA events, inputs larger than L2: encode / decode / fused paged prefill write at 4, 3, 2 bits on
    524 288 vectors, decode attention at 3 and 2 bits and with the hybrid tq35 layout on the headline shapes,
    chunked prefill attention over the packed 4-bit cache."""
    from aitherkvcache_b200 import TQPagedAttention, TurboQuant, fused_tq4_kv_update
    from aitherkvcache_b200.hybrid_quantizer import HybridPagedAttention, HybridTurboQuant
    peak, _ = peak_hbm()
    res = {}
    g = torch.Generator(device=dev).manual_seed(0)
    x = torch.randn(4 * 1024 * 8 * 16, D, generator=g, device=dev).half()       # 524 288 vectors (prefill-write size)
    n = x.shape[0]

    def rate(ms, units, bytes_per_unit):
        gbs = units * bytes_per_unit / ms / 1e6
        return {"Mvec/s": units / ms / 1e3, "GB/s": gbs, "frac_of_measured_peak": gbs / peak, "ms": ms}

    for bits in (4, 3, 2):
        tq = TurboQuant(head_dim=D, bits=bits, device=str(dev))
        packed, norms = tq.encode(x)
        by = 256 + D * bits // 8 + 4
        res[f"tq{bits}_encode"] = rate(_event_time(lambda: tq.encode(x), steps, warmup), n, by)
        res[f"tq{bits}_decode"] = rate(_event_time(lambda: tq.decode(packed, norms), steps, warmup), n, by)
        T = 16 * 2048            # fused prefill write: 16 seqs x 2048 tokens x 8 heads into random paged blocks
        xk = x[:T * H_KV].reshape(T, H_KV, D)
        nblk = T // BS
        perm = torch.randperm(nblk, generator=torch.Generator().manual_seed(1)).to(dev)
        slots = (perm[:, None] * BS + torch.arange(BS, device=dev)[None]).reshape(-1)
        outp = torch.zeros(nblk, BS, H_KV, D * bits // 8, dtype=torch.uint8, device=dev)
        outn = torch.zeros(nblk, BS, H_KV, device=dev)
        ms = _event_time(lambda: fused_tq4_kv_update(xk, slots, outp, outn, tq.rotation, tq.boundaries_inner, BS,
                                                     rotation_t=tq.rotation_T), steps, warmup)
        res[f"tq{bits}_paged_write"] = rate(ms, T * H_KV, by)
    ctx = context_lengths(0)
    total_ctx = int(ctx.sum())
    bt, nblk, total = block_tables_for(ctx, 1)
    bt = bt.to(dev)
    ctx_dev = ctx.to(torch.int32).to(dev)
    q = torch.randn(NUM_SEQS, H_Q, D, generator=g, device=dev).half()
    for bits in (3, 2):
        tq = TurboQuant(head_dim=D, bits=bits, device=str(dev))
        pd = D * bits // 8
        kp = torch.randint(0, 256, (total, BS, H_KV, pd), dtype=torch.uint8, device=dev)
        vp = torch.randint(0, 256, (total, BS, H_KV, pd), dtype=torch.uint8, device=dev)
        kn = torch.rand(total, BS, H_KV, device=dev) + 10.8
        vn = torch.rand(total, BS, H_KV, device=dev) + 10.8
        attn = TQPagedAttention(tq, H_Q)
        ms = _event_time(lambda: attn.forward(q, kp, kn, vp, vn, bt, ctx_dev), steps, warmup)
        by = total_ctx * H_KV * 2 * (pd + 4)
        res[f"tq{bits}_decode_attn"] = {"KV-tokens/s": total_ctx / ms * 1e3, "GB/s": by / ms / 1e6,
                                        "frac_of_measured_peak": by / ms / 1e6 / peak, "ms": ms}
    # chunked prefill over the packed 4-bit cache: a 2048-token chunk of one sequence with 30 000 tokens before it
    tq = TurboQuant(head_dim=D, bits=4, device=str(dev))
    attn = TQPagedAttention(tq, H_Q)
    past, chunk = 30000, 2048
    pnb = (past + chunk + BS - 1) // BS
    kp = torch.randint(0, 256, (pnb, BS, H_KV, D // 2), dtype=torch.uint8, device=dev)
    vp = torch.randint(0, 256, (pnb, BS, H_KV, D // 2), dtype=torch.uint8, device=dev)
    kn = torch.rand(pnb, BS, H_KV, device=dev) + 0.5
    vn = torch.rand(pnb, BS, H_KV, device=dev) + 0.5
    pbt = torch.randperm(pnb, generator=torch.Generator().manual_seed(2)).to(torch.int32).reshape(1, pnb).to(dev)
    qp = torch.randn(chunk, H_Q, D, generator=g, device=dev).half()
    sl = torch.tensor([past + chunk], dtype=torch.int32, device=dev)
    qsl = torch.tensor([0, chunk], dtype=torch.int32, device=dev)
    outp = torch.empty_like(qp)
    pairs = chunk * past + chunk * (chunk + 1) // 2            # (query token, key) pairs under the causal mask
    # "staged": the longest sequence is known on the host (as in vLLM's metadata), so the codes become fp16 operand images
    # once per call; "in_kernel": they are decoded inside the attention kernel, once per 128 query rows
    for name, msl in (("tq4_chunked_prefill", past + chunk), ("tq4_chunked_prefill_in_kernel_decode", None)):
        if attn.prefill(qp, kp, kn, vp, vn, pbt, sl, qsl, block_size=BS, num_kv_heads=H_KV, out=outp, max_seq_len=msl) is None:
            raise RuntimeError("the chunked-prefill kernel refused the benchmark shape")
        calls = max(3, steps // 8)      # a burst at full clock; hundreds of back-to-back calls reach the board's power limit
        ms = _event_time(lambda: attn.prefill(qp, kp, kn, vp, vn, pbt, sl, qsl, block_size=BS, num_kv_heads=H_KV, out=outp,
                                              max_seq_len=msl), calls, 2)
        res[name] = {"ms": ms, "calls_timed": calls, "query_tokens": chunk, "past_tokens": past,
                     "TFLOP/s": pairs * H_Q * D * 4 / ms / 1e9, "query-tokens/s": chunk / ms * 1e3}
    htq = HybridTurboQuant(D, "tq35", device=str(dev))
    htq.calibrate_uniform()
    xh = torch.randn(8 * 4096 * 8, D, generator=g, device=dev).half()
    ph = htq.encode(xh)
    nh = xh.shape[0]
    res["tq35_encode"] = rate(_event_time(lambda: htq.encode(xh), steps, warmup), nh, 320)
    res["tq35_decode"] = rate(_event_time(lambda: htq.decode(ph), steps, warmup), nh, 576)
    kc = torch.randint(0, 256, (total, BS, H_KV, 64), dtype=torch.uint8, device=dev)
    kc[..., 32:36] = htq.encode(torch.randn(1, D, device=dev))[0, 32:36]       # sane fp16 norm fields
    kc[..., 60:64] = kc[..., 32:36]
    hattn = HybridPagedAttention(htq, H_Q)
    ms = _event_time(lambda: hattn.forward(q, kc, kc, bt, ctx_dev), max(3, steps // 4), 3)
    by = total_ctx * H_KV * 128
    res["tq35_decode_attn"] = {"KV-tokens/s": total_ctx / ms * 1e3, "GB/s": by / ms / 1e6,
                               "frac_of_measured_peak": by / ms / 1e6 / peak, "ms": ms}
    # the same prefill chunk over tq35 records (records decoded into the staged operand images, attention in the original domain)
    if hattn.prefill(qp, kc, kc, pbt, sl, qsl, block_size=BS, num_kv_heads=H_KV, out=outp, max_seq_len=past + chunk) is None:
        raise RuntimeError("the chunked-prefill kernel refused the tq35 benchmark shape")
    ms = _event_time(lambda: hattn.prefill(qp, kc, kc, pbt, sl, qsl, block_size=BS, num_kv_heads=H_KV, out=outp,
                                           max_seq_len=past + chunk), max(3, steps // 8), 2)
    res["tq35_chunked_prefill"] = {"ms": ms, "query_tokens": chunk, "past_tokens": past,
                                   "TFLOP/s": pairs * H_Q * D * 4 / ms / 1e9, "query-tokens/s": chunk / ms * 1e3}
    return res


class SplitK:
    """One long-context batch whose key range is split over the ranks.  Every step: the local split-K
    call writes this rank's un-normalised (m, l, acc) partials, the partials are exchanged, a local
    kernel merges them by log-sum-exp.  Two exchanges are measured: "p2p" - the library's own kernels
    over NVLink peer memory (peer stores + flag words, akv_p2p_lse_merge) - and "nccl" - one
    all_gather_into_tensor followed by akv_lse_merge.  With one rank the library's own call (kernel +
    in-library merge) is the step.  Replicas of the local shard are cycled so that a step never finds its
    inputs in L2."""

    def __init__(self, name, world, rank, dev, rows, local_calls, direct_calls, merge, shard_bytes, kv_tokens,
                 workload, rotation=None, out=None, batch=0):
        self.name, self.world, self.rank, self.dev = name, world, rank, dev
        self.local_calls, self.direct_calls, self.merge = local_calls, direct_calls, merge
        self.shard_bytes, self.kv_tokens, self.workload = shard_bytes, kv_tokens, workload
        self.raw = torch.empty(rows, D + 2, dtype=torch.float32, device=dev)
        self.parts = torch.empty(world, rows, D + 2, dtype=torch.float32, device=dev)
        self.nrep = len(local_calls)
        self.rotation, self.out, self.batch = rotation, out, batch
        self.exchange, self.exchange_error = None, None
        if world > 1:
            try:
                from aitherkvcache_b200.parallel import PeerExchange
                self.exchange = PeerExchange(batch, H_Q, D, dev)
            except Exception as exc:      # noqa: BLE001 - symmetric memory is optional; NCCL remains
                self.exchange_error = f"{type(exc).__name__}: {exc}"[:200]

    def step(self, r, ev=None, marks=None, mode="nccl"):
        import torch.distributed as dist
        if self.world == 1:
            self.direct_calls[r % self.nrep](ev)
            return
        self.local_calls[r % self.nrep](self.raw, ev)
        if marks:
            marks[0].record()
        if mode == "p2p":
            from aitherkvcache_b200.parallel import p2p_merge_partials
            p2p_merge_partials(self.exchange, self.raw, rotation=self.rotation, out=self.out)
            if marks:
                marks[1].record()
            return
        dist.all_gather_into_tensor(self.parts, self.raw)
        if marks:
            marks[1].record()
        self.merge(self.parts)

    def measure(self, steps, warmup, barrier, allreduce_max):
        if self.world == 1:
            return self._measure_mode("single", steps, warmup, barrier, allreduce_max)
        res = {"nccl": self._measure_mode("nccl", steps, warmup, barrier, allreduce_max)}
        ref_out = self.out.clone()
        if self.exchange is not None:
            res["p2p"] = self._measure_mode("p2p", steps, warmup, barrier, allreduce_max)
            res["p2p"]["max_abs_diff_vs_nccl"] = float((self.out.float() - ref_out.float()).abs().max())
        best = min(res, key=lambda k: res[k]["ms_per_step"])
        top = dict(res[best])
        top["exchange"] = best
        top["variants"] = {k: {kk: v[kk] for kk in ("ms_per_step", "value", "eager", "launch", "library_launches_per_step")
                               if kk in v} for k, v in res.items()}
        if self.exchange_error:
            top["p2p_unavailable"] = self.exchange_error
        return top

    def _measure_mode(self, mode, steps, warmup, barrier, allreduce_max):
        from aitherkvcache_b200 import _lib
        L = _lib.lib()
        for i in range(warmup):
            self.step(i, mode=mode)
        # eager pass: per-phase times (events between the phases) and the split-K kernel alone
        ev = lambda: torch.cuda.Event(enable_timing=True)      # noqa: E731
        rec = [(ev(), ev(), ev(), ev(), ev(), ev()) for _ in range(steps)]
        barrier()
        for i, (a, k0, k1, m0, m1, b) in enumerate(rec):
            a.record()
            self.step(i, (k0, k1), (m0, m1) if self.world > 1 else None, mode=mode)
            b.record()
        barrier()
        kernel_ms = float(np.mean([k0.elapsed_time(k1) for _, k0, k1, _, _, _ in rec]))
        eager_ms = float(np.mean([a.elapsed_time(b) for a, _, _, _, _, b in rec]))
        if self.world > 1:
            local_ms = float(np.mean([a.elapsed_time(m0) for a, _, _, m0, _, _ in rec]))
            gather_ms = float(np.mean([m0.elapsed_time(m1) for _, _, _, m0, m1, _ in rec]))
            merge_ms = float(np.mean([m1.elapsed_time(b) for _, _, _, _, m1, b in rec]))
        else:
            local_ms, gather_ms, merge_ms = eager_ms, 0.0, 0.0
        kernel_name = L.akv_last_split_kernel().decode()
        # the step as a CUDA graph (the exchange is captured with it), one graph per replica
        launch, graphs = "cuda graph replay", []
        n0 = L.akv_launch_count()
        try:
            side = torch.cuda.Stream(device=self.dev)
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                for r in range(self.nrep):
                    self.step(r, mode=mode)
            torch.cuda.current_stream().wait_stream(side)
            n0 = L.akv_launch_count()
            for r in range(self.nrep):
                gr = torch.cuda.CUDAGraph()
                with torch.cuda.graph(gr):
                    self.step(r, mode=mode)
                graphs.append(gr)
        except Exception as exc:      # noqa: BLE001 - keep measuring, but say how
            graphs, launch = [], f"eager (graph capture failed: {type(exc).__name__}: {exc})"[:200]
            torch.cuda.synchronize()
        launches = (L.akv_launch_count() - n0) // max(1, len(graphs)) if graphs else None
        run = (lambda i: graphs[i % len(graphs)].replay()) if graphs else (lambda i: self.step(i, mode=mode))
        for i in range(warmup):
            run(i)
        regions = []
        for _ in range(5):
            barrier()
            e0, e1 = ev(), ev()
            e0.record()
            for i in range(steps):
                run(i)
            e1.record()
            barrier()
            regions.append(e0.elapsed_time(e1) / steps)
        t = allreduce_max([kernel_ms, local_ms, gather_ms, merge_ms, eager_ms] + regions)
        kernel_ms, local_ms, gather_ms, merge_ms, eager_ms = t[:5]
        regions = t[5:]
        ms = float(np.median(regions))
        peak, _ = peak_hbm()
        achieved = self.shard_bytes / (kernel_ms * 1e-3) / 1e9
        phases = ({"local_call_ms": local_ms, "exchange_and_merge_ms": gather_ms} if mode == "p2p" else
                  {"local_call_ms": local_ms, "all_gather_ms": gather_ms, "merge_ms": merge_ms})
        return {"workload": self.workload, "n_gpus": self.world, "scaling": "strong", "launch": launch,
                "ms_per_step": ms, "ms_per_step_min": float(min(regions)), "ms_per_step_max": float(max(regions)),
                "value": self.kv_tokens / (ms * 1e-3), "unit": UNIT, "kv_tokens_per_step": self.kv_tokens,
                "eager": dict(phases, ms_per_step=eager_ms,
                              note="max over ranks of per-rank means; CUDA events between the phases"),
                "kernel": kernel_name, "kernel_ms": kernel_ms, "library_launches_per_step": launches,
                "replicas_cycled": self.nrep, "shard_bytes_per_rank": self.shard_bytes,
                "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                             "per": "rank (max over ranks of the kernel time)"}}


def splitk_tri(world, rank, dev):
    """TriAttention decode_step, batch 8, 131072 keys, F=12 int4 coefficients (26 B per token, head and side)."""
    from aitherkvcache_b200.parallel import merge_partials, shard_range
    from aitherkvcache_b200.triattention import SpectralEncoding, TriAttention, TriAttentionConfig
    B, S, F = 8, 131072, 12
    cfg = TriAttentionConfig(head_dim=D, num_freqs=F, coeff_bits=4, num_kv_heads=H_KV, num_query_heads=H_Q,
                             rope_base=1_000_000.0)
    tri = TriAttention(cfg, device=str(dev))
    lo, hi = shard_range(S, rank, world, 32)
    gsel = torch.Generator().manual_seed(2)
    s_i = torch.exp(-torch.arange(64, dtype=torch.float32) / 16.0)
    pair_scale = torch.stack([s_i[torch.randperm(64, generator=gsel)] for _ in range(H_KV)]).to(dev)
    gg = torch.Generator(device=dev).manual_seed(2 + rank)
    encs = []
    for is_key in (True, False):
        parts = []
        for b in range(B):          # one batch element at a time keeps the fp16 staging tensor small
            x = torch.randn(hi - lo, H_KV, 64, 2, generator=gg, device=dev)
            if is_key:
                x = x * pair_scale[None, :, :, None]
            parts.append(tri.encoder.encode(x.reshape(1, hi - lo, H_KV, D).half()))
        encs.append(SpectralEncoding(*[torch.cat([p_[i] for p_ in parts]) for i in range(3)]))
    shard_bytes = B * (hi - lo) * H_KV * 2 * (2 * F + 2)
    nrep = max(2, -(-300_000_000 // max(1, shard_bytes)))
    reps = [encs] + [[SpectralEncoding(*[t.clone() for t in e]) for e in encs] for _ in range(nrep - 1)]
    q = torch.randn(B, H_Q, D, generator=torch.Generator().manual_seed(3)).half().to(dev)
    out = torch.empty(B, H_Q, D, dtype=torch.float32, device=dev)
    local = [(lambda raw, ev, k=k, v=v: tri._run(q, k, v, None, None, raw_out=raw, key_pos_start=lo,
                                                 query_pos_default=S, kernel_events=ev)) for k, v in reps]
    direct = [(lambda ev, k=k, v=v: tri._run(q, k, v, None, None, out=out, kernel_events=ev)) for k, v in reps]
    return SplitK("tri128k", world, rank, dev, B * H_Q, local, direct,
                  lambda parts: merge_partials(parts, B, H_Q, D, out=out), shard_bytes, B * S, rotation=None, out=out,
                  batch=B, workload=
                  "TriAttention decode_step: batch 8, 131072 keys (positions 0..131071, query at 131072), F=12 int4 "
                  "coefficients, 32Q/8KV heads, head_dim 128, rope_base 1e6, pre-RoPE keys with shuffled exp(-i/16) "
                  "pair scales; key range split over the ranks"), out


def splitk_tq4(world, rank, dev):
    """tq-t4nc paged decode attention over one long batch: 8 sequences of 131072 tokens, every rank holding a
    contiguous block range of every sequence in its own paged cache."""
    from aitherkvcache_b200 import TQPagedAttention, TurboQuant, fused_tq4_kv_update
    from aitherkvcache_b200.parallel import merge_partials, shard_range
    B, S = 8, 131072
    tq = TurboQuant(head_dim=D, bits=BITS, device=str(dev))
    lo, hi = shard_range(S, rank, world, BS)
    n_loc = hi - lo
    nb = n_loc // BS
    total = B * nb
    perm = torch.randperm(total, generator=torch.Generator().manual_seed(7 + rank))
    bt = perm.reshape(B, nb).to(torch.int32).to(dev)
    kp = torch.zeros(total, BS, H_KV, PD, dtype=torch.uint8, device=dev)
    vp = torch.zeros_like(kp)
    kn = torch.zeros(total, BS, H_KV, device=dev)
    vn = torch.zeros_like(kn)
    gg = torch.Generator(device=dev).manual_seed(11 + rank)
    for s in range(B):
        slots = (bt[s].long()[:, None] * BS + torch.arange(BS, device=dev)[None, :]).reshape(-1)
        for packed, norms in ((kp, kn), (vp, vn)):
            x = torch.randn(n_loc, H_KV, D, generator=gg, device=dev).half()
            fused_tq4_kv_update(x, slots, packed, norms, tq.rotation, tq.boundaries_inner, BS, rotation_t=tq.rotation_T)
            del x
    shard_bytes = B * n_loc * H_KV * 2 * (PD + 4)
    nrep = max(2, -(-300_000_000 // max(1, shard_bytes)))
    reps = [(kp, kn, vp, vn)] + [tuple(t.clone() for t in (kp, kn, vp, vn)) for _ in range(nrep - 1)]
    ctx_loc = torch.full((B,), n_loc, dtype=torch.int32, device=dev)
    q = torch.randn(B, H_Q, D, generator=torch.Generator().manual_seed(5)).half().to(dev)
    out = torch.empty(B, H_Q, D, dtype=torch.float16, device=dev)
    attn = TQPagedAttention(tq, H_Q)
    local = [(lambda raw, ev, c=c: attn.forward(q, c[0], c[1], c[2], c[3], bt, ctx_loc, raw_out=raw, kernel_events=ev))
             for c in reps]
    direct = [(lambda ev, c=c: attn.forward(q, c[0], c[1], c[2], c[3], bt, ctx_loc, out=out, kernel_events=ev))
              for c in reps]
    return SplitK("tq4_128k", world, rank, dev, B * H_Q, local, direct,
                  lambda parts: merge_partials(parts, B, H_Q, D, rotation=tq.rotation, out=out), shard_bytes, B * S,
                  rotation=tq.rotation, out=out, batch=B, workload=
                  "tq-t4nc paged decode attention: 8 sequences x 131072 tokens, 32Q/8KV heads, head_dim 128, "
                  "block_size 16, permuted block tables; each sequence's block range split over the ranks"), out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=None,
                    help="timed steps (default 1000: a timed region of 0.1 s, long enough for the clock sampler; "
                         "10 for --impl reference, whose steps take seconds)")
    ap.add_argument("--warmup", type=int, default=None, help="untimed steps first (default 20; 3 for --impl reference)")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--replicas", type=int, default=2, help="cache copies cycled through (L2 defeat)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-splitk", action="store_true", help="skip the long-context split-K configurations")
    ap.add_argument("--no-secondary", action="store_true", help="skip the secondary kernels (N = 1 only)")
    ap.add_argument("--no-parity", action="store_true")
    ap.add_argument("--e2e-eager", action="store_true", help="end-to-end loop without CUDA-graph capture")
    args = ap.parse_args()
    slow = args.impl == "reference"
    if args.steps is None:
        args.steps = 10 if slow else 1000
    if args.warmup is None:
        args.warmup = 3 if slow else 20
    args.warmup = max(args.warmup, 3)

    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    if args.impl == "reference":
        run_reference(args, rank, world)
        return

    import torch.distributed as dist
    from aitherkvcache_b200 import TQPagedAttention, TurboQuant, _lib
    from aitherkvcache_b200.vllm import ops

    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    L = _lib.lib()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def allreduce_max(values):
        t = torch.tensor(values, dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return [float(v) for v in t]

    tq = TurboQuant(head_dim=D, bits=BITS, device=str(dev))
    ctx = context_lengths(rank)
    total_ctx = int(ctx.sum())
    caches, bt, total_blocks, sample = build_cache(tq, ctx, dev, seed=1 + rank, replicas=args.replicas,
                                                   keep_sample=4096)
    ctx_dev = ctx.to(torch.int32).to(dev)
    q_host = torch.randn(NUM_SEQS, H_Q, D, generator=torch.Generator().manual_seed(2 + rank)).half()
    q = q_host.to(dev)
    attn = TQPagedAttention(tq, H_Q)
    out = torch.empty(NUM_SEQS, H_Q, D, dtype=torch.float16, device=dev)
    kv_bytes = total_ctx * H_KV * 2 * (PD + 4)          # algorithmic packed-KV bytes per step

    def step(i, events=None):
        kp, kn, vp, vn = caches[i % len(caches)]
        attn.forward(q, kp, kn, vp, vn, bt, ctx_dev, out=out, kernel_events=events)

    # ---- per-kernel timing: eager launches with events around the split-K kernel -------
    for i in range(args.warmup):
        step(i)
    kev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
    barrier()
    for i in range(args.steps):
        step(i, kev[i])
    barrier()
    kernel_ms = float(np.mean([a.elapsed_time(b) for a, b in kev]))
    kernel_name = L.akv_last_split_kernel().decode()
    parity = None
    if not args.no_parity and rank == 0:
        step(0)
        torch.cuda.synchronize()
        parity = parity_report(tq, caches[0], bt, ctx, q, out, sample)

    # ---- device-resident timing: one CUDA graph per cache replica, replayed -------------
    launch_mode = "cuda graph replay"
    graphs = []
    launches_per_step = 3
    try:
        side = torch.cuda.Stream(device=dev)
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for r in range(len(caches)):
                step(r)
        torch.cuda.current_stream().wait_stream(side)
        n0 = L.akv_launch_count()
        for r in range(len(caches)):
            gr = torch.cuda.CUDAGraph()
            with torch.cuda.graph(gr):
                step(r)
            graphs.append(gr)
        launches_per_step = int((L.akv_launch_count() - n0) // len(caches))
    except Exception as exc:          # keep measuring, but say how
        graphs, launch_mode = [], f"eager (graph capture failed: {type(exc).__name__})"

    def timed_step(i):
        if graphs:
            graphs[i % len(graphs)].replay()
        else:
            step(i)

    for i in range(args.warmup):
        timed_step(i)
    sampler = ClockSampler(local)
    barrier()
    sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(args.steps):
        timed_step(i)
    e1.record()
    barrier()
    ms_total = e0.elapsed_time(e1)
    # the same region ten more times: the spread of the number above
    regions = [ms_total / args.steps]
    for _ in range(10):
        barrier()
        r0, r1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        r0.record()
        for i in range(args.steps):
            timed_step(i)
        r1.record()
        barrier()
        regions.append(r0.elapsed_time(r1) / args.steps)
    clocks = sampler.stop()

    # ---- end to end through tq::decode_step with host buffers ---------------------
    ops.register_custom_ops()
    ops._quantizers[D] = tq
    kv_cache = torch.zeros(total_blocks, 2, BS, H_KV, PD, dtype=torch.uint8, device=dev)
    kv_cache[:, 0] = caches[0][0]
    kv_cache[:, 1] = caches[0][2]
    k_norms = caches[0][1].unsqueeze(0).contiguous()
    v_norms = caches[0][3].unsqueeze(0).contiguous()
    gen = torch.Generator().manual_seed(3 + rank)
    host = {
        "query": q_host.pin_memory(),
        "key": torch.randn(NUM_SEQS, H_KV, D, generator=gen).half().pin_memory(),
        "value": torch.randn(NUM_SEQS, H_KV, D, generator=gen).half().pin_memory(),
        # the new token overwrites the last context position of each sequence
        "slot_mapping": torch.stack([bt[s, (int(ctx[s]) - 1) // BS].cpu().long() * BS + (int(ctx[s]) - 1) % BS
                                     for s in range(NUM_SEQS)]).pin_memory(),
        "block_table": bt.cpu().pin_memory(),
        "seq_lens": ctx.to(torch.int32).pin_memory(),
    }
    out_host = torch.empty(NUM_SEQS, H_Q, D, dtype=torch.float16).pin_memory()
    out_dev = torch.empty(NUM_SEQS, H_Q, D, dtype=torch.float16, device=dev)
    d2h = out_host.numel() * out_host.element_size()

    # the step's inputs travel as one pinned staging buffer and one host-to-device copy; the typed
    # device views over it are made once
    offs, total = {}, 0
    for k_, v_ in host.items():
        offs[k_] = total
        total += (v_.numel() * v_.element_size() + 255) // 256 * 256
    host_buf = torch.empty(total, dtype=torch.uint8).pin_memory()
    dev_buf = torch.empty(total, dtype=torch.uint8, device=dev)
    d = {}
    for k_, v_ in host.items():
        n = v_.numel() * v_.element_size()
        host_buf[offs[k_]:offs[k_] + n].view(v_.dtype).view(v_.shape).copy_(v_)
        d[k_] = dev_buf[offs[k_]:offs[k_] + n].view(v_.dtype).view(v_.shape)

    h2d = total    # bytes of the staging buffer copied every step (payload padded to 256-byte pieces)

    def e2e_step():
        dev_buf.copy_(host_buf, non_blocking=True)
        res = torch.ops.tq.decode_step(d["query"], d["key"], d["value"], kv_cache, out_dev, k_norms, v_norms,
                                       d["slot_mapping"], d["block_table"], d["seq_lens"], 0, H_Q, H_KV, D,
                                       1.0 / math.sqrt(D), NUM_SEQS)
        out_host.copy_(res, non_blocking=True)
        torch.cuda.current_stream().synchronize()     # the caller reads the result every step

    for _ in range(args.warmup):
        e2e_step()
    eager_out = out_host.clone()                      # what the eager path returned, to check the replay against
    # A serving loop replays its decode step as a CUDA graph: the copy of the staging buffer, the op
    # and the copy of the result back are captured once; every replay moves the bytes again.
    e2e_mode, e2e_graph = "eager", None
    if not args.e2e_eager:
        try:
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                g_ = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g_, stream=side):
                    dev_buf.copy_(host_buf, non_blocking=True)
                    res_ = torch.ops.tq.decode_step(d["query"], d["key"], d["value"], kv_cache, out_dev, k_norms,
                                                    v_norms, d["slot_mapping"], d["block_table"], d["seq_lens"], 0,
                                                    H_Q, H_KV, D, 1.0 / math.sqrt(D), NUM_SEQS)
                    out_host.copy_(res_, non_blocking=True)
            torch.cuda.current_stream().wait_stream(side)
            e2e_graph, e2e_mode = g_, "cuda graph replay (H2D copy + tq::decode_step + D2H copy)"
        except Exception as exc:                      # noqa: BLE001 - capture is an optimisation
            e2e_mode = f"eager (graph capture failed: {type(exc).__name__})"
            torch.cuda.synchronize()

    def e2e_timed():
        if e2e_graph is None:
            e2e_step()
        else:
            e2e_graph.replay()
            torch.cuda.current_stream().synchronize()  # the caller reads the result every step

    for _ in range(args.warmup):
        e2e_timed()
    barrier()
    f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    f0.record()
    for _ in range(args.steps):
        e2e_timed()
    f1.record()
    barrier()
    e2e_ms = f0.elapsed_time(f1)
    if not torch.equal(out_host, eager_out):
        raise RuntimeError("end-to-end replay returned a different result than the eager call")
    e2e_oracle_err = None
    if parity is not None:
        # the op's output (new token written over the last position) against the oracle on the shortest sequence
        from oracle import tq as otq
        s0 = int(np.argmin(ctx.numpy()))
        kc_, vc_ = kv_cache[:, 0].cpu().numpy(), kv_cache[:, 1].cpu().numpy()
        ref = otq.paged_attention_decode_sdpa(q_host.numpy()[s0:s0 + 1], kc_, k_norms[0].cpu().numpy(), vc_,
                                              v_norms[0].cpu().numpy(), bt.cpu().numpy()[s0:s0 + 1],
                                              ctx.numpy()[s0:s0 + 1].astype(np.int64), tq.rotation.cpu().numpy(),
                                              tq.centroids.cpu().numpy(), BITS, 1.0 / math.sqrt(D), BS)
        e2e_oracle_err = float(np.abs(out_host[s0].float().numpy() - ref[0].astype(np.float32)).max())
        parity["e2e_max_abs_err"] = e2e_oracle_err
    status = _lib.device_status()

    # free the headline's buffers before the long-context configurations
    del graphs, e2e_graph, kv_cache, k_norms, v_norms
    cache0 = caches[0]
    caches = [cache0]
    torch.cuda.empty_cache()

    splitk = {}
    if not args.no_splitk:
        for make in (splitk_tri, splitk_tq4):
            job, job_out = make(world, rank, dev)
            res = job.measure(min(args.steps, 200), min(args.warmup, 10), barrier, allreduce_max)
            res["output_finite"] = bool(torch.isfinite(job_out.float()).all())
            splitk[job.name] = res
            del job, job_out
            torch.cuda.empty_cache()

    secondary = None
    if world == 1 and not args.no_secondary:
        secondary = secondary_kernels(min(args.steps, 50), 3, dev)

    t = allreduce_max([ms_total, e2e_ms] + regions)
    ms_total, e2e_ms, regions = t[0], t[1], t[2:]
    job = torch.tensor([float(total_ctx)], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(job, op=dist.ReduceOp.SUM)
    job_ctx = float(job[0])

    if rank == 0:
        peak, peak_src = peak_hbm()
        achieved = kv_bytes / (kernel_ms * 1e-3) / 1e9
        line = {
            "metric": METRIC, "value": job_ctx * args.steps / (ms_total * 1e-3), "unit": UNIT,
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms_total / args.steps, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f16 mma / f32 accumulate over u8 4-bit codes", "data": "synthetic",
            "config": {"workload": WORKLOAD, "kv_tokens_per_gpu": total_ctx, "packed_kv_bytes_per_step": kv_bytes,
                       "l2_policy": f"inputs larger than L2: {args.replicas} cache replicas of {kv_bytes / 1e6:.0f} MB "
                                    "cycled between steps",
                       "launch": launch_mode,
                       "parallelism": f"dp{world} (sequences sharded, no collective)"},
            "timing": {"regions": len(regions), "steps_per_region": args.steps,
                       "ms_per_step_median": float(np.median(regions)), "ms_per_step_min": float(min(regions)),
                       "ms_per_step_max": float(max(regions)),
                       "note": "the first region is the one `value` is computed from; max over ranks per region"},
            "e2e": {"value": job_ctx * args.steps / (e2e_ms * 1e-3), "unit": UNIT,
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "ms_per_step": e2e_ms / args.steps,
                    "launch": e2e_mode,
                    "api": "torch.ops.tq.decode_step (encode new token + attention), host pinned buffers"},
            "gpu_launches": launches_per_step * args.steps,
            "gpu_launches_per_step": launches_per_step,
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                         "frac": achieved / peak,
                         "traffic": NCU_TRAFFIC_BYTES.get(kernel_name) if world == 1 else None,
                         "algorithmic_bytes": kv_bytes, "kernel": kernel_name,
                         "kernel_ms": kernel_ms, "peak_source": peak_src,
                         "frac_of_8TBs_nominal": achieved / 8000.0},
            "clocks": clocks,
            "device_status": status,
        }
        if parity is not None:
            line["parity"] = parity
        if splitk:
            line["splitk"] = splitk
        if secondary is not None:
            line["secondary"] = secondary
        if not args.no_cpu_baseline and world == 1:
            line["cpu_baseline"] = cpu_baseline(tq, cache0, bt, ctx, q)
        print(json.dumps(line))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
