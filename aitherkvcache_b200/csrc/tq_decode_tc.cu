// TurboQuant decode on the 5th-generation tensor cores (tcgen05 / TMEM), head_dim 128.
//
// Same operation as tq_decode_tiled_kernel in tq_codec.cu (reference: quantizer.py:170-212):
//   x_hat[j] = norm * sum_i centroid[code_i] * R[i][j],   rounded to the output type.
// A tile of 128 vectors is one 128 x 128 x 128 GEMM.  Centroids and R are float32, so both are
// split into two fp16 terms of 1024 x the value (c = c1 + c2, R = R1 + R2; the factor keeps
// the second terms out of fp16's subnormal range) and the product is accumulated as
// c1 R1 + c1 R2 + c2 R1 in one float32 TMEM accumulator (the dropped c2 R2 term is 2^-22 of the
// result); the factor 2^-20 is folded into the norm.  Results agree with the float32 FMA kernel
// to a few float32 ulps, i.e. the fp16 outputs differ only where a value sits on a rounding tie.
//
// One persistent CTA per SM: 16 worker warps and one warp whose first lane issues the MMAs.  Worker thread
// (row, q) owns the 32 codes 32q..32q+31 of a row: it prefetches their 4*BITS bytes a tile ahead into registers
// (one 16-byte load for 4-bit rows), turns them into the two fp16 operand rows (per-lane table: code -> (c1, c2))
// in the 128-byte-swizzled K-major layout of operand stage t % 2, and writes out tile t-1 from its half of
// tensor memory (tcgen05.ld: one thread per vector, 32 consecutive outputs).  Nothing in the loop is a CTA-wide
// barrier; the hand-overs are mbarriers:
//   full[s]      16 warp arrivals: the operand rows of stage s are written          -> the MMA warp may issue
//   mma_done[s]  tcgen05.commit: the tile's MMAs are complete                       -> stage s may be refilled,
//                                                                                      accumulator s may be read
//   acc_free[s]  16 warp arrivals: accumulator s has been loaded into registers     -> the MMA warp may reuse it
// so warps drift apart and their unpack, load, convert and store phases overlap.
// Every wait is bounded; a wait that gives up sets g_tc_decode_status and a shared flag that ends all loops,
// and the CTA leaves after releasing its tensor memory.
#include "tq_rowmap.cuh"
#include "umma.cuh"
#include <cuda.h>
#include <stdlib.h>
#include <string.h>

namespace akv {
namespace {

__device__ int g_tc_decode_status;          // 1: a wait on the MMA barrier gave up
__device__ int g_tc_decode_withhold = -1;   // test hook: CTA 0 issues neither the MMAs nor the commit of this tile

constexpr int DT_THREADS = 17 * 32;                    // 16 worker warps + the MMA warp
constexpr int DT_TERMS_R = 0;                          // R1, R2: 2 operands
constexpr int DT_ABUF = 2 * TC_OPER_BYTES;             // 2 stages x (c1, c2) operands
constexpr int DT_LUT = DT_ABUF + 4 * TC_OPER_BYTES;    // 16 entries x 128 B
constexpr int DT_MISC = DT_LUT + 2048;                 // mbarriers, TMEM slot
constexpr int DT_SMEM = DT_MISC + 64 + 1024;           // + slack for the 1024-byte alignment

// Code e (0..31) of a thread's MSB-first stream held as big-endian words B[]; returns the byte
// address of the code's table entry for this lane (entry stride 128 B).
template <int BITS, int E>
__device__ __forceinline__ uint32_t entry_addr(const uint32_t* B, uint32_t lut_lane) {
  constexpr int pos = E * BITS, w = pos >> 5, off = pos & 31, sh = 32 - BITS - off;
  constexpr uint32_t mask = ((1u << BITS) - 1u) << 7;
  uint32_t x;
  if constexpr (sh >= 7) x = B[w] >> (sh - 7);
  else if constexpr (sh >= 0) x = B[w] << (7 - sh);
  else x = __funnelshift_l(B[w + 1], B[w], 7 + BITS + off - 32);   // field straddles two words
  return lut_lane + (x & mask);
}

template <int BITS, int C>
__device__ __forceinline__ void unpack_chunk(const uint32_t* B, uint32_t lut_lane, uint4& c1, uint4& c2) {
  uint32_t r[8];
  r[0] = lds_u32(entry_addr<BITS, 8 * C + 0>(B, lut_lane)); r[1] = lds_u32(entry_addr<BITS, 8 * C + 1>(B, lut_lane));
  r[2] = lds_u32(entry_addr<BITS, 8 * C + 2>(B, lut_lane)); r[3] = lds_u32(entry_addr<BITS, 8 * C + 3>(B, lut_lane));
  r[4] = lds_u32(entry_addr<BITS, 8 * C + 4>(B, lut_lane)); r[5] = lds_u32(entry_addr<BITS, 8 * C + 5>(B, lut_lane));
  r[6] = lds_u32(entry_addr<BITS, 8 * C + 6>(B, lut_lane)); r[7] = lds_u32(entry_addr<BITS, 8 * C + 7>(B, lut_lane));
  c1 = make_uint4(__byte_perm(r[0], r[1], 0x5410), __byte_perm(r[2], r[3], 0x5410),
                  __byte_perm(r[4], r[5], 0x5410), __byte_perm(r[6], r[7], 0x5410));
  c2 = make_uint4(__byte_perm(r[0], r[1], 0x7632), __byte_perm(r[2], r[3], 0x7632),
                  __byte_perm(r[4], r[5], 0x7632), __byte_perm(r[6], r[7], 0x7632));
}

__device__ __forceinline__ void sts128(uint32_t addr, const uint4& v) {
  asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" :: "r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

template <int BITS>
__global__ void __launch_bounds__(DT_THREADS, 1)
tq_decode_tc_kernel(const uint8_t* __restrict__ packed, int64_t p_stride_row, const float* __restrict__ norms,
                    int64_t n_rows, const float* __restrict__ rot, const float* __restrict__ centroids,
                    void* __restrict__ out, int out_dtype, const __grid_constant__ CUtensorMap out_map, int tma_store) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_s = smem_u32(smem_raw);
  const uint32_t base_s = (raw_s + 1023u) & ~1023u;
  uint8_t* base = smem_raw + (base_s - raw_s);
  uint8_t* rterms = base + DT_TERMS_R;
  uint64_t* mbar = reinterpret_cast<uint64_t*>(base + DT_MISC);   // full[2], mma_done[2], acc_free[2], drain
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(mbar + 7);
  const uint32_t failed_s = base_s + DT_MISC + 60;
  const uint32_t abuf_s = base_s + DT_ABUF, lut_s = base_s + DT_LUT, mbar_s = base_s + DT_MISC;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

  // ---------------- one-time setup ----------------
  if (tid == 0) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 16;" :: "r"(mbar_s));          // full[0]
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 16;" :: "r"(mbar_s + 8));      // full[1]
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" :: "r"(mbar_s + 16));      // mma_done[0]
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" :: "r"(mbar_s + 24));      // mma_done[1]
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 16;" :: "r"(mbar_s + 32));     // acc_free[0]
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 16;" :: "r"(mbar_s + 40));     // acc_free[1]
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" :: "r"(mbar_s + 48));      // drain
    asm volatile("st.shared.u32 [%0], %1;" :: "r"(failed_s), "r"(0u) : "memory");
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  const int withhold = blockIdx.x == 0 ? g_tc_decode_withhold : -1;
  __syncwarp();
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], 256;"
                 :: "r"(smem_u32(tmem_slot)) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  // B operand: row n = output coordinate j, K index i, value 1024 R[i][j] in two fp16 terms.  rot is
  // read with j fastest (coalesced) into a float32 staging copy (the A buffers, not yet in use); the
  // XOR on the staging column keeps both passes free of bank conflicts.
  {
    float* stg = reinterpret_cast<float*>(base + DT_ABUF);
    for (int e = tid; e < 128 * 128; e += DT_THREADS) {
      const int i = e >> 7, j = e & 127;
      stg[i * 128 + (j ^ (i & 31))] = rot[e];
    }
    __syncthreads();
    for (int e = tid; e < 128 * 128; e += DT_THREADS) {
      const int j = e >> 7, i = e & 127;
      const float r = stg[i * 128 + (j ^ (i & 31))] * 1024.0f;
      const uint32_t off = tc_operand_offset(j, i);
      const __half t1 = __float2half_rn(r);
      *reinterpret_cast<__half*>(rterms + off) = t1;
      *reinterpret_cast<__half*>(rterms + TC_OPER_BYTES + off) = __float2half_rn(r - __half2float(t1));
    }
  }
  // table: code -> half2(c1, c2), one copy per lane
  for (int e = tid; e < (1 << BITS) * 32; e += DT_THREADS) {
    const float c = centroids[e >> 5] * 1024.0f;
    const __half h1 = __float2half_rn(c), h2 = __float2half_rn(c - __half2float(h1));
    *reinterpret_cast<uint32_t*>(base + DT_LUT + (e >> 5) * 128 + (e & 31) * 4) =
        (uint32_t)__half_as_ushort(h1) | ((uint32_t)__half_as_ushort(h2) << 16);
  }
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_slot;

  // instruction descriptor: D = f32, A/B = f16, both K-major, N = 128, M = 128
  constexpr uint32_t IDESC = (1u << 4) | ((128u >> 3) << 17) | ((128u >> 4) << 24);

  const int64_t num_tiles = (n_rows + 127) >> 7;
  const int n_my = (int)((num_tiles - blockIdx.x + gridDim.x - 1) / gridDim.x);
  auto tile_row0 = [&](int t) { return ((int64_t)blockIdx.x + (int64_t)t * gridDim.x) * 128; };

  // unpack role: thread (row, q) owns codes 32q .. 32q+31 of a row = 4*BITS bytes
  const int urow = tid >> 2, uq = tid & 3;
  const uint32_t lut_lane = lut_s + lane * 4;
  // the four 16-byte chunks of the operand row this thread writes: K = 32 uq + 8 c
  const uint32_t u_off = (uint32_t)((uq >> 1) * TC_HALF_BYTES + urow * 128);
  const uint32_t u_chunk0 = (uint32_t)((4 * uq) & 7), u_swz = (uint32_t)(urow & 7);
  // epilogue role: thread = row, 32 consecutive outputs
  const int w4 = warp & 3, colq = warp >> 2, erow = w4 * 32 + lane;

  uint32_t cw[BITS];      // packed bytes of the tile to unpack next
  uint32_t cw_nx[BITS];   // ... and of the tile after it, in flight while this one is unpacked
  const bool vec_rows = BITS == 4 && (p_stride_row & 15) == 0 && (reinterpret_cast<uintptr_t>(packed) & 15) == 0;
  auto prefetch = [&](int t, uint32_t (&dst)[BITS]) {
    const int64_t n = tile_row0(t) + urow;
#pragma unroll
    for (int k = 0; k < BITS; ++k) dst[k] = 0u;
    if (t < n_my && n < n_rows) {
      const uint32_t* src = reinterpret_cast<const uint32_t*>(packed + n * p_stride_row + 4 * BITS * uq);
      if (BITS == 4 && vec_rows) {
        const uint4 v = __ldg(reinterpret_cast<const uint4*>(src));
        dst[0] = v.x; dst[1] = v.y; dst[2 % BITS] = v.z; dst[3 % BITS] = v.w;
      } else {
#pragma unroll
        for (int k = 0; k < BITS; ++k) dst[k] = __ldg(src + k);
      }
    }
  };
  auto unpack = [&](int t) {      // registers cw -> operand buffers of stage t & 1
    uint32_t B[BITS];
#pragma unroll
    for (int k = 0; k < BITS; ++k) B[k] = bswap32(cw[k]);
    const uint32_t a1 = abuf_s + (uint32_t)(t & 1) * 2 * TC_OPER_BYTES + u_off, a2 = a1 + TC_OPER_BYTES;
    uint4 c1, c2;
    unpack_chunk<BITS, 0>(B, lut_lane, c1, c2);
    sts128(a1 + (((u_chunk0 + 0) ^ u_swz) << 4), c1); sts128(a2 + (((u_chunk0 + 0) ^ u_swz) << 4), c2);
    unpack_chunk<BITS, 1>(B, lut_lane, c1, c2);
    sts128(a1 + (((u_chunk0 + 1) ^ u_swz) << 4), c1); sts128(a2 + (((u_chunk0 + 1) ^ u_swz) << 4), c2);
    unpack_chunk<BITS, 2>(B, lut_lane, c1, c2);
    sts128(a1 + (((u_chunk0 + 2) ^ u_swz) << 4), c1); sts128(a2 + (((u_chunk0 + 2) ^ u_swz) << 4), c2);
    unpack_chunk<BITS, 3>(B, lut_lane, c1, c2);
    sts128(a1 + (((u_chunk0 + 3) ^ u_swz) << 4), c1); sts128(a2 + (((u_chunk0 + 3) ^ u_swz) << 4), c2);
  };

  // Bounded wait; once one wait of the CTA has run out, the others return at once.
  auto wait = [&](uint32_t bar, uint32_t parity) -> bool {
    if (lds_u32(failed_s) != 0u) return false;
    if (mbar_wait(bar, parity)) return true;
    g_tc_decode_status = 1;
    asm volatile("st.shared.u32 [%0], %1;" :: "r"(failed_s), "r"(1u) : "memory");
    return false;
  };
  // the same for a whole warp, with one answer for all its lanes
  auto wait_warp = [&](uint32_t bar, uint32_t parity) -> bool { return __all_sync(0xffffffffu, wait(bar, parity)); };
  const uint32_t full_s = mbar_s, done_s = mbar_s + 16, free_s = mbar_s + 32, drain_s = mbar_s + 48;

  if (warp == 16) {
    // ---- MMA warp: tile t = c1 R1 + c1 R2 + c2 R1 as soon as its operand rows are there and its accumulator is free ----
    if (lane == 0) {
      for (int t = 0; t < n_my; ++t) {
        const uint32_t s = (uint32_t)(t & 1), ph = (uint32_t)((t >> 1) & 1);
        if (!wait(full_s + 8u * s, ph)) break;
        if (t >= 2 && !wait(free_s + 8u * s, (uint32_t)(((t - 2) >> 1) & 1))) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        if (t == withhold) continue;
        const uint32_t a_s = abuf_s + s * 2 * TC_OPER_BYTES;
        const uint32_t d0 = tmem_base + s * 128;
#pragma unroll
        for (int pass = 0; pass < 3; ++pass) {
          const uint32_t ao = pass == 2 ? TC_OPER_BYTES : 0u, bo = pass == 1 ? TC_OPER_BYTES : 0u;
#pragma unroll
          for (int kk = 0; kk < 8; ++kk) {
            const uint32_t koff = (uint32_t)((kk >> 2) * TC_HALF_BYTES + (kk & 3) * 32);
            umma_f16(d0, umma_desc(a_s + ao + koff), umma_desc(base_s + DT_TERMS_R + bo + koff), IDESC,
                     (uint32_t)((pass | kk) != 0));
          }
        }
        umma_commit(done_s + 8u * s);
      }
    }
    __syncwarp();
  } else {
    // ---- worker warps ----
    // 16-bit outputs leave through a transpose in shared memory, so that a store instruction of the warp covers
    // eight 64-byte row segments instead of thirty-two 16-byte pieces.  The staging space is the part of the idle
    // operand stage that this warp itself fills next (operand rows 8 warp .. 8 warp + 7, both K halves = 2 KB).
    const uint32_t stg_lane = (uint32_t)((lane >> 4) * TC_HALF_BYTES + (lane & 15) * 64), stg_swz = (uint32_t)((lane >> 1) & 3);
    prefetch(0, cw);
    float nrm_cur = 0.f;
    for (int t = 0; t <= n_my; ++t) {
      const bool have = t < n_my;
      prefetch(t + 1, cw_nx);
      float nrm_next = 0.f;
      if (have) {
        const int64_t n = tile_row0(t) + erow;
        if (n < n_rows) nrm_next = __ldg(norms + n);
        // ---- tile t: operand rows into stage t % 2, free once the MMAs of tile t-2 are complete ----
        if (t >= 2 && !wait_warp(done_s + 8u * (uint32_t)(t & 1), (uint32_t)(((t - 2) >> 1) & 1))) break;
        if (tma_store) {      // the bulk stores of tile t-2 have read this warp's staging rows (issued an iteration ago)
          if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
          __syncwarp();
        }
        unpack(t);
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncwarp();
        if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" :: "r"(full_s + 8u * (uint32_t)(t & 1)) : "memory");
      }
      // ---- tile t-1: out of tensor memory, scale by the norm, convert, store ----
      if (t >= 1) {
        const uint32_t s1 = (uint32_t)((t - 1) & 1);
        if (!wait_warp(done_s + 8u * s1, (uint32_t)(((t - 1) >> 1) & 1))) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        uint32_t v[32];
        tmem_ld32(tmem_base + ((uint32_t)(w4 * 32) << 16) + (uint32_t)(s1 * 128 + colq * 32), v);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncwarp();
        if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" :: "r"(free_s + 8u * s1) : "memory");
        const int64_t n = tile_row0(t - 1) + erow;
        const float sc = nrm_cur * (1.0f / 1048576.0f);
        if (out_dtype == AKV_F32) {
          if (n < n_rows) {
            float4* dst = reinterpret_cast<float4*>(reinterpret_cast<float*>(out) + n * 128 + colq * 32);
#pragma unroll
            for (int k = 0; k < 8; ++k)
              dst[k] = make_float4(__uint_as_float(v[4 * k]) * sc, __uint_as_float(v[4 * k + 1]) * sc,
                                   __uint_as_float(v[4 * k + 2]) * sc, __uint_as_float(v[4 * k + 3]) * sc);
          }
        } else {
          uint32_t h[16];
#pragma unroll
          for (int k = 0; k < 16; ++k) {
            const float lo = __uint_as_float(v[2 * k]) * sc, hi = __uint_as_float(v[2 * k + 1]) * sc;
            if (out_dtype == AKV_F16) {
              __half2 p = __floats2half2_rn(lo, hi);
              h[k] = *reinterpret_cast<uint32_t*>(&p);
            } else {
              __nv_bfloat162 p = __floats2bfloat162_rn(lo, hi);
              h[k] = *reinterpret_cast<uint32_t*>(&p);
            }
          }
          // stage (t + 1) % 2 is idle: the MMAs of tile t-1 are complete and this warp refills its rows only in
          // the next iteration
          const uint32_t stg = abuf_s + (uint32_t)((t + 1) & 1) * 2 * TC_OPER_BYTES + (uint32_t)warp * 1024u;
#pragma unroll
          for (int c = 0; c < 4; ++c)
            sts128(stg + stg_lane + ((((uint32_t)c) ^ stg_swz) << 4), make_uint4(h[4 * c], h[4 * c + 1], h[4 * c + 2], h[4 * c + 3]));
          const int64_t n0 = tile_row0(t - 1) + w4 * 32;
          if (tma_store) {
            // the staged rows are in the 64-byte-swizzled layout of the output map: two bulk tensor stores of 16 rows
            // x 64 bytes (rows past the end of the output are dropped by the copy engine), no load / store instructions
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            if (lane == 0) {
              const int x = colq * 32, y = (int)n0;
              if (n0 < n_rows)
                asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%1, %2}], [%3];"
                             :: "l"(&out_map), "r"(x), "r"(y), "r"(stg) : "memory");
              if (n0 + 16 < n_rows)
                asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%1, %2}], [%3];"
                             :: "l"(&out_map), "r"(x), "r"(y + 16), "r"(stg + (uint32_t)TC_HALF_BYTES) : "memory");
              asm volatile("cp.async.bulk.commit_group;" ::: "memory");
            }
          } else {
            __syncwarp();
#pragma unroll
            for (int k = 0; k < 4; ++k) {
              const int r = 8 * k + (lane >> 2), c = lane & 3;       // row of the warp's 32, 16-byte piece of its 64 bytes
              uint4 q;
              const uint32_t a = stg + (uint32_t)((r >> 4) * TC_HALF_BYTES + (r & 15) * 64) + ((((uint32_t)c) ^ (uint32_t)((r >> 1) & 3)) << 4);
              asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(q.x), "=r"(q.y), "=r"(q.z), "=r"(q.w) : "r"(a) : "memory");
              if (n0 + r < n_rows)
                *reinterpret_cast<uint4*>(reinterpret_cast<uint16_t*>(out) + (n0 + r) * 128 + colq * 32 + c * 8) = q;
            }
            __syncwarp();        // the staging rows are this warp's to overwrite in the next unpack
          }
        }
      }
#pragma unroll
      for (int k = 0; k < BITS; ++k) cw[k] = cw_nx[k];
      nrm_cur = nrm_next;
    }
    if (tma_store && lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");    // before the CTA's shared memory goes
  }

  // A CTA in which a wait gave up may still have MMAs in flight: before the columns go back, the issuing thread
  // commits once more on the drain barrier (it completes when every MMA that thread issued has) and waits,
  // bounded.  Only if that wait gives up too are the columns kept (status 2): lost to this SM until the context
  // ends, which is better than freeing them under an MMA.
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  int leak = 0;
  if (warp == 16 && lane == 0 && lds_u32(failed_s) != 0u) {
    umma_commit(drain_s);
    leak = mbar_wait(drain_s, 0u) ? 0 : 1;
    if (leak) g_tc_decode_status = 2;
  }
  leak = __syncthreads_or(leak);
  if (warp == 0 && !leak) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, 256;" :: "r"(tmem_base) : "memory");
  }
}

typedef CUresult (*dt_encode_tiled_fn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                       const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                       CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

dt_encode_tiled_fn dt_encoder() {
  static dt_encode_tiled_fn fn = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<dt_encode_tiled_fn>(p);
    else
      cudaGetLastError();
  }
  return fn;
}

// Map of a 16-bit output [n_rows][128] for stores of 16 rows x 32 elements out of 64-byte-swizzled shared memory.
bool dt_out_map(void* out, int64_t n_rows, CUtensorMap* map) {
  static const bool off = getenv("AKV_NO_TMA_STORE") != nullptr;
  if (off || (reinterpret_cast<uintptr_t>(out) & 15) != 0 || n_rows >= (1ll << 31)) return false;
  dt_encode_tiled_fn enc = dt_encoder();
  if (enc == nullptr) return false;
  const cuuint64_t dims[2] = {128, (cuuint64_t)n_rows};
  const cuuint64_t strides[1] = {256};
  const cuuint32_t box[2] = {32, 16}, ones[2] = {1, 1};
  return enc(map, CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, out, dims, strides, box, ones, CU_TENSOR_MAP_INTERLEAVE_NONE,
             CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int BITS>
int launch_dtc(const uint8_t* packed, int64_t ps, const float* norms, int64_t n_rows, const float* rot,
               const float* cent, void* out, int out_dtype, cudaStream_t st) {
  auto kern = tq_decode_tc_kernel<BITS>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, DT_SMEM);
  if (e != cudaSuccess) return fail((int)e, "decode: smem attribute: %s", cudaGetErrorString(e));
  int64_t tiles = (n_rows + 127) / 128;
  int grid = (int)(tiles < sm_count() ? tiles : sm_count());
  CUtensorMap map;
  memset(&map, 0, sizeof(map));
  const int tma_store = (out_dtype != AKV_F32 && dt_out_map(out, n_rows, &map)) ? 1 : 0;
  kern<<<grid, DT_THREADS, DT_SMEM, st>>>(packed, ps, norms, n_rows, rot, cent, out, out_dtype, map, tma_store);
  return check_launch("tq_decode_tc_kernel");
}

}  // namespace

int tc_decode_status(int* host_out, int reset) {
  cudaError_t e = cudaMemcpyFromSymbol(host_out, g_tc_decode_status, sizeof(int));
  if (e == cudaSuccess && reset) { const int z = 0; e = cudaMemcpyToSymbol(g_tc_decode_status, &z, sizeof(int)); }
  return e == cudaSuccess ? AKV_OK : fail((int)e, "decode status: %s", cudaGetErrorString(e));
}

int tc_decode_withhold(int tile) {
  cudaError_t e = cudaMemcpyToSymbol(g_tc_decode_withhold, &tile, sizeof(int));
  return e == cudaSuccess ? AKV_OK : fail((int)e, "decode test hook: %s", cudaGetErrorString(e));
}

int launch_decode_tc(const uint8_t* packed, int64_t packed_row_stride, const float* norms, int64_t n_rows,
                     int bits, const float* rot, const float* centroids, void* out, int out_dtype,
                     cudaStream_t st) {
  if (bits == 4) return launch_dtc<4>(packed, packed_row_stride, norms, n_rows, rot, centroids, out, out_dtype, st);
  if (bits == 3) return launch_dtc<3>(packed, packed_row_stride, norms, n_rows, rot, centroids, out, out_dtype, st);
  if (bits == 2) return launch_dtc<2>(packed, packed_row_stride, norms, n_rows, rot, centroids, out, out_dtype, st);
  return fail(AKV_ERR_ARG, "launch_decode_tc: bits %d", bits);
}

}  // namespace akv
