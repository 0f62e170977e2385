// Persistent 4-bit paged decode attention with a TMA-fed block ring (included by tq_attention.cu
// after its lookup / MMA helpers).
//
// Same stream-K schedule, partial format and 64 KB per-lane lookup table as tq4_attn_streamk4_kernel;
// what differs:
//   * Data movement.  A ninth warp is the producer: for every 64-token stage, lanes 0..3 each issue the
//     four tensor copies of one 16-token block (cp.async.bulk.tensor, completion counted in bytes on an
//     mbarrier): K codes as [head][token][64 B], V codes as [head pair][token][128 B] with the hardware
//     128-byte swizzle, K and V norms as [token][8 heads].  With those shapes the 16-byte K reads and
//     the 8-byte V reads of a warp are conflict-free without any software swizzle.  The eight consumer
//     warps (one per KV head) never issue a copy, never meet at a CTA-wide barrier inside the loop, and
//     give a stage's K slot back right after its scores, before the value products.
//   * Value products.  For up to four query heads per KV head the eight MMA columns are (query head,
//     dim parity): the B operand is P with a zero in the other parity, so a packed byte (two adjacent
//     dims of one token) is a complete A register and no nibbles are moved between tokens; the
//     accumulators shrink from 32 to 16 registers.
// Every wait on an mbarrier is bounded; a wait that runs out sets g_attn_window_status to 2 and the
// thread carries on (the result of that call is then unspecified, the kernel still ends).
#pragma once

#include <cuda.h>
#include <string.h>

namespace akv {

constexpr uint32_t T4_BAR = 2048;                       // 8 mbarriers
constexpr uint32_t T4_K0 = 4096, T4_NRM = T4_K0 + 32768;   // norms of slot s: K at T4_NRM + 4096 s, V 2048 further
constexpr uint32_t T4_K1 = 131072, T4_V0 = T4_K1 + 32768, T4_V1 = T4_V0 + 32768;
constexpr int T4_DYN_SMEM = T4_V1 + 32768;              // 229376: covers every address above for any start >= 0
constexpr int T4_THREADS = 288;
static_assert(T4_NRM + 2 * 4096 <= SK_LUT, "low region overlaps the lookup table");
static_assert(T4_V0 % 1024 == 0 && T4_V1 % 1024 == 0, "swizzled slots start on 1 KB boundaries");

struct T4Maps { CUtensorMap k, v, kn, vn; };

__device__ __forceinline__ void t4_bar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" :: "r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void t4_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" :: "r"(bar) : "memory");
}
__device__ __forceinline__ void t4_arrive_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" :: "r"(bar), "r"(bytes) : "memory");
}
// Bounded wait: about a second of SM cycles at most.  After the first wait of a CTA that runs out, the
// shared word T4_FAILED makes every later wait of the CTA return at once, so a broken run ends quickly.
constexpr uint32_t T4_FAILED = T4_BAR + 64;
constexpr uint32_t T4_PLAN = T4_BAR + 256;     // copy of the stage plan (4 S + 2 words) for up to 64 sequences
__device__ __forceinline__ bool t4_wait(uint32_t bar, uint32_t parity) {
  if (lds32(T4_FAILED) != 0u) return false;
  const long long t0 = clock64();
  for (int it = 0; it < (1 << 24); ++it) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}\n"
        : "=r"(done) : "r"(bar), "r"(parity) : "memory");
    if (done) return true;
    if ((it & 63) == 63 && clock64() - t0 > (1ll << 31)) break;
  }
  g_attn_window_status = 2;
  asm volatile("st.shared.u32 [%0], %1;" :: "r"(T4_FAILED), "r"(1u) : "memory");
  return false;
}
__device__ __forceinline__ void t4_tma4(uint32_t dst, const CUtensorMap* map, int c0, int c1, int c2, int c3, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5}], [%6];"
      :: "r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(bar) : "memory");
}
__device__ __forceinline__ void t4_tma3(uint32_t dst, const CUtensorMap* map, int c0, int c1, int c2, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
      :: "r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(bar) : "memory");
}

__device__ __forceinline__ void mma16816_zero(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                              uint32_t b0, uint32_t b1) {
  asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};\n"
      : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(0.f));
}

// Scores of the four 16-token tiles of one stage for this warp's head, scaled by the K norms.
__device__ __forceinline__ void t4_scores(uint32_t lanebase, const uint32_t (&bq)[8][2], uint32_t k_addr,
                                          uint32_t nk_addr, float (&s)[4][4]) {
  constexpr lut_t lut = 0;
  uint4 ka[4], kb[4];
  float nk[4][2];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    ka[j] = lds128(k_addr + j * 8192);
    kb[j] = lds128(k_addr + j * 8192 + 512);            // token g + 8
    nk[j][0] = __uint_as_float(lds32(nk_addr + j * 512));
    nk[j][1] = __uint_as_float(lds32(nk_addr + j * 512 + 256));
  }
#pragma unroll
  for (int w = 0; w < 4; ++w) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const uint32_t a = w == 0 ? ka[j].x : w == 1 ? ka[j].y : w == 2 ? ka[j].z : ka[j].w;
      const uint32_t b = w == 0 ? kb[j].x : w == 1 ? kb[j].y : w == 2 ? kb[j].z : kb[j].w;
      if (w == 0)
        mma16816_zero(s[j], lut4<0>(lut, a, lanebase), lut4<0>(lut, b, lanebase), lut4<1>(lut, a, lanebase),
                      lut4<1>(lut, b, lanebase), bq[0][0], bq[0][1]);
      else
        mma16816(s[j], lut4<0>(lut, a, lanebase), lut4<0>(lut, b, lanebase), lut4<1>(lut, a, lanebase),
                 lut4<1>(lut, b, lanebase), bq[2 * w][0], bq[2 * w][1]);
      mma16816(s[j], lut4<2>(lut, a, lanebase), lut4<2>(lut, b, lanebase), lut4<3>(lut, a, lanebase),
               lut4<3>(lut, b, lanebase), bq[2 * w + 1][0], bq[2 * w + 1][1]);
    }
  }
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    s[j][0] *= nk[j][0]; s[j][1] *= nk[j][0];
    s[j][2] *= nk[j][1]; s[j][3] *= nk[j][1];
  }
}

// The per-lane lookup table of the consumers (entry stride LUT_STRIDE / LUT3_STRIDE, one copy per lane), written by
// `nthr` threads with 16-byte stores.
template <int BITS>
__device__ __forceinline__ void t4_fill_lut(const float* s_cent, int tid, int nthr) {
  if constexpr (BITS == 4) {          // byte -> half2(c[hi nibble], c[lo nibble])
    for (int i = tid; i < 256 * 8; i += nthr) {          // entry e, lanes 4 q .. 4 q + 3: one 16-byte store
      const int e = i >> 3, q4 = i & 7;
      const uint32_t v = pack_half2(s_cent[e >> 4], s_cent[e & 15]);
      asm volatile("st.shared.v4.u32 [%0], {%1,%1,%1,%1};\n" :: "r"(SK_LUT + e * LUT_STRIDE + q4 * 16), "r"(v));
    }
  } else if constexpr (BITS == 3) {   // 6 bits -> half2(c[hi 3 bits], c[lo 3 bits])
    for (int i = tid; i < 64 * 32; i += nthr) {
      const int e = i >> 5, l = i & 31;
      const uint32_t v = pack_half2(s_cent[e >> 3], s_cent[e & 7]);
      asm volatile("st.shared.u32 [%0], %1;\n" :: "r"(SK_LUT + e * LUT3_STRIDE + l * 4), "r"(v));
    }
  } else {                            // byte -> four halves
    for (int i = tid; i < 256 * 16; i += nthr) {         // entry e, lanes 2 q, 2 q + 1: one 16-byte store
      const int e = i >> 4, q2 = i & 15;
      const uint32_t v0 = pack_half2(s_cent[e >> 6], s_cent[(e >> 4) & 3]);
      const uint32_t v1 = pack_half2(s_cent[(e >> 2) & 3], s_cent[e & 3]);
      asm volatile("st.shared.v4.u32 [%0], {%1,%2,%1,%2};\n" :: "r"(SK_LUT + e * LUT_STRIDE + q2 * 16), "r"(v0), "r"(v1));
    }
  }
}

// BITS = 4: the layouts above.  BITS = 3, 2 (48 / 32 packed bytes per token and head): K and V codes both as
// [head][token][PD] boxes without swizzle, the lookup tables and the natural-order fragment helpers of the
// low-bit kernels (lowbit_k_fragments, lowbit_v_fragments); block slots keep their 8 KB spacing.
template <int BITS>
__global__ void __launch_bounds__(T4_THREADS, 1)
tq_attn_tma_kernel(AttnArgs a, const __grid_constant__ T4Maps maps) {
  constexpr int PD = 16 * BITS;                       // packed bytes per (token, head)
  constexpr uint32_t BLOCK_TX = 8 * 16 * PD + 512;    // bytes of one block's codes and norms (one side)
  extern __shared__ __align__(128) unsigned char smem[];
  __shared__ float s_cent[16];
  const uint32_t dyn0 = (uint32_t)__cvta_generic_to_shared(smem);
  const int b = blockIdx.x, hg = blockIdx.y;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int S = a.num_seqs;
  if (dyn0 > T4_BAR) {          // the host checks the window before choosing this kernel
    if (tid == 0) g_attn_window_status = 1;
    return;
  }
  // the merge launch that follows may be scheduled already; it waits for this whole grid before it reads partials
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  if (warp == 8 && lane < 4) {       // the producer's four tensor maps into the descriptor cache, ahead of the first copy
    const CUtensorMap* mp = lane == 0 ? &maps.k : lane == 1 ? &maps.v : lane == 2 ? &maps.kn : &maps.vn;
    asm volatile("prefetch.tensormap [%0];" :: "l"(mp) : "memory");
  }
  if (tid < 16) s_cent[tid] = tid < (1 << BITS) ? a.centroids[tid] : 0.f;
  if (tid == 0) {
    asm volatile("st.shared.u32 [%0], %1;" :: "r"(T4_FAILED), "r"(0u) : "memory");
#pragma unroll
    for (int i = 0; i < 4; ++i) t4_bar_init(T4_BAR + 8 * i, 4);          // fullK[0..1], fullV[0..1]: four issuing lanes
#pragma unroll
    for (int i = 4; i < 8; ++i) t4_bar_init(T4_BAR + 8 * i, 8);          // emptyK[0..1], emptyV[0..1]: eight consumer warps
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  // Launched as a programmatic dependent of the query-rotation launch (a.pdl), this grid may start while that one
  // still runs: the lookup table, which needs nothing of it, is filled first, then the grid waits for it.
  const bool lut_first = a.pdl != 0;
  if (lut_first) {
    __syncthreads();                 // centroids
    t4_fill_lut<BITS>(s_cent, tid, T4_THREADS);
    asm volatile("griddepcontrol.wait;" ::: "memory");
  }
  // The plan written by the query-rotation launch ([0..S] stage prefix, [S] total, [S+1] stages per CTA, then three
  // words per sequence) comes into shared memory with one round of loads; every later look-up is a shared load.
  const int* __restrict__ Pg = a.sk;
  const bool plan_local = S <= 64;
  if (plan_local)
    for (int i = tid; i < 4 * S + 2; i += T4_THREADS)
      asm volatile("st.shared.u32 [%0], %1;" :: "r"(T4_PLAN + 4 * i), "r"((uint32_t)Pg[i]) : "memory");
  __syncthreads();
  auto P = [&](int i) -> int { return plan_local ? (int)lds32(T4_PLAN + 4 * i) : Pg[i]; };

  // this CTA's range of stages.  The first sequence of the range is the last one whose stage prefix is
  // <= u_begin: found with a ballot for up to 64 sequences, by bisection beyond that.
  const int T = P(S), chunk = P(S + 1);
  const int u_begin = b * chunk;
  const int u_end = (u_begin + chunk < T) ? u_begin + chunk : T;
  if (u_begin >= u_end) return;                      // uniform for the CTA
  const int n_it = u_end - u_begin;
  int seq0;
  if (S <= 64) {
    const int c0 = (lane < S && P(lane) <= u_begin) ? 1 : 0, c1 = (lane + 32 < S && P(lane + 32) <= u_begin) ? 1 : 0;
    seq0 = __popc(__ballot_sync(0xffffffffu, c0)) + __popc(__ballot_sync(0xffffffffu, c1)) - 1;
  } else {
    int lo = 0, hi = S - 1;
    while (lo < hi) {
      const int mid = (lo + hi + 1) >> 1;
      if (P(mid) <= u_begin) lo = mid; else hi = mid - 1;
    }
    seq0 = lo;
  }
  while (seq0 < S - 1 && u_begin >= P(seq0 + 1)) ++seq0;      // skip sequences without stages

  if (warp < 8) {        // the consumers fill the lookup table while the producer already issues copies
    if (!lut_first) t4_fill_lut<BITS>(s_cent, tid, 256);
    asm volatile("bar.sync 1, 256;" ::: "memory");
  }

  if (warp == 8) {
    // ------------------------------ producer ------------------------------
    const bool bt64 = a.bt_dtype == AKV_I64;
    const int nblocks = (int)a.num_blocks;
    int p_seq = seq0, p_base = P(seq0), p_end = P(seq0 + 1), p_nb = P(3 * S + 2 + seq0);
    const char* bt_row = reinterpret_cast<const char*>(a.block_tables) + (int64_t)p_seq * a.bt_stride * (bt64 ? 8 : 4);
    for (int it = 0; it < n_it; ++it) {
      const int u = u_begin + it;
      if (u >= p_end) {
        while (p_seq < S - 1 && u >= P(p_seq + 1)) ++p_seq;
        p_base = P(p_seq); p_end = P(p_seq + 1); p_nb = P(3 * S + 2 + p_seq);
        bt_row = reinterpret_cast<const char*>(a.block_tables) + (int64_t)p_seq * a.bt_stride * (bt64 ? 8 : 4);
      }
      const int bi = 4 * (u - p_base);
      const int n_has = p_nb - bi < 4 ? p_nb - bi : 4;
      int pb = 0;
      if (lane < n_has) {
        pb = bt64 ? (int)reinterpret_cast<const int64_t*>(bt_row)[bi + lane] : reinterpret_cast<const int*>(bt_row)[bi + lane];
        pb = min(max(pb, 0), nblocks - 1);
      }
      const int slot = it & 1;
      const uint32_t par = (uint32_t)(((it >> 1) - 1) & 1);
      const uint32_t k_dst = (slot ? T4_K1 : T4_K0) + lane * 8192, v_dst = (slot ? T4_V1 : T4_V0) + lane * 8192;
      const uint32_t kn_dst = T4_NRM + slot * 4096 + lane * 512, vn_dst = kn_dst + 2048;
      const uint32_t fullK = T4_BAR + 8 * slot, fullV = T4_BAR + 16 + 8 * slot;
      if (it >= 2) t4_wait(T4_BAR + 32 + 8 * slot, par);             // K slot handed back
      if (lane < 4) {
        if (lane < n_has) {
          t4_arrive_tx(fullK, BLOCK_TX);
          t4_tma4(k_dst, &maps.k, 0, 0, hg * 8, pb, fullK);
          t4_tma3(kn_dst, &maps.kn, hg * 8, 0, pb, fullK);
        } else {
          t4_arrive(fullK);
        }
      }
      if (it >= 2) t4_wait(T4_BAR + 48 + 8 * slot, par);             // V slot handed back
      if (lane < 4) {
        if (lane < n_has) {
          t4_arrive_tx(fullV, BLOCK_TX);
          t4_tma4(v_dst, &maps.v, 0, 0, BITS == 4 ? hg * 4 : hg * 8, pb, fullV);
          t4_tma3(vn_dst, &maps.vn, hg * 8, 0, pb, fullV);
        } else {
          t4_arrive(fullV);
        }
      }
    }
    return;
  }

  // ------------------------------ consumers: warp = KV head ------------------------------
  const int g = lane >> 2, t = lane & 3;
  const int hl = warp, h = hg * 8 + hl;
  const int G = a.num_q_heads / a.num_kv_heads;       // <= 4 here
  const uint32_t lanebase = SK_LUT | (lane * 4), lb8 = SK_LUT | (lane * 8);
  const uint32_t k_off = hl * (16 * PD) + g * PD + 4 * BITS * t;
  uint32_t v_off[4];
  const uint32_t v_byte = 2 * BITS * g;               // low-bit: the thread's 2*BITS value bytes inside a token's PD
  const uint32_t v_sh = BITS == 3 ? 8u * (v_byte & 3u) : 0u;
  {
    const int toks[4] = {2 * t, 2 * t + 1, 2 * t + 8, 2 * t + 9};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      if constexpr (BITS == 4)
        v_off[i] = (hl >> 1) * 2048 + toks[i] * 128 + ((((hl & 1) * 4 + (g >> 1)) ^ (toks[i] & 7)) << 4) + (g & 1) * 8;
      else
        v_off[i] = hl * (16 * PD) + toks[i] * PD + (BITS == 3 ? (v_byte & ~3u) : v_byte);
    }
  }
  const uint32_t n_off = (g * 8 + hl) * 4;            // norm of token g; token g + 8 is 256 bytes further
  // B operand of the value products: column g = (query head g & 3, dim parity g >> 2)
  const uint32_t selA = (g >> 2) ? 0x1044u : 0x4410u, selB = (g >> 2) ? 0x3244u : 0x4432u;

  uint32_t bq[8][2];
  float o[4][4];
  SoftmaxState st{-CUDART_INF_F, -CUDART_INF_F, 0.f, 0.f};
  int seq_c = -1, c_base = 0, c_end = 0, ctx_c = 0;
  auto begin_seq = [&](int seq) {
    seq_c = seq;
    c_base = P(seq); c_end = P(seq + 1);
    ctx_c = (int)load_ctx(a.context_lens, a.cl_dtype, seq, (int64_t)a.max_blocks_per_seq * a.block_size);
    const int qg = g & 3;
    const float* qp = a.qrot + ((int64_t)seq * a.num_q_heads + h * G + (qg < G ? qg : 0)) * 128 + 32 * t;
    float4 f[8];
#pragma unroll
    for (int kk = 0; kk < 8; ++kk) f[kk] = *reinterpret_cast<const float4*>(qp + 4 * kk);
#pragma unroll
    for (int kk = 0; kk < 8; ++kk) {
      if (qg >= G) f[kk] = make_float4(0.f, 0.f, 0.f, 0.f);
      bq[kk][0] = pack_half2(f[kk].x, f[kk].y);
      bq[kk][1] = pack_half2(f[kk].z, f[kk].w);
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) { o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f; }
    st = SoftmaxState{-CUDART_INF_F, -CUDART_INF_F, 0.f, 0.f};
  };
  auto end_seq = [&]() {
    float l0 = st.l0, l1 = st.l1;
#pragma unroll
    for (int offs = 4; offs < 32; offs <<= 1) {
      l0 += __shfl_xor_sync(0xffffffffu, l0, offs);
      l1 += __shfl_xor_sync(0xffffffffu, l1, offs);
    }
    const int part = b - P(S + 2 + seq_c);
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      const int n = 2 * t + e, qg = n & 3, ep = n >> 2;      // column -> (query head, dim parity)
      if (qg >= G) continue;
      const int64_t row = (int64_t)seq_c * a.num_q_heads + h * G + qg;
      float* pa = a.part_acc + (row * a.num_parts + part) * 128 + 16 * g + ep;
#pragma unroll
      for (int mt = 0; mt < 4; ++mt) {                       // row g of tile mt: byte 8g + 2mt; row g + 8: the next byte
        pa[4 * mt] = o[mt][e];
        pa[4 * mt + 2] = o[mt][2 + e];
      }
      if (g == 0 && ep == 0) {
        a.part_ml[(row * a.num_parts + part) * 2] = e ? st.m1 : st.m0;
        a.part_ml[(row * a.num_parts + part) * 2 + 1] = e ? l1 : l0;
      }
    }
  };

  int it = 0;
  int seq_next = seq0;
  while (it < n_it) {
    begin_seq(seq_next);
    const int it_end = (c_end - u_begin < n_it) ? c_end - u_begin : n_it;     // stages of this sequence in the range
    for (; it < it_end; ++it) {
      const int slot = it & 1;
      const uint32_t par = (uint32_t)((it >> 1) & 1);
      const uint32_t kb = slot ? T4_K1 : T4_K0, vb = slot ? T4_V1 : T4_V0, nb_ = T4_NRM + slot * 4096;
      const int rem = ctx_c - 64 * (u_begin + it - c_base);
      float s[4][4];
      t4_wait(T4_BAR + 8 * slot, par);                       // K codes and norms of the stage have landed
      if constexpr (BITS == 4) {
        t4_scores(lanebase, bq, kb + k_off, nb_ + n_off, s);
      } else {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          uint32_t na[16], nb2[16];
          lowbit_k_fragments<BITS>(kb + j * 8192 + k_off, lanebase, lb8, na);
          lowbit_k_fragments<BITS>(kb + j * 8192 + k_off + 8 * PD, lanebase, lb8, nb2);
          mma16816_zero(s[j], na[0], nb2[0], na[1], nb2[1], bq[0][0], bq[0][1]);
#pragma unroll
          for (int kk = 1; kk < 8; ++kk)
            mma16816(s[j], na[2 * kk], nb2[2 * kk], na[2 * kk + 1], nb2[2 * kk + 1], bq[kk][0], bq[kk][1]);
          const float nkA = __uint_as_float(lds32(nb_ + n_off + j * 512)), nkB = __uint_as_float(lds32(nb_ + n_off + j * 512 + 256));
          s[j][0] *= nkA; s[j][1] *= nkA; s[j][2] *= nkB; s[j][3] *= nkB;
        }
      }
      __syncwarp();
      if (lane == 0) t4_arrive(T4_BAR + 32 + 8 * slot);      // K slot back to the producer
      t4_wait(T4_BAR + 16 + 8 * slot, par);                  // V codes and norms
      float nv[4][2];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        nv[j][0] = __uint_as_float(lds32(nb_ + 2048 + n_off + j * 512));
        nv[j][1] = __uint_as_float(lds32(nb_ + 2048 + n_off + j * 512 + 256));
      }
      if (rem < 64) {              // warp-uniform: only the last stage of a sequence
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int nvld = rem - 16 * j;
          if (g >= nvld) { s[j][0] = -CUDART_INF_F; s[j][1] = -CUDART_INF_F; nv[j][0] = 0.f; }
          if (g + 8 >= nvld) { s[j][2] = -CUDART_INF_F; s[j][3] = -CUDART_INF_F; nv[j][1] = 0.f; }
        }
      }
      float mx0 = fmaxf(s[0][0], s[0][2]), mx1 = fmaxf(s[0][1], s[0][3]);
#pragma unroll
      for (int j = 1; j < 4; ++j) {
        mx0 = fmaxf(mx0, fmaxf(s[j][0], s[j][2]));
        mx1 = fmaxf(mx1, fmaxf(s[j][1], s[j][3]));
      }
#pragma unroll
      for (int off = 4; off < 32; off <<= 1) {
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, off));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, off));
      }
      const float mn0 = fmaxf(st.m0, mx0), mn1 = fmaxf(st.m1, mx1);
      if (__any_sync(0xffffffffu, (mn0 != st.m0) | (mn1 != st.m1))) {
        const float al0 = ex2_approx(st.m0 - mn0), al1 = ex2_approx(st.m1 - mn1);
        st.l0 *= al0; st.l1 *= al1;
#pragma unroll
        for (int j = 0; j < 4; ++j) { o[j][0] *= al0; o[j][1] *= al1; o[j][2] *= al0; o[j][3] *= al1; }
        st.m0 = mn0; st.m1 = mn1;
      }
      uint32_t pb[4][2][2];        // [tile][token group][k half]
      float ls0 = 0.f, ls1 = 0.f;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float p0 = ex2_approx(s[j][0] - mn0), p1 = ex2_approx(s[j][1] - mn1);
        const float p2 = ex2_approx(s[j][2] - mn0), p3 = ex2_approx(s[j][3] - mn1);
        ls0 += p0 + p2;
        ls1 += p1 + p3;
        const uint32_t x0 = movmatrix_trans(pack_half2(p0 * nv[j][0], p1 * nv[j][0]));   // tokens 2t, 2t+1 of rows 0..7
        const uint32_t x1 = movmatrix_trans(pack_half2(p2 * nv[j][1], p3 * nv[j][1]));   // of rows 8..15
        pb[j][0][0] = __byte_perm(x0, 0u, selA); pb[j][0][1] = __byte_perm(x0, 0u, selB);
        pb[j][1][0] = __byte_perm(x1, 0u, selA); pb[j][1][1] = __byte_perm(x1, 0u, selB);
      }
      st.l0 += ls0;
      st.l1 += ls1;
      constexpr lut_t lut = 0;
      if constexpr (BITS != 4) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          uint32_t n0[8], n1[8], n2[8], n3[8];
          lowbit_v_fragments<BITS>(vb + j * 8192 + v_off[0], v_sh, lanebase, lb8, n0);
          lowbit_v_fragments<BITS>(vb + j * 8192 + v_off[1], v_sh, lanebase, lb8, n1);
          lowbit_v_fragments<BITS>(vb + j * 8192 + v_off[2], v_sh, lanebase, lb8, n2);
          lowbit_v_fragments<BITS>(vb + j * 8192 + v_off[3], v_sh, lanebase, lb8, n3);
#pragma unroll
          for (int mt = 0; mt < 4; ++mt) {
            mma16816(o[mt], n0[2 * mt], n0[2 * mt + 1], n1[2 * mt], n1[2 * mt + 1], pb[j][0][0], pb[j][0][1]);
            mma16816(o[mt], n2[2 * mt], n2[2 * mt + 1], n3[2 * mt], n3[2 * mt + 1], pb[j][1][0], pb[j][1][1]);
          }
        }
      } else {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        uint2 vv[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) vv[i] = lds64(vb + v_off[i] + j * 8192);
#pragma unroll
        for (int hf = 0; hf < 2; ++hf) {
          const uint32_t w0 = hf ? vv[0].y : vv[0].x, w1 = hf ? vv[1].y : vv[1].x;
          const uint32_t w2 = hf ? vv[2].y : vv[2].x, w3 = hf ? vv[3].y : vv[3].x;
          mma16816(o[2 * hf], lut4<0>(lut, w0, lanebase), lut4<1>(lut, w0, lanebase), lut4<0>(lut, w1, lanebase),
                   lut4<1>(lut, w1, lanebase), pb[j][0][0], pb[j][0][1]);
          mma16816(o[2 * hf], lut4<0>(lut, w2, lanebase), lut4<1>(lut, w2, lanebase), lut4<0>(lut, w3, lanebase),
                   lut4<1>(lut, w3, lanebase), pb[j][1][0], pb[j][1][1]);
          mma16816(o[2 * hf + 1], lut4<2>(lut, w0, lanebase), lut4<3>(lut, w0, lanebase), lut4<2>(lut, w1, lanebase),
                   lut4<3>(lut, w1, lanebase), pb[j][0][0], pb[j][0][1]);
          mma16816(o[2 * hf + 1], lut4<2>(lut, w2, lanebase), lut4<3>(lut, w2, lanebase), lut4<2>(lut, w3, lanebase),
                   lut4<3>(lut, w3, lanebase), pb[j][1][0], pb[j][1][1]);
        }
      }
      }
      __syncwarp();
      if (lane == 0) t4_arrive(T4_BAR + 48 + 8 * slot);      // V slot back to the producer
    }
    end_seq();
    if (it < n_it) {
      seq_next = seq_c;
      while (seq_next < S - 1 && u_begin + it >= P(seq_next + 1)) ++seq_next;
    }
  }
}

// ---- host side: tensor maps over the caller's cache (this GPU's memory only) ----
typedef CUresult (*akv_encode_tiled_fn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                        const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                        CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static akv_encode_tiled_fn t4_encoder() {
  static akv_encode_tiled_fn fn = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<akv_encode_tiled_fn>(p);
    else
      cudaGetLastError();
  }
  return fn;
}

// Maps for one (cache, strides) combination; the last one built is kept, a serving loop asks for the
// same one at every step.  False: the layout cannot be described (the caller takes another kernel).
static bool t4_make_maps(const AttnArgs& p, T4Maps* out) {
  const int pd = 16 * p.bits;
  struct Key { int64_t v[19]; };      // pointers, strides, sizes: eight-byte fields only, so memcmp sees no padding
  static thread_local Key last{};
  static thread_local T4Maps last_maps;
  static thread_local bool have = false;
  const Key key{{(int64_t)(uintptr_t)p.k_packed, (int64_t)(uintptr_t)p.v_packed, (int64_t)(uintptr_t)p.k_norms,
                 (int64_t)(uintptr_t)p.v_norms, p.kp_sb, p.kp_sp, p.kp_sh, p.vp_sb, p.vp_sp, p.vp_sh, p.kn_sb, p.kn_sp,
                 p.kn_sh, p.vn_sb, p.vn_sp, p.vn_sh, p.num_blocks, (int64_t)p.num_kv_heads, (int64_t)p.bits}};
  if (have && memcmp(&key, &last, sizeof(Key)) == 0) { *out = last_maps; return true; }
  akv_encode_tiled_fn enc = t4_encoder();
  if (enc == nullptr) return false;
  const cuuint32_t ones[4] = {1, 1, 1, 1};
  T4Maps m;
  {   // K codes: (pd bytes, 16 tokens, heads, blocks); a box holds eight heads of one block as [head][token][pd]
    const cuuint64_t dims[4] = {(cuuint64_t)pd, 16, (cuuint64_t)p.num_kv_heads, (cuuint64_t)p.num_blocks};
    const cuuint64_t strides[3] = {(cuuint64_t)p.kp_sp, (cuuint64_t)p.kp_sh, (cuuint64_t)p.kp_sb};
    const cuuint32_t box[4] = {(cuuint32_t)pd, 16, 8, 1};
    if (enc(&m.k, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, const_cast<uint8_t*>(p.k_packed), dims, strides, box, ones,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS) return false;
  }
  if (p.bits != 4) {   // low-bit V codes: the K layout
    const cuuint64_t dims[4] = {(cuuint64_t)pd, 16, (cuuint64_t)p.num_kv_heads, (cuuint64_t)p.num_blocks};
    const cuuint64_t strides[3] = {(cuuint64_t)p.vp_sp, (cuuint64_t)p.vp_sh, (cuuint64_t)p.vp_sb};
    const cuuint32_t box[4] = {(cuuint32_t)pd, 16, 8, 1};
    if (enc(&m.v, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, const_cast<uint8_t*>(p.v_packed), dims, strides, box, ones,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS) return false;
  } else {   // V codes: (128 bytes = a head pair, 16 tokens, head pairs, blocks), 128-byte swizzle
    const cuuint64_t dims[4] = {128, 16, (cuuint64_t)(p.num_kv_heads / 2), (cuuint64_t)p.num_blocks};
    const cuuint64_t strides[3] = {(cuuint64_t)p.vp_sp, (cuuint64_t)(2 * p.vp_sh), (cuuint64_t)p.vp_sb};
    const cuuint32_t box[4] = {128, 16, 4, 1};
    if (enc(&m.v, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, const_cast<uint8_t*>(p.v_packed), dims, strides, box, ones,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS) return false;
  }
  for (int side = 0; side < 2; ++side) {   // norms: (heads, 16 tokens, blocks) float32; a box is [token][8 heads]
    const float* base = side ? p.v_norms : p.k_norms;
    const int64_t sb = side ? p.vn_sb : p.kn_sb, sp = side ? p.vn_sp : p.kn_sp;
    const cuuint64_t dims[3] = {(cuuint64_t)p.num_kv_heads, 16, (cuuint64_t)p.num_blocks};
    const cuuint64_t strides[2] = {(cuuint64_t)(sp * 4), (cuuint64_t)(sb * 4)};
    const cuuint32_t box[3] = {8, 16, 1};
    if (enc(side ? &m.vn : &m.kn, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<float*>(base), dims, strides, box, ones,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_NONE,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS) return false;
  }
  last = key; last_maps = m; have = true;
  *out = m;
  return true;
}

}  // namespace akv
