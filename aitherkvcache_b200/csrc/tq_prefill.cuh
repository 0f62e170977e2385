// Chunked-prefill attention over the packed 4-bit cache (included by tq_attention.cu).
//
// The reference decompresses every active block to bf16 and calls vLLM's unified attention
// (vllm/backend.py:1093-1244, vllm/hooks.py:726-850).  Here the query tokens of a chunk share one pass over
// their sequence's packed blocks: a CTA takes 64 / G consecutive query tokens of one sequence and one KV head
// (G = query heads per KV head), i.e. 64 (token, head) rows, 16 per warp, and walks over the causal key range in
// tiles of 32 keys (cp.async, three stages).  Per tile the CTA first turns the packed codes into fp16 once
// (every thread 16 key bytes and 16 value bytes through the per-lane lookup table, byte -> two neighbouring
// coordinates) into two 32 x 128 tiles in shared memory; then per warp:
//   scores  S[16 rows][32 keys] = Q K^T on mma.sync m16n8k16: A = the warp's query rows (registers, loaded once),
//           B = the key tile by ldmatrix;
//   softmax online per row, in log2 units, with the causal limit of the row's token; key norms scale the scores;
//   values  O[16 rows][128] += P V: A = the probabilities (times the value norms) straight from the score
//           accumulators (same fragment layout), B = the value tile by ldmatrix.trans.
// The decode work is shared by the 64 rows of the CTA, the stream by all of them.
// Attention runs in the rotated domain like the decode kernels: queries come in rotated (akv_qrot128_kernel),
// the un-normalised result (m, l, acc) of every row goes to the LSE merge kernel, which divides and rotates back.
#pragma once

#include "tq_prefill_args.cuh"

namespace akv {

constexpr int PF_THREADS = 128;
constexpr int PF_LUT_BYTES = 256 * 128;                       // byte -> half2, one copy per lane
constexpr int PF_KT = 32;                                     // keys per tile
constexpr int PF_STAGE_BYTES = PF_KT * (64 + 64 + 4 + 4);     // K codes, V codes, K norms, V norms
constexpr int PF_LD = 136;                                    // halves per row of a decoded tile (272 B: conflict-free ldmatrix)
constexpr int PF_TILE_BYTES = PF_KT * PF_LD * 2;
constexpr int PF_SMEM = PF_LUT_BYTES + 3 * PF_STAGE_BYTES + 2 * PF_TILE_BYTES;

__device__ __forceinline__ void pf_ldmatrix(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void pf_ldmatrix_trans(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}

__device__ __forceinline__ void pf_mma(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

template <int G>
__global__ void __launch_bounds__(PF_THREADS, 3)
tq_prefill_attn_kernel(PrefillArgs a) {
  static_assert(G == 1 || G == 2 || G == 4 || G == 8, "query heads per KV head");
  constexpr int TT = 64 / G;            // query tokens of a CTA
  constexpr int TPW = 16 / G;           // ... of a warp
  extern __shared__ __align__(16) unsigned char pf_smem[];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
  const int kvh = blockIdx.y;

  // ---- which sequence and which of its query tiles ----
  int tile = blockIdx.x, s = 0, q0 = 0, qlen = 0;
  bool found = false;
  for (s = 0; s < a.num_seqs; ++s) {
    q0 = (int)load_index(a.query_start_loc, a.qs_dtype, s);
    const int q1 = (int)load_index(a.query_start_loc, a.qs_dtype, s + 1);
    qlen = q1 - q0;
    if (qlen < 0) qlen = 0;
    const int tiles = (qlen + TT - 1) / TT;
    if (tile < tiles) { found = true; break; }
    tile -= tiles;
  }
  if (!found) return;                   // uniform for the CTA
  const int64_t max_ctx = (int64_t)a.max_blocks_per_seq * a.block_size;
  const int seq_len = (int)load_ctx(a.seq_lens, a.sl_dtype, s, max_ctx);
  int past = seq_len - qlen;            // keys before the chunk
  if (past < 0) past = 0;
  const int tok_lo = tile * TT;
  const int tok_hi = (tok_lo + TT < qlen) ? tok_lo + TT : qlen;       // local query tokens [tok_lo, tok_hi)
  int kend = past + tok_hi;             // keys any row of this CTA may see
  if (kend > seq_len) kend = seq_len;
  const int n_ktiles = (kend + PF_KT - 1) / PF_KT;

  // ---- lookup table: byte -> half2(centroid[high nibble], centroid[low nibble]), one copy per lane ----
  __shared__ float s_cent[16];
  if (tid < 16) s_cent[tid] = a.centroids[tid];
  __syncthreads();
  for (int i = tid; i < 256 * 8; i += PF_THREADS) {
    const int e = i >> 3, q4 = i & 7;
    const uint32_t v = pack_half2(s_cent[e >> 4], s_cent[e & 15]);
    *reinterpret_cast<uint4*>(pf_smem + e * 128 + q4 * 16) = make_uint4(v, v, v, v);
  }
  const uint32_t lut = (uint32_t)__cvta_generic_to_shared(pf_smem) + lane * 4;
  const uint32_t stage0 = (uint32_t)__cvta_generic_to_shared(pf_smem) + PF_LUT_BYTES;
  const uint32_t tiles0 = stage0 + 3 * PF_STAGE_BYTES;        // decoded K tile, then decoded V tile

  // ---- this thread's two rows: (token, head) pairs r = g and g + 8 of the warp's 16 ----
  const int tokA = tok_lo + warp * TPW + g / G, tokB = tok_lo + warp * TPW + (g + 8) / G;
  const int headA = g % G, headB = (g + 8) % G;
  const bool liveA = tokA < qlen && q0 + tokA < a.n_tokens, liveB = tokB < qlen && q0 + tokB < a.n_tokens;
  int limA = liveA ? past + tokA + 1 : 0, limB = liveB ? past + tokB + 1 : 0;     // keys the row may see
  if (limA > seq_len) limA = seq_len;
  if (limB > seq_len) limB = seq_len;
  const int64_t rowA = (int64_t)(q0 + tokA) * a.num_q_heads + kvh * G + headA;
  const int64_t rowB = (int64_t)(q0 + tokB) * a.num_q_heads + kvh * G + headB;

  // query fragments: k-step kk covers coordinates 16 kk .. 16 kk + 15 (columns 2t, 2t+1 and 2t+8, 2t+9)
  uint32_t qa[8][4];
  {
    const float* pa = a.qrot + rowA * 128 + 2 * t;
    const float* pb = a.qrot + rowB * 128 + 2 * t;
#pragma unroll
    for (int kk = 0; kk < 8; ++kk) {
      const float2 z = make_float2(0.f, 0.f);
      const float2 a0 = liveA ? *reinterpret_cast<const float2*>(pa + 16 * kk) : z;
      const float2 a2 = liveA ? *reinterpret_cast<const float2*>(pa + 16 * kk + 8) : z;
      const float2 b0 = liveB ? *reinterpret_cast<const float2*>(pb + 16 * kk) : z;
      const float2 b2 = liveB ? *reinterpret_cast<const float2*>(pb + 16 * kk + 8) : z;
      qa[kk][0] = pack_half2(a0.x, a0.y);
      qa[kk][1] = pack_half2(b0.x, b0.y);
      qa[kk][2] = pack_half2(a2.x, a2.y);
      qa[kk][3] = pack_half2(b2.x, b2.y);
    }
  }

  float o[16][4];
#pragma unroll
  for (int j = 0; j < 16; ++j) { o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f; }
  float mA = -CUDART_INF_F, mB = -CUDART_INF_F, lA = 0.f, lB = 0.f;

  // ---- key tiles of 32 keys.  Thread (key r = tid / 4, chunk c = tid % 4) copies 16 bytes of K and 16 bytes of V
  // and later decodes exactly those bytes itself; threads with c < 2 also copy the key's K or V norm.  Three raw
  // stages (tiles j + 1 and j + 2 in flight while tile j is computed); the physical block of the tile after is
  // looked up one iteration ahead so that the copy never waits for the block table. ----
  const int cr = tid >> 2, cc = tid & 3;
  const int n_table = a.max_blocks_per_seq;
  auto lookup = [&](int j) -> int64_t {
    int blk = (PF_KT * j + (cr & 16)) / a.block_size;
    if (blk >= n_table) blk = n_table - 1;
    if (j >= n_ktiles || blk < 0) return 0;
    const int64_t pb_ = load_index(a.block_tables, a.bt_dtype, (int64_t)s * a.bt_stride + blk);
    return pb_ < 0 ? 0 : (pb_ >= a.num_blocks ? a.num_blocks - 1 : pb_);
  };
  auto issue = [&](int j, int64_t pb_) {
    const int key = PF_KT * j + cr;
    const int pos = key - (key / a.block_size) * a.block_size;
    const uint32_t st = stage0 + (uint32_t)(j % 3) * PF_STAGE_BYTES;
    const uint8_t* ks = a.k_packed + pb_ * a.kp_sb + (int64_t)pos * a.kp_sp + kvh * a.kp_sh + cc * 16;
    const uint8_t* vs = a.v_packed + pb_ * a.vp_sb + (int64_t)pos * a.vp_sp + kvh * a.vp_sh + cc * 16;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" :: "r"(st + tid * 16), "l"(ks) : "memory");
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" :: "r"(st + PF_KT * 64 + tid * 16), "l"(vs) : "memory");
    if (cc < 2) {
      const float* src = cc ? a.v_norms + pb_ * a.vn_sb + (int64_t)pos * a.vn_sp + kvh * a.vn_sh
                            : a.k_norms + pb_ * a.kn_sb + (int64_t)pos * a.kn_sp + kvh * a.kn_sh;
      asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" :: "r"(st + PF_KT * 128 + cc * (PF_KT * 4) + cr * 4), "l"(src) : "memory");
    }
  };

  if (n_ktiles > 0) issue(0, lookup(0));
  asm volatile("cp.async.commit_group;\n" ::: "memory");
  if (n_ktiles > 1) issue(1, lookup(1));
  asm volatile("cp.async.commit_group;\n" ::: "memory");
  int64_t pb_next = lookup(2);
  // decoded halves of word i of the thread's chunk go to 16-byte piece i ^ 2 (c >> 1) first: the eight threads of a
  // quarter warp then hit eight different bank groups with every store
  const uint32_t dk0 = tiles0 + cr * (PF_LD * 2) + cc * 64;
  const uint32_t pxor = (uint32_t)(cc >> 1) << 5;
#pragma unroll 1
  for (int j = 0; j < n_ktiles; ++j) {
    asm volatile("cp.async.wait_group 1;\n" ::: "memory");       // this thread's copies of tile j have landed
    __syncthreads();                                   // everyone has finished with the decoded tiles and the norms of tile j-1
    if (j + 2 < n_ktiles) issue(j + 2, pb_next);      // into the stage tile j-1 used
    asm volatile("cp.async.commit_group;\n" ::: "memory");
    pb_next = lookup(j + 3);
    const uint32_t st = stage0 + (uint32_t)(j % 3) * PF_STAGE_BYTES;
    const int key0 = PF_KT * j;
    // ---- codes -> fp16 tiles, once for the CTA ----
#pragma unroll
    for (int side = 0; side < 2; ++side) {
      uint4 w = lds128(st + side * (PF_KT * 64) + tid * 16);
      if (cc >> 1) { uint32_t x = w.x; w.x = w.z; w.z = x; x = w.y; w.y = w.w; w.w = x; }
      const uint32_t ws[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        uint32_t h[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) h[e] = lds32(lut + (((ws[i] >> (8 * e)) & 0xffu) << 7));
        const uint32_t d = dk0 + side * PF_TILE_BYTES + (((uint32_t)i << 4) ^ pxor);
        asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};\n" :: "r"(d), "r"(h[0]), "r"(h[1]), "r"(h[2]), "r"(h[3]) : "memory");
      }
    }
    __syncthreads();                                   // the decoded tiles are complete, the norms visible

    // ================= scores =================
    float sc[4][4];
#pragma unroll
    for (int n8 = 0; n8 < 4; ++n8) sc[n8][0] = sc[n8][1] = sc[n8][2] = sc[n8][3] = 0.f;
    {
      const uint32_t ka = tiles0 + ((lane & 7) + 8 * (lane >> 4)) * (PF_LD * 2) + 8 * ((lane >> 3) & 1) * 2;
#pragma unroll
      for (int kk = 0; kk < 8; ++kk) {
        uint32_t b0[4], b1[4];      // keys 0..7: (dims 16kk.., 16kk+8..), keys 8..15: the same; then keys 16..31
        pf_ldmatrix(b0, ka + 32 * kk);
        pf_ldmatrix(b1, ka + 32 * kk + 16 * (PF_LD * 2));
        pf_mma(sc[0], qa[kk], b0[0], b0[1]);
        pf_mma(sc[1], qa[kk], b0[2], b0[3]);
        pf_mma(sc[2], qa[kk], b1[0], b1[1]);
        pf_mma(sc[3], qa[kk], b1[2], b1[3]);
      }
    }
    // key norms, causal limits, online softmax (rows A = g, B = g + 8; this thread's keys 8 n8 + 2t, + 1);
    // the probabilities leave multiplied by the value norms, as the A operand of the second product
    uint32_t pa[2][4];
    {
      const float* nk = reinterpret_cast<const float*>(pf_smem + PF_LUT_BYTES + (j % 3) * PF_STAGE_BYTES + PF_KT * 128);
      float mxA = -CUDART_INF_F, mxB = -CUDART_INF_F;
#pragma unroll
      for (int n8 = 0; n8 < 4; ++n8) {
        const float2 k2 = *reinterpret_cast<const float2*>(nk + 8 * n8 + 2 * t);
        const int kx = key0 + 8 * n8 + 2 * t;
        sc[n8][0] = kx < limA ? sc[n8][0] * k2.x : -CUDART_INF_F;
        sc[n8][1] = kx + 1 < limA ? sc[n8][1] * k2.y : -CUDART_INF_F;
        sc[n8][2] = kx < limB ? sc[n8][2] * k2.x : -CUDART_INF_F;
        sc[n8][3] = kx + 1 < limB ? sc[n8][3] * k2.y : -CUDART_INF_F;
        mxA = fmaxf(mxA, fmaxf(sc[n8][0], sc[n8][1]));
        mxB = fmaxf(mxB, fmaxf(sc[n8][2], sc[n8][3]));
      }
      mxA = fmaxf(mxA, __shfl_xor_sync(0xffffffffu, mxA, 1)); mxA = fmaxf(mxA, __shfl_xor_sync(0xffffffffu, mxA, 2));
      mxB = fmaxf(mxB, __shfl_xor_sync(0xffffffffu, mxB, 1)); mxB = fmaxf(mxB, __shfl_xor_sync(0xffffffffu, mxB, 2));
      const float mnA = fmaxf(mA, mxA), mnB = fmaxf(mB, mxB);
      const float refA = mnA == -CUDART_INF_F ? 0.f : mnA, refB = mnB == -CUDART_INF_F ? 0.f : mnB;
      const float alA = ex2_approx(mA - refA), alB = ex2_approx(mB - refB);
      mA = mnA; mB = mnB;
      if (__any_sync(0xffffffffu, (alA != 1.0f) | (alB != 1.0f))) {
#pragma unroll
        for (int jj = 0; jj < 16; ++jj) { o[jj][0] *= alA; o[jj][1] *= alA; o[jj][2] *= alB; o[jj][3] *= alB; }
      }
      float sA = 0.f, sB = 0.f;
#pragma unroll
      for (int n8 = 0; n8 < 4; ++n8) {
        const float p0 = ex2_approx(sc[n8][0] - refA), p1 = ex2_approx(sc[n8][1] - refA);
        const float p2 = ex2_approx(sc[n8][2] - refB), p3 = ex2_approx(sc[n8][3] - refB);
        sA += p0 + p1;
        sB += p2 + p3;
        // a key beyond the sequence may carry any norm: keep it out of the product
        const int kx = key0 + 8 * n8 + 2 * t;
        float2 v2 = *reinterpret_cast<const float2*>(nk + PF_KT + 8 * n8 + 2 * t);
        v2.x = kx < kend ? v2.x : 0.f;
        v2.y = kx + 1 < kend ? v2.y : 0.f;
        pa[n8 >> 1][(n8 & 1) * 2] = pack_half2(p0 * v2.x, p1 * v2.y);          // row A
        pa[n8 >> 1][(n8 & 1) * 2 + 1] = pack_half2(p2 * v2.x, p3 * v2.y);      // row B
      }
      lA = __fmaf_rn(lA, alA, sA);
      lB = __fmaf_rn(lB, alB, sB);
    }

    // ================= values =================
    // B operand of output tiles 2 j2, 2 j2 + 1 (coordinates 16 j2 .. 16 j2 + 15): the value tile transposed
    {
      const uint32_t va = tiles0 + PF_TILE_BYTES + ((lane & 7) + 8 * ((lane >> 3) & 1)) * (PF_LD * 2) + 8 * (lane >> 4) * 2;
#pragma unroll
      for (int j2 = 0; j2 < 8; ++j2) {
        uint32_t b0[4], b1[4];
        pf_ldmatrix_trans(b0, va + 32 * j2);
        pf_ldmatrix_trans(b1, va + 32 * j2 + 16 * (PF_LD * 2));
        pf_mma(o[2 * j2], pa[0], b0[0], b0[1]);
        pf_mma(o[2 * j2 + 1], pa[0], b0[2], b0[3]);
        pf_mma(o[2 * j2], pa[1], b1[0], b1[1]);
        pf_mma(o[2 * j2 + 1], pa[1], b1[2], b1[3]);
      }
    }
  }
  asm volatile("cp.async.wait_group 0;\n" ::: "memory");

  // ---- un-normalised rows for the merge kernel: columns 2t, 2t+1 of tile jj are coordinates 8 jj + 2t, + 1 ----
  lA += __shfl_xor_sync(0xffffffffu, lA, 1); lA += __shfl_xor_sync(0xffffffffu, lA, 2);
  lB += __shfl_xor_sync(0xffffffffu, lB, 1); lB += __shfl_xor_sync(0xffffffffu, lB, 2);
  if (liveA) {
    float* pa_ = a.part_acc + rowA * 128 + 2 * t;
#pragma unroll
    for (int jj = 0; jj < 16; ++jj) *reinterpret_cast<float2*>(pa_ + 8 * jj) = make_float2(o[jj][0], o[jj][1]);
    if (t == 0) { a.part_ml[rowA * 2] = mA; a.part_ml[rowA * 2 + 1] = lA; }
  }
  if (liveB) {
    float* pb_ = a.part_acc + rowB * 128 + 2 * t;
#pragma unroll
    for (int jj = 0; jj < 16; ++jj) *reinterpret_cast<float2*>(pb_ + 8 * jj) = make_float2(o[jj][2], o[jj][3]);
    if (t == 0) { a.part_ml[rowB * 2] = mB; a.part_ml[rowB * 2 + 1] = lB; }
  }
}

}  // namespace akv
