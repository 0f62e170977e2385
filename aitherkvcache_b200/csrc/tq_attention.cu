// Paged decode attention over a TurboQuant-packed KV cache, computed in the
// rotated domain without materialising K/V (reference semantics:
// aither_kvcache/fused_attention.py:91-185; dispatcher :538-748).
//
//   q_rot = R q                                   (akv_qrot_kernel, once per call)
//   s_t   = n^K_t * (q_rot . c[idxK_t]) * scale   (split-K kernels below)
//   acc   = sum_t softmax(s)_t * n^V_t * c[idxV_t]
//   out   = R^T (acc / l)                          (akv_merge_kernel: LSE merge of the
//                                                   split partials + inverse rotation)
//
// Two split-K kernels write the same partial format (m in log2 units, l, acc[D]):
//   * tq_attn_mma_kernel  - head_dim 128, 4/3/2-bit codes, up to 8 query heads per KV
//     head, block_size a multiple of 16.  One warp per (KV head, 16-token tile);
//     codes are turned into fp16 MMA fragments by a shared-memory table lookup
//     (one lookup per code pair) and both products run on mma.sync m16n8k16 with
//     the 4..8 query heads of the group in the N dimension, so every K/V byte is
//     read once for the whole GQA group.
//   * tq_attn_generic_kernel - any power-of-two head_dim in [32, 256], 2/3/4 bits,
//     any GQA ratio.  Scalar; lanes own dims.
#include "common.cuh"
#include "tq_rowmap.cuh"
#include "tq_encode_generic.cuh"
#include <math_constants.h>
#include <stdlib.h>

// 1: one norm load per lane, broadcast by shuffles; 0: four norm loads per thread (slightly faster
// in the shared-memory-staged kernels).
#ifndef AKV_MMA_SEP
#define AKV_MMA_SEP 0
#endif
#ifndef AKV_LDS_NOVOL
#define AKV_LDS_NOVOL 0
#endif
#ifndef AKV_NORM_SHFL
#define AKV_NORM_SHFL 0
#endif

namespace akv {

__device__ int g_attn_window_status;   // 1: a fixed-address kernel found its shared window taken and returned

struct AttnArgs {
  const uint8_t* k_packed; const uint8_t* v_packed;
  int64_t kp_sb, kp_sp, kp_sh;   // bytes: block, position, head
  int64_t vp_sb, vp_sp, vp_sh;
  const float* k_norms; const float* v_norms;
  int64_t kn_sb, kn_sp, kn_sh;   // floats
  int64_t vn_sb, vn_sp, vn_sh;
  const void* block_tables; int bt_dtype; int64_t bt_stride;
  const void* context_lens; int cl_dtype;
  int num_seqs, num_q_heads, num_kv_heads, head_dim, block_size, max_blocks_per_seq;
  int64_t num_blocks;            // physical blocks in the cache (for clamping)
  int bits;
  int pdl;        // launched as a programmatic dependent of the query-rotation launch
  int blocks_per_split, num_splits, warps_per_head, num_parts;
  const float* qrot;             // [S][QH][D] float32, already multiplied by scale*log2(e)
  const float* centroids;
  float* part_acc;               // [S][QH][NP][D]
  float* part_ml;                // [S][QH][NP][2]
  // stream-K plan (persistent kernel): [0..S] prefix of per-sequence stage counts, [S+1] stages per
  // CTA, then first CTA [S], part count [S], block count [S]
  int* sk;
};

__device__ __forceinline__ int64_t phys_block(const AttnArgs& a, int seq, int blk) {
  int64_t b = load_index(a.block_tables, a.bt_dtype, (int64_t)seq * a.bt_stride + blk);
  if (b < 0) b = 0;
  if (b >= a.num_blocks) b = a.num_blocks - 1;
  return b;
}

// ---------------------------------------------------------------------------
// q_rot[s][qh][i] = premul * sum_j R[i][j] q[s][qh][j]   (rot_t[j*D+i] = R[i][j])
// ---------------------------------------------------------------------------
// Stream-K plan: sequence s contributes ceil(blocks_s / 2) two-block stages; the stages of all
// sequences, laid end to end, are cut into `grid` equal ranges, one per persistent CTA.
struct StreamKPlanArgs {
  const void* context_lens; int cl_dtype; int num_seqs; int block_size; int grid;
  int64_t max_ctx;   // max_blocks_per_seq * block_size: context lengths are clamped to [0, max_ctx]
  int* sk;    // nullptr: no plan wanted
  int parts_per_cta;   // partials a CTA writes per (sequence, q head): warps per KV head
  int blocks_per_stage;   // 16-token blocks in a stage (2 or 4)
};

__device__ void streamk_plan(const StreamKPlanArgs& p) {
  __shared__ int s_part[128];
  __shared__ int s_total;
  const int S = p.num_seqs, tid = threadIdx.x, nthr = blockDim.x < 128 ? blockDim.x : 128;
  const int per = (S + nthr - 1) / nthr;
  const bool act = tid < nthr;             // threads past the first 128 only keep the barriers company
  const int s0 = act ? tid * per : S, s1 = (s0 + per < S) ? s0 + per : S;
  int local = 0;
  for (int s = s0; s < s1; ++s) {
    const int64_t ctx = load_ctx(p.context_lens, p.cl_dtype, s, p.max_ctx);
    const int nb = (int)((ctx + p.block_size - 1) / p.block_size);
    p.sk[3 * S + 2 + s] = nb;
    local += (nb + p.blocks_per_stage - 1) / p.blocks_per_stage;
  }
  if (act) s_part[tid] = local;
  __syncthreads();
  if (tid == 0) {
    int run = 0;
    const int used = per > 0 ? (S + per - 1) / per : 0;     // only these threads own sequences and read their prefix
    for (int i = 0; i < used; ++i) { const int v = s_part[i]; s_part[i] = run; run += v; }
    s_total = run;
  }
  __syncthreads();
  const int T = s_total;
  const int chunk = T > 0 ? (T + p.grid - 1) / p.grid : 1;
  int run = act ? s_part[tid] : 0;
  for (int s = s0; s < s1; ++s) {
    const int cnt = (p.sk[3 * S + 2 + s] + p.blocks_per_stage - 1) / p.blocks_per_stage;
    p.sk[s] = run;
    p.sk[S + 2 + s] = cnt > 0 ? run / chunk : 0;
    p.sk[2 * S + 2 + s] = cnt > 0 ? p.parts_per_cta * ((run + cnt - 1) / chunk - run / chunk + 1) : 0;
    run += cnt;
  }
  if (tid == 0) { p.sk[S] = T; p.sk[S + 1] = chunk; }
}

// The new token's K and V vectors of a decode step, written into the paged cache by extra blocks of
// the query-rotation launch (n_rows vectors each; n_rows == 0: nothing to write).
struct NewTokenWrite {
  RowMap k, v;
  int64_t n_rows;
  int bits;
  const float* boundaries;
};

__global__ void akv_qrot_kernel(const void* __restrict__ q, int q_dtype, int64_t q_ss, int64_t q_sh,
                                int num_q_heads, int D, const float* __restrict__ rot_t,
                                float premul, float* __restrict__ qrot, int rows, int plan_blocks,
                                StreamKPlanArgs plan, NewTokenWrite nt) {
  extern __shared__ __align__(16) float qs[];
  if ((int)blockIdx.x >= rows + plan_blocks) {   // blocks past the plan block: one K or V vector each (128 threads)
    const int64_t e = (int64_t)blockIdx.x - rows - plan_blocks;
    const bool is_v = e >= nt.n_rows;
    encode_generic_rows(is_v ? nt.v : nt.k, is_v ? e - nt.n_rows : e, nt.n_rows, nt.n_rows, D, nt.bits, rot_t,
                        nt.boundaries);
    return;
  }
  if ((int)blockIdx.x == rows) {   // the extra block computes the stream-K plan
    streamk_plan(plan);
    return;
  }
  int s = blockIdx.x / num_q_heads, qh = blockIdx.x % num_q_heads;
  for (int j = threadIdx.x; j < D; j += blockDim.x)
    qs[j] = load_as_float(q, q_dtype, s * q_ss + qh * q_sh + j);
  __syncthreads();
  for (int i = threadIdx.x; i < D; i += blockDim.x) {
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    for (int j = 0; j < D; j += 32) {      // 32 loads in flight per round (the matrix sits in L2)
      float r[32];
#pragma unroll
      for (int k = 0; k < 32; ++k) r[k] = rot_t[(int64_t)(j + k) * D + i];
#pragma unroll
      for (int k = 0; k < 32; ++k) acc[k & 3] = __fmaf_rn(r[k], qs[j + k], acc[k & 3]);
    }
    qrot[(int64_t)blockIdx.x * D + i] = ((acc[0] + acc[1]) + (acc[2] + acc[3])) * premul;
  }
}

// ---------------------------------------------------------------------------
// LSE merge of `np` partials per (seq, q head) followed by out = R^T (acc / l).
// Part p of row r: acc at acc + r*acc_row + p*acc_part (+ d), ml at ml + r*ml_row + p*ml_part.
// n_valid (optional, per sequence via context_lens): only parts < n_valid are read.
// mode MERGE_ROTATE: out = R^T (acc / l); MERGE_NORMALIZE: out = acc / l;
// MERGE_RAW: the merged, un-normalised (m, l, acc) goes to raw_out as [row][D+2]
// for a later cross-device merge.
// ---------------------------------------------------------------------------
__global__ void akv_merge_kernel(MergeArgs a) {
  extern __shared__ float sm[];   // [D] merged vector, then [np] weights
  float* wts = sm + a.D;
  __shared__ float s_red[2];
  const int row = blockIdx.x;
  const int seq = row / a.num_q_heads, qh = row % a.num_q_heads;
  int np = a.np;
  if (a.part_counts != nullptr) {
    np = a.part_counts[seq] < np ? a.part_counts[seq] : np;
  } else if (a.context_lens != nullptr) {
    int64_t ctx = load_index(a.context_lens, a.cl_dtype, seq);
    int64_t splits = (ctx + a.tokens_per_split - 1) / a.tokens_per_split;
    int64_t v = splits * a.warps_per_head;
    np = (int)(v < np ? v : np);
  }
  const float* ml = a.ml + merge_half_offset(a) + (int64_t)row * a.ml_row;
  // weights w_p = 2^(m_p - M) for parts with l_p > 0 (first warp), L = sum l_p w_p
  if (threadIdx.x < 32) {
    float M = -CUDART_INF_F;
    for (int p = threadIdx.x; p < np; p += 32) {
      const float m = ml[(int64_t)p * a.ml_part], l = ml[(int64_t)p * a.ml_part + 1];   // both loads in flight together
      if (l > 0.f) M = fmaxf(M, m);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, o));
    float L = 0.f;
    for (int p = threadIdx.x; p < np; p += 32) {
      const float l = ml[(int64_t)p * a.ml_part + 1];
      const float w = (l > 0.f) ? exp2f(ml[(int64_t)p * a.ml_part] - M) : 0.f;
      wts[p] = w;
      L += l * w;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) L += __shfl_xor_sync(0xffffffffu, L, o);
    if (threadIdx.x == 0) { s_red[0] = M; s_red[1] = L; }
  }
  __syncthreads();
  const float M = s_red[0], L = s_red[1];
  const float* acc = a.acc + merge_half_offset(a) + (int64_t)row * a.acc_row;
  for (int d = threadIdx.x; d < a.D; d += blockDim.x) {
    float o4[4] = {0.f, 0.f, 0.f, 0.f};    // independent chains so the loads overlap
    int p = 0;
    for (; p + 8 <= np; p += 8) {          // 8 loads in flight per round
      float v[8];
#pragma unroll
      for (int k = 0; k < 8; ++k) v[k] = acc[(int64_t)(p + k) * a.acc_part + d];
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        const float w = wts[p + k];
        o4[k & 3] = (w != 0.f) ? __fmaf_rn(v[k], w, o4[k & 3]) : o4[k & 3];
      }
    }
    if (p < np) {                          // the last np % 8 parts: one masked round, loads in flight together
      float v[8];
#pragma unroll
      for (int k = 0; k < 8; ++k) v[k] = (p + k < np) ? acc[(int64_t)(p + k) * a.acc_part + d] : 0.f;
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        const float w = (p + k < np) ? wts[p + k] : 0.f;
        o4[k & 3] = (w != 0.f) ? __fmaf_rn(v[k], w, o4[k & 3]) : o4[k & 3];
      }
    }
    const float o = (o4[0] + o4[1]) + (o4[2] + o4[3]);
    if (a.mode == MERGE_RAW) {
      a.raw_out[(int64_t)row * (a.D + 2) + 2 + d] = o;
    } else {
      const float v = (L > 0.f) ? o / L : 0.f;
      if (a.mode == MERGE_NORMALIZE) store_from_float(a.out, a.out_dtype, seq * a.out_ss + qh * a.out_sh + d, v);
      else sm[d] = v;
    }
  }
  if (a.mode == MERGE_RAW) {
    if (threadIdx.x == 0) {
      a.raw_out[(int64_t)row * (a.D + 2)] = M;
      a.raw_out[(int64_t)row * (a.D + 2) + 1] = L;
    }
    return;
  }
  if (a.mode == MERGE_NORMALIZE) return;
  __syncthreads();
  for (int j = threadIdx.x; j < a.D; j += blockDim.x) {
    float x4[4] = {0.f, 0.f, 0.f, 0.f};
    for (int i = 0; i < a.D; i += 32) {
      float r[32];
#pragma unroll
      for (int k = 0; k < 32; ++k) r[k] = a.rot[(int64_t)(i + k) * a.D + j];
#pragma unroll
      for (int k = 0; k < 32; ++k) x4[k & 3] = __fmaf_rn(sm[i + k], r[k], x4[k & 3]);
    }
    const float o = (x4[0] + x4[1]) + (x4[2] + x4[3]);
    store_from_float(a.out, a.out_dtype, seq * a.out_ss + qh * a.out_sh + j, o);
    if (a.out2 != nullptr) store_from_float(a.out2, a.out_dtype, (int64_t)row * a.D + j, o);
  }
}


// ---------------------------------------------------------------------------
// head_dim 128: the same two kernels with the 64 KB rotation matrix staged in shared memory.
// 512 threads; each group of 128 threads owns one (sequence, q head) row at a time, a CTA walks over
// row quads.  The matrix is copied once per CTA with cp.async while the rows' own data arrives, so a
// row costs one trip to L2 for its inputs and none for the matrix.  Summation orders are those of
// akv_qrot_kernel / akv_merge_kernel: results are bit-identical.
// ---------------------------------------------------------------------------
constexpr int ROT128_THREADS = 512;
constexpr int ROT128_MAT_BYTES = 128 * 128 * 4;

__device__ __forceinline__ void stage_matrix128(float* dst, const float* __restrict__ src) {
  const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
  for (int i = threadIdx.x; i < 128 * 128 / 4; i += ROT128_THREADS)
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" :: "r"(d + i * 16), "l"(src + i * 4));
  asm volatile("cp.async.commit_group;\n" ::);
}
__device__ __forceinline__ void group_sync(int g) {      // the 128 threads of row group g
  asm volatile("bar.sync %0, 128;\n" :: "r"(g + 1) : "memory");
}

// The new token's vectors, four per CTA of 512 threads (head_dim 128): threads 128 g .. 128 g + 127 encode vector
// 4 * quad + g (K rows first, then V rows), each group on its own named barrier.  Per vector the arithmetic and its order
// are those of encode_generic_rows: norm by sumsq_8lane, exact division, one accumulation chain j = 0..127 per output.
// `scratch`: 4 x 168 floats of shared memory.
__device__ __forceinline__ void encode128_quad(const RowMap& mk, const RowMap& mv, int64_t n_rows, int64_t quad, int bits,
                                               const float* __restrict__ rot_t, const float* __restrict__ boundaries,
                                               float* scratch) {
  constexpr int D = 128;
  const int g = threadIdx.x >> 7, i = threadIdx.x & 127;
  const int64_t e = quad * 4 + g;
  if (e >= 2 * n_rows) return;              // the whole group leaves; the others only use their own barriers
  const bool is_v = e >= n_rows;
  const RowMap& m = is_v ? mv : mk;
  float* u = scratch + g * 168;                              // [128]
  uint8_t* codes = reinterpret_cast<uint8_t*>(u + D);        // [128]
  float* s_nrm = u + D + 32;
  const int nb = (1 << bits) - 1;
  const int pd = D * bits / 8;
  RowAddr a = map_row(m, is_v ? e - n_rows : e);
  u[i] = load_as_float(a.src_base, m.x_dtype, a.src_off + i);
  group_sync(g);
  if (i < 32) {
    const float tot = sumsq_8lane(u, D, i & 7, 0xffffffffu);
    if (i == 0) *s_nrm = __fsqrt_rn(tot);
  }
  group_sync(g);
  const float nrm = *s_nrm;
  const float den = __fadd_rn(nrm, 1e-10f);
  u[i] = __fdiv_rn(u[i], den);              // the first warp finished reading u before the barrier above
  group_sync(g);
  float y = 0.f;
  for (int j0 = 0; j0 < D; j0 += 32) {      // 32 loads in flight per round: the matrix comes from L2
    float r[32];
#pragma unroll
    for (int k = 0; k < 32; ++k) r[k] = rot_t[(int64_t)(j0 + k) * D + i];
#pragma unroll
    for (int k = 0; k < 32; ++k) y = __fmaf_rn(u[j0 + k], r[k], y);
  }
  int c = 0;
  for (int k = 0; k < nb; ++k) c += (boundaries[k] < y) ? 1 : 0;
  codes[i] = (uint8_t)c;
  group_sync(g);
  if (a.dst != nullptr) {
    if (i < pd) {
      int val = 0;
      for (int bit = 0; bit < 8; ++bit) {
        const int pos = i * 8 + bit;
        const int k = pos / bits, off = pos - k * bits;
        val = (val << 1) | ((codes[k] >> (bits - 1 - off)) & 1);
      }
      a.dst[i] = (uint8_t)val;
    }
    if (i == 0) *a.dst_norm = nrm;
  }
}

__global__ void __launch_bounds__(ROT128_THREADS)
akv_qrot128_kernel(const void* __restrict__ q, int q_dtype, int64_t q_ss, int64_t q_sh, int num_q_heads,
                   const float* __restrict__ rot_t, float premul, float* __restrict__ qrot, int rows,
                   int rot_blocks, int plan_blocks, StreamKPlanArgs plan, NewTokenWrite nt) {
  extern __shared__ __align__(16) float qs[];
  constexpr int D = 128;
  // the attention launch that follows may be scheduled already: it waits (griddepcontrol.wait) for this whole
  // grid before it reads the plan or the rotated queries
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  // block order: the new token's vectors first (the longest-running blocks, so they start at once), then
  // the plan block, then the rotation blocks
  const int enc_blocks = (int)((2 * nt.n_rows + 3) / 4);
  if ((int)blockIdx.x < enc_blocks) {       // four K or V vectors of the new token
    encode128_quad(nt.k, nt.v, nt.n_rows, blockIdx.x, nt.bits, rot_t, nt.boundaries, qs);
    return;
  }
  if ((int)blockIdx.x < enc_blocks + plan_blocks) {
    streamk_plan(plan);
    return;
  }
  const int rb = (int)blockIdx.x - enc_blocks - plan_blocks;      // rotation block index
  float* mat = qs;                          // [128][128]: mat[j * 128 + i] = rot_t[j * 128 + i]
  float* qv = qs + D * D;                   // [4][128]
  stage_matrix128(mat, rot_t);
  const int g = threadIdx.x >> 7, i = threadIdx.x & 127;
  bool first = true;
  for (int r0 = rb * 4; r0 < rows; r0 += rot_blocks * 4) {
    const int row = r0 + g;
    const bool live = row < rows;
    if (live) {
      const int s = row / num_q_heads, qh = row % num_q_heads;
      qv[g * D + i] = load_as_float(q, q_dtype, s * q_ss + qh * q_sh + i);
    }
    if (first) {
      asm volatile("cp.async.wait_group 0;\n" ::: "memory");
      __syncthreads();                      // matrix and the first quad of queries
      first = false;
    } else {
      group_sync(g);
    }
    if (live) {
      float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 8
      for (int j = 0; j < D; j += 4) {
#pragma unroll
        for (int k = 0; k < 4; ++k) acc[k] = __fmaf_rn(mat[(j + k) * D + i], qv[g * D + j + k], acc[k]);
      }
      qrot[(int64_t)row * D + i] = ((acc[0] + acc[1]) + (acc[2] + acc[3])) * premul;
    }
    group_sync(g);                          // qv[g] is free again
  }
  asm volatile("cp.async.wait_group 0;\n" ::: "memory");
}

__global__ void __launch_bounds__(ROT128_THREADS)
akv_merge128_kernel(MergeArgs a, int rows, int np_alloc) {
  extern __shared__ __align__(16) float sm[];
  constexpr int D = 128;
  float* mat = sm;                          // [128][128]: rot[i * 128 + j]
  float* vec = sm + D * D;                  // [4][128] merged vectors
  float* wall = vec + 4 * D;                // [4][np_alloc] weights
  float* red = wall + 4 * np_alloc;         // [4][2]  M, L
  stage_matrix128(mat, a.rot);
  // launched as a programmatic dependent, this grid may start while the attention kernel still runs: the
  // partials are complete only after this wait (a no-op for an ordinary launch)
  asm volatile("griddepcontrol.wait;" ::: "memory");
  const int g = threadIdx.x >> 7, d = threadIdx.x & 127;
  float* wts = wall + g * np_alloc;
  bool first = true;
  for (int r0 = blockIdx.x * 4; r0 < rows; r0 += gridDim.x * 4) {
    const int row = r0 + g;
    const bool live = row < rows;
    const int seq = live ? row / a.num_q_heads : 0, qh = live ? row % a.num_q_heads : 0;
    int np = 0;
    constexpr int MP = 24;
    float v[MP];
    if (live) {
      np = a.np;
      if (a.part_counts != nullptr) {
        np = a.part_counts[seq] < np ? a.part_counts[seq] : np;
      } else if (a.context_lens != nullptr) {
        int64_t ctx = load_index(a.context_lens, a.cl_dtype, seq);
        int64_t splits = (ctx + a.tokens_per_split - 1) / a.tokens_per_split;
        int64_t v = splits * a.warps_per_head;
        np = (int)(v < np ? v : np);
      }
      // the partial sums do not depend on the weights: up to MP parts are requested now and arrive while
      // the group's first warp works the weights out
      if (np <= MP) {
        const float* accp = a.acc + merge_half_offset(a) + (int64_t)row * a.acc_row + d;
#pragma unroll
        for (int k = 0; k < MP; ++k) v[k] = (k < np) ? accp[(int64_t)k * a.acc_part] : 0.f;
      }
      if (d < 32) {                         // first warp of the group: weights, as in akv_merge_kernel
        const float* ml = a.ml + merge_half_offset(a) + (int64_t)row * a.ml_row;
        float M = -CUDART_INF_F;
        for (int p = d; p < np; p += 32) {
          const float m = ml[(int64_t)p * a.ml_part], l = ml[(int64_t)p * a.ml_part + 1];
          if (l > 0.f) M = fmaxf(M, m);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, o));
        float L = 0.f;
        for (int p = d; p < np; p += 32) {
          const float l = ml[(int64_t)p * a.ml_part + 1];
          const float w = (l > 0.f) ? exp2f(ml[(int64_t)p * a.ml_part] - M) : 0.f;
          wts[p] = w;
          L += l * w;
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) L += __shfl_xor_sync(0xffffffffu, L, o);
        if (d == 0) { red[2 * g] = M; red[2 * g + 1] = L; }
      }
    }
    group_sync(g);
    if (live) {
      const float L = red[2 * g + 1];
      const float* acc = a.acc + merge_half_offset(a) + (int64_t)row * a.acc_row;
      float o4[4] = {0.f, 0.f, 0.f, 0.f};
      int p = 0;
      if (np <= MP) {                       // same order of additions as the rounds of eight below
#pragma unroll
        for (int k = 0; k < MP; ++k) {
          const float w = (k < np) ? wts[k] : 0.f;
          o4[k & 3] = (w != 0.f) ? __fmaf_rn(v[k], w, o4[k & 3]) : o4[k & 3];
        }
        p = np;
      }
      for (; p + 8 <= np; p += 8) {
        float v[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) v[k] = acc[(int64_t)(p + k) * a.acc_part + d];
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const float w = wts[p + k];
          o4[k & 3] = (w != 0.f) ? __fmaf_rn(v[k], w, o4[k & 3]) : o4[k & 3];
        }
      }
      if (p < np) {                        // the last np % 8 parts: one masked round
        float v[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) v[k] = (p + k < np) ? acc[(int64_t)(p + k) * a.acc_part + d] : 0.f;
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const float w = (p + k < np) ? wts[p + k] : 0.f;
          o4[k & 3] = (w != 0.f) ? __fmaf_rn(v[k], w, o4[k & 3]) : o4[k & 3];
        }
      }
      const float o = (o4[0] + o4[1]) + (o4[2] + o4[3]);
      vec[g * D + d] = (L > 0.f) ? o / L : 0.f;
    }
    if (first) {
      asm volatile("cp.async.wait_group 0;\n" ::: "memory");
      __syncthreads();                      // matrix and the first quad of merged vectors
      first = false;
    } else {
      group_sync(g);
    }
    if (live) {
      float x4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 8
      for (int i = 0; i < D; i += 4) {
#pragma unroll
        for (int k = 0; k < 4; ++k) x4[k] = __fmaf_rn(vec[g * D + i + k], mat[(i + k) * D + d], x4[k]);
      }
      const float o = (x4[0] + x4[1]) + (x4[2] + x4[3]);
      store_from_float(a.out, a.out_dtype, seq * a.out_ss + qh * a.out_sh + d, o);
      if (a.out2 != nullptr) store_from_float(a.out2, a.out_dtype, (int64_t)row * D + d, o);
    }
    group_sync(g);                          // vec[g], wts and red[g] are free again
  }
  asm volatile("cp.async.wait_group 0;\n" ::: "memory");
}

// Normalise-only LSE merge for many rows, D = 128: one warp per row (lane = four dims), eight rows per CTA, grid-stride.
// Same arithmetic and order of operations per element as akv_merge_kernel (weights 2^(m_p - M) for parts with l_p > 0,
// four accumulation chains by part number modulo 4, one division by L); float32 rows out.
__global__ void __launch_bounds__(256)
akv_merge_norm_rows_kernel(MergeArgs a, int rows) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int row = blockIdx.x * 8 + warp; row < rows; row += gridDim.x * 8) {
    const int seq = row / a.num_q_heads, qh = row % a.num_q_heads;
    int np = a.np;
    if (a.part_counts != nullptr) {
      np = a.part_counts[seq] < np ? a.part_counts[seq] : np;
    } else if (a.context_lens != nullptr) {
      const int64_t ctx = load_index(a.context_lens, a.cl_dtype, seq);
      const int64_t splits = (ctx + a.tokens_per_split - 1) / a.tokens_per_split;
      const int64_t v = splits * a.warps_per_head;
      np = (int)(v < np ? v : np);
    }
    const float* ml = a.ml + merge_half_offset(a) + (int64_t)row * a.ml_row;
    const float* acc = a.acc + merge_half_offset(a) + (int64_t)row * a.acc_row + 4 * lane;
    float M = -CUDART_INF_F;
    for (int p = lane; p < np; p += 32) {
      const float m = ml[(int64_t)p * a.ml_part], l = ml[(int64_t)p * a.ml_part + 1];
      if (l > 0.f) M = fmaxf(M, m);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, o));
    float L = 0.f;
    for (int p = lane; p < np; p += 32) {
      const float l = ml[(int64_t)p * a.ml_part + 1];
      const float w = (l > 0.f) ? exp2f(ml[(int64_t)p * a.ml_part] - M) : 0.f;
      L += l * w;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) L += __shfl_xor_sync(0xffffffffu, L, o);
    float o4[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i) o4[i][0] = o4[i][1] = o4[i][2] = o4[i][3] = 0.f;
    for (int p = 0; p < np; ++p) {
      const float l = ml[(int64_t)p * a.ml_part + 1];                 // the same address in all lanes: one broadcast load
      const float w = (l > 0.f) ? exp2f(ml[(int64_t)p * a.ml_part] - M) : 0.f;
      if (w != 0.f) {
        const float4 x = *reinterpret_cast<const float4*>(acc + (int64_t)p * a.acc_part);
        o4[0][p & 3] = __fmaf_rn(x.x, w, o4[0][p & 3]); o4[1][p & 3] = __fmaf_rn(x.y, w, o4[1][p & 3]);
        o4[2][p & 3] = __fmaf_rn(x.z, w, o4[2][p & 3]); o4[3][p & 3] = __fmaf_rn(x.w, w, o4[3][p & 3]);
      }
    }
    float v[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float o = (o4[i][0] + o4[i][1]) + (o4[i][2] + o4[i][3]);
      v[i] = (L > 0.f) ? o / L : 0.f;
    }
    *reinterpret_cast<float4*>(reinterpret_cast<float*>(a.out) + (int64_t)seq * a.out_ss + (int64_t)qh * a.out_sh + 4 * lane) =
        make_float4(v[0], v[1], v[2], v[3]);
  }
}

int launch_merge(const MergeArgs& a, int rows, cudaStream_t st, bool pdl) {
  const int np_alloc = a.np > 0 ? a.np : 1;
  static const bool no_rot128 = getenv("AKV_NO_ROT128") != nullptr;
  static const bool no_rot_gemm = getenv("AKV_NO_ROT_GEMM") != nullptr;
  if (a.D == 128 && a.mode == MERGE_ROTATE && a.gemm_scratch != nullptr && rows >= 2048 && !no_rot_gemm &&
      rot_rows_ok(a.gemm_scratch, AKV_F32, (int64_t)a.num_q_heads * 128, 128, a.out, a.out_dtype, a.out_ss, a.out_sh)) {
    MergeArgs n = a;                       // LSE merge and division only, float32 rows into the scratch ...
    n.mode = MERGE_NORMALIZE;
    n.out = a.gemm_scratch; n.out_dtype = AKV_F32; n.out_ss = (int64_t)a.num_q_heads * 128; n.out_sh = 128;
    n.gemm_scratch = nullptr;
    const bool vec = ((reinterpret_cast<uintptr_t>(a.acc) | (uintptr_t)(a.acc_row * 4) | (uintptr_t)(a.acc_part * 4) |
                       (uintptr_t)(a.half_stride * 4)) & 15) == 0;
    if (vec) {
      const int ctas = (rows + 7) / 8;
      akv_merge_norm_rows_kernel<<<ctas < 8 * sm_count() ? ctas : 8 * sm_count(), 256, 0, st>>>(n, rows);
      if (int rc = check_launch("akv_merge_norm_rows_kernel")) return rc;
    } else {
      akv_merge_kernel<<<rows, 128, (128 + np_alloc) * sizeof(float), st>>>(n);
      if (int rc = check_launch("akv_merge_kernel")) return rc;
    }
    // ... then out = R^T x for all rows at once
    if (int rc = launch_rot_rows(a.gemm_scratch, AKV_F32, (int64_t)a.num_q_heads * 128, 128, a.num_q_heads, nullptr, 0, a.rot,
                                 1.0f, a.out, a.out_dtype, a.out_ss, a.out_sh, rows, st))
      return rc;
    if (a.out2 == nullptr) return AKV_OK;
    // the second destination: a device copy when `out` is dense itself, else the product once more
    if (a.out_sh == 128 && a.out_ss == (int64_t)a.num_q_heads * 128) {
      const size_t bytes = (size_t)rows * 128 * (a.out_dtype == AKV_F32 ? 4 : 2);
      cudaError_t e = cudaMemcpyAsync(a.out2, a.out, bytes, cudaMemcpyDeviceToDevice, st);
      return e == cudaSuccess ? AKV_OK : fail((int)e, "merge: copy of the result: %s", cudaGetErrorString(e));
    }
    return launch_rot_rows(a.gemm_scratch, AKV_F32, (int64_t)a.num_q_heads * 128, 128, a.num_q_heads, nullptr, 0, a.rot, 1.0f,
                           a.out2, a.out_dtype, (int64_t)a.num_q_heads * 128, 128, rows, st);
  }
  const size_t smem128 = (size_t)ROT128_MAT_BYTES + (size_t)(4 * 128 + 4 * np_alloc + 8) * sizeof(float);
  if (a.D == 128 && a.mode == MERGE_ROTATE && !no_rot128 && rows > 0 && smem128 <= 200 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(akv_merge128_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem128);
    if (e != cudaSuccess) return fail((int)e, "merge: smem attribute: %s", cudaGetErrorString(e));
    const int quads = (rows + 3) / 4;
    const int grid = quads < 2 * sm_count() ? quads : 2 * sm_count();
    if (pdl) {
      cudaLaunchConfig_t cfg{};
      cfg.gridDim = dim3(grid); cfg.blockDim = dim3(ROT128_THREADS); cfg.dynamicSmemBytes = smem128; cfg.stream = st;
      cudaLaunchAttribute at[1];
      at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
      at[0].val.programmaticStreamSerializationAllowed = 1;
      cfg.attrs = at; cfg.numAttrs = 1;
      cudaLaunchKernelEx(&cfg, akv_merge128_kernel, a, rows, np_alloc);
    } else {
      akv_merge128_kernel<<<grid, ROT128_THREADS, smem128, st>>>(a, rows, np_alloc);
    }
    return check_launch("akv_merge128_kernel");
  }
  akv_merge_kernel<<<rows, a.D < 128 ? (a.D < 32 ? 32 : a.D) : 128, (a.D + np_alloc) * sizeof(float), st>>>(a);
  return check_launch("akv_merge_kernel");
}

// ---------------------------------------------------------------------------
// Generic split-K kernel.  grid = (splits, kv heads, seqs), 4 warps; warp j takes
// blocks j, j+4, ... of the split; lane owns D/32 consecutive dims.
// ---------------------------------------------------------------------------
constexpr int GEN_WARPS = 4;
constexpr int GEN_QCH = 4;   // query heads processed per pass over the tokens

__global__ void __launch_bounds__(GEN_WARPS * 32)
tq_attn_generic_kernel(AttnArgs a) {
  const int split = blockIdx.x, h = blockIdx.y, seq = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int D = a.head_dim, bits = a.bits, pd = D * bits / 8;
  const int dpl = D / 32;
  const int G = a.num_q_heads / a.num_kv_heads;
  const int64_t ctx = load_ctx(a.context_lens, a.cl_dtype, seq, (int64_t)a.max_blocks_per_seq * a.block_size);
  const int bs = a.block_size;
  const int64_t nblk = (ctx + bs - 1) / bs;
  const int64_t blk_begin = (int64_t)split * a.blocks_per_split;
  if (blk_begin >= nblk) return;
  const int64_t blk_end = (blk_begin + a.blocks_per_split < nblk) ? blk_begin + a.blocks_per_split : nblk;
  const int part = split * GEN_WARPS + warp;
  __shared__ float cent[16];
  if (threadIdx.x < (1 << bits)) cent[threadIdx.x] = a.centroids[threadIdx.x];
  __syncthreads();

  for (int g0 = 0; g0 < G; g0 += GEN_QCH) {
    const int ng = (G - g0 < GEN_QCH) ? G - g0 : GEN_QCH;
    float q[GEN_QCH][8], acc[GEN_QCH][8], m[GEN_QCH], l[GEN_QCH];
#pragma unroll
    for (int gi = 0; gi < GEN_QCH; ++gi) {
      m[gi] = -CUDART_INF_F; l[gi] = 0.f;
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        acc[gi][k] = 0.f;
        q[gi][k] = (gi < ng && k < dpl)
            ? a.qrot[((int64_t)seq * a.num_q_heads + h * G + g0 + gi) * D + lane * dpl + k] : 0.f;
      }
    }
    for (int64_t blk = blk_begin + warp; blk < blk_end; blk += GEN_WARPS) {
      const int64_t pb = phys_block(a, seq, (int)blk);
      const int ntok = (int)((ctx - blk * bs < bs) ? ctx - blk * bs : bs);
      for (int t = 0; t < ntok; ++t) {
        const uint8_t* krow = a.k_packed + pb * a.kp_sb + t * a.kp_sp + h * a.kp_sh;
        const uint8_t* vrow = a.v_packed + pb * a.vp_sb + t * a.vp_sp + h * a.vp_sh;
        const float nk = a.k_norms[pb * a.kn_sb + t * a.kn_sp + h * a.kn_sh];
        const float nv = a.v_norms[pb * a.vn_sb + t * a.vn_sp + h * a.vn_sh];
        float kc[8], vc[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          if (k < dpl) {
            kc[k] = cent[extract_code(krow, lane * dpl + k, bits, pd)];
            vc[k] = cent[extract_code(vrow, lane * dpl + k, bits, pd)] * nv;
          } else { kc[k] = 0.f; vc[k] = 0.f; }
        }
#pragma unroll
        for (int gi = 0; gi < GEN_QCH; ++gi) {
          if (gi >= ng) continue;
          float d = 0.f;
#pragma unroll
          for (int k = 0; k < 8; ++k) d = __fmaf_rn(q[gi][k], kc[k], d);
#pragma unroll
          for (int o = 16; o > 0; o >>= 1) d += __shfl_xor_sync(0xffffffffu, d, o);
          const float s = d * nk;
          const float mn = fmaxf(m[gi], s);
          const float alpha = exp2f(m[gi] - mn);
          const float p = exp2f(s - mn);
          l[gi] = l[gi] * alpha + p;
#pragma unroll
          for (int k = 0; k < 8; ++k) acc[gi][k] = __fmaf_rn(p, vc[k], acc[gi][k] * alpha);
          m[gi] = mn;
        }
      }
    }
    for (int gi = 0; gi < ng; ++gi) {
      const int64_t row = (int64_t)seq * a.num_q_heads + h * G + g0 + gi;
      float* pa = a.part_acc + (row * a.num_parts + part) * D;
      for (int k = 0; k < dpl; ++k) pa[lane * dpl + k] = acc[gi][k];
      if (lane == 0) {
        a.part_ml[(row * a.num_parts + part) * 2] = m[gi];
        a.part_ml[(row * a.num_parts + part) * 2 + 1] = l[gi];
      }
    }
  }
}

// ---------------------------------------------------------------------------
// Tensor-core split-K kernel (head_dim 128).
// ---------------------------------------------------------------------------
constexpr int LUT_STRIDE = 256;                 // bytes between table entries
constexpr int LUT_BYTES = 256 * LUT_STRIDE;     // 64 KB: entry e, lane l at e*256 + l*4

__device__ __forceinline__ void mma16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                         uint32_t a3, uint32_t b0, uint32_t b1) {
#if AKV_MMA_SEP
  float e0, e1, e2, e3;
  asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%11,%12,%13};\n"
      : "=f"(e0), "=f"(e1), "=f"(e2), "=f"(e3)
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(d[0]), "f"(d[1]), "f"(d[2]), "f"(d[3]));
  d[0] = e0; d[1] = e1; d[2] = e2; d[3] = e3;
  return;
#endif
#if AKV_LUT_VOLATILE
  asm volatile(
#else
  asm(
#endif
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};\n"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t x) {
  uint32_t y;
  asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;\n" : "=r"(y) : "r"(x));
  return y;
}

__device__ __forceinline__ uint32_t pack_half2(float lo, float hi) {
  __half2 h = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&h);
}

// Table lookup: byte `k` of `w` selects the entry; the result is
// half2(c[byte >> 4], c[byte & 15]).  lanebase = lane * 4.
// All table reads go through explicit 32-bit shared-space addresses: `lut` is the table's address
// in the shared window (not a generic pointer), so a lookup is one PRMT, one add and one LDS.
using lut_t = uint32_t;

__device__ __forceinline__ uint32_t lds32(uint32_t addr) {
  uint32_t v;
#if AKV_LDS_NOVOL
  asm("ld.shared.u32 %0, [%1];\n" : "=r"(v) : "r"(addr));
#else
  asm volatile("ld.shared.u32 %0, [%1];\n" : "=r"(v) : "r"(addr));
#endif
  return v;
}
__device__ __forceinline__ uint2 lds64(uint32_t addr) {
  uint2 v;
  asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];\n" : "=r"(v.x), "=r"(v.y) : "r"(addr));
  return v;
}
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];\n" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
  return v;
}

// Table reads are not volatile: the table is constant once filled (a barrier before the first
// lookup), and every address depends on tile data read after the barriers, so the compiler may
// schedule them - and the MMAs they feed - freely.
__device__ __forceinline__ uint32_t lds32_table(uint32_t addr) {
  uint32_t v;
#if AKV_LUT_VOLATILE
  asm volatile("ld.shared.u32 %0, [%1];\n" : "=r"(v) : "r"(addr));
#else
  asm("ld.shared.u32 %0, [%1];\n" : "=r"(v) : "r"(addr));
#endif
  return v;
}
template <int K>
__device__ __forceinline__ uint32_t lut4(lut_t lut, uint32_t w, uint32_t lanebase) {
  return lds32_table(lut + __byte_perm(w, lanebase, 0x7604 + (K << 4)));
}

template <bool VEC16>
__device__ __forceinline__ uint4 load16(const uint8_t* p) {
  if (VEC16) return *reinterpret_cast<const uint4*>(p);
  const uint32_t* q = reinterpret_cast<const uint32_t*>(p);
  return make_uint4(q[0], q[1], q[2], q[3]);
}
template <bool VEC16>
__device__ __forceinline__ uint2 load8(const uint8_t* p) {
  if (VEC16) return *reinterpret_cast<const uint2*>(p);
  const uint32_t* q = reinterpret_cast<const uint32_t*>(p);
  return make_uint2(q[0], q[1]);
}

__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Per-thread packed data of one 16-token tile of one KV head.  With `BITS` bits per code a
// thread holds, for the score product, dims 32t..32t+31 of tokens g and g+8 (4*BITS bytes each)
// and, for the value product, dims 16g..16g+15 of tokens 2t, 2t+1, 2t+8, 2t+9 (2*BITS bytes each).
template <int BITS>
struct TileData {
  uint32_t kA[BITS], kB[BITS];   // little-endian words of the K bytes
  uint32_t v[4][2];              // V bytes of the four tokens (3-bit: 6 bytes, 2-bit: 4 bytes)
#if AKV_NORM_SHFL
  float nrm;             // lanes 0..15: K norm of token `lane`; lanes 16..31: V norm of token lane-16
#else
  float nkA, nkB, nvA, nvB;   // norms of tokens g, g+8
#endif
};

// Byte / element offsets that do not change from tile to tile (block_size 16: one tile per block).
struct ThreadOffsets {
  int kA, kB, v0, v1, v2, v3;   // from the block's base in k_packed / v_packed
  int nrm;                      // from the block's base in k_norms (lanes 0..15) or v_norms
  int nkA, nkB, nvA, nvB;
};

template <int BITS, bool VEC16>
__device__ __forceinline__ void load_k(const uint8_t* p, uint32_t (&w)[BITS]) {
  if constexpr (BITS == 4 && VEC16) {
    const uint4 q = *reinterpret_cast<const uint4*>(p);
    w[0] = q.x; w[1] = q.y; w[2] = q.z; w[3] = q.w;
  } else {
#pragma unroll
    for (int i = 0; i < BITS; ++i) w[i] = reinterpret_cast<const uint32_t*>(p)[i];
  }
}

template <int BITS, bool VEC16>
__device__ __forceinline__ void load_v(const uint8_t* p, uint32_t (&w)[2]) {
  if constexpr (BITS == 4) {
    if (VEC16) { const uint2 q = *reinterpret_cast<const uint2*>(p); w[0] = q.x; w[1] = q.y; }
    else { w[0] = reinterpret_cast<const uint32_t*>(p)[0]; w[1] = reinterpret_cast<const uint32_t*>(p)[1]; }
  } else if constexpr (BITS == 3) {   // 6 bytes at a 2-byte aligned address
    const uint16_t* h = reinterpret_cast<const uint16_t*>(p);
    w[0] = (uint32_t)h[0] | ((uint32_t)h[1] << 16);
    w[1] = h[2];
  } else {
    w[0] = *reinterpret_cast<const uint32_t*>(p);
    w[1] = 0;
  }
}

template <int BITS, bool VEC16>
__device__ __forceinline__ void load_tile(const AttnArgs& a, const ThreadOffsets& off, int64_t pb,
                                          int tok0, int lane, TileData<BITS>& d) {
  const uint8_t* kb = a.k_packed + pb * a.kp_sb + (int64_t)tok0 * a.kp_sp;
  const uint8_t* vb = a.v_packed + pb * a.vp_sb + (int64_t)tok0 * a.vp_sp;
  load_k<BITS, VEC16>(kb + off.kA, d.kA);
  load_k<BITS, VEC16>(kb + off.kB, d.kB);
  load_v<BITS, VEC16>(vb + off.v0, d.v[0]);
  load_v<BITS, VEC16>(vb + off.v1, d.v[1]);
  load_v<BITS, VEC16>(vb + off.v2, d.v[2]);
  load_v<BITS, VEC16>(vb + off.v3, d.v[3]);
#if AKV_NORM_SHFL
  const float* nb = (lane < 16) ? a.k_norms + pb * a.kn_sb + (int64_t)tok0 * a.kn_sp
                                : a.v_norms + pb * a.vn_sb + (int64_t)tok0 * a.vn_sp;
  d.nrm = nb[off.nrm];
#else
  const float* kn = a.k_norms + pb * a.kn_sb + (int64_t)tok0 * a.kn_sp;
  const float* vn = a.v_norms + pb * a.vn_sb + (int64_t)tok0 * a.vn_sp;
  d.nkA = kn[off.nkA]; d.nkB = kn[off.nkB]; d.nvA = vn[off.nvA]; d.nvB = vn[off.nvB];
#endif
}

struct SoftmaxState {
  float m0, m1, l0, l1;   // running max (log2 units) and sum for q-head columns 2t, 2t+1
};

// ---- code -> fp16 fragment lookups for 3 and 2 bits ----
// 3-bit table: entry e (two codes, 6 bits) -> half2(c[e >> 3], c[e & 7]) at e*128 + lane*4.
// 2-bit table: entry e (four codes, one byte) -> 4 halves at e*256 + lane*8.
constexpr int LUT3_STRIDE = 128;

// Pair P of an MSB-first 3-bit stream held as big-endian words B[0], B[1], ...
template <int P>
__device__ __forceinline__ uint32_t lut3(lut_t lut, const uint32_t* B, uint32_t lanebase) {
  constexpr int o = 6 * P, w = o >> 5, pos = o & 31;
  uint32_t x;
  if constexpr (pos <= 26) x = B[w] >> (26 - pos);
  else x = __funnelshift_r(B[w + 1], B[w], 58 - pos);
  return lds32(lut + (((x & 63u) << 7) | lanebase));
}

template <int K>
__device__ __forceinline__ uint2 lut2(lut_t lut, uint32_t w, uint32_t lanebase8) {
  return lds64(lut + __byte_perm(w, lanebase8, 0x7604 + (K << 4)));
}

__device__ __forceinline__ uint32_t bswap32(uint32_t w) { return __byte_perm(w, 0, 0x0123); }

// Natural-order fragments of one token's K bytes: n[p] = half2(dim 32t+2p, dim 32t+2p+1), p = 0..15.
template <int BITS>
__device__ __forceinline__ void k_natural(lut_t lut, const uint32_t (&w)[BITS], uint32_t lanebase,
                                          uint32_t (&n)[16]) {
  if constexpr (BITS == 3) {
    const uint32_t B[3] = {bswap32(w[0]), bswap32(w[1]), bswap32(w[2])};
    n[0] = lut3<0>(lut, B, lanebase);   n[1] = lut3<1>(lut, B, lanebase);   n[2] = lut3<2>(lut, B, lanebase);
    n[3] = lut3<3>(lut, B, lanebase);   n[4] = lut3<4>(lut, B, lanebase);   n[5] = lut3<5>(lut, B, lanebase);
    n[6] = lut3<6>(lut, B, lanebase);   n[7] = lut3<7>(lut, B, lanebase);   n[8] = lut3<8>(lut, B, lanebase);
    n[9] = lut3<9>(lut, B, lanebase);   n[10] = lut3<10>(lut, B, lanebase); n[11] = lut3<11>(lut, B, lanebase);
    n[12] = lut3<12>(lut, B, lanebase); n[13] = lut3<13>(lut, B, lanebase); n[14] = lut3<14>(lut, B, lanebase);
    n[15] = lut3<15>(lut, B, lanebase);
  } else {   // 2 bits: byte b holds dims 32t+4b .. 32t+4b+3
    const uint32_t lb8 = lanebase * 2;
    uint2 r;
    r = lut2<0>(lut, w[0], lb8); n[0] = r.x;  n[1] = r.y;
    r = lut2<1>(lut, w[0], lb8); n[2] = r.x;  n[3] = r.y;
    r = lut2<2>(lut, w[0], lb8); n[4] = r.x;  n[5] = r.y;
    r = lut2<3>(lut, w[0], lb8); n[6] = r.x;  n[7] = r.y;
    r = lut2<0>(lut, w[1], lb8); n[8] = r.x;  n[9] = r.y;
    r = lut2<1>(lut, w[1], lb8); n[10] = r.x; n[11] = r.y;
    r = lut2<2>(lut, w[1], lb8); n[12] = r.x; n[13] = r.y;
    r = lut2<3>(lut, w[1], lb8); n[14] = r.x; n[15] = r.y;
  }
}

// Natural-order fragments of one token's V bytes: n[j] = half2(dim 16g+2j, dim 16g+2j+1), j = 0..7.
template <int BITS>
__device__ __forceinline__ void v_natural(lut_t lut, const uint32_t (&w)[2], uint32_t lanebase,
                                          uint32_t (&n)[8]) {
  if constexpr (BITS == 3) {
    // bytes b0..b5 of the stream: w[0] = b0 | b1<<8 | b2<<16 | b3<<24, w[1] = b4 | b5<<8
    const uint32_t B[2] = {bswap32(w[0]), __byte_perm(w[1], 0, 0x0144)};   // b4 b5 0 0 (big-endian)
    n[0] = lut3<0>(lut, B, lanebase); n[1] = lut3<1>(lut, B, lanebase); n[2] = lut3<2>(lut, B, lanebase);
    n[3] = lut3<3>(lut, B, lanebase); n[4] = lut3<4>(lut, B, lanebase); n[5] = lut3<5>(lut, B, lanebase);
    n[6] = lut3<6>(lut, B, lanebase); n[7] = lut3<7>(lut, B, lanebase);
  } else {
    const uint32_t lb8 = lanebase * 2;
    uint2 r;
    r = lut2<0>(lut, w[0], lb8); n[0] = r.x; n[1] = r.y;
    r = lut2<1>(lut, w[0], lb8); n[2] = r.x; n[3] = r.y;
    r = lut2<2>(lut, w[0], lb8); n[4] = r.x; n[5] = r.y;
    r = lut2<3>(lut, w[0], lb8); n[6] = r.x; n[7] = r.y;
  }
}

// One 16-token tile: scores, online softmax, value accumulation.
// `n_valid` (1..16) masks the tail of the last tile of a sequence.
template <int BITS>
__device__ __forceinline__ void process_tile(lut_t lut, uint32_t lanebase, int g,
                                             const uint32_t (&bq)[8][2], const TileData<BITS>& cur,
                                             int n_valid, float (&o)[8][4], SoftmaxState& st) {
  // ---- scores: S^T[16 tokens][8 q heads], two independent accumulation chains ----
  float s[4] = {0.f, 0.f, 0.f, 0.f}, s2[4] = {0.f, 0.f, 0.f, 0.f};
  if constexpr (BITS == 4) {
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      mma16816(s, lut4<0>(lut, cur.kA[w], lanebase), lut4<0>(lut, cur.kB[w], lanebase),
               lut4<1>(lut, cur.kA[w], lanebase), lut4<1>(lut, cur.kB[w], lanebase),
               bq[2 * w][0], bq[2 * w][1]);
      mma16816(s2, lut4<2>(lut, cur.kA[w], lanebase), lut4<2>(lut, cur.kB[w], lanebase),
               lut4<3>(lut, cur.kA[w], lanebase), lut4<3>(lut, cur.kB[w], lanebase),
               bq[2 * w + 1][0], bq[2 * w + 1][1]);
    }
  } else {
    uint32_t na[16], nb[16];
    k_natural<BITS>(lut, cur.kA, lanebase, na);
    k_natural<BITS>(lut, cur.kB, lanebase, nb);
#pragma unroll
    for (int kk = 0; kk < 8; kk += 2) {
      mma16816(s, na[2 * kk], nb[2 * kk], na[2 * kk + 1], nb[2 * kk + 1], bq[kk][0], bq[kk][1]);
      mma16816(s2, na[2 * kk + 2], nb[2 * kk + 2], na[2 * kk + 3], nb[2 * kk + 3], bq[kk + 1][0], bq[kk + 1][1]);
    }
  }
#if AKV_NORM_SHFL
  const float nkA = __shfl_sync(0xffffffffu, cur.nrm, g);
  const float nkB = __shfl_sync(0xffffffffu, cur.nrm, g + 8);
  float nvA = __shfl_sync(0xffffffffu, cur.nrm, g + 16);
  float nvB = __shfl_sync(0xffffffffu, cur.nrm, g + 24);
#else
  const float nkA = cur.nkA, nkB = cur.nkB;
  float nvA = cur.nvA, nvB = cur.nvB;
#endif
  s[0] = (s[0] + s2[0]) * nkA;
  s[1] = (s[1] + s2[1]) * nkA;
  s[2] = (s[2] + s2[2]) * nkB;
  s[3] = (s[3] + s2[3]) * nkB;
  if (n_valid < 16) {   // warp-uniform: only the last tile of a sequence
    if (g >= n_valid) { s[0] = -CUDART_INF_F; s[1] = -CUDART_INF_F; nvA = 0.f; }
    if (g + 8 >= n_valid) { s[2] = -CUDART_INF_F; s[3] = -CUDART_INF_F; nvB = 0.f; }
  }

  // ---- online softmax over the 16 tokens (columns 2t, 2t+1 of this thread) ----
  float mx0 = fmaxf(s[0], s[2]), mx1 = fmaxf(s[1], s[3]);
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
    for (int j = 0; j < 8; ++j) { o[j][0] *= al0; o[j][1] *= al1; o[j][2] *= al0; o[j][3] *= al1; }
    st.m0 = mn0; st.m1 = mn1;
  }
  const float p0 = ex2_approx(s[0] - mn0), p1 = ex2_approx(s[1] - mn1);
  const float p2 = ex2_approx(s[2] - mn0), p3 = ex2_approx(s[3] - mn1);
  st.l0 += p0 + p2;
  st.l1 += p1 + p3;
  // weights times value norms, transposed into the B-operand layout
  const uint32_t pb0 = movmatrix_trans(pack_half2(p0 * nvA, p1 * nvA));
  const uint32_t pb1 = movmatrix_trans(pack_half2(p2 * nvB, p3 * nvB));

  // ---- values: O^T[128 dims][8 q heads] += V^T P^T ----
  if constexpr (BITS == 4) {
#pragma unroll
    for (int w = 0; w < 2; ++w) {
      const uint32_t va = cur.v[0][w], vb = cur.v[1][w], vc = cur.v[2][w], vd = cur.v[3][w];
      // index byte = (code of the first token) << 4 | (code of the second token), same dim
      const uint32_t x01 = (va & 0xF0F0F0F0u) | ((vb >> 4) & 0x0F0F0F0Fu);
      const uint32_t y01 = ((va << 4) & 0xF0F0F0F0u) | (vb & 0x0F0F0F0Fu);
      const uint32_t x23 = (vc & 0xF0F0F0F0u) | ((vd >> 4) & 0x0F0F0F0Fu);
      const uint32_t y23 = ((vc << 4) & 0xF0F0F0F0u) | (vd & 0x0F0F0F0Fu);
      mma16816(o[4 * w + 0], lut4<0>(lut, x01, lanebase), lut4<0>(lut, y01, lanebase),
               lut4<0>(lut, x23, lanebase), lut4<0>(lut, y23, lanebase), pb0, pb1);
      mma16816(o[4 * w + 1], lut4<1>(lut, x01, lanebase), lut4<1>(lut, y01, lanebase),
               lut4<1>(lut, x23, lanebase), lut4<1>(lut, y23, lanebase), pb0, pb1);
      mma16816(o[4 * w + 2], lut4<2>(lut, x01, lanebase), lut4<2>(lut, y01, lanebase),
               lut4<2>(lut, x23, lanebase), lut4<2>(lut, y23, lanebase), pb0, pb1);
      mma16816(o[4 * w + 3], lut4<3>(lut, x01, lanebase), lut4<3>(lut, y01, lanebase),
               lut4<3>(lut, x23, lanebase), lut4<3>(lut, y23, lanebase), pb0, pb1);
    }
  } else {
    // dequantise each token in natural order, then pair the same dim of two tokens
    uint32_t n0[8], n1[8], n2[8], n3[8];
    v_natural<BITS>(lut, cur.v[0], lanebase, n0);
    v_natural<BITS>(lut, cur.v[1], lanebase, n1);
    v_natural<BITS>(lut, cur.v[2], lanebase, n2);
    v_natural<BITS>(lut, cur.v[3], lanebase, n3);
#pragma unroll
    for (int j = 0; j < 8; ++j)
      mma16816(o[j], __byte_perm(n0[j], n1[j], 0x5410), __byte_perm(n0[j], n1[j], 0x7632),
               __byte_perm(n2[j], n3[j], 0x5410), __byte_perm(n2[j], n3[j], 0x7632), pb0, pb1);
  }
}

// Two 16-token tiles of one KV head at once (4-bit codes): the score products of both tiles are
// independent, one softmax update covers the 32 tokens, and both value products accumulate into the
// same output fragments.  Twice the independent work per warp for the 8-warp persistent kernel.
// n_valid_b may be 0 (no second tile): its scores are masked and its weights are zero.
__device__ __forceinline__ void process_tile_pair4(uint32_t lanebase, int g, const uint32_t (&bq)[8][2],
                                                   const TileData<4>& ta, const TileData<4>& tb,
                                                   int n_valid_a, int n_valid_b, float (&o)[8][4],
                                                   SoftmaxState& st) {
  constexpr lut_t lut = 0;
  float sa[4] = {0.f, 0.f, 0.f, 0.f}, sa2[4] = {0.f, 0.f, 0.f, 0.f};
  float sb[4] = {0.f, 0.f, 0.f, 0.f}, sb2[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
  for (int w = 0; w < 4; ++w) {
    mma16816(sa, lut4<0>(lut, ta.kA[w], lanebase), lut4<0>(lut, ta.kB[w], lanebase),
             lut4<1>(lut, ta.kA[w], lanebase), lut4<1>(lut, ta.kB[w], lanebase), bq[2 * w][0], bq[2 * w][1]);
    mma16816(sb, lut4<0>(lut, tb.kA[w], lanebase), lut4<0>(lut, tb.kB[w], lanebase),
             lut4<1>(lut, tb.kA[w], lanebase), lut4<1>(lut, tb.kB[w], lanebase), bq[2 * w][0], bq[2 * w][1]);
    mma16816(sa2, lut4<2>(lut, ta.kA[w], lanebase), lut4<2>(lut, ta.kB[w], lanebase),
             lut4<3>(lut, ta.kA[w], lanebase), lut4<3>(lut, ta.kB[w], lanebase), bq[2 * w + 1][0], bq[2 * w + 1][1]);
    mma16816(sb2, lut4<2>(lut, tb.kA[w], lanebase), lut4<2>(lut, tb.kB[w], lanebase),
             lut4<3>(lut, tb.kA[w], lanebase), lut4<3>(lut, tb.kB[w], lanebase), bq[2 * w + 1][0], bq[2 * w + 1][1]);
  }
  float nvAa = ta.nvA, nvBa = ta.nvB, nvAb = tb.nvA, nvBb = tb.nvB;
  sa[0] = (sa[0] + sa2[0]) * ta.nkA; sa[1] = (sa[1] + sa2[1]) * ta.nkA;
  sa[2] = (sa[2] + sa2[2]) * ta.nkB; sa[3] = (sa[3] + sa2[3]) * ta.nkB;
  sb[0] = (sb[0] + sb2[0]) * tb.nkA; sb[1] = (sb[1] + sb2[1]) * tb.nkA;
  sb[2] = (sb[2] + sb2[2]) * tb.nkB; sb[3] = (sb[3] + sb2[3]) * tb.nkB;
  if (n_valid_a < 16 || n_valid_b < 16) {   // warp-uniform: only at the end of a sequence
    if (g >= n_valid_a) { sa[0] = -CUDART_INF_F; sa[1] = -CUDART_INF_F; nvAa = 0.f; }
    if (g + 8 >= n_valid_a) { sa[2] = -CUDART_INF_F; sa[3] = -CUDART_INF_F; nvBa = 0.f; }
    if (g >= n_valid_b) { sb[0] = -CUDART_INF_F; sb[1] = -CUDART_INF_F; nvAb = 0.f; }
    if (g + 8 >= n_valid_b) { sb[2] = -CUDART_INF_F; sb[3] = -CUDART_INF_F; nvBb = 0.f; }
  }
  float mx0 = fmaxf(fmaxf(sa[0], sa[2]), fmaxf(sb[0], sb[2]));
  float mx1 = fmaxf(fmaxf(sa[1], sa[3]), fmaxf(sb[1], sb[3]));
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
    for (int j = 0; j < 8; ++j) { o[j][0] *= al0; o[j][1] *= al1; o[j][2] *= al0; o[j][3] *= al1; }
    st.m0 = mn0; st.m1 = mn1;
  }
  const float pa0 = ex2_approx(sa[0] - mn0), pa1 = ex2_approx(sa[1] - mn1);
  const float pa2 = ex2_approx(sa[2] - mn0), pa3 = ex2_approx(sa[3] - mn1);
  const float pb0f = ex2_approx(sb[0] - mn0), pb1f = ex2_approx(sb[1] - mn1);
  const float pb2f = ex2_approx(sb[2] - mn0), pb3f = ex2_approx(sb[3] - mn1);
  st.l0 += (pa0 + pa2) + (pb0f + pb2f);
  st.l1 += (pa1 + pa3) + (pb1f + pb3f);
  const uint32_t qa0 = movmatrix_trans(pack_half2(pa0 * nvAa, pa1 * nvAa));
  const uint32_t qa1 = movmatrix_trans(pack_half2(pa2 * nvBa, pa3 * nvBa));
  const uint32_t qb0 = movmatrix_trans(pack_half2(pb0f * nvAb, pb1f * nvAb));
  const uint32_t qb1 = movmatrix_trans(pack_half2(pb2f * nvBb, pb3f * nvBb));
#pragma unroll
  for (int w = 0; w < 2; ++w) {
    uint32_t x01[2], y01[2], x23[2], y23[2];
#pragma unroll
    for (int k = 0; k < 2; ++k) {
      const TileData<4>& tt = k ? tb : ta;
      const uint32_t va = tt.v[0][w], vb = tt.v[1][w], vc = tt.v[2][w], vd = tt.v[3][w];
      x01[k] = (va & 0xF0F0F0F0u) | ((vb >> 4) & 0x0F0F0F0Fu);
      y01[k] = ((va << 4) & 0xF0F0F0F0u) | (vb & 0x0F0F0F0Fu);
      x23[k] = (vc & 0xF0F0F0F0u) | ((vd >> 4) & 0x0F0F0F0Fu);
      y23[k] = ((vc << 4) & 0xF0F0F0F0u) | (vd & 0x0F0F0F0Fu);
    }
#define AKV_PV(J, K)                                                                                        \
    mma16816(o[4 * w + J], lut4<J>(lut, x01[K], lanebase), lut4<J>(lut, y01[K], lanebase),                  \
             lut4<J>(lut, x23[K], lanebase), lut4<J>(lut, y23[K], lanebase), K ? qb0 : qa0, K ? qb1 : qa1);
    AKV_PV(0, 0) AKV_PV(1, 0) AKV_PV(2, 0) AKV_PV(3, 0)
    AKV_PV(0, 1) AKV_PV(1, 1) AKV_PV(2, 1) AKV_PV(3, 1)
#undef AKV_PV
  }
}

template <int BITS, bool VEC16>
__global__ void __launch_bounds__(256, 2)
tq_attn_mma_kernel(AttnArgs a) {
  extern __shared__ __align__(16) unsigned char lut[];
  const int split = blockIdx.x, hg = blockIdx.y, seq = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int64_t ctx = load_ctx(a.context_lens, a.cl_dtype, seq, (int64_t)a.max_blocks_per_seq * a.block_size);
  const int tpb = a.block_size / 16;
  const int64_t tiles_total = (ctx + 15) / 16;
  const int64_t tile_begin = (int64_t)split * a.blocks_per_split * tpb;
  if (tile_begin >= tiles_total) return;   // uniform for the CTA
  int64_t tile_end = tile_begin + (int64_t)a.blocks_per_split * tpb;
  if (tile_end > tiles_total) tile_end = tiles_total;

  // lookup table, one copy per lane (bank = lane); a warp fills one entry
  if constexpr (BITS == 4) {          // byte -> half2(c[hi nibble], c[lo nibble])
    for (int i = threadIdx.x; i < 256 * 32; i += blockDim.x) {
      const int e = i >> 5, l = i & 31;
      *reinterpret_cast<uint32_t*>(lut + e * LUT_STRIDE + l * 4) =
          pack_half2(a.centroids[e >> 4], a.centroids[e & 15]);
    }
  } else if constexpr (BITS == 3) {   // 6 bits -> half2(c[hi 3 bits], c[lo 3 bits])
    for (int i = threadIdx.x; i < 64 * 32; i += blockDim.x) {
      const int e = i >> 5, l = i & 31;
      *reinterpret_cast<uint32_t*>(lut + e * LUT3_STRIDE + l * 4) =
          pack_half2(a.centroids[e >> 3], a.centroids[e & 7]);
    }
  } else {                            // byte -> four halves
    for (int i = threadIdx.x; i < 256 * 32; i += blockDim.x) {
      const int e = i >> 5, l = i & 31;
      *reinterpret_cast<uint2*>(lut + e * LUT_STRIDE + l * 8) =
          make_uint2(pack_half2(a.centroids[e >> 6], a.centroids[(e >> 4) & 3]),
                     pack_half2(a.centroids[(e >> 2) & 3], a.centroids[e & 3]));
    }
  }
  __syncthreads();

  const int wph = a.warps_per_head;
  const int hl = warp / wph, wj = warp - hl * wph;
  const int h = hg * 8 + hl;
  if (h >= a.num_kv_heads) return;
  const int G = a.num_q_heads / a.num_kv_heads;
  const uint32_t lanebase = lane * 4;
  const lut_t lut_s = (lut_t)__cvta_generic_to_shared(lut);

  // query fragments (B operand of the score product): thread (g,t) holds
  // q_rot[qh = g][32t .. 32t+31]; k-tile kk uses dims 32t+4kk .. 32t+4kk+3.
  uint32_t bq[8][2];
  {
    const float* qp = a.qrot + ((int64_t)seq * a.num_q_heads + h * G + (g < G ? g : 0)) * 128 + 32 * t;
#pragma unroll
    for (int kk = 0; kk < 8; ++kk) {
      float4 f = *reinterpret_cast<const float4*>(qp + 4 * kk);
      if (g >= G) f = make_float4(0.f, 0.f, 0.f, 0.f);
      bq[kk][0] = pack_half2(f.x, f.y);
      bq[kk][1] = pack_half2(f.z, f.w);
    }
  }

  ThreadOffsets off;
  off.kA = (int)(g * a.kp_sp + h * a.kp_sh + 4 * BITS * t);
  off.kB = (int)(off.kA + 8 * a.kp_sp);
  off.v0 = (int)(2 * t * a.vp_sp + h * a.vp_sh + 2 * BITS * g);
  off.v1 = (int)(off.v0 + a.vp_sp);
  off.v2 = (int)(off.v0 + 8 * a.vp_sp);
  off.v3 = (int)(off.v0 + 9 * a.vp_sp);
  off.nkA = (int)(g * a.kn_sp + h * a.kn_sh); off.nkB = (int)(off.nkA + 8 * a.kn_sp);
  off.nvA = (int)(g * a.vn_sp + h * a.vn_sh); off.nvB = (int)(off.nvA + 8 * a.vn_sp);
  off.nrm = (lane < 16) ? (int)(lane * a.kn_sp + h * a.kn_sh) : (int)((lane - 16) * a.vn_sp + h * a.vn_sh);

  float o[8][4];
#pragma unroll
  for (int j = 0; j < 8; ++j) { o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f; }
  SoftmaxState st{-CUDART_INF_F, -CUDART_INF_F, 0.f, 0.f};

  // This warp's tiles: tile_begin + wj, + wph, ...  Block ids are fetched 32 tiles at
  // a time (lane i holds the block of the i-th tile of the batch) and broadcast.
  const int64_t first = tile_begin + wj;
  const int n_tiles = first < tile_end ? (int)((tile_end - first + wph - 1) / wph) : 0;
  for (int base = 0; base < n_tiles; base += 32) {
    const int cnt = n_tiles - base < 32 ? n_tiles - base : 32;
    int64_t my_pb = 0;
    if (lane < cnt) my_pb = phys_block(a, seq, (int)((first + (int64_t)(base + lane) * wph) / tpb));
    TileData<BITS> buf0, buf1;
    {
      const int64_t tile = first + (int64_t)base * wph;
      load_tile<BITS, VEC16>(a, off, __shfl_sync(0xffffffffu, my_pb, 0), (int)(tile % tpb) * 16, lane, buf0);
    }
#pragma unroll 1
    for (int i = 0; i < cnt; i += 2) {
      const int64_t tile = first + (int64_t)(base + i) * wph;
      if (i + 1 < cnt) {
        const int64_t pb = __shfl_sync(0xffffffffu, my_pb, i + 1);
        load_tile<BITS, VEC16>(a, off, pb, (int)((tile + wph) % tpb) * 16, lane, buf1);
      }
      {
        const int64_t rem = ctx - tile * 16;
        process_tile<BITS>(lut_s, lanebase, g, bq, buf0, rem < 16 ? (int)rem : 16, o, st);
      }
      if (i + 1 < cnt) {
        if (i + 2 < cnt) {
          const int64_t pb = __shfl_sync(0xffffffffu, my_pb, i + 2);
          load_tile<BITS, VEC16>(a, off, pb, (int)((tile + 2 * wph) % tpb) * 16, lane, buf0);
        }
        const int64_t rem = ctx - (tile + wph) * 16;
        process_tile<BITS>(lut_s, lanebase, g, bq, buf1, rem < 16 ? (int)rem : 16, o, st);
      }
    }
  }

  // ---- partial for this warp ----
  float l0 = st.l0, l1 = st.l1;
#pragma unroll
  for (int offs = 4; offs < 32; offs <<= 1) {
    l0 += __shfl_xor_sync(0xffffffffu, l0, offs);
    l1 += __shfl_xor_sync(0xffffffffu, l1, offs);
  }
  const int part = split * wph + wj;
#pragma unroll
  for (int e = 0; e < 2; ++e) {
    const int qg = 2 * t + e;
    if (qg >= G) continue;
    const int64_t row = (int64_t)seq * a.num_q_heads + h * G + qg;
    float* pa = a.part_acc + (row * a.num_parts + part) * 128;
#pragma unroll
    for (int j = 0; j < 8; ++j)   // M-tile j: row g -> dim 16g+2j, row g+8 -> dim 16g+2j+1
      *reinterpret_cast<float2*>(pa + 16 * g + 2 * j) = make_float2(o[j][e], o[j][2 + e]);
    if (g == 0) {
      a.part_ml[(row * a.num_parts + part) * 2] = e ? st.m1 : st.m0;
      a.part_ml[(row * a.num_parts + part) * 2 + 1] = e ? l1 : l0;
    }
  }
}


// ---------------------------------------------------------------------------
// Pipelined variant for the common cache layout (4-bit, 8 KV heads per CTA, block_size 16,
// token rows of 8 x 64 contiguous bytes, norms [block][16][heads] contiguous).
//
// A CTA of 16 warps streams whole 16-token blocks (8 KB of K codes, 8 KB of V codes, 2 x 512 B
// of norms) into a 4-stage shared-memory ring with 16-byte asynchronous copies, two blocks per
// stage; warp (head, j) consumes block j of every stage.  Copies are written through an XOR
// swizzle so that the fragment reads below are free of bank conflicts:
//   K: 64-byte head slot h is stored at slot h ^ (token & 1)      (two token rows per 128-bit read phase)
//   V: 32-byte slot s is stored at slot s ^ ((token >> 1) & 3)    (four token rows per 64-bit read phase)
// ---------------------------------------------------------------------------
constexpr int PIPE_STAGES = 4;
constexpr int PIPE_STAGE_BYTES = 2 * 8192 + 2 * 8192 + 4 * 512;       // K, V, norms of two blocks
constexpr int PIPE_SMEM = LUT_BYTES + PIPE_STAGES * PIPE_STAGE_BYTES;  // 204800
constexpr int PIPE_MAX_BLOCKS = 256;                                   // blocks per split

__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gsrc) {
  const uint32_t d = (uint32_t)__cvta_generic_to_shared(smem_dst);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" :: "r"(d), "l"(gsrc));
}

__global__ void __launch_bounds__(512, 1)
tq4_attn_pipe_kernel(AttnArgs a) {
  extern __shared__ __align__(128) unsigned char smem[];
  __shared__ int s_pb[PIPE_MAX_BLOCKS];
  __shared__ float s_cent[16];
  unsigned char* lut = smem;
  unsigned char* ring = smem + LUT_BYTES;
  const uint32_t ring_s = (uint32_t)__cvta_generic_to_shared(ring);
  const int split = blockIdx.x, hg = blockIdx.y, seq = blockIdx.z;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t = lane & 3;
  const int64_t ctx = load_ctx(a.context_lens, a.cl_dtype, seq, (int64_t)a.max_blocks_per_seq * a.block_size);
  const int64_t nblk = (ctx + 15) / 16;
  const int64_t blk_begin = (int64_t)split * a.blocks_per_split;
  if (blk_begin >= nblk) return;   // uniform for the CTA
  const int nb = (int)((blk_begin + a.blocks_per_split < nblk ? blk_begin + a.blocks_per_split : nblk) - blk_begin);
  const int n_ss = (nb + 1) / 2;

  for (int i = tid; i < nb; i += 512) s_pb[i] = (int)phys_block(a, seq, (int)(blk_begin + i));
  if (tid < 16) s_cent[tid] = a.centroids[tid];
  __syncthreads();

  // producer role of this thread: one 16-byte chunk of K and of V per block
  const int c_tok = tid >> 5, c_r = tid & 31;
  const int k_dst = c_tok * 512 + (((c_r >> 2) ^ (c_tok & 1)) << 6) + (c_r & 3) * 16;
  const int v_dst = c_tok * 512 + (((c_r >> 1) ^ ((c_tok >> 1) & 3)) << 5) + (c_r & 1) * 16;
  const int64_t k_src = (int64_t)c_tok * a.kp_sp + hg * 512 + c_r * 16;
  const int64_t v_src = (int64_t)c_tok * a.vp_sp + hg * 512 + c_r * 16;
  auto issue = [&](int ss) {
    unsigned char* st = ring + (ss % PIPE_STAGES) * PIPE_STAGE_BYTES;
#pragma unroll
    for (int b2 = 0; b2 < 2; ++b2) {
      const int bi = 2 * ss + b2;
      if (bi >= nb) break;
      const int64_t pb = s_pb[bi];
      cp_async16(st + b2 * 8192 + k_dst, a.k_packed + pb * a.kp_sb + k_src);
      cp_async16(st + 16384 + b2 * 8192 + v_dst, a.v_packed + pb * a.vp_sb + v_src);
    }
    if (tid < 128) {   // norms: 32 chunks of 16 bytes per (K|V, block)
      const int which = tid >> 5, ch = tid & 31, b2 = which & 1;
      const int bi = 2 * ss + b2;
      if (bi < nb) {
        const int64_t pb = s_pb[bi];
        const int tok = ch >> 1, half = ch & 1;
        const float* src = (which < 2)
            ? a.k_norms + pb * a.kn_sb + (int64_t)tok * a.kn_sp + hg * 8 + half * 4
            : a.v_norms + pb * a.vn_sb + (int64_t)tok * a.vn_sp + hg * 8 + half * 4;
        cp_async16(st + 32768 + which * 512 + ch * 16, src);
      }
    }
    asm volatile("cp.async.commit_group;\n" ::);
  };

  // start the copies first; the table fill and the query loads below overlap their latency
#pragma unroll
  for (int ss = 0; ss < PIPE_STAGES - 1; ++ss) {
    if (ss < n_ss) issue(ss);
    else asm volatile("cp.async.commit_group;\n" ::);
  }
  for (int i = tid; i < 256 * 32; i += 512) {
    const int e = i >> 5, l = i & 31;
    *reinterpret_cast<uint32_t*>(lut + e * LUT_STRIDE + l * 4) = pack_half2(s_cent[e >> 4], s_cent[e & 15]);
  }

  const int hl = warp & 7, wj = warp >> 3;
  const int h = hg * 8 + hl;
  const int G = a.num_q_heads / a.num_kv_heads;
  const uint32_t lanebase = lane * 4;
  const lut_t lut_s = (lut_t)__cvta_generic_to_shared(lut);
  uint32_t bq[8][2];
  {
    const float* qp = a.qrot + ((int64_t)seq * a.num_q_heads + h * G + (g < G ? g : 0)) * 128 + 32 * t;
    float4 f[8];
#pragma unroll
    for (int kk = 0; kk < 8; ++kk) f[kk] = *reinterpret_cast<const float4*>(qp + 4 * kk);
#pragma unroll
    for (int kk = 0; kk < 8; ++kk) {
      if (g >= G) f[kk] = make_float4(0.f, 0.f, 0.f, 0.f);
      bq[kk][0] = pack_half2(f[kk].x, f[kk].y);
      bq[kk][1] = pack_half2(f[kk].z, f[kk].w);
    }
  }
  // consumer offsets inside a stage
  const int kA_off = wj * 8192 + g * 512 + ((hl ^ (g & 1)) << 6) + 16 * t;          // token g (g+8: +4096)
  int v_off[4];
  {
    const int toks[4] = {2 * t, 2 * t + 1, 2 * t + 8, 2 * t + 9};
#pragma unroll
    for (int i = 0; i < 4; ++i)
      v_off[i] = 16384 + wj * 8192 + toks[i] * 512 + (((2 * hl + (g >> 2)) ^ ((toks[i] >> 1) & 3)) << 5) + (g & 3) * 8;
  }

  float o[8][4];
#pragma unroll
  for (int j = 0; j < 8; ++j) { o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f; }
  SoftmaxState st{-CUDART_INF_F, -CUDART_INF_F, 0.f, 0.f};

  for (int it = 0; it < n_ss; ++it) {
    asm volatile("cp.async.wait_group %0;\n" :: "n"(PIPE_STAGES - 2) : "memory");
    __syncthreads();                 // stage `it` has landed; stage it-1 is free again
    if (it + PIPE_STAGES - 1 < n_ss) issue(it + PIPE_STAGES - 1);
    else asm volatile("cp.async.commit_group;\n" ::);
    const int bi = 2 * it + wj;
    if (bi < nb) {
      const uint32_t sb = ring_s + (it % PIPE_STAGES) * PIPE_STAGE_BYTES;
      TileData<4> cur;
      const uint4 ka = lds128(sb + kA_off);
      const uint4 kb = lds128(sb + kA_off + 4096);
      cur.kA[0] = ka.x; cur.kA[1] = ka.y; cur.kA[2] = ka.z; cur.kA[3] = ka.w;
      cur.kB[0] = kb.x; cur.kB[1] = kb.y; cur.kB[2] = kb.z; cur.kB[3] = kb.w;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const uint2 v = lds64(sb + v_off[i]);
        cur.v[i][0] = v.x; cur.v[i][1] = v.y;
      }
#if AKV_NORM_SHFL
      cur.nrm = __uint_as_float(lds32(sb + n_off));
#else
      cur.nkA = __uint_as_float(lds32(sb + 32768 + wj * 512 + (g * 8 + hl) * 4));
      cur.nkB = __uint_as_float(lds32(sb + 32768 + wj * 512 + ((g + 8) * 8 + hl) * 4));
      cur.nvA = __uint_as_float(lds32(sb + 33792 + wj * 512 + (g * 8 + hl) * 4));
      cur.nvB = __uint_as_float(lds32(sb + 33792 + wj * 512 + ((g + 8) * 8 + hl) * 4));
#endif
      const int64_t rem = ctx - (blk_begin + bi) * 16;
      process_tile<4>(lut_s, lanebase, g, bq, cur, rem < 16 ? (int)rem : 16, o, st);
    }
  }
  asm volatile("cp.async.wait_group 0;\n" ::: "memory");

  float l0 = st.l0, l1 = st.l1;
#pragma unroll
  for (int offs = 4; offs < 32; offs <<= 1) {
    l0 += __shfl_xor_sync(0xffffffffu, l0, offs);
    l1 += __shfl_xor_sync(0xffffffffu, l1, offs);
  }
  // the two warps of a head combine their partials through shared memory (the ring is free now)
  __syncthreads();
  float* xch = reinterpret_cast<float*>(ring) + (hl * 32 + lane) * 37;   // 36 floats + 1 pad
  if (wj == 1) {
    xch[0] = st.m0; xch[1] = st.m1; xch[2] = l0; xch[3] = l1;
#pragma unroll
    for (int j = 0; j < 8; ++j) { xch[4 + 4 * j] = o[j][0]; xch[5 + 4 * j] = o[j][1]; xch[6 + 4 * j] = o[j][2]; xch[7 + 4 * j] = o[j][3]; }
  }
  __syncthreads();
  if (wj == 1) return;
  {
    const float om0 = xch[0], om1 = xch[1];
    const float mn0 = fmaxf(st.m0, om0), mn1 = fmaxf(st.m1, om1);
    // a side that saw no token has m = -inf and l = 0: its weight is 0
    const float a0 = (st.m0 == mn0) ? 1.f : ex2_approx(st.m0 - mn0), b0 = (om0 == mn0) ? 1.f : ex2_approx(om0 - mn0);
    const float a1 = (st.m1 == mn1) ? 1.f : ex2_approx(st.m1 - mn1), b1 = (om1 == mn1) ? 1.f : ex2_approx(om1 - mn1);
    l0 = l0 * a0 + xch[2] * b0;
    l1 = l1 * a1 + xch[3] * b1;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      o[j][0] = o[j][0] * a0 + xch[4 + 4 * j] * b0;
      o[j][1] = o[j][1] * a1 + xch[5 + 4 * j] * b1;
      o[j][2] = o[j][2] * a0 + xch[6 + 4 * j] * b0;
      o[j][3] = o[j][3] * a1 + xch[7 + 4 * j] * b1;
    }
    st.m0 = mn0; st.m1 = mn1;
  }
  const int part = split;
#pragma unroll
  for (int e = 0; e < 2; ++e) {
    const int qg = 2 * t + e;
    if (qg >= G) continue;
    const int64_t row = (int64_t)seq * a.num_q_heads + h * G + qg;
    float* pa = a.part_acc + (row * a.num_parts + part) * 128;
#pragma unroll
    for (int j = 0; j < 8; ++j)
      *reinterpret_cast<float2*>(pa + 16 * g + 2 * j) = make_float2(o[j][e], o[j][2 + e]);
    if (g == 0) {
      a.part_ml[(row * a.num_parts + part) * 2] = e ? st.m1 : st.m0;
      a.part_ml[(row * a.num_parts + part) * 2 + 1] = e ? l1 : l0;
    }
  }
}

// ---------------------------------------------------------------------------
// Persistent ("stream-K") form of the pipelined kernel.  The two-block stages of all sequences
// are laid end to end and cut into gridDim.x equal ranges (plan in a.sk); every CTA streams its
// range through the copy ring without draining between sequences, so all CTAs finish together
// and a sequence produces only as many partials as CTAs touch it.  Partial slot of (sequence, CTA
// b, warp j): 2 * (b - first_cta[sequence]) + j.
// ---------------------------------------------------------------------------
constexpr int SK_MAX_SEQS = 1024;
// Shared-memory map in ABSOLUTE shared-window addresses.  The lookup table sits at exactly 64 KB so
// that its address bits 8..15 are free: the PRMT that inserts the code byte then yields the complete
// address and a lookup is two instructions (PRMT, LDS).
//   [dyn start, 64 KB)   plan arrays (8.2 KB) + ring stage 0
//   [64 KB, 128 KB)      lookup table
//   [128 KB, ...)        ring stages 1, 2
constexpr int SK_STAGES = 3;
constexpr uint32_t SK_LUT = 65536;
constexpr uint32_t SK_END = 131072 + (SK_STAGES - 1) * PIPE_STAGE_BYTES;   // 200704
constexpr uint32_t SK_LOW_BYTES = (SK_MAX_SEQS + 2) * 4 + SK_MAX_SEQS * 4 + PIPE_STAGE_BYTES;   // below 64 KB
constexpr int SK_DYN_SMEM = SK_END;        // requested dynamic bytes: covers [start, SK_END) for any start >= 0

__device__ __forceinline__ void cp_async16_s(uint32_t smem_dst, const void* gsrc) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" :: "r"(smem_dst), "l"(gsrc));
}

// WPH = warps per KV head: 2 -> 16 warps, warp (head, j) takes block j of every stage and writes its own
// partial; 1 -> 8 warps with twice the registers, a warp takes both blocks of its head's stage.
template <int WPH, bool PAIR>
__global__ void __launch_bounds__(256 * WPH, 1)
tq4_attn_streamk_kernel(AttnArgs a) {
  constexpr int NT = 256 * WPH;
  extern __shared__ __align__(128) unsigned char smem[];
  __shared__ float s_cent[16];
  const uint32_t dyn0 = (uint32_t)__cvta_generic_to_shared(smem);
  // generic pointers into the low region (all shared addresses below are absolute)
  int* s_P = reinterpret_cast<int*>(smem + (SK_LUT - SK_LOW_BYTES - dyn0));   // stage prefix, total, chunk
  int* s_nb = s_P + (SK_MAX_SEQS + 2);                                        // blocks per sequence
  const uint32_t stage0_s = SK_LUT - PIPE_STAGE_BYTES;
  auto stage_addr = [&](int slot) -> uint32_t { return slot == 0 ? stage0_s : 131072u + (uint32_t)(slot - 1) * PIPE_STAGE_BYTES; };
  const int b = blockIdx.x, hg = blockIdx.y;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t = lane & 3;
  const int S = a.num_seqs;
  for (int i = tid; i < S + 2; i += NT) s_P[i] = a.sk[i];
  for (int i = tid; i < S; i += NT) s_nb[i] = a.sk[3 * S + 2 + i];
  if (tid < 16) s_cent[tid] = a.centroids[tid];
  __syncthreads();
  const int T = s_P[S], chunk = s_P[S + 1];
  const int u_begin = b * chunk;
  const int u_end = (u_begin + chunk < T) ? u_begin + chunk : T;
  if (u_begin >= u_end) return;            // uniform for the CTA
  const int n_it = u_end - u_begin;

  // sequence that owns stage u: the one with P[s] <= u < P[s+1] (empty sequences are skipped)
  auto locate = [&](int u, int hint) {
    while (u >= s_P[hint + 1]) ++hint;
    return hint;
  };
  int seq0;
  {
    int lo = 0, hi = S - 1;                // binary search for the first stage
    while (lo < hi) {
      const int mid = (lo + hi + 1) >> 1;
      if (s_P[mid] <= u_begin) lo = mid; else hi = mid - 1;
    }
    seq0 = locate(u_begin, lo);
  }

  // ---- producer ----
  // thread -> (token, 16-byte piece) of a block; with 8 warps a thread copies tokens c_tok and c_tok + 8
  // (same swizzle: token parity and (token >> 1) & 3 are unchanged by +8)
  constexpr int TOK_PASSES = 2 / WPH;
  const int c_tok = tid >> 5, c_r = tid & 31;
  const int k_dst = c_tok * 512 + (((c_r >> 2) ^ (c_tok & 1)) << 6) + (c_r & 3) * 16;
  const int v_dst = c_tok * 512 + (((c_r >> 1) ^ ((c_tok >> 1) & 3)) << 5) + (c_r & 1) * 16;
  const int64_t k_src = (int64_t)c_tok * a.kp_sp + hg * 512 + c_r * 16;
  const int64_t v_src = (int64_t)c_tok * a.vp_sp + hg * 512 + c_r * 16;
  const int64_t k_step = 8 * a.kp_sp, v_step = 8 * a.vp_sp;
  // 32-bit strides (checked on the host) keep the address arithmetic to one wide multiply-add
  const int kp_sb = (int)a.kp_sb, vp_sb = (int)a.vp_sb, kn_sb = (int)a.kn_sb, vn_sb = (int)a.vn_sb;
  const bool bt64 = a.bt_dtype == AKV_I64;
  int up = u_begin;                        // next stage to issue
  int p_seq = seq0 - 1, p_base = 0, p_end = u_begin, p_nb = 0;   // its sequence: stages [p_base, p_end), p_nb blocks
  const char* bt_row = nullptr;
  int pb0 = 0, pb1 = 0;                    // physical blocks of stage `up` (raw table entries until issue())
  bool has1 = false;
  // Block ids of stage `up` (all threads read the same entries).  Only the loads are issued here;
  // the values are first touched (clamped) by the next issue(), one iteration later, so no warp
  // waits on them.
  auto load_pb = [&]() {
    if (up >= p_end) {                     // next sequence (rare)
      p_seq = locate(up, p_seq < 0 ? 0 : p_seq);
      p_base = s_P[p_seq]; p_end = s_P[p_seq + 1]; p_nb = s_nb[p_seq];
      bt_row = reinterpret_cast<const char*>(a.block_tables) + (int64_t)p_seq * a.bt_stride * (bt64 ? 8 : 4);
    }
    const int bi = 2 * (up - p_base);
    has1 = bi + 1 < p_nb;
    const int bj = bi + (has1 ? 1 : 0);
    if (bt64) {
      pb0 = (int)reinterpret_cast<const int64_t*>(bt_row)[bi];
      pb1 = (int)reinterpret_cast<const int64_t*>(bt_row)[bj];
    } else {
      pb0 = reinterpret_cast<const int*>(bt_row)[bi];
      pb1 = reinterpret_cast<const int*>(bt_row)[bj];
    }
  };
  const int nblocks = (int)a.num_blocks;
  auto issue = [&](int slot) {
    pb0 = min(max(pb0, 0), nblocks - 1);
    pb1 = min(max(pb1, 0), nblocks - 1);
    const uint32_t st = stage_addr(slot);
#pragma unroll
    for (int tp = 0; tp < TOK_PASSES; ++tp) {
      cp_async16_s(st + k_dst + tp * 4096, a.k_packed + ((int64_t)pb0 * kp_sb + k_src + tp * k_step));
      cp_async16_s(st + 16384 + v_dst + tp * 4096, a.v_packed + ((int64_t)pb0 * vp_sb + v_src + tp * v_step));
      if (has1) {
        cp_async16_s(st + 8192 + k_dst + tp * 4096, a.k_packed + ((int64_t)pb1 * kp_sb + k_src + tp * k_step));
        cp_async16_s(st + 16384 + 8192 + v_dst + tp * 4096, a.v_packed + ((int64_t)pb1 * vp_sb + v_src + tp * v_step));
      }
    }
    if (tid < 128) {
      const int which = tid >> 5, ch = tid & 31, b2 = which & 1;
      if (b2 == 0 || has1) {
        const int pb = b2 ? pb1 : pb0;
        const int tok = ch >> 1, half = ch & 1;
        const float* src = (which < 2)
            ? a.k_norms + ((int64_t)pb * kn_sb + (int64_t)tok * a.kn_sp + hg * 8 + half * 4)
            : a.v_norms + ((int64_t)pb * vn_sb + (int64_t)tok * a.vn_sp + hg * 8 + half * 4);
        cp_async16_s(st + 32768 + which * 512 + ch * 16, src);
      }
    }
    asm volatile("cp.async.commit_group;\n" ::);
    ++up;
    if (up < u_end) load_pb();             // for the next issue, one iteration from now
  };
  load_pb();
#pragma unroll
  for (int ss = 0; ss < SK_STAGES - 1; ++ss) {
    if (ss < n_it) issue(ss);
    else asm volatile("cp.async.commit_group;\n" ::);
  }
  for (int i = tid; i < 256 * 32; i += NT) {
    const int e = i >> 5, l = i & 31;
    const uint32_t v = pack_half2(s_cent[e >> 4], s_cent[e & 15]);
    asm volatile("st.shared.u32 [%0], %1;\n" :: "r"(SK_LUT + e * LUT_STRIDE + l * 4), "r"(v));
  }

  // ---- consumer ----
  const int hl = warp & 7, wj0 = (WPH == 2) ? (warp >> 3) : 0;
  const int h = hg * 8 + hl;
  const int G = a.num_q_heads / a.num_kv_heads;
  const uint32_t lanebase = SK_LUT | (lane * 4);   // upper address bytes ride along in the PRMT
  constexpr lut_t lut_s = 0;
  const int kA_off = wj0 * 8192 + g * 512 + ((hl ^ (g & 1)) << 6) + 16 * t;
  int v_off[4];
  {
    const int toks[4] = {2 * t, 2 * t + 1, 2 * t + 8, 2 * t + 9};
#pragma unroll
    for (int i = 0; i < 4; ++i)
      v_off[i] = 16384 + wj0 * 8192 + toks[i] * 512 + (((2 * hl + (g >> 2)) ^ ((toks[i] >> 1) & 3)) << 5) + (g & 3) * 8;
  }

  uint32_t bq[8][2];
  float o[8][4];
  SoftmaxState st{-CUDART_INF_F, -CUDART_INF_F, 0.f, 0.f};
  int seq_c = -1, c_base = 0, c_end = 0, c_nb = 0, ctx_c = 0;
  auto begin_seq = [&](int seq) {          // query fragments and fresh accumulators
    seq_c = seq;
    c_base = s_P[seq]; c_end = s_P[seq + 1]; c_nb = s_nb[seq];
    ctx_c = (int)load_ctx(a.context_lens, a.cl_dtype, seq, (int64_t)a.max_blocks_per_seq * a.block_size);
    const float* qp = a.qrot + ((int64_t)seq * a.num_q_heads + h * G + (g < G ? g : 0)) * 128 + 32 * t;
    float4 f[8];
#pragma unroll
    for (int kk = 0; kk < 8; ++kk) f[kk] = *reinterpret_cast<const float4*>(qp + 4 * kk);
#pragma unroll
    for (int kk = 0; kk < 8; ++kk) {
      if (g >= G) f[kk] = make_float4(0.f, 0.f, 0.f, 0.f);
      bq[kk][0] = pack_half2(f[kk].x, f[kk].y);
      bq[kk][1] = pack_half2(f[kk].z, f[kk].w);
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) { o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f; }
    st = SoftmaxState{-CUDART_INF_F, -CUDART_INF_F, 0.f, 0.f};
  };
  auto end_seq = [&]() {                   // this CTA's partial of sequence seq_c
    float l0 = st.l0, l1 = st.l1;
#pragma unroll
    for (int offs = 4; offs < 32; offs <<= 1) {
      l0 += __shfl_xor_sync(0xffffffffu, l0, offs);
      l1 += __shfl_xor_sync(0xffffffffu, l1, offs);
    }
    const int part = WPH * (b - a.sk[S + 2 + seq_c]) + wj0;
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      const int qg = 2 * t + e;
      if (qg >= G) continue;
      const int64_t row = (int64_t)seq_c * a.num_q_heads + h * G + qg;
      float* pa = a.part_acc + (row * a.num_parts + part) * 128;
#pragma unroll
      for (int j = 0; j < 8; ++j)
        *reinterpret_cast<float2*>(pa + 16 * g + 2 * j) = make_float2(o[j][e], o[j][2 + e]);
      if (g == 0) {
        a.part_ml[(row * a.num_parts + part) * 2] = e ? st.m1 : st.m0;
        a.part_ml[(row * a.num_parts + part) * 2 + 1] = e ? l1 : l0;
      }
    }
  };
  begin_seq(seq0);

  for (int it = 0; it < n_it; ++it) {
    asm volatile("cp.async.wait_group %0;\n" :: "n"(SK_STAGES - 2) : "memory");
    __syncthreads();
    if (it + SK_STAGES - 1 < n_it) issue((it + SK_STAGES - 1) % SK_STAGES);
    else asm volatile("cp.async.commit_group;\n" ::);
    const int u = u_begin + it;
    if (u >= c_end) { end_seq(); begin_seq(locate(u, seq_c)); }     // next sequence (rare)
    auto load_tile_s = [&](int jj, TileData<4>& cur) {
      const uint32_t sb = stage_addr(it % SK_STAGES) + jj * 8192;
      const uint32_t nb_ = stage_addr(it % SK_STAGES) + 32768 + (wj0 + jj) * 512;
      const uint4 ka = lds128(sb + kA_off);
      const uint4 kb = lds128(sb + kA_off + 4096);
      cur.kA[0] = ka.x; cur.kA[1] = ka.y; cur.kA[2] = ka.z; cur.kA[3] = ka.w;
      cur.kB[0] = kb.x; cur.kB[1] = kb.y; cur.kB[2] = kb.z; cur.kB[3] = kb.w;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const uint2 v = lds64(sb + v_off[i]);
        cur.v[i][0] = v.x; cur.v[i][1] = v.y;
      }
      cur.nkA = __uint_as_float(lds32(nb_ + (g * 8 + hl) * 4));
      cur.nkB = __uint_as_float(lds32(nb_ + ((g + 8) * 8 + hl) * 4));
      cur.nvA = __uint_as_float(lds32(nb_ + 1024 + (g * 8 + hl) * 4));
      cur.nvB = __uint_as_float(lds32(nb_ + 1024 + ((g + 8) * 8 + hl) * 4));
    };
    if constexpr (WPH == 1 && PAIR) {
      // both blocks of the stage at once; a missing second block (odd block count) is masked out:
      // its shared-memory slot holds stale but decodable bytes
      const int bi = 2 * (u - c_base);
      TileData<4> ta, tb;
      load_tile_s(0, ta);
      load_tile_s(1, tb);
      const int rem_a = ctx_c - bi * 16, rem_b = rem_a - 16;
      process_tile_pair4(lanebase, g, bq, ta, tb, rem_a < 16 ? rem_a : 16,
                         rem_b < 0 ? 0 : (rem_b < 16 ? rem_b : 16), o, st);
    } else {
#pragma unroll
      for (int jj = 0; jj < 2 / WPH; ++jj) {
        const int bi = 2 * (u - c_base) + wj0 + jj;
        if (bi < c_nb) {
          TileData<4> cur;
          load_tile_s(jj, cur);
          const int rem = ctx_c - bi * 16;
          process_tile<4>(lut_s, lanebase, g, bq, cur, rem < 16 ? rem : 16, o, st);
        }
      }
    }
  }
  asm volatile("cp.async.wait_group 0;\n" ::: "memory");
  end_seq();
}

// ---------------------------------------------------------------------------
// Four tiles at once: the persistent kernel with 4-block stages.
//
// Same schedule, copies, swizzles and lookups as tq4_attn_streamk_kernel; a stage is now four
// 16-token blocks of a sequence (64 tokens) and a warp runs the four tiles of its head through one
// code path: four independent score products, one softmax update per 64 tokens, four value
// products into the same fragments.  Two ring slots of 68 KB; their pieces sit where the fixed
// lookup-table address leaves room (absolute shared addresses):
//   [4 KB, 12.5 KB) plan arrays  [12.5 KB, 44.5 KB) slot 0 K  [44.5 KB, 52.5 KB) norms of slots 0, 1
//   [64 KB, 128 KB) lookup table [128 KB, 160 KB) slot 1 K    [160 KB, 192 KB) slot 1 V   [192 KB, 224 KB) slot 0 V
// Blocks missing from the last stage of a sequence are not copied; their tiles are masked.
// ---------------------------------------------------------------------------
constexpr uint32_t SK4_PLAN = 4096;        // dynamic shared memory starts at about 1.1 KB (system-reserved 1 KB + statics)
constexpr uint32_t SK4_K0 = 12800, SK4_N0 = SK4_K0 + 32768, SK4_N1 = SK4_N0 + 4096;
constexpr uint32_t SK4_K1 = 131072, SK4_V1 = SK4_K1 + 32768, SK4_V0 = SK4_V1 + 32768;
constexpr int SK4_DYN_SMEM = SK4_V0 + 32768;     // 229376: covers every address above for any start >= 0
static_assert(SK4_PLAN + (SK_MAX_SEQS + 2) * 4 + SK_MAX_SEQS * 4 <= SK4_K0, "plan arrays overlap the ring");
static_assert(SK4_N1 + 4096 <= SK_LUT, "low region overlaps the lookup table");

// K data, norms and scores of NTILE tiles, one softmax update, then V data and the value products.
template <int NTILE>
__device__ __forceinline__ void process_tiles4(uint32_t lanebase, int g, const uint32_t (&bq)[8][2],
                                               uint32_t k_addr, const uint32_t (&v_addr)[4], uint32_t n_addr,
                                               int rem, float (&o)[8][4], SoftmaxState& st) {
  constexpr lut_t lut = 0;
  float s[NTILE][4], s2[NTILE][4];
  float nk[NTILE][2], nv[NTILE][2];
  {
    uint4 ka[NTILE], kb[NTILE];
#pragma unroll
    for (int j = 0; j < NTILE; ++j) {
      ka[j] = lds128(k_addr + j * 8192);
      kb[j] = lds128(k_addr + j * 8192 + 4096);
      nk[j][0] = __uint_as_float(lds32(n_addr + j * 512));
      nk[j][1] = __uint_as_float(lds32(n_addr + j * 512 + 256));
      nv[j][0] = __uint_as_float(lds32(n_addr + 2048 + j * 512));
      nv[j][1] = __uint_as_float(lds32(n_addr + 2048 + j * 512 + 256));
      s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
      s2[j][0] = s2[j][1] = s2[j][2] = s2[j][3] = 0.f;
    }
#pragma unroll
    for (int w = 0; w < 4; ++w) {
#pragma unroll
      for (int j = 0; j < NTILE; ++j) {
        const uint32_t a = w == 0 ? ka[j].x : w == 1 ? ka[j].y : w == 2 ? ka[j].z : ka[j].w;
        const uint32_t b = w == 0 ? kb[j].x : w == 1 ? kb[j].y : w == 2 ? kb[j].z : kb[j].w;
        mma16816(s[j], lut4<0>(lut, a, lanebase), lut4<0>(lut, b, lanebase),
                 lut4<1>(lut, a, lanebase), lut4<1>(lut, b, lanebase), bq[2 * w][0], bq[2 * w][1]);
        mma16816(s2[j], lut4<2>(lut, a, lanebase), lut4<2>(lut, b, lanebase),
                 lut4<3>(lut, a, lanebase), lut4<3>(lut, b, lanebase), bq[2 * w + 1][0], bq[2 * w + 1][1]);
      }
    }
  }
#pragma unroll
  for (int j = 0; j < NTILE; ++j) {
    s[j][0] = (s[j][0] + s2[j][0]) * nk[j][0]; s[j][1] = (s[j][1] + s2[j][1]) * nk[j][0];
    s[j][2] = (s[j][2] + s2[j][2]) * nk[j][1]; s[j][3] = (s[j][3] + s2[j][3]) * nk[j][1];
  }
  if (rem < 16 * NTILE) {     // warp-uniform: only the last stage of a sequence
#pragma unroll
    for (int j = 0; j < NTILE; ++j) {
      const int nvld = rem - 16 * j;
      if (g >= nvld) { s[j][0] = -CUDART_INF_F; s[j][1] = -CUDART_INF_F; nv[j][0] = 0.f; }
      if (g + 8 >= nvld) { s[j][2] = -CUDART_INF_F; s[j][3] = -CUDART_INF_F; nv[j][1] = 0.f; }
    }
  }
  float mx0 = fmaxf(s[0][0], s[0][2]), mx1 = fmaxf(s[0][1], s[0][3]);
#pragma unroll
  for (int j = 1; j < NTILE; ++j) {
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
    for (int j = 0; j < 8; ++j) { o[j][0] *= al0; o[j][1] *= al1; o[j][2] *= al0; o[j][3] *= al1; }
    st.m0 = mn0; st.m1 = mn1;
  }
  uint32_t pq[NTILE][2];
  float ls0 = 0.f, ls1 = 0.f;
#pragma unroll
  for (int j = 0; j < NTILE; ++j) {
    const float p0 = ex2_approx(s[j][0] - mn0), p1 = ex2_approx(s[j][1] - mn1);
    const float p2 = ex2_approx(s[j][2] - mn0), p3 = ex2_approx(s[j][3] - mn1);
    ls0 += p0 + p2;
    ls1 += p1 + p3;
    pq[j][0] = movmatrix_trans(pack_half2(p0 * nv[j][0], p1 * nv[j][0]));
    pq[j][1] = movmatrix_trans(pack_half2(p2 * nv[j][1], p3 * nv[j][1]));
  }
  st.l0 += ls0;
  st.l1 += ls1;
#pragma unroll
  for (int j = 0; j < NTILE; ++j) {
    uint2 vv[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) vv[i] = lds64(v_addr[i] + j * 8192);
#pragma unroll
    for (int w = 0; w < 2; ++w) {
      const uint32_t va = w ? vv[0].y : vv[0].x, vb = w ? vv[1].y : vv[1].x;
      const uint32_t vc = w ? vv[2].y : vv[2].x, vd = w ? vv[3].y : vv[3].x;
      const uint32_t x01 = (va & 0xF0F0F0F0u) | ((vb >> 4) & 0x0F0F0F0Fu);
      const uint32_t y01 = ((va << 4) & 0xF0F0F0F0u) | (vb & 0x0F0F0F0Fu);
      const uint32_t x23 = (vc & 0xF0F0F0F0u) | ((vd >> 4) & 0x0F0F0F0Fu);
      const uint32_t y23 = ((vc << 4) & 0xF0F0F0F0u) | (vd & 0x0F0F0F0Fu);
      mma16816(o[4 * w + 0], lut4<0>(lut, x01, lanebase), lut4<0>(lut, y01, lanebase),
               lut4<0>(lut, x23, lanebase), lut4<0>(lut, y23, lanebase), pq[j][0], pq[j][1]);
      mma16816(o[4 * w + 1], lut4<1>(lut, x01, lanebase), lut4<1>(lut, y01, lanebase),
               lut4<1>(lut, x23, lanebase), lut4<1>(lut, y23, lanebase), pq[j][0], pq[j][1]);
      mma16816(o[4 * w + 2], lut4<2>(lut, x01, lanebase), lut4<2>(lut, y01, lanebase),
               lut4<2>(lut, x23, lanebase), lut4<2>(lut, y23, lanebase), pq[j][0], pq[j][1]);
      mma16816(o[4 * w + 3], lut4<3>(lut, x01, lanebase), lut4<3>(lut, y01, lanebase),
               lut4<3>(lut, x23, lanebase), lut4<3>(lut, y23, lanebase), pq[j][0], pq[j][1]);
    }
  }
}

__global__ void __launch_bounds__(256, 1)
tq4_attn_streamk4_kernel(AttnArgs a) {
  extern __shared__ __align__(128) unsigned char smem[];
  __shared__ float s_cent[16];
  const uint32_t dyn0 = (uint32_t)__cvta_generic_to_shared(smem);
  int* s_P = reinterpret_cast<int*>(smem + (SK4_PLAN - dyn0));   // stage prefix, total, chunk
  int* s_nb = s_P + (SK_MAX_SEQS + 2);                           // blocks per sequence
  const int b = blockIdx.x, hg = blockIdx.y;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t = lane & 3;
  const int S = a.num_seqs;
  if (dyn0 > SK4_PLAN) {       // the window below the plan arrays is taken (static + system-reserved bytes)
    if (tid == 0) g_attn_window_status = 1;      // the host checks the window before launching; see run_tq_attn
    return;
  }
  for (int i = tid; i < S + 2; i += 256) s_P[i] = a.sk[i];
  for (int i = tid; i < S; i += 256) s_nb[i] = a.sk[3 * S + 2 + i];
  if (tid < 16) s_cent[tid] = a.centroids[tid];
  __syncthreads();
  const int T = s_P[S], chunk = s_P[S + 1];
  const int u_begin = b * chunk;
  const int u_end = (u_begin + chunk < T) ? u_begin + chunk : T;
  if (u_begin >= u_end) return;            // uniform for the CTA
  const int n_it = u_end - u_begin;

  auto locate = [&](int u, int hint) {
    while (hint < S - 1 && u >= s_P[hint + 1]) ++hint;
    return hint;
  };
  int seq0;
  {
    int lo = 0, hi = S - 1;
    while (lo < hi) {
      const int mid = (lo + hi + 1) >> 1;
      if (s_P[mid] <= u_begin) lo = mid; else hi = mid - 1;
    }
    seq0 = locate(u_begin, lo);
  }

  // ---- producer: thread -> (token c_tok and c_tok + 8, 16-byte piece c_r) of every block ----
  const int c_tok = tid >> 5, c_r = tid & 31;
  const int k_dst = c_tok * 512 + (((c_r >> 2) ^ (c_tok & 1)) << 6) + (c_r & 3) * 16;
  const int v_dst = c_tok * 512 + (((c_r >> 1) ^ ((c_tok >> 1) & 3)) << 5) + (c_r & 1) * 16;
  const int64_t k_src = (int64_t)c_tok * a.kp_sp + hg * 512 + c_r * 16;
  const int64_t v_src = (int64_t)c_tok * a.vp_sp + hg * 512 + c_r * 16;
  const int64_t k_step = 8 * a.kp_sp, v_step = 8 * a.vp_sp;
  const int kp_sb = (int)a.kp_sb, vp_sb = (int)a.vp_sb, kn_sb = (int)a.kn_sb, vn_sb = (int)a.vn_sb;
  const bool bt64 = a.bt_dtype == AKV_I64;
  int up = u_begin;
  int p_seq = seq0 - 1, p_base = 0, p_end = u_begin, p_nb = 0;
  const char* bt_row = nullptr;
  int pb[4] = {0, 0, 0, 0};                // physical blocks of stage `up` (raw table entries until issue())
  int n_has = 0;                           // blocks present in stage `up` (1..4)
  auto load_pb = [&]() {
    if (up >= p_end) {
      p_seq = locate(up, p_seq < 0 ? 0 : p_seq);
      p_base = s_P[p_seq]; p_end = s_P[p_seq + 1]; p_nb = s_nb[p_seq];
      bt_row = reinterpret_cast<const char*>(a.block_tables) + (int64_t)p_seq * a.bt_stride * (bt64 ? 8 : 4);
    }
    const int bi = 4 * (up - p_base);
    n_has = p_nb - bi < 4 ? p_nb - bi : 4;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int bj = bi + (j < n_has ? j : 0);
      pb[j] = bt64 ? (int)reinterpret_cast<const int64_t*>(bt_row)[bj] : reinterpret_cast<const int*>(bt_row)[bj];
    }
  };
  const int nblocks = (int)a.num_blocks;
  auto issue = [&](int slot) {
    const uint32_t kb = slot ? SK4_K1 : SK4_K0, vb = slot ? SK4_V1 : SK4_V0, nb_ = slot ? SK4_N1 : SK4_N0;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      pb[j] = min(max(pb[j], 0), nblocks - 1);
      if (j < n_has) {
#pragma unroll
        for (int tp = 0; tp < 2; ++tp) {
          cp_async16_s(kb + j * 8192 + k_dst + tp * 4096, a.k_packed + ((int64_t)pb[j] * kp_sb + k_src + tp * k_step));
          cp_async16_s(vb + j * 8192 + v_dst + tp * 4096, a.v_packed + ((int64_t)pb[j] * vp_sb + v_src + tp * v_step));
        }
      }
    }
    {   // norms: 8 x 512 B, one 16-byte piece per thread
      const int which = tid >> 5, ch = tid & 31, j = which & 3;
      if (j < n_has) {
        const int tok = ch >> 1, half = ch & 1;
        const int pbj = j == 0 ? pb[0] : j == 1 ? pb[1] : j == 2 ? pb[2] : pb[3];
        const float* src = (which < 4)
            ? a.k_norms + ((int64_t)pbj * kn_sb + (int64_t)tok * a.kn_sp + hg * 8 + half * 4)
            : a.v_norms + ((int64_t)pbj * vn_sb + (int64_t)tok * a.vn_sp + hg * 8 + half * 4);
        cp_async16_s(nb_ + which * 512 + ch * 16, src);
      }
    }
    asm volatile("cp.async.commit_group;\n" ::);
    ++up;
    if (up < u_end) load_pb();             // for the next issue, one iteration from now
  };
  load_pb();
  issue(0);
  for (int i = tid; i < 256 * 32; i += 256) {
    const int e = i >> 5, l = i & 31;
    const uint32_t v = pack_half2(s_cent[e >> 4], s_cent[e & 15]);
    asm volatile("st.shared.u32 [%0], %1;\n" :: "r"(SK_LUT + e * LUT_STRIDE + l * 4), "r"(v));
  }

  // ---- consumer: warp = KV head ----
  const int hl = warp;
  const int h = hg * 8 + hl;
  const int G = a.num_q_heads / a.num_kv_heads;
  const uint32_t lanebase = SK_LUT | (lane * 4);
  const int kA_off = g * 512 + ((hl ^ (g & 1)) << 6) + 16 * t;
  int v_off[4];
  {
    const int toks[4] = {2 * t, 2 * t + 1, 2 * t + 8, 2 * t + 9};
#pragma unroll
    for (int i = 0; i < 4; ++i)
      v_off[i] = toks[i] * 512 + (((2 * hl + (g >> 2)) ^ ((toks[i] >> 1) & 3)) << 5) + (g & 3) * 8;
  }
  const int n_off = (g * 8 + hl) * 4;      // norm of token g; token g + 8 is 256 bytes further

  uint32_t bq[8][2];
  float o[8][4];
  SoftmaxState st{-CUDART_INF_F, -CUDART_INF_F, 0.f, 0.f};
  int seq_c = -1, c_base = 0, c_end = 0, ctx_c = 0;
  auto begin_seq = [&](int seq) {
    seq_c = seq;
    c_base = s_P[seq]; c_end = s_P[seq + 1];
    ctx_c = (int)load_ctx(a.context_lens, a.cl_dtype, seq, (int64_t)a.max_blocks_per_seq * a.block_size);
    const float* qp = a.qrot + ((int64_t)seq * a.num_q_heads + h * G + (g < G ? g : 0)) * 128 + 32 * t;
    float4 f[8];
#pragma unroll
    for (int kk = 0; kk < 8; ++kk) f[kk] = *reinterpret_cast<const float4*>(qp + 4 * kk);
#pragma unroll
    for (int kk = 0; kk < 8; ++kk) {
      if (g >= G) f[kk] = make_float4(0.f, 0.f, 0.f, 0.f);
      bq[kk][0] = pack_half2(f[kk].x, f[kk].y);
      bq[kk][1] = pack_half2(f[kk].z, f[kk].w);
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) { o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f; }
    st = SoftmaxState{-CUDART_INF_F, -CUDART_INF_F, 0.f, 0.f};
  };
  auto end_seq = [&]() {
    float l0 = st.l0, l1 = st.l1;
#pragma unroll
    for (int offs = 4; offs < 32; offs <<= 1) {
      l0 += __shfl_xor_sync(0xffffffffu, l0, offs);
      l1 += __shfl_xor_sync(0xffffffffu, l1, offs);
    }
    const int part = b - a.sk[S + 2 + seq_c];
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      const int qg = 2 * t + e;
      if (qg >= G) continue;
      const int64_t row = (int64_t)seq_c * a.num_q_heads + h * G + qg;
      float* pa = a.part_acc + (row * a.num_parts + part) * 128;
#pragma unroll
      for (int j = 0; j < 8; ++j)
        *reinterpret_cast<float2*>(pa + 16 * g + 2 * j) = make_float2(o[j][e], o[j][2 + e]);
      if (g == 0) {
        a.part_ml[(row * a.num_parts + part) * 2] = e ? st.m1 : st.m0;
        a.part_ml[(row * a.num_parts + part) * 2 + 1] = e ? l1 : l0;
      }
    }
  };
  // outer loop: the sequences this CTA's range touches; inner loop: their stages, with nothing but
  // copy, barrier and tile code in it
  int it = 0;
  int seq_next = seq0;
  while (it < n_it) {
    begin_seq(seq_next);
    const int it_end = (c_end - u_begin < n_it) ? c_end - u_begin : n_it;   // stages of this sequence in the range
    for (; it < it_end; ++it) {
      asm volatile("cp.async.wait_group 0;\n" ::: "memory");
      __syncthreads();                     // stage `it` has landed; the other slot is free again
      if (it + 1 < n_it) issue((it + 1) & 1);
      const int u = u_begin + it;
      const int slot = it & 1;
      const uint32_t kb = slot ? SK4_K1 : SK4_K0, vb = slot ? SK4_V1 : SK4_V0, nb_ = slot ? SK4_N1 : SK4_N0;
      const uint32_t va[4] = {vb + v_off[0], vb + v_off[1], vb + v_off[2], vb + v_off[3]};
      const int rem = ctx_c - 64 * (u - c_base);
      process_tiles4<4>(lanebase, g, bq, kb + kA_off, va, nb_ + n_off, rem, o, st);
    }
    end_seq();
    if (it < n_it) seq_next = locate(u_begin + it, seq_c);
  }
}

// ---------------------------------------------------------------------------
// The persistent 4-block-stage kernel for 3-bit and 2-bit codes.
//
// Same schedule, ring slots and plan as tq4_attn_streamk4_kernel.  Token rows of a block are
// 8 heads x PD bytes (PD = 48 or 32); they are copied in 16-byte pieces into rows of a padded pitch
// (400 / 288 bytes) instead of an XOR swizzle: with those pitches the 12-byte (3-bit) and 8-byte
// (2-bit) K fragment reads of the 8 tokens x 4 dim-quarters of a warp fall on distinct banks.
// Tables at absolute shared address 64 KB: 3-bit - 64 entries x 128 B, a 6-bit code pair -> half2;
// 2-bit - 256 entries x 256 B, a byte of four codes -> four halves.  A warp runs the four tiles of
// its head with one softmax update per 64 tokens; scores are built tile by tile (each tile's 32
// natural-order fragments are transient), the value products likewise.
// ---------------------------------------------------------------------------
template <int BITS> struct LowBit {
  static constexpr int PD = 16 * BITS;                   // packed bytes per (token, head)
  static constexpr int ROW = 8 * PD;                     // bytes of a token row (8 heads)
  static constexpr int PITCH = BITS == 3 ? 400 : 288;    // padded row pitch in shared memory
  static constexpr int BLK = 16 * PITCH;                 // one block's K (or V) in shared memory
  static constexpr int PPT = ROW / 16;                   // 16-byte pieces per token row
};

// k-tile fragments of one token in natural order from its 4*BITS packed bytes at `addr`
// (n[p] = half2(dim 32t+2p, 32t+2p+1)); lb4 / lb8 = table base | lane*4 / lane*8.
template <int BITS>
__device__ __forceinline__ void lowbit_k_fragments(uint32_t addr, uint32_t lb4, uint32_t lb8, uint32_t (&n)[16]) {
  if constexpr (BITS == 3) {
    const uint32_t B[3] = {bswap32(lds32(addr)), bswap32(lds32(addr + 4)), bswap32(lds32(addr + 8))};
    n[0] = lut3<0>(0, B, lb4);   n[1] = lut3<1>(0, B, lb4);   n[2] = lut3<2>(0, B, lb4);   n[3] = lut3<3>(0, B, lb4);
    n[4] = lut3<4>(0, B, lb4);   n[5] = lut3<5>(0, B, lb4);   n[6] = lut3<6>(0, B, lb4);   n[7] = lut3<7>(0, B, lb4);
    n[8] = lut3<8>(0, B, lb4);   n[9] = lut3<9>(0, B, lb4);   n[10] = lut3<10>(0, B, lb4); n[11] = lut3<11>(0, B, lb4);
    n[12] = lut3<12>(0, B, lb4); n[13] = lut3<13>(0, B, lb4); n[14] = lut3<14>(0, B, lb4); n[15] = lut3<15>(0, B, lb4);
  } else {
    const uint2 w = lds64(addr);
    uint2 r;
    r = lut2<0>(0, w.x, lb8); n[0] = r.x;  n[1] = r.y;
    r = lut2<1>(0, w.x, lb8); n[2] = r.x;  n[3] = r.y;
    r = lut2<2>(0, w.x, lb8); n[4] = r.x;  n[5] = r.y;
    r = lut2<3>(0, w.x, lb8); n[6] = r.x;  n[7] = r.y;
    r = lut2<0>(0, w.y, lb8); n[8] = r.x;  n[9] = r.y;
    r = lut2<1>(0, w.y, lb8); n[10] = r.x; n[11] = r.y;
    r = lut2<2>(0, w.y, lb8); n[12] = r.x; n[13] = r.y;
    r = lut2<3>(0, w.y, lb8); n[14] = r.x; n[15] = r.y;
  }
}

// value fragments of one token: n[j] = half2(dim 16g+2j, 16g+2j+1), from its 2*BITS bytes at addr
// (3-bit: the 6 bytes start 0 or 2 bytes into the aligned word at addr; sh = 8 * that offset)
template <int BITS>
__device__ __forceinline__ void lowbit_v_fragments(uint32_t addr, uint32_t sh, uint32_t lb4, uint32_t lb8,
                                                   uint32_t (&n)[8]) {
  if constexpr (BITS == 3) {
    const uint32_t wa = lds32(addr), wb = lds32(addr + 4);
    const uint32_t w0 = __funnelshift_r(wa, wb, sh), w1 = wb >> sh;
    const uint32_t B[2] = {bswap32(w0), __byte_perm(w1, 0, 0x0144)};
    n[0] = lut3<0>(0, B, lb4); n[1] = lut3<1>(0, B, lb4); n[2] = lut3<2>(0, B, lb4); n[3] = lut3<3>(0, B, lb4);
    n[4] = lut3<4>(0, B, lb4); n[5] = lut3<5>(0, B, lb4); n[6] = lut3<6>(0, B, lb4); n[7] = lut3<7>(0, B, lb4);
  } else {
    const uint32_t w = lds32(addr);
    uint2 r;
    r = lut2<0>(0, w, lb8); n[0] = r.x; n[1] = r.y;
    r = lut2<1>(0, w, lb8); n[2] = r.x; n[3] = r.y;
    r = lut2<2>(0, w, lb8); n[4] = r.x; n[5] = r.y;
    r = lut2<3>(0, w, lb8); n[6] = r.x; n[7] = r.y;
  }
}

// PAR (at most four query heads per KV head): the eight MMA columns of the value products are (query head,
// dim parity) as in tq4_attn_tma_kernel, so the natural-order pair fragments of a token are complete A
// registers (no transposes between tokens) and the accumulators are 16 registers instead of 32.
template <int BITS, bool PAR>
__global__ void __launch_bounds__(256, 1)
tq_attn_streamk4_lowbit_kernel(AttnArgs a) {
  using LB = LowBit<BITS>;
  extern __shared__ __align__(128) unsigned char smem[];
  __shared__ float s_cent[16];
  const uint32_t dyn0 = (uint32_t)__cvta_generic_to_shared(smem);
  int* s_P = reinterpret_cast<int*>(smem + (SK4_PLAN - dyn0));
  int* s_nb = s_P + (SK_MAX_SEQS + 2);
  const int b = blockIdx.x, hg = blockIdx.y;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t = lane & 3;
  const int S = a.num_seqs;
  if (dyn0 > SK4_PLAN) {
    if (tid == 0) g_attn_window_status = 1;
    return;
  }
  for (int i = tid; i < S + 2; i += 256) s_P[i] = a.sk[i];
  for (int i = tid; i < S; i += 256) s_nb[i] = a.sk[3 * S + 2 + i];
  if (tid < 16) s_cent[tid] = tid < (1 << BITS) ? a.centroids[tid] : 0.f;
  __syncthreads();
  const int T = s_P[S], chunk = s_P[S + 1];
  const int u_begin = b * chunk;
  const int u_end = (u_begin + chunk < T) ? u_begin + chunk : T;
  if (u_begin >= u_end) return;            // uniform for the CTA
  const int n_it = u_end - u_begin;

  auto locate = [&](int u, int hint) {
    while (hint < S - 1 && u >= s_P[hint + 1]) ++hint;
    return hint;
  };
  int seq0;
  {
    int lo = 0, hi = S - 1;
    while (lo < hi) {
      const int mid = (lo + hi + 1) >> 1;
      if (s_P[mid] <= u_begin) lo = mid; else hi = mid - 1;
    }
    seq0 = locate(u_begin, lo);
  }

  // ---- producer: 16 x PPT pieces of 16 bytes per block and side, spread over the 256 threads ----
  const int kp_sb = (int)a.kp_sb, vp_sb = (int)a.vp_sb, kn_sb = (int)a.kn_sb, vn_sb = (int)a.vn_sb;
  const bool bt64 = a.bt_dtype == AKV_I64;
  int up = u_begin;
  int p_seq = seq0 - 1, p_base = 0, p_end = u_begin, p_nb = 0;
  const char* bt_row = nullptr;
  int pb[4] = {0, 0, 0, 0};
  int n_has = 0;
  auto load_pb = [&]() {
    if (up >= p_end) {
      p_seq = locate(up, p_seq < 0 ? 0 : p_seq);
      p_base = s_P[p_seq]; p_end = s_P[p_seq + 1]; p_nb = s_nb[p_seq];
      bt_row = reinterpret_cast<const char*>(a.block_tables) + (int64_t)p_seq * a.bt_stride * (bt64 ? 8 : 4);
    }
    const int bi = 4 * (up - p_base);
    n_has = p_nb - bi < 4 ? p_nb - bi : 4;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int bj = bi + (j < n_has ? j : 0);
      pb[j] = bt64 ? (int)reinterpret_cast<const int64_t*>(bt_row)[bj] : reinterpret_cast<const int*>(bt_row)[bj];
    }
  };
  const int nblocks = (int)a.num_blocks;
  constexpr int PIECES = 16 * LB::PPT;      // per block and side
  auto issue = [&](int slot) {
    const uint32_t kb = slot ? SK4_K1 : SK4_K0, vb = slot ? SK4_V1 : SK4_V0, nb_ = slot ? SK4_N1 : SK4_N0;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      pb[j] = min(max(pb[j], 0), nblocks - 1);
      if (j < n_has) {
        for (int e = tid; e < PIECES; e += 256) {
          const int tok = e / LB::PPT, pc = e - tok * LB::PPT;
          const uint32_t d = (uint32_t)(j * LB::BLK + tok * LB::PITCH + pc * 16);
          cp_async16_s(kb + d, a.k_packed + ((int64_t)pb[j] * kp_sb + (int64_t)tok * a.kp_sp + hg * LB::ROW + pc * 16));
          cp_async16_s(vb + d, a.v_packed + ((int64_t)pb[j] * vp_sb + (int64_t)tok * a.vp_sp + hg * LB::ROW + pc * 16));
        }
      }
    }
    {
      const int which = tid >> 5, ch = tid & 31, j = which & 3;
      if (j < n_has) {
        const int tok = ch >> 1, half = ch & 1;
        const int pbj = j == 0 ? pb[0] : j == 1 ? pb[1] : j == 2 ? pb[2] : pb[3];
        const float* src = (which < 4)
            ? a.k_norms + ((int64_t)pbj * kn_sb + (int64_t)tok * a.kn_sp + hg * 8 + half * 4)
            : a.v_norms + ((int64_t)pbj * vn_sb + (int64_t)tok * a.vn_sp + hg * 8 + half * 4);
        cp_async16_s(nb_ + which * 512 + ch * 16, src);
      }
    }
    asm volatile("cp.async.commit_group;\n" ::);
    ++up;
    if (up < u_end) load_pb();
  };
  load_pb();
  issue(0);
  if constexpr (BITS == 3) {          // 6 bits -> half2(c[hi 3 bits], c[lo 3 bits])
    for (int i = tid; i < 64 * 32; i += 256) {
      const int e = i >> 5, l = i & 31;
      const uint32_t v = pack_half2(s_cent[e >> 3], s_cent[e & 7]);
      asm volatile("st.shared.u32 [%0], %1;\n" :: "r"(SK_LUT + e * LUT3_STRIDE + l * 4), "r"(v));
    }
  } else {                            // byte -> four halves
    for (int i = tid; i < 256 * 32; i += 256) {
      const int e = i >> 5, l = i & 31;
      const uint32_t v0 = pack_half2(s_cent[e >> 6], s_cent[(e >> 4) & 3]);
      const uint32_t v1 = pack_half2(s_cent[(e >> 2) & 3], s_cent[e & 3]);
      asm volatile("st.shared.v2.u32 [%0], {%1,%2};\n" :: "r"(SK_LUT + e * LUT_STRIDE + l * 8), "r"(v0), "r"(v1));
    }
  }

  // ---- consumer: warp = KV head ----
  const int hl = warp;
  const int h = hg * 8 + hl;
  const int G = a.num_q_heads / a.num_kv_heads;
  const uint32_t lb4 = SK_LUT | (lane * 4), lb8 = SK_LUT | (lane * 8);
  const uint32_t kA_off = (uint32_t)(g * LB::PITCH + hl * LB::PD + 4 * BITS * t);
  uint32_t v_off[4];
  const uint32_t v_byte = (uint32_t)(hl * LB::PD + 2 * BITS * g);
  const uint32_t v_sh = BITS == 3 ? 8u * (v_byte & 3u) : 0u;
  {
    const int toks[4] = {2 * t, 2 * t + 1, 2 * t + 8, 2 * t + 9};
#pragma unroll
    for (int i = 0; i < 4; ++i) v_off[i] = (uint32_t)(toks[i] * LB::PITCH) + (BITS == 3 ? (v_byte & ~3u) : v_byte);
  }
  const int n_off = (g * 8 + hl) * 4;

  constexpr int NO = PAR ? 4 : 8;
  const uint32_t selA = (g >> 2) ? 0x1044u : 0x4410u, selB = (g >> 2) ? 0x3244u : 0x4432u;   // PAR: P with a zero parity
  uint32_t bq[8][2];
  float o[NO][4];
  SoftmaxState st{-CUDART_INF_F, -CUDART_INF_F, 0.f, 0.f};
  int seq_c = -1, c_base = 0, c_end = 0, ctx_c = 0;
  auto begin_seq = [&](int seq) {
    seq_c = seq;
    c_base = s_P[seq]; c_end = s_P[seq + 1];
    ctx_c = (int)load_ctx(a.context_lens, a.cl_dtype, seq, (int64_t)a.max_blocks_per_seq * a.block_size);
    const int qg = PAR ? (g & 3) : g;        // PAR: columns 4..7 repeat the query heads 0..3
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
    for (int j = 0; j < NO; ++j) { o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f; }
    st = SoftmaxState{-CUDART_INF_F, -CUDART_INF_F, 0.f, 0.f};
  };
  auto end_seq = [&]() {
    float l0 = st.l0, l1 = st.l1;
#pragma unroll
    for (int offs = 4; offs < 32; offs <<= 1) {
      l0 += __shfl_xor_sync(0xffffffffu, l0, offs);
      l1 += __shfl_xor_sync(0xffffffffu, l1, offs);
    }
    const int part = b - a.sk[S + 2 + seq_c];
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      const int n = 2 * t + e, qg = PAR ? (n & 3) : n, ep = PAR ? (n >> 2) : 0;      // column -> (query head, dim parity)
      if (qg >= G) continue;
      const int64_t row = (int64_t)seq_c * a.num_q_heads + h * G + qg;
      float* pa = a.part_acc + (row * a.num_parts + part) * 128;
      if constexpr (PAR) {
#pragma unroll
        for (int mt = 0; mt < 4; ++mt) {                     // rows g, g + 8 of tile mt: pair slots 2mt, 2mt + 1 of dims 16g..
          pa[16 * g + 4 * mt + ep] = o[mt][e];
          pa[16 * g + 4 * mt + 2 + ep] = o[mt][2 + e];
        }
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j)
          *reinterpret_cast<float2*>(pa + 16 * g + 2 * j) = make_float2(o[j][e], o[j][2 + e]);
      }
      if (g == 0 && ep == 0) {
        a.part_ml[(row * a.num_parts + part) * 2] = e ? st.m1 : st.m0;
        a.part_ml[(row * a.num_parts + part) * 2 + 1] = e ? l1 : l0;
      }
    }
  };
  // outer loop: the sequences of this CTA's range; inner loop: their stages
  int it = 0;
  int seq_next = seq0;
  while (it < n_it) {
  begin_seq(seq_next);
  const int it_end = (c_end - u_begin < n_it) ? c_end - u_begin : n_it;
  for (; it < it_end; ++it) {
    asm volatile("cp.async.wait_group 0;\n" ::: "memory");
    __syncthreads();
    if (it + 1 < n_it) issue((it + 1) & 1);
    const int u = u_begin + it;
    const int slot = it & 1;
    const uint32_t kb = slot ? SK4_K1 : SK4_K0, vb = slot ? SK4_V1 : SK4_V0, nb_ = (slot ? SK4_N1 : SK4_N0) + n_off;
    const int rem = ctx_c - 64 * (u - c_base);

    // ---- scores of the four tiles ----
    float s[4][4];
    float nv[4][2];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      uint32_t na[16], nb2[16];
      lowbit_k_fragments<BITS>(kb + j * LB::BLK + kA_off, lb4, lb8, na);
      lowbit_k_fragments<BITS>(kb + j * LB::BLK + kA_off + 8 * LB::PITCH, lb4, lb8, nb2);
      float sa[4] = {0.f, 0.f, 0.f, 0.f}, sb[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int kk = 0; kk < 8; kk += 2) {
        mma16816(sa, na[2 * kk], nb2[2 * kk], na[2 * kk + 1], nb2[2 * kk + 1], bq[kk][0], bq[kk][1]);
        mma16816(sb, na[2 * kk + 2], nb2[2 * kk + 2], na[2 * kk + 3], nb2[2 * kk + 3], bq[kk + 1][0], bq[kk + 1][1]);
      }
      const float nkA = __uint_as_float(lds32(nb_ + j * 512)), nkB = __uint_as_float(lds32(nb_ + j * 512 + 256));
      nv[j][0] = __uint_as_float(lds32(nb_ + 2048 + j * 512));
      nv[j][1] = __uint_as_float(lds32(nb_ + 2048 + j * 512 + 256));
      s[j][0] = (sa[0] + sb[0]) * nkA; s[j][1] = (sa[1] + sb[1]) * nkA;
      s[j][2] = (sa[2] + sb[2]) * nkB; s[j][3] = (sa[3] + sb[3]) * nkB;
    }
    if (rem < 64) {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int nvld = rem - 16 * j;
        if (g >= nvld) { s[j][0] = -CUDART_INF_F; s[j][1] = -CUDART_INF_F; nv[j][0] = 0.f; }
        if (g + 8 >= nvld) { s[j][2] = -CUDART_INF_F; s[j][3] = -CUDART_INF_F; nv[j][1] = 0.f; }
      }
    }
    // ---- one softmax update for the 64 tokens ----
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
      for (int j = 0; j < NO; ++j) { o[j][0] *= al0; o[j][1] *= al1; o[j][2] *= al0; o[j][3] *= al1; }
      st.m0 = mn0; st.m1 = mn1;
    }
    uint32_t pq[4][2];
    float ls0 = 0.f, ls1 = 0.f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float p0 = ex2_approx(s[j][0] - mn0), p1 = ex2_approx(s[j][1] - mn1);
      const float p2 = ex2_approx(s[j][2] - mn0), p3 = ex2_approx(s[j][3] - mn1);
      ls0 += p0 + p2;
      ls1 += p1 + p3;
      pq[j][0] = movmatrix_trans(pack_half2(p0 * nv[j][0], p1 * nv[j][0]));
      pq[j][1] = movmatrix_trans(pack_half2(p2 * nv[j][1], p3 * nv[j][1]));
    }
    st.l0 += ls0;
    st.l1 += ls1;
    // ---- values ----
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      uint32_t n0[8], n1[8], n2[8], n3[8];
      lowbit_v_fragments<BITS>(vb + j * LB::BLK + v_off[0], v_sh, lb4, lb8, n0);
      lowbit_v_fragments<BITS>(vb + j * LB::BLK + v_off[1], v_sh, lb4, lb8, n1);
      lowbit_v_fragments<BITS>(vb + j * LB::BLK + v_off[2], v_sh, lb4, lb8, n2);
      lowbit_v_fragments<BITS>(vb + j * LB::BLK + v_off[3], v_sh, lb4, lb8, n3);
      if constexpr (PAR) {
        const uint32_t b00 = __byte_perm(pq[j][0], 0u, selA), b01 = __byte_perm(pq[j][0], 0u, selB);   // tokens 2t, 2t+1
        const uint32_t b10 = __byte_perm(pq[j][1], 0u, selA), b11 = __byte_perm(pq[j][1], 0u, selB);   // tokens 2t+8, 2t+9
#pragma unroll
        for (int mt = 0; mt < 4; ++mt) {
          mma16816(o[mt], n0[2 * mt], n0[2 * mt + 1], n1[2 * mt], n1[2 * mt + 1], b00, b01);
          mma16816(o[mt], n2[2 * mt], n2[2 * mt + 1], n3[2 * mt], n3[2 * mt + 1], b10, b11);
        }
      } else {
#pragma unroll
        for (int m = 0; m < 8; ++m)
          mma16816(o[m], __byte_perm(n0[m], n1[m], 0x5410), __byte_perm(n0[m], n1[m], 0x7632),
                   __byte_perm(n2[m], n3[m], 0x5410), __byte_perm(n2[m], n3[m], 0x7632), pq[j][0], pq[j][1]);
      }
    }
  }
  end_seq();
  if (it < n_it) seq_next = locate(u_begin + it, seq_c);
  }
}

}  // namespace akv
#include "tq_attention_tma.cuh"
#include "tq_prefill.cuh"
namespace akv {

int attn_window_status(int* host_out, int reset) {
  cudaError_t e = cudaMemcpyFromSymbol(host_out, g_attn_window_status, sizeof(int));
  if (e == cudaSuccess && reset) { const int z = 0; e = cudaMemcpyToSymbol(g_attn_window_status, &z, sizeof(int)); }
  return e == cudaSuccess ? AKV_OK : fail((int)e, "attention status: %s", cudaGetErrorString(e));
}

static inline size_t align256(size_t v) { return (v + 255) & ~(size_t)255; }

struct Plan {
  bool mma;
  bool persist_shape;     // shapes allow the persistent stream-K kernel (strides are checked at run time)
  int sk_grid;            // persistent CTAs per head group
  int blocks_per_split, num_splits, warps_per_head, num_parts;
  size_t parts_alloc;     // partial slots per (sequence, q head) the buffers are sized for
  size_t off_qrot, off_acc, off_ml, off_sk, total;
};

static bool persist_enabled() {
  static const bool on = getenv("AKV_NO_PERSIST") == nullptr;
  return on;
}

static Plan make_plan(int num_seqs, int num_q_heads, int num_kv_heads, int head_dim, int bits,
                      int block_size, int max_blocks_per_seq, int blocks_per_split, bool persist_ok = true) {
  Plan p;
  const int G = num_q_heads / num_kv_heads;
  p.mma = (head_dim == 128 && G >= 1 && G <= 8 && block_size % 16 == 0);
  if (blocks_per_split <= 0) blocks_per_split = (64 * 16 + block_size - 1) / block_size;  // ~1024 tokens
  if (blocks_per_split > max_blocks_per_seq) blocks_per_split = max_blocks_per_seq > 0 ? max_blocks_per_seq : 1;
  p.blocks_per_split = blocks_per_split;
  p.num_splits = max_blocks_per_seq > 0 ? (max_blocks_per_seq + blocks_per_split - 1) / blocks_per_split : 1;
  if (p.mma) {
    int nh = num_kv_heads < 8 ? num_kv_heads : 8;
    p.warps_per_head = 8 / nh;
  } else {
    p.warps_per_head = GEN_WARPS;
  }
  p.num_parts = p.num_splits * p.warps_per_head;
  const int head_groups = (num_kv_heads + 7) / 8;
  p.sk_grid = sm_count() / head_groups > 0 ? sm_count() / head_groups : 1;
  p.persist_shape = persist_ok && persist_enabled() && p.mma && block_size == 16 &&
                    num_kv_heads % 8 == 0 && num_seqs <= SK_MAX_SEQS && max_blocks_per_seq > 0;
  p.parts_alloc = (size_t)p.num_parts;
  if (p.persist_shape && (size_t)2 * p.sk_grid > p.parts_alloc) p.parts_alloc = (size_t)2 * p.sk_grid;
  size_t rows = (size_t)num_seqs * num_q_heads;
  p.off_qrot = 0;
  p.off_acc = align256(rows * head_dim * sizeof(float));
  p.off_ml = p.off_acc + align256(rows * p.parts_alloc * head_dim * sizeof(float));
  p.off_sk = p.off_ml + align256(rows * p.parts_alloc * 2 * sizeof(float));
  p.total = p.off_sk + align256(((size_t)4 * num_seqs + 4) * sizeof(int));
  return p;
}

}  // namespace akv

using namespace akv;

// Field-for-field mirror of akv_tq_attn_params in include/akv_b200.h.
struct akv_tq_attn_params {
  const void* query; int q_dtype; int64_t q_stride_seq, q_stride_head;
  const uint8_t* k_packed; int64_t kp_stride_blk, kp_stride_pos, kp_stride_head;
  const float* k_norms; int64_t kn_stride_blk, kn_stride_pos, kn_stride_head;
  const uint8_t* v_packed; int64_t vp_stride_blk, vp_stride_pos, vp_stride_head;
  const float* v_norms; int64_t vn_stride_blk, vn_stride_pos, vn_stride_head;
  const void* block_tables; int bt_dtype; int64_t bt_stride_seq;
  const void* context_lens; int cl_dtype;
  int num_seqs, num_q_heads, num_kv_heads, head_dim, block_size, max_blocks_per_seq;
  int64_t num_blocks;
  int bits;
  const float* rotation; const float* rotation_t; const float* centroids;
  float scale;
  void* out; int out_dtype; int64_t out_stride_seq, out_stride_head;
  float* raw_out;            // if non-null: write merged (m, l, acc) instead of `out`
  void* workspace; size_t workspace_bytes;
  int blocks_per_split;      // 0 = default
  void* stream;
  void* ev_kernel_start;     // optional cudaEvent_t recorded right before / after the
  void* ev_kernel_stop;      // split-K kernel (for per-kernel timing); may be null
  void* out_copy;            // optional dense [num_seqs][num_q_heads][head_dim] second copy of `out`
};

AKV_EXPORT size_t akv_tq_paged_attn_workspace_bytes(int num_seqs, int num_q_heads, int num_kv_heads,
                                                    int head_dim, int bits, int block_size,
                                                    int max_blocks_per_seq, int blocks_per_split) {
  if (num_seqs <= 0 || num_q_heads <= 0 || num_kv_heads <= 0) return 0;
  return make_plan(num_seqs, num_q_heads, num_kv_heads, head_dim, bits, block_size,
                   max_blocks_per_seq, blocks_per_split).total;
}

namespace akv {
// new_token (optional): K and V vectors to write into the cache by the first launch; once the arguments
// have passed validation that launch always happens.
int run_tq_attn(const akv_tq_attn_params* p, void* workspace, size_t workspace_bytes, bool allow_persist = true,
                const NewTokenWrite* new_token = nullptr);
}

int akv::run_tq_attn(const akv_tq_attn_params* p, void* workspace, size_t workspace_bytes, bool allow_persist,
                     const NewTokenWrite* new_token) {
  if (!p) return fail(AKV_ERR_ARG, "null params");
  if (p->bits != 2 && p->bits != 3 && p->bits != 4)
    return fail(AKV_ERR_ARG, "Supported bit-widths: 2, 3, 4. Got %d", p->bits);
  const int D = p->head_dim;
  if (!is_pow2(D) || D < 32 || D > 256)
    return fail(AKV_ERR_ARG, "paged attention needs a power-of-two head_dim in [32, 256], got %d", D);
  if (p->num_seqs < 0 || p->num_q_heads <= 0 || p->num_kv_heads <= 0 ||
      p->num_q_heads % p->num_kv_heads != 0 || p->block_size <= 0 || p->max_blocks_per_seq < 0)
    return fail(AKV_ERR_ARG, "paged attention: bad sizes");
  if (p->num_seqs == 0) return AKV_OK;
  if (!p->query || !p->k_packed || !p->v_packed || !p->k_norms || !p->v_norms || !p->block_tables ||
      !p->context_lens || !p->rotation_t || !p->centroids || (!p->raw_out && (!p->out || !p->rotation)))
    return fail(AKV_ERR_ARG, "paged attention: null pointer");
  if (p->num_blocks <= 0) return fail(AKV_ERR_ARG, "paged attention: num_blocks must be > 0");
  cudaStream_t st = (cudaStream_t)p->stream;
  Plan plan = make_plan(p->num_seqs, p->num_q_heads, p->num_kv_heads, D, p->bits, p->block_size,
                        p->max_blocks_per_seq, p->blocks_per_split, allow_persist);
  if (workspace == nullptr || workspace_bytes < plan.total)
    return fail(AKV_ERR_WORKSPACE, "workspace too small: need %zu bytes, got %zu", plan.total, workspace_bytes);
  char* ws = reinterpret_cast<char*>(workspace);
  float* qrot = reinterpret_cast<float*>(ws + plan.off_qrot);
  float* part_acc = reinterpret_cast<float*>(ws + plan.off_acc);
  float* part_ml = reinterpret_cast<float*>(ws + plan.off_ml);
  const int rows = p->num_seqs * p->num_q_heads;

  // which split-K kernel serves this call
  const bool aligned4 = (p->kp_stride_blk % 4 == 0) && (p->kp_stride_pos % 4 == 0) && (p->kp_stride_head % 4 == 0) &&
                        (p->vp_stride_blk % 4 == 0) && (p->vp_stride_pos % 4 == 0) && (p->vp_stride_head % 4 == 0) &&
                        (reinterpret_cast<uintptr_t>(p->k_packed) % 4 == 0) &&
                        (reinterpret_cast<uintptr_t>(p->v_packed) % 4 == 0);
  if (plan.mma && !aligned4) return fail(AKV_ERR_UNSUPPORTED, "packed cache rows must be 4-byte aligned");
  const bool vec16 = (p->kp_stride_blk % 16 == 0) && (p->kp_stride_pos % 16 == 0) && (p->kp_stride_head % 16 == 0) &&
                     (p->vp_stride_blk % 16 == 0) && (p->vp_stride_pos % 16 == 0) && (p->vp_stride_head % 16 == 0) &&
                     (reinterpret_cast<uintptr_t>(p->k_packed) % 16 == 0) &&
                     (reinterpret_cast<uintptr_t>(p->v_packed) % 16 == 0);
  static const bool no_pipe = getenv("AKV_NO_PIPE") != nullptr;
  const bool pipe = plan.mma && !no_pipe && vec16 && p->bits == 4 && p->block_size == 16 && p->num_kv_heads % 8 == 0 &&
                    p->kp_stride_head == 64 && p->vp_stride_head == 64 && p->kn_stride_head == 1 &&
                    p->vn_stride_head == 1 && p->kn_stride_pos % 4 == 0 && p->vn_stride_pos % 4 == 0 &&
                    p->kn_stride_blk % 4 == 0 && p->vn_stride_blk % 4 == 0 &&
                    reinterpret_cast<uintptr_t>(p->k_norms) % 16 == 0 &&
                    reinterpret_cast<uintptr_t>(p->v_norms) % 16 == 0 && p->max_blocks_per_seq > 0;
  const int64_t lim = (int64_t)1 << 31;
  // the same layout test for any bit width: heads contiguous in a token row, rows readable in 16-byte pieces
  const int pd_bytes = 16 * p->bits;
  const bool ring_layout = plan.mma && vec16 && p->block_size == 16 && p->num_kv_heads % 8 == 0 &&
                           p->kp_stride_head == pd_bytes && p->vp_stride_head == pd_bytes && p->kn_stride_head == 1 &&
                           p->vn_stride_head == 1 && p->kn_stride_pos % 4 == 0 && p->vn_stride_pos % 4 == 0 &&
                           p->kn_stride_blk % 4 == 0 && p->vn_stride_blk % 4 == 0 &&
                           reinterpret_cast<uintptr_t>(p->k_norms) % 16 == 0 &&
                           reinterpret_cast<uintptr_t>(p->v_norms) % 16 == 0 && p->max_blocks_per_seq > 0;
  static const bool sk4 = getenv("AKV_NO_SK4") == nullptr;    // 4-block stages, four tiles per warp at once
  static const bool no_lowbit_ring = getenv("AKV_NO_LOWBIT_RING") != nullptr;
  const bool ring = p->bits == 4 ? pipe : (ring_layout && sk4 && !no_pipe && !no_lowbit_ring);
  // the 4-block-stage kernels address their plan arrays and tables at fixed shared addresses; they are
  // used only where the dynamic window starts at or below the first of them (else: the per-split kernels)
  static const bool sk4_window_ok =
      dyn_smem_window_start(reinterpret_cast<const void*>(tq4_attn_streamk4_kernel)) <= SK4_PLAN &&
      dyn_smem_window_start(reinterpret_cast<const void*>(tq_attn_streamk4_lowbit_kernel<3, true>)) <= SK4_PLAN &&
      dyn_smem_window_start(reinterpret_cast<const void*>(tq_attn_streamk4_lowbit_kernel<2, true>)) <= SK4_PLAN &&
      dyn_smem_window_start(reinterpret_cast<const void*>(tq_attn_streamk4_lowbit_kernel<3, false>)) <= SK4_PLAN &&
      dyn_smem_window_start(reinterpret_cast<const void*>(tq_attn_streamk4_lowbit_kernel<2, false>)) <= SK4_PLAN;
  const bool persist = ring && (!sk4 || sk4_window_ok) && plan.persist_shape && p->kp_stride_blk < lim && p->vp_stride_blk < lim &&
                       p->kn_stride_blk < lim && p->vn_stride_blk < lim && p->num_blocks < lim;
  int* sk = reinterpret_cast<int*>(ws + plan.off_sk);

  StreamKPlanArgs pl{};
  pl.context_lens = p->context_lens; pl.cl_dtype = p->cl_dtype; pl.num_seqs = p->num_seqs;
  pl.block_size = p->block_size; pl.grid = plan.sk_grid; pl.sk = persist ? sk : nullptr;
  pl.max_ctx = (int64_t)p->max_blocks_per_seq * p->block_size;
  static const int sk_wph = (getenv("AKV_SK_WPH") && atoi(getenv("AKV_SK_WPH")) == 2) ? 2 : 1;
  pl.parts_per_cta = sk4 ? 1 : sk_wph;
  pl.blocks_per_stage = sk4 ? 4 : 2;
  NewTokenWrite nt{};
  size_t qrot_smem = D * sizeof(float);
  if (new_token != nullptr && new_token->n_rows > 0) {       // D >= 128 here (the caller checked): 128-thread blocks
    nt = *new_token;
    qrot_smem = (size_t)(D + D / 4 + 16) * sizeof(float);
  }
  const int plan_blocks = persist ? 1 : 0;
  static const bool no_rot128 = getenv("AKV_NO_ROT128") != nullptr;
  // Large batches (2048+ rows; below that the per-row kernels are as fast): the query rotation is one tensor-core product over all rows (rot_rows.cu); the
  // plan block and the new token's vectors keep their launch
  static const bool no_rot_gemm = getenv("AKV_NO_ROT_GEMM") != nullptr;
  const bool gemm_q = D == 128 && rows >= 2048 && !no_rot_gemm && !no_rot128 &&
                      rot_rows_ok(p->query, p->q_dtype, p->q_stride_seq, p->q_stride_head, qrot, AKV_F32,
                                  (int64_t)p->num_q_heads * 128, 128);
  if (gemm_q) {
    if (int rc = launch_rot_rows(p->query, p->q_dtype, p->q_stride_seq, p->q_stride_head, p->num_q_heads, nullptr, 0,
                                 p->rotation_t, p->scale * 1.4426950408889634f, qrot, AKV_F32,
                                 (int64_t)p->num_q_heads * 128, 128, rows, st))
      return rc;
  }
  if (D == 128 && !no_rot128) {            // rotation matrix staged in shared memory, four rows per CTA pass
    const size_t smem128 = (size_t)ROT128_MAT_BYTES + 4 * 128 * sizeof(float);
    cudaError_t e = cudaFuncSetAttribute(akv_qrot128_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem128);
    if (e != cudaSuccess) return fail((int)e, "attention: smem attribute: %s", cudaGetErrorString(e));
    const int quads = gemm_q ? 0 : (rows + 3) / 4;
    const int rot_blocks = quads < 2 * sm_count() ? quads : 2 * sm_count();
    const unsigned enc_blocks = (unsigned)((2 * nt.n_rows + 3) / 4);      // four vectors of the new token per block
    if (rot_blocks + plan_blocks + enc_blocks > 0) {
      akv_qrot128_kernel<<<rot_blocks + plan_blocks + enc_blocks, ROT128_THREADS, smem128, st>>>(
          p->query, p->q_dtype, p->q_stride_seq, p->q_stride_head, p->num_q_heads, p->rotation_t,
          p->scale * 1.4426950408889634f, qrot, rows, rot_blocks, plan_blocks, pl, nt);
      if (int rc = check_launch("akv_qrot128_kernel")) return rc;
    }
  } else {
    const int qrot_threads = D < 128 ? D : 128;
    akv_qrot_kernel<<<rows + plan_blocks + (unsigned)(2 * nt.n_rows), qrot_threads, qrot_smem, st>>>(
        p->query, p->q_dtype, p->q_stride_seq, p->q_stride_head, p->num_q_heads, D, p->rotation_t,
        p->scale * 1.4426950408889634f, qrot, rows, plan_blocks, pl, nt);
    if (int rc = check_launch("akv_qrot_kernel")) return rc;
  }

  AttnArgs a{};
  a.k_packed = p->k_packed; a.v_packed = p->v_packed;
  a.kp_sb = p->kp_stride_blk; a.kp_sp = p->kp_stride_pos; a.kp_sh = p->kp_stride_head;
  a.vp_sb = p->vp_stride_blk; a.vp_sp = p->vp_stride_pos; a.vp_sh = p->vp_stride_head;
  a.k_norms = p->k_norms; a.v_norms = p->v_norms;
  a.kn_sb = p->kn_stride_blk; a.kn_sp = p->kn_stride_pos; a.kn_sh = p->kn_stride_head;
  a.vn_sb = p->vn_stride_blk; a.vn_sp = p->vn_stride_pos; a.vn_sh = p->vn_stride_head;
  a.block_tables = p->block_tables; a.bt_dtype = p->bt_dtype; a.bt_stride = p->bt_stride_seq;
  a.context_lens = p->context_lens; a.cl_dtype = p->cl_dtype;
  a.num_seqs = p->num_seqs; a.num_q_heads = p->num_q_heads; a.num_kv_heads = p->num_kv_heads;
  a.head_dim = D; a.block_size = p->block_size; a.max_blocks_per_seq = p->max_blocks_per_seq;
  a.num_blocks = p->num_blocks; a.bits = p->bits;
  a.blocks_per_split = plan.blocks_per_split; a.num_splits = plan.num_splits;
  a.warps_per_head = plan.warps_per_head; a.num_parts = plan.num_parts;
  a.qrot = qrot; a.centroids = p->centroids; a.part_acc = part_acc; a.part_ml = part_ml;
  a.sk = sk;
  int merge_parts = plan.num_parts;          // stride (and upper bound) of the partial slots the merge reads

  // 4-bit codes, at most four query heads per KV head, cache strides a tensor map can describe: the kernel
  // with the TMA-fed ring (tensor maps cover the caller's cache on this GPU only)
  static const bool no_tma = getenv("AKV_NO_TMA") != nullptr;
  static const bool tma_window_ok =
      dyn_smem_window_start(reinterpret_cast<const void*>(tq_attn_tma_kernel<4>)) <= T4_BAR &&
      dyn_smem_window_start(reinterpret_cast<const void*>(tq_attn_tma_kernel<3>)) <= T4_BAR &&
      dyn_smem_window_start(reinterpret_cast<const void*>(tq_attn_tma_kernel<2>)) <= T4_BAR;
  static const bool no_tma_lowbit = getenv("AKV_NO_TMA_LOWBIT") != nullptr;
  T4Maps maps;
  const bool tma = persist && sk4 && !no_tma && tma_window_ok && (p->bits == 4 || !no_tma_lowbit) && p->max_blocks_per_seq > 0 &&
                   p->num_q_heads / p->num_kv_heads <= 4 && p->kp_stride_pos % 16 == 0 && p->vp_stride_pos % 16 == 0 &&
                   p->kp_stride_blk % 16 == 0 && p->vp_stride_blk % 16 == 0 && t4_make_maps(a, &maps);

  // The three launches of a step overlap their ends and beginnings (programmatic dependent launch) unless the
  // caller brackets the attention kernel with events, which have to sit between whole launches.
  static const bool no_pdl = getenv("AKV_NO_PDL") != nullptr;
  const bool pdl = tma && !no_pdl && D == 128 && !no_rot128 && !p->ev_kernel_start && !p->ev_kernel_stop;
  if (p->ev_kernel_start) cudaEventRecord((cudaEvent_t)p->ev_kernel_start, st);
  if (p->max_blocks_per_seq > 0) {
    if (tma) {
      a.num_parts = plan.sk_grid;
      merge_parts = a.num_parts;
      auto kern = p->bits == 4 ? tq_attn_tma_kernel<4> : (p->bits == 3 ? tq_attn_tma_kernel<3> : tq_attn_tma_kernel<2>);
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, T4_DYN_SMEM);
      if (e != cudaSuccess) return fail((int)e, "attention: smem attribute: %s", cudaGetErrorString(e));
      dim3 grid(plan.sk_grid, p->num_kv_heads / 8);
      if (pdl) {
        // programmatic dependent launch: the grid may be scheduled while the query-rotation launch drains; the
        // kernel fills its lookup table and then waits for that launch before reading anything it produced
        a.pdl = 1;
        cudaLaunchConfig_t cfg{};
        cfg.gridDim = grid; cfg.blockDim = dim3(T4_THREADS); cfg.dynamicSmemBytes = T4_DYN_SMEM; cfg.stream = st;
        cudaLaunchAttribute at[1];
        at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        at[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = at; cfg.numAttrs = 1;
        cudaLaunchKernelEx(&cfg, kern, a, maps);
      } else {
        kern<<<grid, T4_THREADS, T4_DYN_SMEM, st>>>(a, maps);
      }
      if (int rc = check_launch(p->bits == 4 ? "tq4_attn_tma_kernel" : "tq_lowbit_attn_tma_kernel")) return rc;
    } else if (persist && sk4) {
      a.num_parts = plan.sk_grid;
      merge_parts = a.num_parts;
      const bool par = p->num_q_heads / p->num_kv_heads <= 4;
      auto kern = p->bits == 4 ? tq4_attn_streamk4_kernel
                  : p->bits == 3 ? (par ? tq_attn_streamk4_lowbit_kernel<3, true> : tq_attn_streamk4_lowbit_kernel<3, false>)
                                 : (par ? tq_attn_streamk4_lowbit_kernel<2, true> : tq_attn_streamk4_lowbit_kernel<2, false>);
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SK4_DYN_SMEM);
      if (e != cudaSuccess) return fail((int)e, "attention: smem attribute: %s", cudaGetErrorString(e));
      dim3 grid(plan.sk_grid, p->num_kv_heads / 8);
      kern<<<grid, 256, SK4_DYN_SMEM, st>>>(a);
      if (int rc = check_launch(p->bits == 4 ? "tq4_attn_streamk4_kernel" : "tq_attn_streamk4_lowbit_kernel")) return rc;
    } else if (persist) {
      a.num_parts = sk_wph * plan.sk_grid;
      merge_parts = a.num_parts;
      static const bool sk_pair = getenv("AKV_SK_NO_PAIR") == nullptr;   // two tiles per warp at once
      auto kern = sk_wph == 2 ? tq4_attn_streamk_kernel<2, false>
                              : (sk_pair ? tq4_attn_streamk_kernel<1, true> : tq4_attn_streamk_kernel<1, false>);
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SK_DYN_SMEM);
      if (e != cudaSuccess) return fail((int)e, "attention: smem attribute: %s", cudaGetErrorString(e));
      dim3 grid(plan.sk_grid, p->num_kv_heads / 8);
      kern<<<grid, 256 * sk_wph, SK_DYN_SMEM, st>>>(a);
      if (int rc = check_launch("tq4_attn_streamk_kernel")) return rc;
    } else if (pipe && plan.blocks_per_split <= PIPE_MAX_BLOCKS) {
      cudaError_t e = cudaFuncSetAttribute(tq4_attn_pipe_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, PIPE_SMEM);
      if (e != cudaSuccess) return fail((int)e, "attention: smem attribute: %s", cudaGetErrorString(e));
      dim3 grid(plan.num_splits, p->num_kv_heads / 8, p->num_seqs);
      tq4_attn_pipe_kernel<<<grid, 512, PIPE_SMEM, st>>>(a);
      if (int rc = check_launch("tq4_attn_pipe_kernel")) return rc;
    } else if (plan.mma) {
      int nh = p->num_kv_heads < 8 ? p->num_kv_heads : 8;
      dim3 grid(plan.num_splits, (p->num_kv_heads + 7) / 8, p->num_seqs);
      dim3 block(32 * nh * plan.warps_per_head);
      void (*kern)(AttnArgs) = nullptr;
      int lut_bytes = LUT_BYTES;
      if (p->bits == 4) kern = vec16 ? tq_attn_mma_kernel<4, true> : tq_attn_mma_kernel<4, false>;
      else if (p->bits == 3) { kern = tq_attn_mma_kernel<3, false>; lut_bytes = 64 * LUT3_STRIDE; }
      else kern = tq_attn_mma_kernel<2, false>;
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, lut_bytes);
      if (e != cudaSuccess) return fail((int)e, "attention: smem attribute: %s", cudaGetErrorString(e));
      kern<<<grid, block, lut_bytes, st>>>(a);
      if (int rc = check_launch("tq_attn_mma_kernel")) return rc;
    } else {
      dim3 grid(plan.num_splits, p->num_kv_heads, p->num_seqs);
      tq_attn_generic_kernel<<<grid, GEN_WARPS * 32, 0, st>>>(a);
      if (int rc = check_launch("tq_attn_generic_kernel")) return rc;
    }
  }
  if (p->ev_kernel_stop) cudaEventRecord((cudaEvent_t)p->ev_kernel_stop, st);

  MergeArgs mg{};
  mg.acc = part_acc; mg.acc_row = (int64_t)merge_parts * D; mg.acc_part = D;
  mg.ml = part_ml; mg.ml_row = (int64_t)merge_parts * 2; mg.ml_part = 2;
  mg.np = p->max_blocks_per_seq > 0 ? merge_parts : 0;
  mg.part_counts = (persist && p->max_blocks_per_seq > 0) ? sk + 2 * p->num_seqs + 2 : nullptr;
  mg.context_lens = p->context_lens; mg.cl_dtype = p->cl_dtype; mg.num_q_heads = p->num_q_heads;
  mg.tokens_per_split = plan.blocks_per_split * p->block_size; mg.warps_per_head = plan.warps_per_head;
  mg.D = D;
  mg.mode = p->raw_out ? MERGE_RAW : MERGE_ROTATE;
  mg.rot = p->rotation;
  mg.out = p->out; mg.out_dtype = p->out_dtype; mg.out_ss = p->out_stride_seq; mg.out_sh = p->out_stride_head;
  mg.out2 = p->raw_out ? nullptr : p->out_copy;
  mg.raw_out = p->raw_out;
  mg.gemm_scratch = qrot;        // the rotated queries are dead once the attention kernel has run
  return launch_merge(mg, rows, st, pdl && p->max_blocks_per_seq > 0);
}

AKV_EXPORT int akv_tq_paged_attn(const akv_tq_attn_params* p) {
  if (!p) return fail(AKV_ERR_ARG, "null params");
  return run_tq_attn(p, p->workspace, p->workspace_bytes);
}

// Mirror of akv_tq_decode_step_params in include/akv_b200.h.
struct akv_tq_decode_step_params {
  const void* key; const void* value; int kv_dtype;
  int64_t num_tokens;
  int64_t k_stride_tok, k_stride_head, v_stride_tok, v_stride_head;
  const int64_t* slot_mapping;
  const float* boundaries;
  int64_t max_blocks;
  akv_tq_attn_params attn;
};

extern "C" int akv_tq_kv_update(const void* x, int x_dtype, int64_t num_tokens, int num_kv_heads, int head_dim,
                                int64_t x_stride_tok, int64_t x_stride_head, const int64_t* slot_mapping,
                                uint8_t* out_packed, int64_t p_stride_blk, int64_t p_stride_pos,
                                int64_t p_stride_head, float* out_norms, int64_t n_stride_blk,
                                int64_t n_stride_pos, int64_t n_stride_head, int bits, const float* rotation_t,
                                const float* boundaries, int block_size, int64_t max_blocks, void* stream);

// One serving step in one call: write the new tokens' K and V into the packed cache, then attend.
AKV_EXPORT int akv_tq_decode_step(const akv_tq_decode_step_params* p) {
  if (!p) return fail(AKV_ERR_ARG, "null params");
  const akv_tq_attn_params& a = p->attn;
  if (p->num_tokens > 0) {
    if (!p->key || !p->value || !p->slot_mapping || !p->boundaries)
      return fail(AKV_ERR_ARG, "akv_tq_decode_step: null pointer");
    // a decode step writes few vectors: K and V go out as one launch when the arguments are plainly valid
    // (anything else takes the two calls below, which report what is wrong)
    const int64_t rows = p->num_tokens * (int64_t)a.num_kv_heads;
    const int D = a.head_dim;
    if (rows > 0 && rows < 2048 && p->max_blocks > 0 && a.block_size > 0 && a.bits >= 2 && a.bits <= 4 &&
        D >= 8 && D <= 1024 && (D & (D - 1)) == 0 && p->kv_dtype >= AKV_F16 && p->kv_dtype <= AKV_F32 &&
        a.rotation_t && a.k_packed && a.v_packed && a.k_norms && a.v_norms) {
      RowMap mk{}, mv{};
      mk.x = p->key; mk.x_dtype = p->kv_dtype; mk.x_stride_tok = p->k_stride_tok; mk.x_stride_head = p->k_stride_head;
      mk.packed = const_cast<uint8_t*>(a.k_packed); mk.norms = const_cast<float*>(a.k_norms);
      mk.slot_mapping = p->slot_mapping; mk.num_heads = a.num_kv_heads; mk.block_size = a.block_size;
      mk.max_blocks = p->max_blocks;
      mk.p_stride_blk = a.kp_stride_blk; mk.p_stride_pos = a.kp_stride_pos; mk.p_stride_head = a.kp_stride_head;
      mk.n_stride_blk = a.kn_stride_blk; mk.n_stride_pos = a.kn_stride_pos; mk.n_stride_head = a.kn_stride_head;
      mv = mk;
      mv.x = p->value; mv.x_stride_tok = p->v_stride_tok; mv.x_stride_head = p->v_stride_head;
      mv.packed = const_cast<uint8_t*>(a.v_packed); mv.norms = const_cast<float*>(a.v_norms);
      mv.p_stride_blk = a.vp_stride_blk; mv.p_stride_pos = a.vp_stride_pos; mv.p_stride_head = a.vp_stride_head;
      mv.n_stride_blk = a.vn_stride_blk; mv.n_stride_pos = a.vn_stride_pos; mv.n_stride_head = a.vn_stride_head;
      // head_dim 128 or 256 and at least one sequence: the vectors ride in the attention's first launch (if the
      // attention arguments are rejected nothing is written and the error is returned)
      if (D >= 128 && D <= 256 && a.num_seqs > 0) {
        NewTokenWrite nt{};
        nt.k = mk; nt.v = mv; nt.n_rows = rows; nt.bits = a.bits; nt.boundaries = p->boundaries;
        return run_tq_attn(&p->attn, a.workspace, a.workspace_bytes, true, &nt);
      }
      if (int rc = launch_encode_generic_pair(mk, mv, rows, D, a.bits, a.rotation_t, p->boundaries, (cudaStream_t)a.stream))
        return rc;
      return run_tq_attn(&p->attn, a.workspace, a.workspace_bytes);
    }
    int rc = akv_tq_kv_update(p->key, p->kv_dtype, p->num_tokens, a.num_kv_heads, a.head_dim, p->k_stride_tok,
                              p->k_stride_head, p->slot_mapping, const_cast<uint8_t*>(a.k_packed), a.kp_stride_blk,
                              a.kp_stride_pos, a.kp_stride_head, const_cast<float*>(a.k_norms), a.kn_stride_blk,
                              a.kn_stride_pos, a.kn_stride_head, a.bits, a.rotation_t, p->boundaries, a.block_size,
                              p->max_blocks, a.stream);
    if (rc) return rc;
    rc = akv_tq_kv_update(p->value, p->kv_dtype, p->num_tokens, a.num_kv_heads, a.head_dim, p->v_stride_tok,
                          p->v_stride_head, p->slot_mapping, const_cast<uint8_t*>(a.v_packed), a.vp_stride_blk,
                          a.vp_stride_pos, a.vp_stride_head, const_cast<float*>(a.v_norms), a.vn_stride_blk,
                          a.vn_stride_pos, a.vn_stride_head, a.bits, a.rotation_t, p->boundaries, a.block_size,
                          p->max_blocks, a.stream);
    if (rc) return rc;
  }
  return run_tq_attn(&p->attn, a.workspace, a.workspace_bytes);
}

// ---------------------------------------------------------------------------
// Allocation-free variant of akv_tq_paged_attn.
//
// Some callers are not allowed to allocate device memory around the call: a
// serving engine that has already handed every free byte to its KV-cache pool,
// or a plugin that runs inside someone else's memory plan and may not touch
// cudaMalloc (nor torch's caching allocator).  For them the split-K scratch -
// rotated queries plus the (m, l, acc) partials - lives in a fixed array that is
// part of the loaded library image, so each GPU that loads the library holds
// AKV_STATIC_SCRATCH_BYTES of it until the process exits.
//
// In host code `g_static_scratch` is only a handle for the symbol, not a device
// address; the address every kernel receives comes from cudaGetSymbolAddress,
// asked once per device with that device current.
// ---------------------------------------------------------------------------
#define AKV_STATIC_SCRATCH_BYTES (8u << 20)
static __device__ __align__(256) unsigned char g_static_scratch[AKV_STATIC_SCRATCH_BYTES];

namespace akv {
static int static_scratch_ptr(void** out) {
  constexpr int kMaxDevices = 64;
  static void* ptrs[kMaxDevices] = {nullptr};
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return fail((int)e, "cudaGetDevice: %s", cudaGetErrorString(e));
  if (dev < 0 || dev >= kMaxDevices) return fail(AKV_ERR_UNSUPPORTED, "device index %d out of range", dev);
  void* p = __atomic_load_n(&ptrs[dev], __ATOMIC_ACQUIRE);
  if (p == nullptr) {
    e = cudaGetSymbolAddress(&p, g_static_scratch);
    if (e != cudaSuccess || p == nullptr)
      return fail(e != cudaSuccess ? (int)e : AKV_ERR_UNSUPPORTED, "cudaGetSymbolAddress(static scratch): %s",
                  cudaGetErrorString(e));
    __atomic_store_n(&ptrs[dev], p, __ATOMIC_RELEASE);   // same value from any thread
  }
  *out = p;
  return AKV_OK;
}
}  // namespace akv

// Mirror of akv_tq_prefill_params in include/akv_b200.h.
struct akv_tq_prefill_params {
  const void* query; int q_dtype; int64_t q_stride_tok, q_stride_head;
  const uint8_t* k_packed; int64_t kp_stride_blk, kp_stride_pos, kp_stride_head;
  const float* k_norms; int64_t kn_stride_blk, kn_stride_pos, kn_stride_head;
  const uint8_t* v_packed; int64_t vp_stride_blk, vp_stride_pos, vp_stride_head;
  const float* v_norms; int64_t vn_stride_blk, vn_stride_pos, vn_stride_head;
  const void* block_tables; int bt_dtype; int64_t bt_stride_seq;
  const void* seq_lens; int sl_dtype;
  const void* query_start_loc; int qs_dtype;
  int num_seqs, num_tokens, num_q_heads, num_kv_heads, head_dim, block_size, max_blocks_per_seq;
  int64_t num_blocks;
  int bits;
  const float* rotation; const float* rotation_t; const float* centroids;
  float scale;
  void* out; int out_dtype; int64_t out_stride_tok, out_stride_head;
  void* workspace; size_t workspace_bytes;
  void* stream;
  int max_seq_len;
  const void* hybrid_tables;
};

// Chunks of up to PREFILL_SPLIT_ROWS rows get room for PREFILL_MAX_SPLITS partials per row (key-range splits of the
// tensor-core kernels).
constexpr int PREFILL_MAX_SPLITS = 4;
constexpr size_t PREFILL_SPLIT_ROWS = 65536;
static int prefill_parts(size_t rows) { return rows <= PREFILL_SPLIT_ROWS ? PREFILL_MAX_SPLITS : 1; }

// Key-range splits of the tensor-core kernels: `ctas` CTAs of equal length run in ceil(ctas / SMs) rounds; s splits make
// it ceil(s ctas / SMs) rounds of 1 / s the length.  The smallest s within 2 % of the best is taken (every split adds a
// partial per row to the merge), with at least 16 key tiles per split when the caller gave max_seq_len.
static int prefill_splits(int64_t ctas, int parts, int max_seq_len) {
  if (ctas <= 0 || parts <= 1) return 1;
  const int sms = sm_count();
  int limit = parts;
  if (max_seq_len > 0) {
    const int by_len = (max_seq_len / 128) / 16;
    limit = by_len < 1 ? 1 : (by_len < limit ? by_len : limit);
  } else {            // lengths unknown: only the case of fewer CTAs than SMs
    const int by_sms = (int)(sms / ctas);
    limit = by_sms < 1 ? 1 : (by_sms < limit ? by_sms : limit);
  }
  int best = 1;
  double best_cost = (double)((ctas + sms - 1) / sms);
  for (int s = 2; s <= limit; ++s) {
    const double cost = (double)((ctas * s + sms - 1) / sms) / s * (1.0 + 0.02 * (s - 1));
    if (cost < best_cost * 0.98) { best = s; best_cost = cost; }
  }
  return best;
}

static void prefill_plan(int num_tokens, int num_q_heads, size_t* off_acc, size_t* off_ml, size_t* total) {
  const size_t rows = (size_t)num_tokens * num_q_heads, parts = (size_t)prefill_parts(rows);
  auto al = [](size_t v) { return (v + 255) & ~(size_t)255; };
  *off_acc = al(rows * 128 * sizeof(float));
  *off_ml = *off_acc + al(rows * parts * 128 * sizeof(float));
  *total = *off_ml + al(rows * parts * 2 * sizeof(float));
}

AKV_EXPORT size_t akv_tq_prefill_attn_workspace_bytes(int num_tokens, int num_q_heads) {
  if (num_tokens <= 0 || num_q_heads <= 0) return 0;
  size_t a, m, total;
  prefill_plan(num_tokens, num_q_heads, &a, &m, &total);
  return total;
}

// Returns AKV_ERR_UNSUPPORTED (without touching anything) for shapes the kernel is not built for; the caller
// then attends row by row with akv_tq_paged_attn.
AKV_EXPORT size_t akv_tq_prefill_attn_workspace_bytes_staged(int num_tokens, int num_q_heads, int num_kv_heads, int num_seqs,
                                                             int max_seq_len) {
  size_t a, m, total;
  prefill_plan(num_tokens, num_q_heads, &a, &m, &total);
  const size_t staged = prefill_staged_bytes(num_seqs, num_kv_heads, max_seq_len);
  return staged ? ((total + 1023) & ~(size_t)1023) + staged : total;
}

AKV_EXPORT int akv_tq_prefill_attn(const akv_tq_prefill_params* p) {
  if (!p) return fail(AKV_ERR_ARG, "null params");
  if (p->num_tokens < 0 || p->num_seqs < 0 || p->num_q_heads <= 0 || p->num_kv_heads <= 0 ||
      p->num_q_heads % p->num_kv_heads || p->block_size <= 0 || p->max_blocks_per_seq < 0 || p->num_blocks <= 0)
    return fail(AKV_ERR_ARG, "prefill attention: bad sizes");
  const int G = p->num_q_heads / p->num_kv_heads;
  auto al16 = [](const void* q, int64_t a, int64_t b, int64_t c) {
    return ((reinterpret_cast<uintptr_t>(q) | (uintptr_t)a | (uintptr_t)b | (uintptr_t)c) & 15) == 0;
  };
  const bool hybrid = p->hybrid_tables != nullptr;         // tq35 records: staged tensor-core kernel only, like ...
  // ... 3- and 2-bit codes and 4-bit rows that cannot be read in 16-byte pieces (68-byte records with the norm inside)
  const bool rows16 = al16(p->k_packed, p->kp_stride_blk, p->kp_stride_pos, p->kp_stride_head) &&
                      al16(p->v_packed, p->vp_stride_blk, p->vp_stride_pos, p->vp_stride_head);
  const bool low_bits = p->bits == 3 || p->bits == 2 || hybrid || (p->bits == 4 && !rows16);
  if (hybrid && ((reinterpret_cast<uintptr_t>(p->k_packed) | reinterpret_cast<uintptr_t>(p->v_packed) | (uintptr_t)p->kp_stride_blk |
                  (uintptr_t)p->kp_stride_pos | (uintptr_t)p->kp_stride_head | (uintptr_t)p->vp_stride_blk |
                  (uintptr_t)p->vp_stride_pos | (uintptr_t)p->vp_stride_head) & 3) != 0)
    return fail(AKV_ERR_UNSUPPORTED, "prefill attention over hybrid records needs records readable in 4-byte pieces");
  if (p->head_dim != 128 || (p->bits != 4 && !low_bits) || (G != 1 && G != 2 && G != 4 && G != 8) || p->block_size % 16 != 0)
    return fail(AKV_ERR_UNSUPPORTED, "prefill attention is built for head_dim 128, 1/2/4/8 query heads per KV head, block sizes "
                                     "that are multiples of 16 and 4-bit caches readable in 16-byte pieces (3- and 2-bit "
                                     "caches: staged kernel only)");
  if (p->num_tokens == 0 || p->num_seqs == 0) return AKV_OK;
  if (!p->query || !p->k_packed || !p->v_packed || (!hybrid && (!p->k_norms || !p->v_norms || !p->centroids)) ||
      !p->block_tables || !p->seq_lens || !p->query_start_loc || !p->rotation || !p->rotation_t || !p->out)
    return fail(AKV_ERR_ARG, "prefill attention: null pointer");
  size_t off_acc, off_ml, total;
  prefill_plan(p->num_tokens, p->num_q_heads, &off_acc, &off_ml, &total);
  if (!p->workspace || p->workspace_bytes < total)
    return fail(AKV_ERR_WORKSPACE, "workspace too small: need %zu bytes, got %zu", total, p->workspace_bytes);
  char* ws = reinterpret_cast<char*>(p->workspace);
  float* qrot = reinterpret_cast<float*>(ws);
  float* part_acc = reinterpret_cast<float*>(ws + off_acc);
  float* part_ml = reinterpret_cast<float*>(ws + off_ml);
  cudaStream_t st = (cudaStream_t)p->stream;
  const int rows = p->num_tokens * p->num_q_heads;
  // tcgen05 kernel (128 rows per CTA) when its row tiles would be at least half full - chunks of prefill tokens, not a
  // batch of single decode tokens (the host cannot see query_start_loc: a sequence adds at most one ragged tile);
  // AKV_PREFILL_TC=0 / 1 forces one or the other
  static const char* tc_env = getenv("AKV_PREFILL_TC");
  const int64_t tc_rows = (int64_t)p->num_tokens * G;
  const int64_t tc_tiles = (tc_rows + 127) / 128 + p->num_seqs - 1;
  const bool use_tc = tc_env ? tc_env[0] == '1' : tc_rows >= 64 * tc_tiles;
  // the key range of every row tile may be split over up to four CTAs, whose partials the merge kernel combines: few row
  // tiles (a short chunk, possibly on a long context), or a CTA count that leaves the last round of CTAs half empty
  const int splits = use_tc ? prefill_splits(tc_tiles * p->num_kv_heads, prefill_parts((size_t)rows), p->max_seq_len) : 1;
  // 3- and 2-bit caches: only the staged tensor-core kernel reads them; say so before anything is launched
  {
    static const bool no_staged_env = getenv("AKV_PREFILL_STAGED") != nullptr && getenv("AKV_PREFILL_STAGED")[0] == '0';
    const size_t need = prefill_staged_bytes(p->num_seqs, p->num_kv_heads, p->max_seq_len);
    if (low_bits && (!use_tc || no_staged_env || need == 0 || p->workspace_bytes < ((total + 1023) & ~(size_t)1023) + need))
      return fail(AKV_ERR_UNSUPPORTED, "prefill attention over 3- / 2-bit codes or tq35 records needs a chunk that fills "
                                       "128-row tiles, max_seq_len and the staged workspace");
  }
  // Many rows: both rotations are [rows, 128] x [128, 128] products on the tensor cores (rot_rows.cu); a few rows: the
  // kernels of the decode path
  const bool gemm_q = rows >= 2048 && rot_rows_ok(p->query, p->q_dtype, p->q_stride_tok, p->q_stride_head, qrot, AKV_F32,
                                                    (int64_t)p->num_q_heads * 128, 128);
  const bool gemm_o = splits == 1 && rows >= 2048 && rot_rows_ok(part_acc, AKV_F32, (int64_t)p->num_q_heads * 128, 128, p->out, p->out_dtype,
                                                    p->out_stride_tok, p->out_stride_head);
  if (gemm_q) {
    if (int rc = launch_rot_rows(p->query, p->q_dtype, p->q_stride_tok, p->q_stride_head, p->num_q_heads, nullptr, 0,
                                 p->rotation_t, p->scale * 1.4426950408889634f, qrot, AKV_F32,
                                 (int64_t)p->num_q_heads * 128, 128, rows, st))
      return rc;
  } else {   // rotated, scaled queries of every token
    const size_t smem128 = (size_t)ROT128_MAT_BYTES + 4 * 128 * sizeof(float);
    cudaError_t e = cudaFuncSetAttribute(akv_qrot128_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem128);
    if (e != cudaSuccess) return fail((int)e, "prefill attention: smem attribute: %s", cudaGetErrorString(e));
    const int quads = (rows + 3) / 4;
    const int rot_blocks = quads < 2 * sm_count() ? quads : 2 * sm_count();
    StreamKPlanArgs no_plan{};
    NewTokenWrite no_write{};
    akv_qrot128_kernel<<<rot_blocks, ROT128_THREADS, smem128, st>>>(
        p->query, p->q_dtype, p->q_stride_tok, p->q_stride_head, p->num_q_heads, p->rotation_t,
        p->scale * 1.4426950408889634f, qrot, rows, rot_blocks, 0, no_plan, no_write);
    if (int rc = check_launch("akv_qrot128_kernel")) return rc;
  }
  // rows that no sequence of the chunk owns (padding) stay at l = 0 and come out as zeros
  cudaMemsetAsync(part_ml, 0, (size_t)rows * splits * 2 * sizeof(float), st);
  PrefillArgs a{};
  a.qrot = qrot;
  a.k_packed = p->k_packed; a.kp_sb = p->kp_stride_blk; a.kp_sp = p->kp_stride_pos; a.kp_sh = p->kp_stride_head;
  a.k_norms = p->k_norms; a.kn_sb = p->kn_stride_blk; a.kn_sp = p->kn_stride_pos; a.kn_sh = p->kn_stride_head;
  a.v_packed = p->v_packed; a.vp_sb = p->vp_stride_blk; a.vp_sp = p->vp_stride_pos; a.vp_sh = p->vp_stride_head;
  a.v_norms = p->v_norms; a.vn_sb = p->vn_stride_blk; a.vn_sp = p->vn_stride_pos; a.vn_sh = p->vn_stride_head;
  a.block_tables = p->block_tables; a.bt_dtype = p->bt_dtype; a.bt_stride = p->bt_stride_seq;
  a.seq_lens = p->seq_lens; a.sl_dtype = p->sl_dtype;
  a.query_start_loc = p->query_start_loc; a.qs_dtype = p->qs_dtype;
  a.num_seqs = p->num_seqs; a.n_tokens = p->num_tokens; a.num_q_heads = p->num_q_heads; a.num_kv_heads = p->num_kv_heads;
  a.block_size = p->block_size; a.max_blocks_per_seq = p->max_blocks_per_seq; a.num_blocks = p->num_blocks;
  a.centroids = p->centroids; a.part_acc = part_acc; a.part_ml = part_ml;
  if (use_tc) {
    // with the longest sequence known on the host and room in the workspace, the codes are turned into fp16 operand
    // images once (instead of once per row tile) and the tensor-core kernel is fed by bulk copies; AKV_PREFILL_STAGED=0
    // keeps the decode inside the kernel
    static const bool no_staged = getenv("AKV_PREFILL_STAGED") != nullptr && getenv("AKV_PREFILL_STAGED")[0] == '0';
    const size_t staged = no_staged ? 0 : prefill_staged_bytes(p->num_seqs, p->num_kv_heads, p->max_seq_len);
    const size_t staged_off = (total + 1023) & ~(size_t)1023;
    a.bits = p->bits;
    a.byte_rows = rows16 ? 0 : 1;
    a.hybrid_tables = p->hybrid_tables;
    a.splits = splits;
    if (staged != 0 && p->workspace_bytes >= staged_off + staged && (reinterpret_cast<uintptr_t>(ws) & 15) == 0) {
      a.staged = reinterpret_cast<uint8_t*>(ws + staged_off);
      a.tiles_per_seq = (p->max_seq_len + prefill_staged_tile_keys() - 1) / prefill_staged_tile_keys();
    }
    if (low_bits && a.staged == nullptr)
      return fail(AKV_ERR_UNSUPPORTED, "prefill attention over 3- / 2-bit codes needs max_seq_len and the staged workspace");
    if (int rc = launch_prefill_tc(a, G, st)) return rc;
  } else {
  if (low_bits) return fail(AKV_ERR_UNSUPPORTED, "prefill attention over 3- / 2-bit codes: chunk too ragged for the staged kernel");
  const int TT = 64 / G;
  dim3 grid((p->num_tokens + TT - 1) / TT + p->num_seqs, p->num_kv_heads);
  cudaError_t e = cudaSuccess;
#define AKV_PF(GG)                                                                                                  \
  e = cudaFuncSetAttribute(tq_prefill_attn_kernel<GG>, cudaFuncAttributeMaxDynamicSharedMemorySize, PF_SMEM);         \
  if (e == cudaSuccess) tq_prefill_attn_kernel<GG><<<grid, PF_THREADS, PF_SMEM, st>>>(a);
  if (G == 1) { AKV_PF(1) } else if (G == 2) { AKV_PF(2) } else if (G == 4) { AKV_PF(4) } else { AKV_PF(8) }
#undef AKV_PF
  if (e != cudaSuccess) return fail((int)e, "prefill attention: smem attribute: %s", cudaGetErrorString(e));
  if (int rc = check_launch("tq_prefill_attn_kernel")) return rc;
  }
  if (gemm_o)      // out = R^T (acc / l): one partial per row, nothing to merge
    return launch_rot_rows(part_acc, AKV_F32, (int64_t)p->num_q_heads * 128, 128, p->num_q_heads, part_ml + 1, 2, p->rotation,
                           1.0f, p->out, p->out_dtype, p->out_stride_tok, p->out_stride_head, rows, st);
  MergeArgs mg{};
  mg.acc = part_acc; mg.acc_row = (int64_t)splits * 128; mg.acc_part = 128;
  mg.ml = part_ml; mg.ml_row = (int64_t)splits * 2; mg.ml_part = 2;
  mg.np = splits;
  mg.num_q_heads = p->num_q_heads;
  mg.D = 128;
  mg.mode = MERGE_ROTATE;
  mg.rot = p->rotation;
  mg.out = p->out; mg.out_dtype = p->out_dtype; mg.out_ss = p->out_stride_tok; mg.out_sh = p->out_stride_head;
  mg.gemm_scratch = qrot;        // the rotated queries are dead by now
  return launch_merge(mg, rows, st);
}

AKV_EXPORT size_t akv_tq_paged_attn_static_scratch_bytes(void) { return AKV_STATIC_SCRATCH_BYTES; }

// Same arguments and results as akv_tq_paged_attn; params->workspace and
// params->workspace_bytes are ignored.  If params->blocks_per_split is 0 the
// split size is grown until the partials fit the static array; a problem that
// does not fit even with one split per sequence (or an explicit
// blocks_per_split that needs more) is rejected with AKV_ERR_WORKSPACE.
//
// The first call on a device looks up the array's address; make that call
// before any stream capture starts.  All calls on a device share the array and
// it keeps whatever the previous call left (nothing in it needs to start at
// zero: every partial that is read has been written by the same call), so two
// calls that may overlap on the GPU - different streams, or graphs replayed
// concurrently - race on it; serialise them.
AKV_EXPORT int akv_tq_paged_attn_static(const akv_tq_attn_params* p) {
  if (!p) return fail(AKV_ERR_ARG, "null params");
  if (p->num_seqs <= 0 || p->num_q_heads <= 0 || p->num_kv_heads <= 0 || p->block_size <= 0 ||
      p->max_blocks_per_seq < 0)
    return run_tq_attn(p, nullptr, 0);   // reports the argument error (or returns for 0 sequences)
  akv_tq_attn_params q = *p;
  int bps = p->blocks_per_split;
  Plan plan = make_plan(p->num_seqs, p->num_q_heads, p->num_kv_heads, p->head_dim, p->bits,
                        p->block_size, p->max_blocks_per_seq, bps, false);
  if (bps <= 0) {
    bps = plan.blocks_per_split;
    while (plan.total > AKV_STATIC_SCRATCH_BYTES && plan.num_splits > 1) {
      bps *= 2;
      plan = make_plan(p->num_seqs, p->num_q_heads, p->num_kv_heads, p->head_dim, p->bits,
                       p->block_size, p->max_blocks_per_seq, bps, false);
    }
    q.blocks_per_split = plan.blocks_per_split;
  }
  if (plan.total > AKV_STATIC_SCRATCH_BYTES)
    return fail(AKV_ERR_WORKSPACE,
                "akv_tq_paged_attn_static: needs %zu bytes of scratch but the built-in array holds %u "
                "(num_seqs*num_q_heads = %d rows, %d partials each); use akv_tq_paged_attn with a workspace",
                plan.total, (unsigned)AKV_STATIC_SCRATCH_BYTES, p->num_seqs * p->num_q_heads, plan.num_parts);
  void* scratch = nullptr;
  if (int rc = static_scratch_ptr(&scratch)) return rc;
  return run_tq_attn(&q, scratch, AKV_STATIC_SCRATCH_BYTES, false);
}

// Merge `num_parts` raw partials laid out [part][row][D+2] (m in log2 units, l,
// acc[D]) - e.g. the all-gathered raw_out of several devices - and write
// out = R^T (acc / l), or out = acc / l when `rotation` is null.
AKV_EXPORT int akv_lse_merge(const float* parts, int num_parts, int num_seqs, int num_q_heads,
                             int head_dim, const float* rotation, void* out, int out_dtype,
                             int64_t out_stride_seq, int64_t out_stride_head, void* stream) {
  if (num_parts <= 0 || num_seqs < 0 || num_q_heads <= 0 || head_dim <= 0 || head_dim > 1024 ||
      (rotation != nullptr && head_dim % 16 != 0))
    return fail(AKV_ERR_ARG, "akv_lse_merge: bad sizes");
  if (num_seqs == 0) return AKV_OK;
  if (!parts || !out) return fail(AKV_ERR_ARG, "akv_lse_merge: null pointer");
  const int rows = num_seqs * num_q_heads;
  MergeArgs mg{};
  mg.acc = parts + 2; mg.acc_row = head_dim + 2; mg.acc_part = (int64_t)rows * (head_dim + 2);
  mg.ml = parts; mg.ml_row = head_dim + 2; mg.ml_part = (int64_t)rows * (head_dim + 2);
  mg.np = num_parts;
  mg.context_lens = nullptr; mg.num_q_heads = num_q_heads;
  mg.D = head_dim;
  mg.mode = rotation ? MERGE_ROTATE : MERGE_NORMALIZE;
  mg.rot = rotation;
  mg.out = out; mg.out_dtype = out_dtype; mg.out_ss = out_stride_seq; mg.out_sh = out_stride_head;
  return launch_merge(mg, rows, (cudaStream_t)stream);
}
