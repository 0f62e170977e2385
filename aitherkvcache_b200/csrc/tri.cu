// TriAttention: spectral KV codec (top-F RoPE pairs, int4 coefficients) and the
// trig-series decode step.
//
// Reference: aither_kvcache/triattention/encoder.py:73-149 (encode),
// scorer.py:84-208 (scores), attention.py:186-280 (softmax + scattered value sum).
//
// decode step, per (batch, kv head), for every cached token:
//   k0,k1   = dequantised pair coefficients of the F retained pairs
//   phi     = float32( float(pos_k) - float(pos_q) ) * theta[pair]      (same float32 product
//             as the reference; reduced mod 2*pi with a three-term Cody-Waite step)
//   k'      = the pair rotated by phi: (k0 cos - k1 sin, k1 cos + k0 sin)
//   score_h = scale * sum_f ( q_h[2i] k'_0 + q_h[2i+1] k'_1 )
// which equals the reference's c*cos + s*sin series.  The rotated sparse keys and the
// sparse values of a 32-token tile are written into dense fp16 tiles in shared memory
// (zero elsewhere) and both products run on mma.sync m16n8k16, the 4..8 query heads of the
// GQA group in the N dimension; softmax is online over tiles, partials (m, l, acc) are
// merged by the common LSE merge kernel.
#include "common.cuh"
#include <math_constants.h>
#include <stdlib.h>

namespace akv {

// ---------------------------------------------------------------------------
// encode: one thread per vector
// ---------------------------------------------------------------------------
constexpr int TE_THREADS = 64;
constexpr int TE_LD = 129;

template <int F>
__global__ void __launch_bounds__(TE_THREADS)
tri_encode_kernel(const void* __restrict__ x, int x_dtype, int64_t n_rows, int64_t x_row_stride, int coeff_bits,
                  uint8_t* __restrict__ indices, uint8_t* __restrict__ packed, __half* __restrict__ scales) {
  constexpr int D = 128, P = 64;
  __shared__ float xs[TE_THREADS * TE_LD];
  const int tid = threadIdx.x;
  const int64_t row0 = (int64_t)blockIdx.x * TE_THREADS;
  for (int e = tid; e < TE_THREADS * D; e += TE_THREADS) {
    const int r = e / D, c = e % D;
    const int64_t n = row0 + r;
    xs[r * TE_LD + c] = (n < n_rows) ? load_as_float(x, x_dtype, n * x_row_stride + c) : 0.f;
  }
  __syncthreads();
  const int64_t n = row0 + tid;
  if (n >= n_rows) return;
  const float* v = xs + tid * TE_LD;
  float e[P];
#pragma unroll
  for (int i = 0; i < P; ++i) e[i] = __fadd_rn(__fmul_rn(v[2 * i], v[2 * i]), __fmul_rn(v[2 * i + 1], v[2 * i + 1]));
  // F rounds of arg-max; ties go to the lower pair id
  unsigned long long mask = 0ull;
  for (int r = 0; r < F; ++r) {
    float best = -1.f;
    int bi = 0;
#pragma unroll
    for (int i = 0; i < P; ++i) {
      const bool taken = (mask >> i) & 1ull;
      if (!taken && e[i] > best) { best = e[i]; bi = i; }
    }
    mask |= 1ull << bi;
  }
  int ids[F];
  int c = 0;
  for (int i = 0; i < P && c < F; ++i)
    if ((mask >> i) & 1ull) ids[c++] = i;
  if (coeff_bits == 16) {       // the pair values as fp16, no scale (encoder.py:104-112)
    __half* ph = reinterpret_cast<__half*>(packed) + n * (2 * F);
    for (int f = 0; f < F; ++f) {
      indices[n * F + f] = (uint8_t)ids[f];
      ph[2 * f] = __float2half_rn(v[2 * ids[f]]);
      ph[2 * f + 1] = __float2half_rn(v[2 * ids[f] + 1]);
    }
    scales[n] = __float2half_rn(1.0f);
    return;
  }
  float amax = 0.f;
  for (int f = 0; f < F; ++f) {
    amax = fmaxf(amax, fabsf(v[2 * ids[f]]));
    amax = fmaxf(amax, fabsf(v[2 * ids[f] + 1]));
  }
  const float scale = fmaxf(amax, 1e-8f);
  const float half_code = coeff_bits == 8 ? 127.5f : 7.5f, max_code = coeff_bits == 8 ? 255.f : 15.f;
  for (int f = 0; f < F; ++f) {
    float q0 = rintf(__fmul_rn(__fadd_rn(__fdiv_rn(v[2 * ids[f]], scale), 1.0f), half_code));
    float q1 = rintf(__fmul_rn(__fadd_rn(__fdiv_rn(v[2 * ids[f] + 1], scale), 1.0f), half_code));
    q0 = fminf(fmaxf(q0, 0.f), max_code);
    q1 = fminf(fmaxf(q1, 0.f), max_code);
    indices[n * F + f] = (uint8_t)ids[f];
    if (coeff_bits == 8) {        // both components as bytes, pair by pair (encoder.py:136-145)
      packed[n * (2 * F) + 2 * f] = (uint8_t)(int)q0;
      packed[n * (2 * F) + 2 * f + 1] = (uint8_t)(int)q1;
    } else {
      packed[n * F + f] = (uint8_t)(((int)q0 << 4) | (int)q1);
    }
  }
  scales[n] = __float2half_rn(scale);
}

// ---------------------------------------------------------------------------
// decode step
// ---------------------------------------------------------------------------
struct TriArgs {
  const uint8_t* k_idx; const uint8_t* k_packed; const __half* k_scales;
  const uint8_t* v_idx; const uint8_t* v_packed; const __half* v_scales;
  int B, S, KVH, QH, F;
  const void* query; int q_dtype; int64_t q_sb, q_sh;   // [B,QH,128]
  const int64_t* key_positions;   // [B,S] or null: position = key_pos_start + s
  int64_t key_pos_start;
  const int64_t* query_pos;       // [B] or null: query_pos_default
  int64_t query_pos_default;
  const float* theta;             // [64]
  float premul;                   // scale * log2(e)
  int tokens_per_split, num_parts;
  float* part_acc;                // [B*QH][NP][128]
  float* part_ml;                 // [B*QH][NP][2]
  float* scores_out;              // optional [B][QH][S] pre-softmax logits (natural units)
  // paged mode (block_tables != nullptr): the arrays are [num_blocks][block_size][KVH]...; token s of batch b
  // lives in physical block block_tables[b][s / block_size], slot s % block_size; S = table width * block_size
  const void* block_tables; int bt_dtype; int64_t bt_stride;
  int block_size; int64_t num_blocks;
  const void* context_lens; int cl_dtype;      // optional [B]: tokens of each batch element (clamped to S)
  int post_rope;                               // keys were rotated before encoding: all phases are zero (scorer.py:201-203)
};

// Row of (batch b, token s) in the record arrays, before the head index.
__device__ __forceinline__ int64_t tri_token_row(const TriArgs& a, int b, int s) {
  if (a.block_tables == nullptr) return (int64_t)b * a.S + s;
  const int blk = s / a.block_size;
  int64_t phys = load_index(a.block_tables, a.bt_dtype, (int64_t)b * a.bt_stride + blk);
  phys = phys < 0 ? 0 : (phys >= a.num_blocks ? a.num_blocks - 1 : phys);
  return phys * a.block_size + (s - blk * a.block_size);
}

constexpr int TD_LD = 136;                       // halves per row of the dense tiles (272 B: conflict-free ldmatrix)
constexpr int TD_TILE_HALVES = 32 * TD_LD;

__device__ __forceinline__ void mma16816_tri(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const __half* p) {
  const uint32_t addr = (uint32_t)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}

__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const __half* p) {
  const uint32_t addr = (uint32_t)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}

__device__ __forceinline__ uint32_t movmatrix_trans_tri(uint32_t x) {
  uint32_t y;
  asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;\n" : "=r"(y) : "r"(x));
  return y;
}

__device__ __forceinline__ uint32_t pack_h2(float lo, float hi) {
  __half2 h = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&h);
}

__device__ __forceinline__ float ex2a(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// The phase phi = float32(delta) * theta of magnitude up to ~2e5 rad is reduced by n * 2*pi with 2*pi split
// into two float32 terms (each FMA product is exact; the third term of the split would contribute below
// 2e-10 rad at these magnitudes), then sin.approx / cos.approx on [-pi, pi] (absolute error ~5e-7).
__device__ __forceinline__ void cp_async4(void* smem_dst, const void* gsrc) {
  const uint32_t d = (uint32_t)__cvta_generic_to_shared(smem_dst);
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" :: "r"(d), "l"(gsrc));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;\n" ::: "memory"); }

// Shared-memory plan of one CTA (nh <= 8 KV heads, one warp each):
//   dense tile per warp  [32 tokens][TD_LD halves]   (rotated keys, then values; all-zero between uses)
//   two staging buffers  4 arrays x [nh][32 tokens][F bytes] + 2 x [32 tokens][nh] fp16 scales
// CB = bits of one coefficient: 4 (two per byte), 8 (bytes k0, k1 per pair) or 16 (fp16 k0, k1 per pair, no scale).
template <int F, int CB>
struct TriSmem {
  static constexpr int WORDS = F / 4;                       // words of ids per record
  static constexpr int PWORDS = F * CB / 16;                // words of coefficients per record
  static constexpr int HEAD = 32 * WORDS + WORDS;            // words per head, padded so that the async
                                                            // copies of one token row hit distinct banks
  static constexpr int PHEAD = 32 * PWORDS + PWORDS;
  static constexpr int ARR = 8 * HEAD;                      // words per staged id array (8 heads)
  static constexpr int PARR = 8 * PHEAD;                    // words per staged coefficient array
  static constexpr int OFF_KP = ARR, OFF_VI = ARR + PARR, OFF_VP = 2 * ARR + PARR, OFF_SC = 2 * (ARR + PARR);
  static constexpr int STAGE_WORDS = OFF_SC + 2 * 128;      // + scales: 2 x 32 x 8 halves = 2 x 128 words
  static constexpr int THETA_BYTES = 64 * 32 * 4;           // phase table, one copy per lane
  static constexpr size_t bytes(int nh) { return (size_t)nh * TD_TILE_HALVES * 2 + 2 * STAGE_WORDS * 4 + THETA_BYTES; }
};

template <int F, int CB>
__device__ __forceinline__ void tri_stage_load(const TriArgs& a, uint32_t* stage, int b, int hg0, int nh,
                                               int s0, int s_end) {
  using SM = TriSmem<F, CB>;
  {   // ids
    const int row_words = nh * SM::WORDS;                     // words per token of this head group
    for (int i = threadIdx.x; i < 32 * row_words; i += blockDim.x) {
      const int tok = i / row_words, j = i - tok * row_words;
      if (s0 + tok >= s_end) continue;
      const int head = j / SM::WORDS, wj = j - head * SM::WORDS;
      const int64_t g_off = (tri_token_row(a, b, s0 + tok) * a.KVH + hg0) * F + 4 * j;
      const int s_off = head * SM::HEAD + tok * SM::WORDS + wj;
      cp_async4(stage + s_off, a.k_idx + g_off);
      cp_async4(stage + SM::OFF_VI + s_off, a.v_idx + g_off);
    }
  }
  {   // coefficients
    const int row_words = nh * SM::PWORDS;
    for (int i = threadIdx.x; i < 32 * row_words; i += blockDim.x) {
      const int tok = i / row_words, j = i - tok * row_words;
      if (s0 + tok >= s_end) continue;
      const int head = j / SM::PWORDS, wj = j - head * SM::PWORDS;
      const int64_t g_off = (tri_token_row(a, b, s0 + tok) * a.KVH + hg0) * (4 * SM::PWORDS) + 4 * j;
      const int s_off = head * SM::PHEAD + tok * SM::PWORDS + wj;
      cp_async4(stage + SM::OFF_KP + s_off, a.k_packed + g_off);
      cp_async4(stage + SM::OFF_VP + s_off, a.v_packed + g_off);
    }
  }
  // scales, staged as [tok][8] halves: pairs of heads by 4-byte async copies when the layout
  // allows it, single halves through registers otherwise
  __half* sk = reinterpret_cast<__half*>(stage + SM::OFF_SC);
  __half* sv = sk + 256;
  if (((nh | a.KVH) & 1) == 0) {
    const int hp = nh / 2;
    for (int i = threadIdx.x; i < 32 * hp; i += blockDim.x) {
      const int tok = i / hp, pr = i - tok * hp;
      if (s0 + tok >= s_end) continue;
      const int64_t rec = tri_token_row(a, b, s0 + tok) * a.KVH + hg0 + 2 * pr;
      cp_async4(sk + tok * 8 + 2 * pr, a.k_scales + rec);
      cp_async4(sv + tok * 8 + 2 * pr, a.v_scales + rec);
    }
  } else {
    for (int i = threadIdx.x; i < 32 * nh; i += blockDim.x) {
      const int tok = i / nh, head = i - tok * nh;
      if (s0 + tok >= s_end) continue;
      const int64_t rec = tri_token_row(a, b, s0 + tok) * a.KVH + hg0 + head;
      sk[tok * 8 + head] = a.k_scales[rec];
      sv[tok * 8 + head] = a.v_scales[rec];
    }
  }
}

// Coefficient pair f of a record as the integers (or, for fp16 coefficients, the values) the tiles hold;
// the common factor scale / 15 (4-bit), scale / 255 (8-bit) or 1 (fp16) goes onto the scores and onto P.
template <int CB>
__device__ __forceinline__ void tri_coeff_pair(const uint32_t* pw, int f, float& c0, float& c1) {
  if (CB == 4) {
    const uint32_t byte = (pw[f >> 2] >> (8 * (f & 3))) & 0xffu;
    c0 = (float)(2 * (int)(byte >> 4) - 15);
    c1 = (float)(2 * (int)(byte & 15u) - 15);
  } else if (CB == 8) {
    const uint32_t two = (pw[f >> 1] >> (16 * (f & 1))) & 0xffffu;
    c0 = (float)(2 * (int)(two & 0xffu) - 255);
    c1 = (float)(2 * (int)(two >> 8) - 255);
  } else {
    const float2 v = __half22float2(*reinterpret_cast<const __half2*>(&pw[f]));
    c0 = v.x;
    c1 = v.y;
  }
}

template <int F, int CB>
__global__ void __launch_bounds__(256, 2)
tri_decode_kernel(TriArgs a) {
  using SM = TriSmem<F, CB>;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int hg = blockIdx.x, split = blockIdx.y, b = blockIdx.z;
  const int hg0 = hg * 8;
  const int nh = (a.KVH - hg0 < 8) ? a.KVH - hg0 : 8;        // heads (= warps) of this CTA
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  __half* tile = reinterpret_cast<__half*>(smem_raw) + (size_t)warp * TD_TILE_HALVES;
  uint32_t* stage0 = reinterpret_cast<uint32_t*>(smem_raw + (size_t)nh * TD_TILE_HALVES * 2);
  float* theta_rep = reinterpret_cast<float*>(stage0 + 2 * SM::STAGE_WORDS);      // [64][32 lanes]: conflict-free lookups
  for (int i = threadIdx.x; i < 64 * 32; i += blockDim.x) theta_rep[i] = a.theta[i >> 5];
  const float* const my_theta = theta_rep + lane;
  const int kvh = hg0 + warp;
  const int G = a.QH / a.KVH;

  {   // the dense tile starts (and is left after every use) all zero
    uint4* row = reinterpret_cast<uint4*>(tile + lane * TD_LD);
#pragma unroll
    for (int i = 0; i < 17; ++i) row[i] = make_uint4(0, 0, 0, 0);
  }

  // query fragments: B operand [k = dim][n = q head of the group]
  uint32_t bq[8][2];
  {
    const int qh = kvh * G + (g < G ? g : 0);
    const int64_t base = (int64_t)b * a.q_sb + (int64_t)qh * a.q_sh;
#pragma unroll
    for (int kk = 0; kk < 8; ++kk) {
      float f0 = load_as_float(a.query, a.q_dtype, base + 16 * kk + 2 * t) * a.premul;
      float f1 = load_as_float(a.query, a.q_dtype, base + 16 * kk + 2 * t + 1) * a.premul;
      float f2 = load_as_float(a.query, a.q_dtype, base + 16 * kk + 2 * t + 8) * a.premul;
      float f3 = load_as_float(a.query, a.q_dtype, base + 16 * kk + 2 * t + 9) * a.premul;
      if (g >= G) { f0 = f1 = f2 = f3 = 0.f; }
      bq[kk][0] = pack_h2(f0, f1);
      bq[kk][1] = pack_h2(f2, f3);
    }
  }
  const float qpos = (float)(a.query_pos ? a.query_pos[b] : a.query_pos_default);

  float o[8][4];
#pragma unroll
  for (int j = 0; j < 8; ++j) { o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f; }
  float m0 = -CUDART_INF_F, m1 = -CUDART_INF_F, l0 = 0.f, l1 = 0.f;

  const int s_begin = split * a.tokens_per_split;
  int s_end = s_begin + a.tokens_per_split;
  const int s_lim = a.context_lens ? (int)load_ctx(a.context_lens, a.cl_dtype, b, a.S) : a.S;
  if (s_end > s_lim) s_end = s_lim;
  const int n_iter = s_end > s_begin ? (s_end - s_begin + 31) / 32 : 0;

  constexpr float COEFF_DIV = CB == 4 ? 1.0f / 15.0f : (CB == 8 ? 1.0f / 255.0f : 1.0f);
  if (n_iter > 0) tri_stage_load<F, CB>(a, stage0, b, hg0, nh, s_begin, s_end);
  cp_async_commit();
  for (int it = 0; it < n_iter; ++it) {
    const int s0 = s_begin + it * 32;
    uint32_t* st = stage0 + (it & 1) * SM::STAGE_WORDS;
    cp_async_wait_all();
    __syncthreads();            // stage `it` is complete; everyone is done with stage it-1
    if (it + 1 < n_iter) tri_stage_load<F, CB>(a, stage0 + ((it + 1) & 1) * SM::STAGE_WORDS, b, hg0, nh, s0 + 32, s_end);
    cp_async_commit();

    const int s = s0 + lane;
    const bool valid = s < s_end;
    uint32_t kiw[SM::WORDS], kpw[SM::PWORDS], viw[SM::WORDS], vpw[SM::PWORDS];
    float ks = 0.f, vs = 0.f, delta = 0.f;
    if (valid) {
      const int r = warp * SM::HEAD + lane * SM::WORDS, rp = warp * SM::PHEAD + lane * SM::PWORDS;
#pragma unroll
      for (int w = 0; w < SM::WORDS; ++w) {
        kiw[w] = st[r + w];
        viw[w] = st[SM::OFF_VI + r + w];
      }
#pragma unroll
      for (int w = 0; w < SM::PWORDS; ++w) {
        kpw[w] = st[SM::OFF_KP + rp + w];
        vpw[w] = st[SM::OFF_VP + rp + w];
      }
      const __half* sk = reinterpret_cast<const __half*>(st + SM::OFF_SC);
      ks = CB == 16 ? 1.0f : __half2float(sk[lane * 8 + warp]);       // fp16 coefficients carry no scale
      vs = CB == 16 ? 1.0f : __half2float(sk[256 + lane * 8 + warp]);
      const float kpos = (float)(a.key_positions ? a.key_positions[(int64_t)b * a.S + s] : a.key_pos_start + s);
      delta = a.post_rope ? 0.f : __fsub_rn(kpos, qpos);
    }
    __half2* row = reinterpret_cast<__half2*>(tile + lane * TD_LD);
    // ---- rotated keys into the dense tile: integer coefficients 2n - 15 (the factor scale / 15 goes
    //      onto the scores), exponent trick instead of int-to-float conversions ----
    if (valid) {
      if (CB == 4) {
#pragma unroll
        for (int w = 0; w < SM::WORDS; ++w) {
          const uint32_t hi2 = (kpw[w] >> 3) & 0x1E1E1E1Eu, lo2 = (kpw[w] << 1) & 0x1E1E1E1Eu;     // 2n per byte
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            const uint32_t id = __byte_perm(kiw[w], 0u, 0x4440 + c) & 63u;
            const float phi = __fmul_rn(delta, my_theta[id * 32]);
            const float n = rintf(phi * 0.15915494309189535f);
            float r = __fmaf_rn(-n, 6.2831854820251465f, phi);
            r = __fmaf_rn(-n, -1.7484555314695172e-07f, r);
            const float sn = __sinf(r), cs = __cosf(r);
            const float k0 = __uint_as_float(__byte_perm(hi2, 0x4B000000u, 0x7440 + c)) - 8388623.0f;   // 8388608 + 2n - 8388623
            const float k1 = __uint_as_float(__byte_perm(lo2, 0x4B000000u, 0x7440 + c)) - 8388623.0f;
            row[id] = __floats2half2_rn(__fmaf_rn(k0, cs, -k1 * sn), __fmaf_rn(k1, cs, k0 * sn));
          }
        }
      } else {
#pragma unroll
        for (int f = 0; f < F; ++f) {
          const uint32_t id = __byte_perm(kiw[f >> 2], 0u, 0x4440 + (f & 3)) & 63u;
          const float phi = __fmul_rn(delta, my_theta[id * 32]);
          const float n = rintf(phi * 0.15915494309189535f);
          float r = __fmaf_rn(-n, 6.2831854820251465f, phi);
          r = __fmaf_rn(-n, -1.7484555314695172e-07f, r);
          const float sn = __sinf(r), cs = __cosf(r);
          float k0, k1;
          tri_coeff_pair<CB>(kpw, f, k0, k1);
          row[id] = __floats2half2_rn(__fmaf_rn(k0, cs, -k1 * sn), __fmaf_rn(k1, cs, k0 * sn));
        }
      }
    }
    __syncwarp();

    // ---- scores for the two 16-token halves: S^T[tokens][q heads] ----
    float sc[2][4];
#pragma unroll
    for (int mt = 0; mt < 2; ++mt) {
      sc[mt][0] = sc[mt][1] = sc[mt][2] = sc[mt][3] = 0.f;
#pragma unroll
      for (int kk = 0; kk < 8; ++kk) {
        uint32_t af[4];
        ldmatrix_x4(af, tile + (mt * 16 + (lane & 7) + 8 * ((lane >> 3) & 1)) * TD_LD + kk * 16 + 8 * (lane >> 4));
        mma16816_tri(sc[mt], af, bq[kk][0], bq[kk][1]);
      }
    }
    {   // rows of the score tiles are tokens g, g+8 (+16): their key scales come from the lanes that hold them
      const float ksc = ks * COEFF_DIV;
#pragma unroll
      for (int mt = 0; mt < 2; ++mt) {
        const float ka = __shfl_sync(0xffffffffu, ksc, mt * 16 + g), kb = __shfl_sync(0xffffffffu, ksc, mt * 16 + g + 8);
        sc[mt][0] *= ka; sc[mt][1] *= ka; sc[mt][2] *= kb; sc[mt][3] *= kb;
      }
    }
    __syncwarp();
    // ---- take the keys out again, put the integer values in (the factor scale / 15 goes onto P) ----
    if (valid) {
#pragma unroll
      for (int f = 0; f < F; ++f) row[__byte_perm(kiw[f >> 2], 0u, 0x4440 + (f & 3)) & 63u] = __floats2half2_rn(0.f, 0.f);
      if (CB == 4) {
#pragma unroll
        for (int w = 0; w < SM::WORDS; ++w) {
          const uint32_t hi2 = (vpw[w] >> 3) & 0x1E1E1E1Eu, lo2 = (vpw[w] << 1) & 0x1E1E1E1Eu;
          const uint32_t t01 = __byte_perm(hi2, lo2, 0x5140), t23 = __byte_perm(hi2, lo2, 0x7362);
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            const uint32_t idv = __byte_perm(viw[w], 0u, 0x4440 + c) & 63u;
            // halves 0x6400 | 2n = 1024 + 2n, minus 1039: 2n - 15, exactly
            const uint32_t hb = __byte_perm(c < 2 ? t01 : t23, 0x64646464u, (c & 1) ? 0x4342 : 0x4140);
            row[idv] = __hsub2(*reinterpret_cast<const __half2*>(&hb), __floats2half2_rn(1039.f, 1039.f));
          }
        }
      } else {
#pragma unroll
        for (int f = 0; f < F; ++f) {
          const uint32_t idv = __byte_perm(viw[f >> 2], 0u, 0x4440 + (f & 3)) & 63u;
          float v0, v1;
          tri_coeff_pair<CB>(vpw, f, v0, v1);      // integers up to 255, or the fp16 values: exact in fp16
          row[idv] = __floats2half2_rn(v0, v1);
        }
      }
    }
    const int rem = s_end - s0;    // tokens of this tile that exist
    if (a.scores_out != nullptr) {
#pragma unroll
      for (int mt = 0; mt < 2; ++mt)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int tok = mt * 16 + g + 8 * (e >> 1), qg = 2 * t + (e & 1);
          if (tok < rem && qg < G)
            a.scores_out[((int64_t)b * a.QH + kvh * G + qg) * a.S + s0 + tok] = sc[mt][e] * 0.6931471805599453f;
        }
    }
#pragma unroll
    for (int mt = 0; mt < 2; ++mt) {
      if (mt * 16 + g >= rem) { sc[mt][0] = -CUDART_INF_F; sc[mt][1] = -CUDART_INF_F; }
      if (mt * 16 + g + 8 >= rem) { sc[mt][2] = -CUDART_INF_F; sc[mt][3] = -CUDART_INF_F; }
    }
    float mx0 = fmaxf(fmaxf(sc[0][0], sc[0][2]), fmaxf(sc[1][0], sc[1][2]));
    float mx1 = fmaxf(fmaxf(sc[0][1], sc[0][3]), fmaxf(sc[1][1], sc[1][3]));
#pragma unroll
    for (int off = 4; off < 32; off <<= 1) {
      mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, off));
      mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, off));
    }
    const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
    if (__any_sync(0xffffffffu, (mn0 != m0) | (mn1 != m1))) {
      const float al0 = ex2a(m0 - mn0), al1 = ex2a(m1 - mn1);
      l0 *= al0; l1 *= al1;
#pragma unroll
      for (int j = 0; j < 8; ++j) { o[j][0] *= al0; o[j][1] *= al1; o[j][2] *= al0; o[j][3] *= al1; }
      m0 = mn0; m1 = mn1;
    }
    uint32_t pb[2][2];
#pragma unroll
    for (int mt = 0; mt < 2; ++mt) {
      const float p0 = ex2a(sc[mt][0] - mn0), p1 = ex2a(sc[mt][1] - mn1);
      const float p2 = ex2a(sc[mt][2] - mn0), p3 = ex2a(sc[mt][3] - mn1);
      l0 += p0 + p2;
      l1 += p1 + p3;
      const float vsc = vs * COEFF_DIV;        // 0 for lanes past the end
      const float va = __shfl_sync(0xffffffffu, vsc, mt * 16 + g), vb = __shfl_sync(0xffffffffu, vsc, mt * 16 + g + 8);
      pb[mt][0] = movmatrix_trans_tri(pack_h2(p0 * va, p1 * va));
      pb[mt][1] = movmatrix_trans_tri(pack_h2(p2 * vb, p3 * vb));
    }
    __syncwarp();
    // ---- values: O^T[dims][q heads] += V^T P^T ----
#pragma unroll
    for (int j = 0; j < 8; ++j) {
#pragma unroll
      for (int mt = 0; mt < 2; ++mt) {
        uint32_t af[4];
        ldmatrix_x4_trans(af, tile + (mt * 16 + (lane & 7) + 8 * (lane >> 4)) * TD_LD + j * 16 + 8 * ((lane >> 3) & 1));
        mma16816_tri(o[j], af, pb[mt][0], pb[mt][1]);
      }
    }
    __syncwarp();
    if (valid) {
#pragma unroll
      for (int f = 0; f < F; ++f) row[__byte_perm(viw[f >> 2], 0u, 0x4440 + (f & 3)) & 63u] = __floats2half2_rn(0.f, 0.f);
    }
  }

#pragma unroll
  for (int off = 4; off < 32; off <<= 1) {
    l0 += __shfl_xor_sync(0xffffffffu, l0, off);
    l1 += __shfl_xor_sync(0xffffffffu, l1, off);
  }
  const int part = split;
#pragma unroll
  for (int e = 0; e < 2; ++e) {
    const int qg = 2 * t + e;
    if (qg >= G) continue;
    const int64_t rowi = (int64_t)b * a.QH + kvh * G + qg;
    float* pa = a.part_acc + (rowi * a.num_parts + part) * 128;
#pragma unroll
    for (int j = 0; j < 8; ++j) {   // M-tile j: rows g, g+8 -> dims 16j+g, 16j+g+8
      pa[16 * j + g] = o[j][e];
      pa[16 * j + g + 8] = o[j][2 + e];
    }
    if (g == 0) {
      a.part_ml[(rowi * a.num_parts + part) * 2] = e ? m1 : m0;
      a.part_ml[(rowi * a.num_parts + part) * 2 + 1] = e ? l1 : l0;
    }
  }
}

// ---------------------------------------------------------------------------
// decode step, record-lane kernel (8 KV heads, up to 4 query heads per KV head)
//
// The 32-token x 8-head tile of a step is 256 records, one per thread, in memory order (thread r holds
// token r / 8, head r % 8), so the staged arrays are read as they lie in global memory: six bulk copies
// per 16 tokens bring them in, completing on an mbarrier, three tiles deep.
//   Scores run on the CUDA cores: per retained pair one 16-byte load fetches the pair's (even, odd) query
//   values of the group's four heads from a table laid out [pair][KV head] (the eight lanes of a quarter
//   warp are eight different heads, so the load never conflicts), the coefficient pair is rotated by the
//   phase and the four dot products advance.  Nothing dense is built for the keys.
//   Values go through the tensor cores: every lane drops its record's coefficient pairs (2n - 15, exact
//   in e4m3) as 16-bit entries into the head's [pair][token] tile, and warp h multiplies head h's tile with
//   the softmax weights: A = tile (M = pairs, K = (token, parity)), B = weights with N = (query head,
//   parity) and zero where the parities differ, so 16 accumulators per thread cover 4 heads x 128 dims.
//   The reader clears each 16 bytes of the tile as it takes them.
// Scores and value scales cross from the record lanes to the head warps through a small float array.
// ---------------------------------------------------------------------------
template <int F>
struct TriLanes {
  static constexpr int W = F / 4;                 // words per record
  static constexpr int ROW = 8 * F;               // bytes of one token's records of an array (8 heads)
  static constexpr int ARR = 32 * ROW;            // one staged array of a tile
  static constexpr int SC = 32 * 16;              // one side's scales of a tile
  static constexpr int STAGE = 4 * ARR + 2 * SC;  // K ids, K coefficients, V ids, V coefficients, K scales, V scales
  static constexpr int NSTAGE = 3;
  static constexpr int OFF_BAR = 0;               // NSTAGE "stage full" mbarriers, "tile free" mbarrier at +32, the CTA's
                                                  // "a wait ran out" word at +64
  static constexpr int OFF_TAB = 256;             // [64 pairs] x 256 B: theta, one copy per lane (128 B), then the pair's
                                                  // query values [8 heads] x 4 half2 (128 B)
  static constexpr int OFF_SC = OFF_TAB + 16384;  // [8 heads][4 scores + value scale][32 tokens] float
  static constexpr int OFF_TILE = OFF_SC + 8 * 160 * 4;   // [8 heads][64 pairs][32 tokens] e4m3x2
  static constexpr int OFF_STAGE = OFF_TILE + 8 * 4096;
  static constexpr int BYTES = OFF_STAGE + NSTAGE * STAGE;
};

__device__ int g_tri_status;    // 2: a bounded wait for a bulk copy ran out; the step's output is not valid

__device__ __forceinline__ uint32_t tri_s32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ bool tri_wait_raw(uint32_t bar, uint32_t parity) {
  const long long t0 = clock64();
  for (int it = 0; it < (1 << 24); ++it) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}\n"
        : "=r"(done) : "r"(bar), "r"(parity) : "memory");
    if (done) return true;
    if ((it & 63) == 63 && clock64() - t0 > (1ll << 31)) break;     // about a second
  }
  return false;
}

// Bounded wait; once one wait of the CTA has run out, the others return at once.
__device__ __forceinline__ bool tri_wait(uint32_t bar, uint32_t parity, uint32_t failed_addr) {
  uint32_t f;
  asm volatile("ld.shared.u32 %0, [%1];" : "=r"(f) : "r"(failed_addr) : "memory");
  if (f != 0u) return false;
  if (tri_wait_raw(bar, parity)) return true;
  g_tri_status = 2;
  asm volatile("st.shared.u32 [%0], %1;" :: "r"(failed_addr), "r"(1u) : "memory");
  return false;
}

__device__ __forceinline__ void tri_bulk(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               :: "r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}

// One thread: the copies of the tile that starts at token s0 (two units of 16 tokens; a unit lies in one
// cache block), rows past s_end left out.
template <int F>
__device__ __forceinline__ void tri_lanes_issue(const TriArgs& a, uint32_t stage, uint32_t bar, int b, int s0, int s_end) {
  using L = TriLanes<F>;
  int n[2];
  n[0] = s_end - s0;      n[0] = n[0] < 0 ? 0 : (n[0] > 16 ? 16 : n[0]);
  n[1] = s_end - s0 - 16; n[1] = n[1] < 0 ? 0 : (n[1] > 16 ? 16 : n[1]);
  const uint32_t total = (uint32_t)(n[0] + n[1]) * (4 * L::ROW + 2 * 16);
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" :: "r"(bar), "r"(total) : "memory");
  const uint8_t* const srcs[4] = {a.k_idx, a.k_packed, a.v_idx, a.v_packed};
#pragma unroll
  for (int u = 0; u < 2; ++u) {
    if (n[u] == 0) continue;
    const int64_t row = tri_token_row(a, b, s0 + 16 * u);
#pragma unroll
    for (int arr = 0; arr < 4; ++arr)
      tri_bulk(stage + arr * L::ARR + u * 16 * L::ROW, srcs[arr] + row * L::ROW, (uint32_t)n[u] * L::ROW, bar);
    tri_bulk(stage + 4 * L::ARR + u * 256, reinterpret_cast<const char*>(a.k_scales) + row * 16, (uint32_t)n[u] * 16, bar);
    tri_bulk(stage + 4 * L::ARR + L::SC + u * 256, reinterpret_cast<const char*>(a.v_scales) + row * 16, (uint32_t)n[u] * 16, bar);
  }
}

__device__ __forceinline__ uint32_t e4m3x2_to_h2(uint32_t e16) {
  uint32_t h;
  asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(h) : "h"((unsigned short)e16));
  return h;
}

template <int F>
__global__ void __launch_bounds__(256, 2)
tri_decode_lanes_kernel(TriArgs a) {
  using L = TriLanes<F>;
  extern __shared__ __align__(128) unsigned char smem[];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int split = blockIdx.y, b = blockIdx.z;
  const int G = a.QH / a.KVH;
  const uint32_t sb = tri_s32(smem);
  const uint32_t failed_addr = sb + L::OFF_BAR + 64;

  const int s_begin = split * a.tokens_per_split;
  int s_end = s_begin + a.tokens_per_split;
  const int s_lim = a.context_lens ? (int)load_ctx(a.context_lens, a.cl_dtype, b, a.S) : a.S;
  if (s_end > s_lim) s_end = s_lim;
  const int n_iter = s_end > s_begin ? (s_end - s_begin + 31) / 32 : 0;

  if (tid == 0) {
#pragma unroll
    for (int i = 0; i < L::NSTAGE; ++i)
      asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" :: "r"(sb + L::OFF_BAR + 8 * i), "r"(1u) : "memory");
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" :: "r"(sb + L::OFF_BAR + 32), "r"(8u) : "memory");
    asm volatile("st.shared.u32 [%0], %1;" :: "r"(failed_addr), "r"(0u) : "memory");
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (n_iter > 0) {
    // query table: entry (pair, KV head) = four half2 (even, odd) of the group's query heads, scaled
    uint32_t* tab = reinterpret_cast<uint32_t*>(smem + L::OFF_TAB);
    for (int i = tid; i < 64 * 8 * 4; i += 256) {
      const int pair = i >> 5, head = (i >> 2) & 7, h = i & 3;
      uint32_t v = 0u;
      if (h < G) {
        const int64_t base = (int64_t)b * a.q_sb + (int64_t)(head * G + h) * a.q_sh + 2 * pair;
        v = pack_h2(load_as_float(a.query, a.q_dtype, base) * a.premul, load_as_float(a.query, a.q_dtype, base + 1) * a.premul);
      }
      tab[pair * 64 + 32 + (i & 31)] = v;
    }
    for (int i = tid; i < 64 * 32; i += 256) tab[(i >> 5) * 64 + (i & 31)] = __float_as_uint(a.theta[i >> 5]);
    uint4* tz = reinterpret_cast<uint4*>(smem + L::OFF_TILE);
    for (int i = tid; i < 8 * 4096 / 16; i += 256) tz[i] = make_uint4(0, 0, 0, 0);
  }
  __syncthreads();
  if (tid == 0)
    for (int i = 0; i < L::NSTAGE && i < n_iter; ++i)
      tri_lanes_issue<F>(a, sb + L::OFF_STAGE + i * L::STAGE, sb + L::OFF_BAR + 8 * i, b, s_begin + 32 * i, s_end);

  // record-lane role: token jA of the tile, KV head headA; the head's tile and score rows are rotated by
  // 4 * head tokens so that the 32 lanes of a warp store to distinct banks
  const int headA = lane & 7, jA = 4 * warp + (lane >> 3);
  const int tokp = (jA + 4 * headA) & 31;
  const unsigned char* const tab = smem + L::OFF_TAB;
  const uint32_t theta_part = lane * 4, q_part = 128 + headA * 16;     // this lane's bytes inside a pair's table row
  const uint32_t free_bar = sb + L::OFF_BAR + 32;
  float* const my_sc = reinterpret_cast<float*>(smem + L::OFF_SC) + headA * 160 + tokp;
  const uint32_t my_tile = sb + L::OFF_TILE + headA * 4096 + tokp * 2;
  const float qpos = (float)(a.query_pos ? a.query_pos[b] : a.query_pos_default);
  // head-warp role: KV head `warp`; thread (g, t) weighs query head g / 2 into parity g % 2 and keeps the
  // accumulators of query head t
  const int g = lane >> 2, t = lane & 3, hq = g >> 1, par = g & 1;
  float o[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }
  float m_run = -CUDART_INF_F, l_run = 0.f;

  const int64_t* const key_positions = a.key_positions;
  const int64_t key_pos_start = a.key_pos_start;
  float* const scores_out = a.scores_out;
  const bool post_rope = a.post_rope != 0;
  int it = 0;
  bool broken = false;
  for (; it < n_iter; ++it) {
    const int s0 = s_begin + it * 32;
    const int stg = it % L::NSTAGE;
    const uint32_t bar = sb + L::OFF_BAR + 8 * stg;
    const bool ok = tri_wait(bar, (uint32_t)((it / L::NSTAGE) & 1), failed_addr);
    const uint32_t* stw = reinterpret_cast<const uint32_t*>(smem + L::OFF_STAGE + stg * L::STAGE);
    const int s = s0 + jA;
    const bool valid = ok && s < s_end;
    // ---- scores of this lane's record ----
    float sc4[4] = {-CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F};
    float vsc = 0.f;
    if (valid) {
      uint32_t kiw[L::W], kpw[L::W];
#pragma unroll
      for (int w = 0; w < L::W; ++w) {
        kiw[w] = stw[tid * L::W + w] & 0x3F3F3F3Fu;
        kpw[w] = stw[L::ARR / 4 + tid * L::W + w];
      }
      const __half* sch = reinterpret_cast<const __half*>(stw + L::ARR);      // byte offset 4 * ARR
      const float ks = __half2float(sch[tid]);
      vsc = __half2float(sch[L::SC / 2 + tid]) * (1.0f / 15.0f);
      const float kpos = (float)(key_positions ? key_positions[(int64_t)b * a.S + s] : key_pos_start + s);
      const float delta = post_rope ? 0.f : __fsub_rn(kpos, qpos);
      float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int w = 0; w < L::W; ++w) {
        const uint32_t hi2 = (kpw[w] >> 3) & 0x1E1E1E1Eu, lo2 = (kpw[w] << 1) & 0x1E1E1E1Eu;     // 2n per byte
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          // byte c of the id word lands in byte 1 (id * 256 = the pair's table row), the lane's part in byte 0
          const uint32_t th_off = __byte_perm(kiw[w], theta_part, 0x6504 + 16 * c);
          const uint32_t q_off = __byte_perm(kiw[w], q_part, 0x6504 + 16 * c);
          const float phi = __fmul_rn(delta, *reinterpret_cast<const float*>(tab + th_off));
          const float n = __fadd_rn(__fmaf_rn(phi, 0.15915494309189535f, 12582912.0f), -12582912.0f);   // nearest integer
          float r = __fmaf_rn(-n, 6.2831854820251465f, phi);
          r = __fmaf_rn(-n, -1.7484555314695172e-07f, r);
          const float sn = __sinf(r), cs = __cosf(r);
          const float k0 = __uint_as_float(__byte_perm(hi2, 0x4B000000u, 0x7440 + c)) - 8388623.0f;   // 2n - 15
          const float k1 = __uint_as_float(__byte_perm(lo2, 0x4B000000u, 0x7440 + c)) - 8388623.0f;
          const float k0r = __fmaf_rn(k0, cs, -k1 * sn), k1r = __fmaf_rn(k1, cs, k0 * sn);
          const uint4 q = *reinterpret_cast<const uint4*>(tab + q_off);
          // the rotated pair goes to fp16 like the query values; products and sums are float32
          const uint32_t kr = pack_h2(k0r, k1r);
          const unsigned short h0 = (unsigned short)(kr & 0xffffu), h1 = (unsigned short)(kr >> 16);
          const uint32_t qq[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
          for (int h = 0; h < 4; ++h) {
            asm("fma.rn.f32.f16 %0, %1, %2, %0;" : "+f"(acc[h]) : "h"((unsigned short)(qq[h] & 0xffffu)), "h"(h0));
            asm("fma.rn.f32.f16 %0, %1, %2, %0;" : "+f"(acc[h]) : "h"((unsigned short)(qq[h] >> 16)), "h"(h1));
          }
        }
      }
      const float ksc = ks * (1.0f / 15.0f);
#pragma unroll
      for (int h = 0; h < 4; ++h) sc4[h] = acc[h] * ksc;
      if (scores_out != nullptr) {
#pragma unroll
        for (int h = 0; h < 4; ++h)
          if (h < G) scores_out[((int64_t)b * a.QH + headA * G + h) * a.S + s] = sc4[h] * 0.6931471805599453f;
      }
    }
    // the head warps have taken the previous tile's scores and emptied its value tiles
    if (it > 0) tri_wait(free_bar, (uint32_t)((it - 1) & 1), failed_addr);
    my_sc[0] = sc4[0]; my_sc[32] = sc4[1]; my_sc[64] = sc4[2]; my_sc[96] = sc4[3]; my_sc[128] = vsc;
    if (valid) {
      // ---- this record's value coefficients into the head's tile ----
#pragma unroll
      for (int w = 0; w < L::W; ++w) {
        const uint32_t viw = stw[2 * (L::ARR / 4) + tid * L::W + w] & 0x3F3F3F3Fu, vpw = stw[3 * (L::ARR / 4) + tid * L::W + w];
        const uint32_t hi2 = (vpw >> 3) & 0x1E1E1E1Eu, lo2 = (vpw << 1) & 0x1E1E1E1Eu;
        const uint32_t t01 = __byte_perm(hi2, lo2, 0x5140), t23 = __byte_perm(hi2, lo2, 0x7362);
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const uint32_t idv = __byte_perm(viw, 0u, 0x4440 + c);
          // halves 0x6400 | 2n = 1024 + 2n, minus 1039: 2n - 15, exactly; odd integers up to 15 are exact in e4m3
          const uint32_t hb = __byte_perm(c < 2 ? t01 : t23, 0x64646464u, (c & 1) ? 0x4342 : 0x4140);
          const __half2 d = __hsub2(*reinterpret_cast<const __half2*>(&hb), __floats2half2_rn(1039.f, 1039.f));
          unsigned short e;
          asm("cvt.rn.satfinite.e4m3x2.f16x2 %0, %1;" : "=h"(e) : "r"(*reinterpret_cast<const uint32_t*>(&d)));
          asm volatile("st.shared.u16 [%0], %1;" :: "r"(my_tile + idv * 64), "h"(e) : "memory");
        }
      }
    }
    __syncthreads();        // the tile's scores and value entries are in place; the stage has been read
    {
      uint32_t f;
      asm volatile("ld.shared.u32 %0, [%1];" : "=r"(f) : "r"(failed_addr) : "memory");
      if (f != 0u) { broken = true; break; }
    }
    if (tid == 0 && it + L::NSTAGE < n_iter)
      tri_lanes_issue<F>(a, sb + L::OFF_STAGE + stg * L::STAGE, bar, b, s0 + 32 * L::NSTAGE, s_end);

    // ---- head warp: online softmax of its head's 32 tokens, then values ----
    const float* scr = reinterpret_cast<const float*>(smem + L::OFF_SC) + warp * 160;
    const float4 sa = *reinterpret_cast<const float4*>(scr + hq * 32 + 8 * t);
    const float4 sb4 = *reinterpret_cast<const float4*>(scr + hq * 32 + 8 * t + 4);
    const float4 va = *reinterpret_cast<const float4*>(scr + 128 + 8 * t);
    const float4 vb = *reinterpret_cast<const float4*>(scr + 128 + 8 * t + 4);
    const float sv[8] = {sa.x, sa.y, sa.z, sa.w, sb4.x, sb4.y, sb4.z, sb4.w};
    const float vv[8] = {va.x, va.y, va.z, va.w, vb.x, vb.y, vb.z, vb.w};
    float mx = fmaxf(fmaxf(fmaxf(sv[0], sv[1]), fmaxf(sv[2], sv[3])), fmaxf(fmaxf(sv[4], sv[5]), fmaxf(sv[6], sv[7])));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
    const float mn = fmaxf(m_run, mx);
    const float mref = (mn == -CUDART_INF_F) ? 0.f : mn;
    const float alpha = ex2a(m_run - mref);
    m_run = mn;
    const float alpha_o = __shfl_sync(0xffffffffu, alpha, 8 * t);      // lane 8t weighs query head t
    if (__any_sync(0xffffffffu, alpha_o != 1.0f)) {
#pragma unroll
      for (int i = 0; i < 4; ++i) { o[i][0] *= alpha_o; o[i][1] *= alpha_o; o[i][2] *= alpha_o; o[i][3] *= alpha_o; }
    }
    float psum = 0.f;
    uint32_t b0[4], b1[4];
#pragma unroll
    for (int ks = 0; ks < 4; ++ks) {
      const float p0 = ex2a(sv[2 * ks] - mref), p1 = ex2a(sv[2 * ks + 1] - mref);
      psum += p0 + p1;
      const float w0 = p0 * vv[2 * ks], w1 = p1 * vv[2 * ks + 1];
      b0[ks] = par ? pack_h2(0.f, w0) : pack_h2(w0, 0.f);
      b1[ks] = par ? pack_h2(0.f, w1) : pack_h2(w1, 0.f);
    }
    l_run = __fmaf_rn(l_run, alpha, psum);
    const uint32_t trow = sb + L::OFF_TILE + warp * 4096 + g * 64 + t * 16;
#pragma unroll
    for (int mt = 0; mt < 4; ++mt) {
      uint32_t r0[4], r1[4];
      asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(r0[0]), "=r"(r0[1]), "=r"(r0[2]), "=r"(r0[3]) : "r"(trow + mt * 1024) : "memory");
      asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(r1[0]), "=r"(r1[1]), "=r"(r1[2]), "=r"(r1[3]) : "r"(trow + mt * 1024 + 512) : "memory");
      asm volatile("st.shared.v4.u32 [%0], {%1,%1,%1,%1};" :: "r"(trow + mt * 1024), "r"(0u) : "memory");
      asm volatile("st.shared.v4.u32 [%0], {%1,%1,%1,%1};" :: "r"(trow + mt * 1024 + 512), "r"(0u) : "memory");
#pragma unroll
      for (int ks = 0; ks < 4; ++ks) {
        uint32_t af[4];
        af[0] = e4m3x2_to_h2(r0[ks] & 0xffffu);
        af[1] = e4m3x2_to_h2(r1[ks] & 0xffffu);
        af[2] = e4m3x2_to_h2(r0[ks] >> 16);
        af[3] = e4m3x2_to_h2(r1[ks] >> 16);
        mma16816_tri(o[mt], af, b0[ks], b1[ks]);
      }
    }
    __syncwarp();
    if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" :: "r"(free_bar) : "memory");
  }
  if (broken && tid == 0) {
    // copies of later tiles may still be landing in this CTA's shared memory: wait for them (bounded) before leaving
    for (int j = it + 1; j < n_iter && j < it + L::NSTAGE; ++j)
      tri_wait_raw(sb + L::OFF_BAR + 8 * (j % L::NSTAGE), (uint32_t)((j / L::NSTAGE) & 1));
  }

  l_run += __shfl_xor_sync(0xffffffffu, l_run, 1);
  l_run += __shfl_xor_sync(0xffffffffu, l_run, 2);
  const int part = split;
  if (t == 0 && par == 0 && hq < G) {
    const int64_t rowi = (int64_t)b * a.QH + warp * G + hq;
    a.part_ml[(rowi * a.num_parts + part) * 2] = m_run;
    a.part_ml[(rowi * a.num_parts + part) * 2 + 1] = l_run;
  }
  if (t < G) {
    const int64_t rowi = (int64_t)b * a.QH + warp * G + t;
    float* pa = a.part_acc + (rowi * a.num_parts + part) * 128;
#pragma unroll
    for (int mt = 0; mt < 4; ++mt) {
      *reinterpret_cast<float2*>(pa + 2 * (16 * mt + g)) = make_float2(o[mt][0], o[mt][1]);
      *reinterpret_cast<float2*>(pa + 2 * (16 * mt + g + 8)) = make_float2(o[mt][2], o[mt][3]);
    }
  }
}

int tri_status(int* host_out, int reset) {
  cudaError_t e = cudaMemcpyFromSymbol(host_out, g_tri_status, sizeof(int));
  if (e == cudaSuccess && reset) { const int z = 0; e = cudaMemcpyToSymbol(g_tri_status, &z, sizeof(int)); }
  return e == cudaSuccess ? AKV_OK : fail((int)e, "tri status: %s", cudaGetErrorString(e));
}

static void tri_plan(int B, int QH, int S, int tps_in, int* tps, int* parts, size_t* off_ml, size_t* total) {
  int tp = tps_in > 0 ? tps_in : 2048;
  if (tps_in <= 0) {     // the grid should be whole waves of 296 CTAs (two per SM): the fewest waves whose CTAs take at
                         // most 2048 tokens each, split evenly over the batch; never below 128 tokens per CTA
    const long long tokens = (long long)B * S;
    const long long waves = (tokens + 296ll * 2048 - 1) / (296ll * 2048);
    long long per_batch = (296 * waves) / (B > 0 ? B : 1);
    if (per_batch < 1) per_batch = 1;
    long long want = (S + per_batch - 1) / per_batch;
    want = (want + 31) / 32 * 32;
    if (want < 128) want = 128;
    if (want < tp) tp = (int)want;
  }
  if (tp > S) tp = S > 0 ? S : 1;
  tp = (tp + 31) / 32 * 32;
  const int splits = S > 0 ? (S + tp - 1) / tp : 1;
  *tps = tp;
  *parts = splits;
  const size_t rows = (size_t)B * QH;
  auto al = [](size_t v) { return (v + 255) & ~(size_t)255; };
  *off_ml = al(rows * (size_t)*parts * 128 * sizeof(float));
  *total = *off_ml + al(rows * (size_t)*parts * 2 * sizeof(float));
}

}  // namespace akv

using namespace akv;

AKV_EXPORT int akv_tri_encode_bits(const void* x, int x_dtype, int64_t n_rows, int64_t x_row_stride, int head_dim,
                                   int num_freqs, int coeff_bits, uint8_t* indices, void* packed, void* scales_f16,
                                   void* stream) {
  if (head_dim != 128) return fail(AKV_ERR_UNSUPPORTED, "tri encode is built for head_dim 128, got %d", head_dim);
  if (coeff_bits != 4 && coeff_bits != 8 && coeff_bits != 16)
    return fail(AKV_ERR_UNSUPPORTED, "tri encode: coeff_bits must be 4, 8 or 16, got %d", coeff_bits);
  if (n_rows < 0) return fail(AKV_ERR_ARG, "n_rows < 0");
  if (n_rows == 0) return AKV_OK;
  if (!x || !indices || !packed || !scales_f16) return fail(AKV_ERR_ARG, "akv_tri_encode: null pointer");
  if (x_dtype < AKV_F16 || x_dtype > AKV_F32) return fail(AKV_ERR_ARG, "bad x_dtype %d", x_dtype);
  const int grid = (int)((n_rows + TE_THREADS - 1) / TE_THREADS);
  cudaStream_t st = (cudaStream_t)stream;
  __half* sc = reinterpret_cast<__half*>(scales_f16);
  uint8_t* pk = reinterpret_cast<uint8_t*>(packed);
  switch (num_freqs) {
    case 8: tri_encode_kernel<8><<<grid, TE_THREADS, 0, st>>>(x, x_dtype, n_rows, x_row_stride, coeff_bits, indices, pk, sc); break;
    case 12: tri_encode_kernel<12><<<grid, TE_THREADS, 0, st>>>(x, x_dtype, n_rows, x_row_stride, coeff_bits, indices, pk, sc); break;
    case 16: tri_encode_kernel<16><<<grid, TE_THREADS, 0, st>>>(x, x_dtype, n_rows, x_row_stride, coeff_bits, indices, pk, sc); break;
    default: return fail(AKV_ERR_UNSUPPORTED, "tri encode: num_freqs must be 8, 12 or 16, got %d", num_freqs);
  }
  return check_launch("tri_encode_kernel");
}

AKV_EXPORT int akv_tri_encode(const void* x, int x_dtype, int64_t n_rows, int64_t x_row_stride, int head_dim,
                              int num_freqs, uint8_t* indices, uint8_t* packed, void* scales_f16, void* stream) {
  return akv_tri_encode_bits(x, x_dtype, n_rows, x_row_stride, head_dim, num_freqs, 4, indices, packed, scales_f16, stream);
}

// Mirror of akv_tri_decode_params in include/akv_b200.h.
struct akv_tri_decode_params {
  const void* query; int q_dtype; int64_t q_stride_batch, q_stride_head;
  const uint8_t* k_indices; const uint8_t* k_packed; const void* k_scales;
  const uint8_t* v_indices; const uint8_t* v_packed; const void* v_scales;
  int batch, seq_len, num_kv_heads, num_q_heads, head_dim, num_freqs;
  const int64_t* key_positions; int64_t key_pos_start;
  const int64_t* query_pos; int64_t query_pos_default;
  const float* theta;
  float scale;
  float* out;          // [batch, num_q_heads, head_dim] float32, or NULL with raw_out
  float* raw_out;      // [batch*num_q_heads, head_dim+2]: un-normalised (m, l, acc)
  void* workspace; size_t workspace_bytes;
  int tokens_per_split;
  void* stream;
  void* ev_kernel_start; void* ev_kernel_stop;
  float* scores_out;
  const void* block_tables; int bt_dtype; int64_t bt_stride_batch;
  int block_size; int64_t num_blocks;
  const void* context_lens; int cl_dtype;
  int coeff_bits, post_rope;
};

AKV_EXPORT size_t akv_tri_decode_workspace_bytes(int batch, int num_q_heads, int seq_len, int tokens_per_split) {
  if (batch <= 0 || num_q_heads <= 0) return 0;
  int tps, parts; size_t off_ml, total;
  tri_plan(batch, num_q_heads, seq_len, tokens_per_split, &tps, &parts, &off_ml, &total);
  return total;
}

AKV_EXPORT int akv_tri_decode_step(const akv_tri_decode_params* p) {
  if (!p) return fail(AKV_ERR_ARG, "null params");
  if (p->head_dim != 128) return fail(AKV_ERR_UNSUPPORTED, "tri decode is built for head_dim 128");
  if (p->num_freqs != 8 && p->num_freqs != 12 && p->num_freqs != 16)
    return fail(AKV_ERR_UNSUPPORTED, "tri decode: num_freqs must be 8, 12 or 16");
  if (p->batch < 0 || p->seq_len < 0 || p->num_kv_heads <= 0 || p->num_q_heads <= 0 ||
      p->num_q_heads % p->num_kv_heads)
    return fail(AKV_ERR_ARG, "tri decode: bad sizes");
  const int G = p->num_q_heads / p->num_kv_heads;
  if (G > 8) return fail(AKV_ERR_UNSUPPORTED, "tri decode: at most 8 query heads per KV head");
  const int cb = p->coeff_bits == 0 ? 4 : p->coeff_bits;
  if (cb != 4 && cb != 8 && cb != 16) return fail(AKV_ERR_UNSUPPORTED, "tri decode: coeff_bits must be 4, 8 or 16, got %d", cb);
  if (p->batch == 0) return AKV_OK;
  if (!p->query || !p->theta || (!p->out && !p->raw_out) ||
      (p->seq_len > 0 && (!p->k_indices || !p->k_packed || !p->k_scales || !p->v_indices || !p->v_packed || !p->v_scales)))
    return fail(AKV_ERR_ARG, "tri decode: null pointer");
  int tps, parts; size_t off_ml, total;
  tri_plan(p->batch, p->num_q_heads, p->seq_len, p->tokens_per_split, &tps, &parts, &off_ml, &total);
  if (!p->workspace || p->workspace_bytes < total)
    return fail(AKV_ERR_WORKSPACE, "workspace too small: need %zu bytes, got %zu", total, p->workspace_bytes);
  char* ws = reinterpret_cast<char*>(p->workspace);
  cudaStream_t st = (cudaStream_t)p->stream;
  TriArgs a{};
  a.k_idx = p->k_indices; a.k_packed = p->k_packed; a.k_scales = reinterpret_cast<const __half*>(p->k_scales);
  a.v_idx = p->v_indices; a.v_packed = p->v_packed; a.v_scales = reinterpret_cast<const __half*>(p->v_scales);
  a.B = p->batch; a.S = p->seq_len; a.KVH = p->num_kv_heads; a.QH = p->num_q_heads; a.F = p->num_freqs;
  a.query = p->query; a.q_dtype = p->q_dtype; a.q_sb = p->q_stride_batch; a.q_sh = p->q_stride_head;
  a.key_positions = p->key_positions; a.key_pos_start = p->key_pos_start;
  a.query_pos = p->query_pos; a.query_pos_default = p->query_pos_default;
  a.theta = p->theta; a.premul = p->scale * 1.4426950408889634f;
  a.tokens_per_split = tps; a.num_parts = parts;
  a.part_acc = reinterpret_cast<float*>(ws); a.part_ml = reinterpret_cast<float*>(ws + off_ml);
  a.scores_out = p->scores_out;
  if (p->block_tables != nullptr) {
    if (p->block_size <= 0 || p->num_blocks <= 0 || p->seq_len % p->block_size != 0)
      return fail(AKV_ERR_ARG, "tri decode (paged): seq_len must be block-table width x block_size, num_blocks > 0");
    if (p->key_positions != nullptr) return fail(AKV_ERR_UNSUPPORTED, "tri decode (paged): explicit key positions are not supported");
    a.block_tables = p->block_tables; a.bt_dtype = p->bt_dtype; a.bt_stride = p->bt_stride_batch;
    a.block_size = p->block_size; a.num_blocks = p->num_blocks;
  }
  a.context_lens = p->context_lens; a.cl_dtype = p->cl_dtype;
  a.post_rope = p->post_rope;
  if (p->ev_kernel_start) cudaEventRecord((cudaEvent_t)p->ev_kernel_start, st);
  if (p->seq_len > 0) {
    const int nh = p->num_kv_heads < 8 ? p->num_kv_heads : 8;
    dim3 grid((p->num_kv_heads + 7) / 8, parts, p->batch);
    cudaError_t e = cudaSuccess;
    auto al16 = [](const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15) == 0; };
    static const bool dense_tiles_only = getenv("AKV_TRI_DENSE_TILES") != nullptr;
    const bool lanes = !dense_tiles_only && cb == 4 && p->num_kv_heads == 8 && G <= 4 && al16(p->k_indices) && al16(p->k_packed) &&
                       al16(p->k_scales) && al16(p->v_indices) && al16(p->v_packed) && al16(p->v_scales) &&
                       (p->block_tables == nullptr || p->block_size % 16 == 0);
    if (lanes) {
#define AKV_TRI_L(FF)                                                                                    \
      e = cudaFuncSetAttribute(tri_decode_lanes_kernel<FF>, cudaFuncAttributeMaxDynamicSharedMemorySize,  \
                               TriLanes<FF>::BYTES);                                                      \
      if (e == cudaSuccess) tri_decode_lanes_kernel<FF><<<grid, 256, TriLanes<FF>::BYTES, st>>>(a);
      if (p->num_freqs == 8) { AKV_TRI_L(8) } else if (p->num_freqs == 12) { AKV_TRI_L(12) } else { AKV_TRI_L(16) }
#undef AKV_TRI_L
      if (e != cudaSuccess) return fail((int)e, "tri decode: smem attribute: %s", cudaGetErrorString(e));
      if (int rc = check_launch("tri_decode_lanes_kernel")) return rc;
    } else {
#define AKV_TRI(FF, CC)                                                                              \
    e = cudaFuncSetAttribute(tri_decode_kernel<FF, CC>, cudaFuncAttributeMaxDynamicSharedMemorySize,      \
                             (int)TriSmem<FF, CC>::bytes(8));                                            \
    if (e == cudaSuccess) tri_decode_kernel<FF, CC><<<grid, 32 * nh, TriSmem<FF, CC>::bytes(nh), st>>>(a);
#define AKV_TRI_F(CC)                                                                                \
    if (p->num_freqs == 8) { AKV_TRI(8, CC) } else if (p->num_freqs == 12) { AKV_TRI(12, CC) } else { AKV_TRI(16, CC) }
    if (cb == 4) { AKV_TRI_F(4) } else if (cb == 8) { AKV_TRI_F(8) } else { AKV_TRI_F(16) }
#undef AKV_TRI_F
#undef AKV_TRI
    if (e != cudaSuccess) return fail((int)e, "tri decode: smem attribute: %s", cudaGetErrorString(e));
    if (int rc = check_launch("tri_decode_kernel")) return rc;
    }
  }
  if (p->ev_kernel_stop) cudaEventRecord((cudaEvent_t)p->ev_kernel_stop, st);
  const int rows = p->batch * p->num_q_heads;
  MergeArgs mg{};
  mg.mode = p->raw_out ? MERGE_RAW : MERGE_NORMALIZE;
  mg.acc = a.part_acc; mg.acc_row = (int64_t)parts * 128; mg.acc_part = 128;
  mg.ml = a.part_ml; mg.ml_row = (int64_t)parts * 2; mg.ml_part = 2;
  mg.np = p->seq_len > 0 ? parts : 0;
  mg.context_lens = nullptr; mg.num_q_heads = p->num_q_heads;
  mg.D = 128; mg.rot = nullptr;
  mg.out = p->out; mg.out_dtype = AKV_F32; mg.out_ss = (int64_t)p->num_q_heads * 128; mg.out_sh = 128;
  mg.raw_out = p->raw_out;
  return launch_merge(mg, rows, st);
}
