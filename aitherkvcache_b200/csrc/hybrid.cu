// Hybrid split-group codec (tq35 / tq25): two dim groups, each L2-normalised,
// sign-flipped + Walsh-Hadamard transformed, quantised with a Beta-Lloyd-Max
// codebook, plus a 1-bit sketch of the quantisation residual (QJL) and two fp16
// norms - all in one byte record per vector.
//
// Reference: aither_kvcache/hybrid_quantizer.py
//   layout :52-123, FWHT :130-234, packing :310-410, encode :616-779, decode :785-933.
// Every step of the reference encode is element-wise float32, so the kernels
// reproduce its bytes exactly: same butterfly order (h = 1, 2, 4, ...), same
// 8-lane norm reduction, no FMA contraction where the reference rounds twice.
//
// Record of one vector: [g0: codes | sign bits | fp16 norm | fp16 residual norm][g1: same]
//   tq35 (d=128): 24+8+2+2 | 16+8+2+2 = 64 bytes;  tq25: 8+4+2+2 | 12+12+2+2 = 44 bytes.
#include "common.cuh"
#include "tq_prefill_args.cuh"
#include <math_constants.h>
#include <stdlib.h>

namespace akv {

struct HybridTables {
  const int* group_index;     // [num_index_heads][head_dim]: g0 dims then g1 dims
  int num_index_heads;        // rows cycle over heads when > 1 (reference :640-661)
  const float* had_signs;     // [head_dim]: g0 signs then g1 signs
  const float* qjl_signs;     // [head_dim]
  const float* centroids;     // [2][8]: group 0 then group 1, padded
  const float* boundaries;    // [2][8]: padded with +inf
  float qjl_scale0, qjl_scale1;
};

// Where row n of an encode call comes from and where its record goes.  Contiguous mode
// (slot_mapping == nullptr): rows x_stride_row elements apart, records out_stride_row bytes apart.
// Paged mode: row n is (token n / num_heads, head n % num_heads); the record goes to the cache slot
// slot_mapping[token] (block = slot / block_size, position = slot % block_size); tokens with a
// negative slot or a block >= max_blocks are skipped (vllm/hooks.py:259-296 in the reference
// writes them by index-put; a negative slot there wraps to the last block).
struct HyRowMap {
  int64_t x_stride_row, out_stride_row;
  const int64_t* slot_mapping;
  int num_heads, block_size;
  int64_t max_blocks;
  int64_t x_stride_tok, x_stride_head;
  int64_t p_stride_blk, p_stride_pos, p_stride_head;
};

__device__ __forceinline__ int64_t hy_src_off(const HyRowMap& m, int64_t n) {
  if (m.slot_mapping == nullptr) return n * m.x_stride_row;
  const int64_t tok = n / m.num_heads;
  return tok * m.x_stride_tok + (n - tok * m.num_heads) * m.x_stride_head;
}

__device__ __forceinline__ uint8_t* hy_dst(const HyRowMap& m, uint8_t* out, int64_t n) {
  if (m.slot_mapping == nullptr) return out + n * m.out_stride_row;
  const int64_t tok = n / m.num_heads;
  const int64_t slot = m.slot_mapping[tok];
  if (slot < 0) return nullptr;
  const int64_t blk = slot / m.block_size;
  if (blk >= m.max_blocks) return nullptr;
  return out + blk * m.p_stride_blk + (slot - blk * m.block_size) * m.p_stride_pos + (n - tok * m.num_heads) * m.p_stride_head;
}

static inline HyRowMap hy_contiguous(int64_t x_row_stride, int64_t out_row_stride) {
  HyRowMap m{};
  m.x_stride_row = x_row_stride; m.out_stride_row = out_row_stride;
  return m;
}


// Butterfly stages h = 1, 2, 4, ... as a compile-time recursion, so that every index is a
// constant and the array stays in registers.
template <int N, int H>
__device__ __forceinline__ void fwht_stage(float* w) {
  if constexpr (H < N) {
#pragma unroll
    for (int i = 0; i < N; i += 2 * H) {
#pragma unroll
      for (int j = 0; j < H; ++j) {
        const float a = w[i + j], b = w[i + j + H];
        w[i + j] = __fadd_rn(a, b);
        w[i + j + H] = __fsub_rn(a, b);
      }
    }
    fwht_stage<N, 2 * H>(w);
  }
}

template <int N>
__device__ __forceinline__ void fwht_pow2(float* w) { fwht_stage<N, 1>(w); }

// Block-diagonal transform for sizes that are a sum of two powers of two (96 = 64 + 32).
template <int G>
__device__ __forceinline__ void fwht(float* w) {
  if constexpr ((G & (G - 1)) == 0) {
    fwht_pow2<G>(w);
  } else {
    constexpr int P = G >= 64 ? 64 : 32;
    fwht_pow2<P>(w);
    fwht_pow2<G - P>(w + P);
  }
}

template <int G>
__device__ __forceinline__ float norm8(const float* v) {
  float s[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) s[j] = 0.f;
#pragma unroll
  for (int i = 0; i < G; ++i) s[i & 7] = __fadd_rn(s[i & 7], __fmul_rn(v[i], v[i]));
  float t = s[0];
#pragma unroll
  for (int j = 1; j < 8; ++j) t = __fadd_rn(t, s[j]);
  return __fsqrt_rn(t);
}

// MSB-first bit stream writer with compile-time positions.
template <int BITS, int G>
__device__ __forceinline__ void pack_stream(const int* codes, uint8_t* out) {
  constexpr int NBYTES = (G * BITS + 7) / 8;
#pragma unroll
  for (int b = 0; b < NBYTES; ++b) out[b] = 0;
#pragma unroll
  for (int k = 0; k < G; ++k) {
    const int pos = k * BITS, byte = pos >> 3, off = pos & 7;
    const int v16 = (codes[k] & ((1 << BITS) - 1)) << (16 - BITS - off);
    out[byte] |= (uint8_t)(v16 >> 8);
    if (off + BITS > 8) out[byte + 1] |= (uint8_t)(v16 & 0xFF);
  }
}

template <int BITS>
__device__ __forceinline__ int stream_code(const uint8_t* bytes, int k, int nbytes) {
  const int pos = k * BITS, byte = pos >> 3, off = pos & 7;
  const int hi = bytes[byte], lo = (byte + 1 < nbytes) ? bytes[byte + 1] : 0;
  return (((hi << 8) | lo) >> (16 - BITS - off)) & ((1 << BITS) - 1);
}

template <int G, int BITS>
__device__ __forceinline__ void encode_group(const float* xrow, const int* gidx, const float* had,
                                             const float* qjl, const float* cent, const float* bnd,
                                             uint8_t* out) {
  constexpr int MSE = (G * BITS + 7) / 8, QJL = (G + 7) / 8;
  const float sq = sqrtf((float)G);
  float u[G], w[G];
#pragma unroll
  for (int k = 0; k < G; ++k) u[k] = xrow[gidx[k]];
  const float n = norm8<G>(u);
  const float den = __fadd_rn(n, 1e-10f);
#pragma unroll
  for (int k = 0; k < G; ++k) {
    u[k] = __fdiv_rn(u[k], den);
    w[k] = __fmul_rn(u[k], had[k]);
  }
  fwht<G>(w);
  int codes[G];
#pragma unroll
  for (int k = 0; k < G; ++k) {
    const float r = __fdiv_rn(w[k], sq);
    int c = 0;
#pragma unroll
    for (int b = 0; b < (1 << BITS) - 1; ++b) c += (bnd[b] < r) ? 1 : 0;
    codes[k] = c;
    w[k] = cent[c];
  }
  pack_stream<BITS, G>(codes, out);
  fwht<G>(w);
#pragma unroll
  for (int k = 0; k < G; ++k)
    w[k] = __fsub_rn(u[k], __fdiv_rn(__fmul_rn(w[k], had[k]), sq));   // residual on the unit sphere
  const float rho = norm8<G>(w);
#pragma unroll
  for (int k = 0; k < G; ++k) w[k] = __fmul_rn(w[k], qjl[k]);
  fwht<G>(w);
#pragma unroll
  for (int k = 0; k < G; ++k) codes[k] = (__fdiv_rn(w[k], sq) >= 0.f) ? 1 : 0;
  pack_stream<1, G>(codes, out + MSE);
  const __half hn = __float2half_rn(n), hr = __float2half_rn(rho);
  const uint16_t bn = *reinterpret_cast<const uint16_t*>(&hn), br = *reinterpret_cast<const uint16_t*>(&hr);
  out[MSE + QJL + 0] = (uint8_t)(bn & 0xFF);
  out[MSE + QJL + 1] = (uint8_t)(bn >> 8);
  out[MSE + QJL + 2] = (uint8_t)(br & 0xFF);
  out[MSE + QJL + 3] = (uint8_t)(br >> 8);
}

constexpr int HY_THREADS = 64;   // vectors per CTA (one thread each)
constexpr int HY_LD = 129;       // row pitch of the float staging tile: bank = (tid + col) % 32

template <int G0, int B0, int G1, int B1>
__global__ void __launch_bounds__(HY_THREADS)
hybrid_encode_kernel(const void* __restrict__ x, int x_dtype, int64_t n_rows, HyRowMap map,
                     HybridTables t, uint8_t* __restrict__ out) {
  constexpr int D = G0 + G1;
  constexpr int BYTES0 = (G0 * B0 + 7) / 8 + (G0 + 7) / 8 + 4;
  constexpr int BYTES1 = (G1 * B1 + 7) / 8 + (G1 + 7) / 8 + 4;
  __shared__ float xs[HY_THREADS * HY_LD];
  __shared__ float s_had[D], s_qjl[D], s_cent[16], s_bnd[16];
  __shared__ int s_idx[D];
  const int tid = threadIdx.x;
  for (int i = tid; i < D; i += HY_THREADS) { s_had[i] = t.had_signs[i]; s_qjl[i] = t.qjl_signs[i]; }
  if (tid < 16) { s_cent[tid] = t.centroids[tid]; s_bnd[tid] = t.boundaries[tid]; }
  const int64_t row0 = (int64_t)blockIdx.x * HY_THREADS;
  // coalesced load of the CTA's rows
  for (int e = tid; e < HY_THREADS * D; e += HY_THREADS) {
    const int r = e / D, c = e % D;
    const int64_t n = row0 + r;
    xs[r * HY_LD + c] = (n < n_rows) ? load_as_float(x, x_dtype, hy_src_off(map, n) + c) : 0.f;
  }
  const int64_t n = row0 + tid;
  const int head = (t.num_index_heads > 1) ? (int)(n % t.num_index_heads) : 0;
  __syncthreads();
  // The index map can differ per head: every thread reads its own head's map from global
  // memory when there are several, the shared copy otherwise.
  const int* gidx = t.group_index + head * D;
  if (t.num_index_heads <= 1) {
    for (int i = tid; i < D; i += HY_THREADS) s_idx[i] = t.group_index[i];
    __syncthreads();
    gidx = s_idx;
  }
  if (n >= n_rows) return;
  uint8_t* dst = hy_dst(map, out, n);
  if (dst == nullptr) return;
  uint8_t rec[BYTES0 + BYTES1];
  encode_group<G0, B0>(xs + tid * HY_LD, gidx, s_had, s_qjl, s_cent, s_bnd, rec);
  encode_group<G1, B1>(xs + tid * HY_LD, gidx + G0, s_had + G0, s_qjl + G0, s_cent + 8, s_bnd + 8,
                       rec + BYTES0);
  static_assert((BYTES0 + BYTES1) % 4 == 0, "record size must be a multiple of 4");
  if ((reinterpret_cast<uintptr_t>(dst) & 3) == 0) {
#pragma unroll
    for (int wd = 0; wd < (BYTES0 + BYTES1) / 4; ++wd)
      reinterpret_cast<uint32_t*>(dst)[wd] = (uint32_t)rec[4 * wd] | ((uint32_t)rec[4 * wd + 1] << 8) |
                                             ((uint32_t)rec[4 * wd + 2] << 16) | ((uint32_t)rec[4 * wd + 3] << 24);
  } else {
#pragma unroll
    for (int b = 0; b < BYTES0 + BYTES1; ++b) dst[b] = rec[b];
  }
}

// ---------------------------------------------------------------------------
// Encode for 16-bit inputs: 128 vectors per CTA, one thread per vector, same
// arithmetic as encode_group (byte-identical records) with
//   * the rows staged once as raw 16-bit words (16-byte coalesced loads, word index
//     XOR-swizzled by row so that a warp's gathers of one coordinate hit 32 banks),
//   * the normalised vector parked in shared memory between the two uses (one live
//     G-element register array instead of two),
//   * codes and sign bits accumulated straight into big-endian 32-bit words,
//   * division by sqrt(G) done as a multiplication when sqrt(G) is a power of two
//     (exact either way), and dropped where only the sign of the quotient is used.
// ---------------------------------------------------------------------------
constexpr int HE_THREADS = 128;

template <int G> struct SqrtG {
  static constexpr bool POW2 = (G == 4 || G == 16 || G == 64 || G == 256);
};

template <int G>
__device__ __forceinline__ float div_sqrt_g(float v, float sq) {
  if constexpr (SqrtG<G>::POW2) return __fmul_rn(v, 1.0f / sq);
  else return __fdiv_rn(v, sq);
}

template <int BITS>
__device__ __forceinline__ void stream_put(uint32_t* W, int k, uint32_t c) {
  const int pos = k * BITS, j = pos >> 5, off = pos & 31;
  if (off + BITS <= 32) {
    W[j] |= c << (32 - BITS - off);
  } else {
    W[j] |= c >> (off + BITS - 32);
    W[j + 1] |= c << (64 - BITS - off);
  }
}

template <int G, int BITS, bool BF16>
__device__ __forceinline__ void encode_group16(const uint8_t* xrow, int swz, const int* gidx,
                                               const float* had, const float* qjl, const float* cent,
                                               const float* bnd, float* us, uint32_t* out_words) {
  constexpr int MSE_W = G * BITS / 32, QJL_W = G / 32;
  static_assert((G * BITS) % 32 == 0 && G % 32 == 0, "group streams must fill whole words");
  const float sq = sqrtf((float)G);
  float w[G];
#pragma unroll
  for (int k = 0; k < G; ++k) {
    const int idx = gidx[k];
    const uint16_t h = *reinterpret_cast<const uint16_t*>(xrow + ((((idx >> 1) ^ swz) << 2) | ((idx & 1) << 1)));
    w[k] = BF16 ? __uint_as_float((uint32_t)h << 16) : __half2float(__ushort_as_half(h));
  }
  const float n = norm8<G>(w);
  const float den = __fadd_rn(n, 1e-10f);
#pragma unroll
  for (int k = 0; k < G; ++k) {
    const float u = __fdiv_rn(w[k], den);
    us[k * HE_THREADS] = u;
    w[k] = __fmul_rn(u, had[k]);
  }
  fwht<G>(w);
  uint32_t W[MSE_W + QJL_W];
#pragma unroll
  for (int j = 0; j < MSE_W + QJL_W; ++j) W[j] = 0u;
#pragma unroll
  for (int k = 0; k < G; ++k) {
    const float r = div_sqrt_g<G>(w[k], sq);
    uint32_t c = 0;
#pragma unroll
    for (int b = 0; b < (1 << BITS) - 1; ++b) c += (bnd[b] < r) ? 1u : 0u;
    stream_put<BITS>(W, k, c);
    w[k] = cent[c];
  }
  fwht<G>(w);
#pragma unroll
  for (int k = 0; k < G; ++k)
    w[k] = __fsub_rn(us[k * HE_THREADS], div_sqrt_g<G>(__fmul_rn(w[k], had[k]), sq));
  const float rho = norm8<G>(w);
#pragma unroll
  for (int k = 0; k < G; ++k) w[k] = __fmul_rn(w[k], qjl[k]);
  fwht<G>(w);
#pragma unroll
  for (int k = 0; k < G; ++k) {
    // sign of w / sqrt(G): the quotient of a non-NaN w keeps w's sign (and its zero)
    const uint32_t bit = SqrtG<G>::POW2 ? ((w[k] >= 0.f) ? 1u : 0u) : ((__fdiv_rn(w[k], sq) >= 0.f) ? 1u : 0u);
    stream_put<1>(W + MSE_W, k, bit);
  }
#pragma unroll
  for (int j = 0; j < MSE_W + QJL_W; ++j) out_words[j] = __byte_perm(W[j], 0u, 0x0123);
  const uint32_t bn = __half_as_ushort(__float2half_rn(n)), br = __half_as_ushort(__float2half_rn(rho));
  out_words[MSE_W + QJL_W] = bn | (br << 16);
}

template <int G0, int B0, int G1, int B1, bool BF16>
#ifndef AKV_HE_MINB
#define AKV_HE_MINB 2
#endif
__global__ void __launch_bounds__(HE_THREADS, AKV_HE_MINB)
hybrid_encode16_kernel(const uint16_t* __restrict__ x, int64_t n_rows, HyRowMap map,
                       HybridTables t, uint8_t* __restrict__ out) {
  constexpr int D = G0 + G1;
  static_assert(D == 128, "rows are staged as 16 chunks of 16 bytes");
  constexpr int W0 = G0 * B0 / 32 + G0 / 32 + 1, W1 = G1 * B1 / 32 + G1 / 32 + 1;
  extern __shared__ __align__(16) uint8_t he_smem[];
  uint32_t* xs = reinterpret_cast<uint32_t*>(he_smem);                 // [128 rows][64 words]
  float* us = reinterpret_cast<float*>(he_smem + HE_THREADS * 256);     // [max(G0, G1)][128]
  __shared__ float s_had[D], s_qjl[D], s_cent[16], s_bnd[16];
  __shared__ int s_idx[D];
  const int tid = threadIdx.x;
  if (tid < D) { s_had[tid] = t.had_signs[tid]; s_qjl[tid] = t.qjl_signs[tid]; s_idx[tid] = t.group_index[tid]; }
  if (tid < 16) { s_cent[tid] = t.centroids[tid]; s_bnd[tid] = t.boundaries[tid]; }
  const int64_t row0 = (int64_t)blockIdx.x * HE_THREADS;
  const bool vec = (reinterpret_cast<uintptr_t>(x) & 15) == 0 &&
                   ((map.x_stride_row | map.x_stride_tok | map.x_stride_head) & 7) == 0;
#pragma unroll
  for (int i0 = 0; i0 < 16; i0 += 8) {
    uint4 v[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int e = (i0 + i) * HE_THREADS + tid, r = e >> 4, c = e & 15;
      const int64_t n = row0 + r;
      v[i] = make_uint4(0u, 0u, 0u, 0u);
      if (n < n_rows) {
        const uint16_t* src = x + hy_src_off(map, n) + c * 8;
        if (vec) {
          v[i] = *reinterpret_cast<const uint4*>(src);
        } else {
          v[i].x = src[0] | ((uint32_t)src[1] << 16); v[i].y = src[2] | ((uint32_t)src[3] << 16);
          v[i].z = src[4] | ((uint32_t)src[5] << 16); v[i].w = src[6] | ((uint32_t)src[7] << 16);
        }
      }
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int e = (i0 + i) * HE_THREADS + tid, r = e >> 4, c = e & 15;
      uint32_t* dst = xs + r * 64;
      const int sw = r & 31;
      dst[(4 * c + 0) ^ sw] = v[i].x; dst[(4 * c + 1) ^ sw] = v[i].y;
      dst[(4 * c + 2) ^ sw] = v[i].z; dst[(4 * c + 3) ^ sw] = v[i].w;
    }
  }
  __syncthreads();
  const int64_t n = row0 + tid;
  if (n >= n_rows) return;
  // The index map can differ per head: then every thread reads its own head's map from
  // global memory, the shared copy otherwise.
  const int* gidx = s_idx;
  if (t.num_index_heads > 1) gidx = t.group_index + (int)(n % t.num_index_heads) * D;
  uint32_t rec[W0 + W1];
  const uint8_t* xrow = reinterpret_cast<const uint8_t*>(xs + tid * 64);
  encode_group16<G0, B0, BF16>(xrow, tid & 31, gidx, s_had, s_qjl, s_cent, s_bnd, us + tid, rec);
  encode_group16<G1, B1, BF16>(xrow, tid & 31, gidx + G0, s_had + G0, s_qjl + G0, s_cent + 8, s_bnd + 8,
                               us + tid, rec + W0);
  uint8_t* dst = hy_dst(map, out, n);
  if (dst == nullptr) return;
  if ((reinterpret_cast<uintptr_t>(dst) & 3) == 0) {
#pragma unroll
    for (int wd = 0; wd < W0 + W1; ++wd) reinterpret_cast<uint32_t*>(dst)[wd] = rec[wd];
  } else {
#pragma unroll
    for (int b = 0; b < 4 * (W0 + W1); ++b) dst[b] = (uint8_t)(rec[b >> 2] >> (8 * (b & 3)));
  }
}

template <int G0, int B0, int G1, int B1>
static int launch_hybrid_encode16(const void* x, int x_dtype, int64_t n_rows, const HyRowMap& map,
                                  const HybridTables& t, uint8_t* out, cudaStream_t st) {
  constexpr int GMAX = G0 > G1 ? G0 : G1;
  constexpr size_t SMEM = (size_t)HE_THREADS * 256 + (size_t)GMAX * HE_THREADS * 4;
  const int grid = (int)((n_rows + HE_THREADS - 1) / HE_THREADS);
  const uint16_t* xp = reinterpret_cast<const uint16_t*>(x);
  cudaError_t e;
  if (x_dtype == AKV_BF16) {
    auto kern = hybrid_encode16_kernel<G0, B0, G1, B1, true>;
    e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM);
    if (e == cudaSuccess) kern<<<grid, HE_THREADS, SMEM, st>>>(xp, n_rows, map, t, out);
  } else {
    auto kern = hybrid_encode16_kernel<G0, B0, G1, B1, false>;
    e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM);
    if (e == cudaSuccess) kern<<<grid, HE_THREADS, SMEM, st>>>(xp, n_rows, map, t, out);
  }
  if (e != cudaSuccess) return fail((int)e, "hybrid encode: smem attribute: %s", cudaGetErrorString(e));
  return check_launch("hybrid_encode16_kernel");
}

// ---------------------------------------------------------------------------
// tq35 encode for 16-bit inputs, four lanes per vector.
//
// Same arithmetic as encode_group (byte-identical records).  A 64-coordinate group is spread over
// four lanes: lane q holds coordinates k = 8 m + 2 q + b (m = 0..7, b = 0, 1), i.e. the index bits
// 1..2 select the lane.  With that split
//   * the eight-lane norm sums (s_j over k = j mod 8, in the order m = 0..7) are complete chains
//     inside one lane (j = 2q, 2q+1); only the final fold s_0 + s_1 + ... hops over the lanes;
//   * the Walsh-Hadamard butterflies of stages h = 1, 8, 16, 32 pair registers of one lane, stages
//     h = 2, 4 pair lanes q ^ 1, q ^ 2 (one shuffle per element);
//   * every lane quantises and packs its own 16 coordinates into its bit positions of the stream
//     words, and the words are OR-reduced over the four lanes.
// Sixteen live values per lane instead of 64 per thread: small code (the thread-per-vector kernel
// stalled on instruction fetch) and enough warps per SM to hide latencies.
// ---------------------------------------------------------------------------
constexpr int HC_THREADS = 128;                 // 32 vectors per CTA
constexpr int HC_ROW_WORDS = 68;                // staged row pitch in 32-bit words (64 + 4: conflict-free gathers)

// element slot i = 2 m + b of a lane <-> coordinate k = 8 m + 2 q + b
__device__ __forceinline__ int hc_coord(int i, int q) { return 8 * (i >> 1) + 2 * q + (i & 1); }

// In-lane butterfly over the slots whose index differs in bit `bit` (slot bit 0 = coordinate bit 0,
// slot bits 1..3 = coordinate bits 3..5).
template <int BIT>
__device__ __forceinline__ void hc_stage_local(float (&w)[16]) {
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    if (!(i & (1 << BIT))) {
      const float a = w[i], b = w[i | (1 << BIT)];
      w[i] = __fadd_rn(a, b);
      w[i | (1 << BIT)] = __fsub_rn(a, b);
    }
  }
}

// Butterfly between lanes q and q ^ MASK: the lane whose bit is clear holds the lower coordinate.
template <int MASK>
__device__ __forceinline__ void hc_stage_cross(float (&w)[16], uint32_t neg_mask) {
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    const float p = __shfl_xor_sync(0xffffffffu, w[i], MASK);
    // lower lane: w + p; upper lane: p - w  (= (-w) + p, same rounding)
    w[i] = __fadd_rn(__uint_as_float(__float_as_uint(w[i]) ^ neg_mask), p);
  }
}

// 64-point transform in the reference's stage order h = 1, 2, 4, 8, 16, 32.
__device__ __forceinline__ void hc_fwht64(float (&w)[16], int q) {
  hc_stage_local<0>(w);                                          // h = 1
  hc_stage_cross<1>(w, (q & 1) ? 0x80000000u : 0u);              // h = 2
  hc_stage_cross<2>(w, (q & 2) ? 0x80000000u : 0u);              // h = 4
  hc_stage_local<1>(w);                                          // h = 8
  hc_stage_local<2>(w);                                          // h = 16
  hc_stage_local<3>(w);                                          // h = 32
}

// sqrt of the eight-lane sum of squares of the group (every lane of the quad returns it).
__device__ __forceinline__ float hc_norm(const float (&v)[16], int q, int lane) {
  float s0 = 0.f, s1 = 0.f;        // lanes j = 2q and 2q + 1 of the reference's reduction
#pragma unroll
  for (int m = 0; m < 8; ++m) {
    s0 = __fadd_rn(s0, __fmul_rn(v[2 * m], v[2 * m]));
    s1 = __fadd_rn(s1, __fmul_rn(v[2 * m + 1], v[2 * m + 1]));
  }
  // fold ((((s_0 + s_1) + s_2) + s_3) + ...) + s_7 across the quad
  float acc = __fadd_rn(s0, s1);
#pragma unroll
  for (int step = 1; step < 4; ++step) {
    const float prev = __shfl_sync(0xffffffffu, acc, (lane & ~3) + step - 1);
    if (q == step) acc = __fadd_rn(__fadd_rn(prev, s0), s1);
  }
  return __fsqrt_rn(__shfl_sync(0xffffffffu, acc, (lane & ~3) + 3));
}

// x / den for one den and many x: with r = RN(1 / den), q0 = RN(x r), rem = x - q0 den (exact, FMA),
// q1 = RN(q0 + rem r) is the correctly rounded quotient unless den's significand is all ones
// (Markstein); that case and non-finite / tiny operands take the IEEE division.
struct HcDivisor { float den, rcp; bool fast; };

__device__ __forceinline__ HcDivisor hc_divisor(float d) {
  HcDivisor v;
  v.den = d;
  v.rcp = __frcp_rn(d);
  const uint32_t bits = __float_as_uint(d);
  const uint32_t ex = (bits >> 23) & 0xffu;
  v.fast = (bits & 0x7fffffu) != 0x7fffffu && ex > 32u && ex < 222u;
  return v;
}

__device__ __forceinline__ float hc_div(const HcDivisor& v, float x) {
  if (v.fast && x != 0.f) {
    const float q0 = __fmul_rn(x, v.rcp);
    const float rem = __fmaf_rn(-q0, v.den, x);
    const float q1 = __fmaf_rn(rem, v.rcp, q0);
    // the shortcut needs a normal, finite quotient; anything unusual goes the long way
    const uint32_t qe = (__float_as_uint(q1) >> 23) & 0xffu;
    if (qe > 1u && qe < 254u) return q1;
  }
  return __fdiv_rn(x, v.den);
}

template <int BITS, bool BF16>
__device__ __forceinline__ void hc_encode_group(const uint32_t* xrow, const int* gidx, const float* had,
                                                const float* qjl, const float* cent, const float* bnd,
                                                int q, int lane, uint32_t* out_words, bool store) {
  constexpr int MSE_W = 64 * BITS / 32, QJL_W = 2, NB = (1 << BITS) - 1;
  float u[16], w[16];
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    const int idx = gidx[hc_coord(i, q)];
    const uint32_t word = xrow[idx >> 1];
    const uint32_t h = (idx & 1) ? (word >> 16) : (word & 0xffffu);
    w[i] = BF16 ? __uint_as_float(h << 16) : __half2float(__ushort_as_half((unsigned short)h));
  }
  const float n = hc_norm(w, q, lane);
  const HcDivisor dv = hc_divisor(__fadd_rn(n, 1e-10f));
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    u[i] = hc_div(dv, w[i]);
    w[i] = __fmul_rn(u[i], had[hc_coord(i, q)]);
  }
  hc_fwht64(w, q);
  uint32_t W[MSE_W + QJL_W];
#pragma unroll
  for (int j = 0; j < MSE_W + QJL_W; ++j) W[j] = 0u;
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    const float r = __fmul_rn(w[i], 0.125f);          // / sqrt(64), exact
    uint32_t c = 0;
#pragma unroll
    for (int b = 0; b < NB; ++b) c += (bnd[b] < r) ? 1u : 0u;
    // code of coordinate k goes to stream bits [k BITS, (k+1) BITS), MSB first; k depends on q at run
    // time only through the term 2 q BITS, a shift inside the 8-code (8 BITS-bit) group of slot pair m
    const int m = i >> 1, b01 = i & 1;
    // group m occupies stream bits [8 m BITS, 8 (m+1) BITS); inside it the code sits (2 q + b01) BITS from the top
    const uint32_t in_group = c << (8 * BITS - BITS - b01 * BITS);     // still to be shifted right by 2 q BITS
    const uint32_t placed = in_group >> (2 * BITS * q);                // 8 BITS-bit value
    // append the group value to the stream words (compile-time positions)
    const int pos = 8 * m * BITS, j = pos >> 5, off = pos & 31;       // group start bit
    if (off + 8 * BITS <= 32) {
      W[j] |= placed << (32 - 8 * BITS - off);
    } else {
      W[j] |= placed >> (off + 8 * BITS - 32);
      W[j + 1] |= placed << (64 - 8 * BITS - off);
    }
    w[i] = cent[c];
  }
  hc_fwht64(w, q);
#pragma unroll
  for (int i = 0; i < 16; ++i)
    w[i] = __fsub_rn(u[i], __fmul_rn(__fmul_rn(w[i], had[hc_coord(i, q)]), 0.125f));
  const float rho = hc_norm(w, q, lane);
#pragma unroll
  for (int i = 0; i < 16; ++i) w[i] = __fmul_rn(w[i], qjl[hc_coord(i, q)]);
  hc_fwht64(w, q);
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    const uint32_t bit = (w[i] >= 0.f) ? 1u : 0u;      // sign of w / 8
    const int m = i >> 1, b01 = i & 1;
    // byte m of the sign stream holds coordinates 8 m .. 8 m + 7, MSB first
    const uint32_t placed = (bit << (7 - b01)) >> (2 * q);
    W[MSE_W + (m >> 2)] |= placed << (24 - 8 * (m & 3));
  }
  // OR the four lanes' contributions, convert to the byte order of the record, spread the stores
#pragma unroll
  for (int j = 0; j < MSE_W + QJL_W; ++j) {
    W[j] |= __shfl_xor_sync(0xffffffffu, W[j], 1);
    W[j] |= __shfl_xor_sync(0xffffffffu, W[j], 2);
  }
#pragma unroll
  for (int j = 0; j < MSE_W + QJL_W; ++j)
    if (store && (j & 3) == q) out_words[j] = __byte_perm(W[j], 0u, 0x0123);
  if (store && q == 3) {
    const uint32_t bn = __half_as_ushort(__float2half_rn(n)), br = __half_as_ushort(__float2half_rn(rho));
    out_words[MSE_W + QJL_W] = bn | (br << 16);
  }
}

// Body of the tq35 four-lanes-per-vector encoder for the 32 rows starting at row0 (a CTA of HC_THREADS).
template <bool BF16>
__device__ __forceinline__ void hc_encode35_rows(const uint16_t* __restrict__ x, int64_t n_rows, int64_t row0,
                                                 const HyRowMap& map, const HybridTables& t,
                                                 uint8_t* __restrict__ out, uint32_t* xs, float* s_had, float* s_qjl,
                                                 float* s_cent, float* s_bnd, int* s_idx) {
  const int tid = threadIdx.x, lane = tid & 31;
  if (tid < 128) { s_had[tid] = t.had_signs[tid]; s_qjl[tid] = t.qjl_signs[tid]; s_idx[tid] = t.group_index[tid]; }
  if (tid < 16) { s_cent[tid] = t.centroids[tid]; s_bnd[tid] = t.boundaries[tid]; }
  // stage 32 rows: 512 pieces of 16 bytes, 4 per thread, coalesced
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int e = i * HC_THREADS + tid, r = e >> 4, c = e & 15;
    const int64_t n = row0 + r;
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (n < n_rows) v = *reinterpret_cast<const uint4*>(x + hy_src_off(map, n) + c * 8);
    *reinterpret_cast<uint4*>(xs + r * HC_ROW_WORDS + 4 * c) = v;
  }
  __syncthreads();
  const int vec = tid >> 2, q = tid & 3;
  const int64_t n = row0 + vec;
  // whole quads leave together (n is the same for the four lanes); the shuffles below name all 32
  // lanes, so a warp with some finished quads keeps them running on zeros instead
  uint8_t* rec = n < n_rows ? hy_dst(map, out, n) : nullptr;     // nullptr: past the end, or a skipped slot
  const bool live = rec != nullptr;
  const int* gidx = s_idx;
  if (t.num_index_heads > 1 && n < n_rows) gidx = t.group_index + (int)(n % t.num_index_heads) * 128;
  uint32_t* dst = reinterpret_cast<uint32_t*>(live ? rec : out);
  hc_encode_group<3, BF16>(xs + vec * HC_ROW_WORDS, gidx, s_had, s_qjl, s_cent, s_bnd, q, lane, dst, live);
  hc_encode_group<2, BF16>(xs + vec * HC_ROW_WORDS, gidx + 64, s_had + 64, s_qjl + 64, s_cent + 8, s_bnd + 8, q, lane,
                           dst + 9, live);
}

template <bool BF16>
__global__ void __launch_bounds__(HC_THREADS, 4)
hybrid_encode35_coop_kernel(const uint16_t* __restrict__ x, int64_t n_rows, HyRowMap map,
                            HybridTables t, uint8_t* __restrict__ out) {
  __shared__ __align__(16) uint32_t xs[32 * HC_ROW_WORDS];
  __shared__ float s_had[128], s_qjl[128], s_cent[16], s_bnd[16];
  __shared__ int s_idx[128];
  hc_encode35_rows<BF16>(x, n_rows, (int64_t)blockIdx.x * 32, map, t, out, xs, s_had, s_qjl, s_cent, s_bnd, s_idx);
}

// ---------------------------------------------------------------------------
// tq35 decode, four lanes per vector (same lane <-> coordinate split as the encoder above):
// records staged in shared memory, codes and sign bits picked out of the big-endian stream
// words, two 64-point transforms per group (centroids, signs), the reference's float32
// arithmetic step for step (bit-identical output), results staged and written as whole rows.
// ---------------------------------------------------------------------------
template <int BITS>
__device__ __forceinline__ void hc_decode_group(const uint32_t* rec /* this group's words, staged */,
                                                const int* gidx, const float* had, const float* qjl,
                                                const float* cent, float qjl_scale, int q, float* orow) {
  constexpr int MSE_W = 64 * BITS / 32;
  uint32_t W[MSE_W + 2];
#pragma unroll
  for (int j = 0; j < MSE_W + 2; ++j) W[j] = __byte_perm(rec[j], 0u, 0x0123);    // big-endian stream words
  const uint32_t sc = rec[MSE_W + 2];
  const float n = __half2float(__ushort_as_half((unsigned short)(sc & 0xffffu)));
  const float rho = __half2float(__ushort_as_half((unsigned short)(sc >> 16)));
  float a[16], b[16];
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    const int m = i >> 1, b01 = i & 1;
    // 8-code group m: stream bits [8 m BITS, 8 (m+1) BITS)
    const int pos = 8 * m * BITS, j = pos >> 5, off = pos & 31;
    uint32_t grp;
    if (off + 8 * BITS <= 32) grp = W[j] >> (32 - 8 * BITS - off);
    else grp = __funnelshift_l(W[j + 1], W[j], off + 8 * BITS - 32);
    const uint32_t code = (grp >> (BITS * (7 - b01) - 2 * BITS * q)) & ((1u << BITS) - 1u);
    a[i] = cent[code];
    const uint32_t byte = (W[MSE_W + (m >> 2)] >> (24 - 8 * (m & 3))) & 0xffu;
    const uint32_t bit = (byte >> (7 - b01 - 2 * q)) & 1u;
    b[i] = __fmul_rn(bit ? 1.f : -1.f, qjl_scale);
  }
  hc_fwht64(a, q);
  hc_fwht64(b, q);
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    const int k = hc_coord(i, q);
    const float mse_hat = __fmul_rn(__fmul_rn(a[i], had[k]), 0.125f);     // / sqrt(64), exact
    const float qjl_hat = __fmul_rn(__fmul_rn(b[i], qjl[k]), 0.125f);
    orow[gidx[k]] = __fmul_rn(__fadd_rn(mse_hat, __fmul_rn(qjl_hat, rho)), n);
  }
}

constexpr int HD_ROW = 132;       // staged output row pitch in floats (128 + 4: quads of a warp hit distinct banks)

__global__ void __launch_bounds__(HC_THREADS, 4)
hybrid_decode35_coop_kernel(const uint8_t* __restrict__ packed, int64_t p_row_stride, int64_t n_rows,
                            HybridTables t, void* __restrict__ out, int out_dtype) {
  __shared__ uint32_t recs[32 * 17];                // 16 words per record, pitch 17
  __shared__ __align__(16) float outs[32 * HD_ROW];
  __shared__ float s_had[128], s_qjl[128], s_cent[16];
  __shared__ int s_idx[128];
  const int tid = threadIdx.x;
  if (tid < 128) { s_had[tid] = t.had_signs[tid]; s_qjl[tid] = t.qjl_signs[tid]; s_idx[tid] = t.group_index[tid]; }
  if (tid < 16) s_cent[tid] = t.centroids[tid];
  const int64_t row0 = (int64_t)blockIdx.x * 32;
  {   // 32 records x 16 words, one 16-byte piece per thread
    const int r = tid >> 2, c = tid & 3;
    const int64_t n = row0 + r;
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (n < n_rows) v = *reinterpret_cast<const uint4*>(packed + n * p_row_stride + c * 16);
    uint32_t* d = recs + r * 17 + 4 * c;
    d[0] = v.x; d[1] = v.y; d[2] = v.z; d[3] = v.w;
  }
  __syncthreads();
  const int vec = tid >> 2, q = tid & 3;
  const int64_t n = row0 + vec;
  const int* gidx = s_idx;
  if (t.num_index_heads > 1 && n < n_rows) gidx = t.group_index + (int)(n % t.num_index_heads) * 128;
  hc_decode_group<3>(recs + vec * 17, gidx, s_had, s_qjl, s_cent, t.qjl_scale0, q, outs + vec * HD_ROW);
  hc_decode_group<2>(recs + vec * 17 + 9, gidx + 64, s_had + 64, s_qjl + 64, s_cent + 8, t.qjl_scale1, q,
                     outs + vec * HD_ROW);
  __syncthreads();
  // 32 rows x 128 values, coalesced
  for (int e = tid; e < 32 * 32; e += HC_THREADS) {
    const int r = e >> 5, c4 = (e & 31) * 4;
    const int64_t nn = row0 + r;
    if (nn >= n_rows) continue;
    const float4 v = *reinterpret_cast<const float4*>(outs + r * HD_ROW + c4);
    if (out_dtype == AKV_F32) {
      *reinterpret_cast<float4*>(reinterpret_cast<float*>(out) + nn * 128 + c4) = v;
    } else {
      uint2 h;
      if (out_dtype == AKV_F16) {
        __half2 lo = __floats2half2_rn(v.x, v.y), hi = __floats2half2_rn(v.z, v.w);
        h = make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
      } else {
        __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
        h = make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
      }
      *reinterpret_cast<uint2*>(reinterpret_cast<uint16_t*>(out) + nn * 128 + c4) = h;
    }
  }
}

static int launch_hybrid_encode35_coop(const void* x, int x_dtype, int64_t n_rows, const HyRowMap& map,
                                       const HybridTables& t, uint8_t* out, cudaStream_t st) {
  const int grid = (int)((n_rows + 31) / 32);
  const uint16_t* xp = reinterpret_cast<const uint16_t*>(x);
  if (x_dtype == AKV_BF16)
    hybrid_encode35_coop_kernel<true><<<grid, HC_THREADS, 0, st>>>(xp, n_rows, map, t, out);
  else
    hybrid_encode35_coop_kernel<false><<<grid, HC_THREADS, 0, st>>>(xp, n_rows, map, t, out);
  return check_launch("hybrid_encode35_coop_kernel");
}

template <int G, int BITS>
__device__ __forceinline__ void decode_group(const uint8_t* rec, const int* gidx, const float* had,
                                             const float* qjl, const float* cent, float qjl_scale,
                                             float* orow) {
  constexpr int MSE = (G * BITS + 7) / 8, QJL = (G + 7) / 8;
  const float sq = sqrtf((float)G);
  float a[G], b[G];
#pragma unroll
  for (int k = 0; k < G; ++k) {
    a[k] = cent[stream_code<BITS>(rec, k, MSE)];
    const int bit = (rec[MSE + (k >> 3)] >> (7 - (k & 7))) & 1;
    b[k] = __fmul_rn(bit ? 1.f : -1.f, qjl_scale);
  }
  fwht<G>(a);
  fwht<G>(b);
  const uint16_t bn = (uint16_t)rec[MSE + QJL] | ((uint16_t)rec[MSE + QJL + 1] << 8);
  const uint16_t br = (uint16_t)rec[MSE + QJL + 2] | ((uint16_t)rec[MSE + QJL + 3] << 8);
  const float n = __half2float(*reinterpret_cast<const __half*>(&bn));
  const float rho = __half2float(*reinterpret_cast<const __half*>(&br));
#pragma unroll
  for (int k = 0; k < G; ++k) {
    const float mse_hat = __fdiv_rn(__fmul_rn(a[k], had[k]), sq);
    const float qjl_hat = __fdiv_rn(__fmul_rn(b[k], qjl[k]), sq);
    orow[gidx[k]] = __fmul_rn(__fadd_rn(mse_hat, __fmul_rn(qjl_hat, rho)), n);
  }
}

template <int G0, int B0, int G1, int B1>
__global__ void __launch_bounds__(HY_THREADS)
hybrid_decode_kernel(const uint8_t* __restrict__ packed, int64_t p_row_stride, int64_t n_rows,
                     HybridTables t, void* __restrict__ out, int out_dtype) {
  constexpr int D = G0 + G1;
  constexpr int BYTES0 = (G0 * B0 + 7) / 8 + (G0 + 7) / 8 + 4;
  constexpr int BYTES1 = (G1 * B1 + 7) / 8 + (G1 + 7) / 8 + 4;
  __shared__ float xs[HY_THREADS * HY_LD];
  __shared__ float s_had[D], s_qjl[D], s_cent[16];
  __shared__ int s_idx[D];
  const int tid = threadIdx.x;
  for (int i = tid; i < D; i += HY_THREADS) { s_had[i] = t.had_signs[i]; s_qjl[i] = t.qjl_signs[i]; }
  if (tid < 16) s_cent[tid] = t.centroids[tid];
  if (t.num_index_heads <= 1)
    for (int i = tid; i < D; i += HY_THREADS) s_idx[i] = t.group_index[i];
  __syncthreads();
  const int64_t row0 = (int64_t)blockIdx.x * HY_THREADS;
  const int64_t n = row0 + tid;
  if (n < n_rows) {
    const int head = (t.num_index_heads > 1) ? (int)(n % t.num_index_heads) : 0;
    const int* gidx = (t.num_index_heads > 1) ? t.group_index + head * D : s_idx;
    uint8_t rec[BYTES0 + BYTES1];
    const uint8_t* src = packed + n * p_row_stride;
    if ((reinterpret_cast<uintptr_t>(src) & 3) == 0) {
#pragma unroll
      for (int wd = 0; wd < (BYTES0 + BYTES1) / 4; ++wd) {
        const uint32_t v = reinterpret_cast<const uint32_t*>(src)[wd];
        rec[4 * wd] = (uint8_t)v; rec[4 * wd + 1] = (uint8_t)(v >> 8);
        rec[4 * wd + 2] = (uint8_t)(v >> 16); rec[4 * wd + 3] = (uint8_t)(v >> 24);
      }
    } else {
#pragma unroll
      for (int b = 0; b < BYTES0 + BYTES1; ++b) rec[b] = src[b];
    }
    decode_group<G0, B0>(rec, gidx, s_had, s_qjl, s_cent, t.qjl_scale0, xs + tid * HY_LD);
    decode_group<G1, B1>(rec + BYTES0, gidx + G0, s_had + G0, s_qjl + G0, s_cent + 8, t.qjl_scale1,
                         xs + tid * HY_LD);
  }
  __syncthreads();
  for (int e = tid; e < HY_THREADS * D; e += HY_THREADS) {
    const int r = e / D, c = e % D;
    const int64_t nn = row0 + r;
    if (nn < n_rows) store_from_float(out, out_dtype, nn * D + c, xs[r * HY_LD + c]);
  }
}

// ---------------------------------------------------------------------------
// Paged decode attention over tq35 records (head_dim 128, uniform dim split).
//
// With q'_g = FWHT(q_g . s_g) / sqrt(G) (the Hadamard matrix is symmetric) the score of a
// token is   scale * sum_g n_g [ q'_had,g . c_g[idx] + rho_g kappa_g (q'_qjl,g . sigma) ]
// and the value sum can be accumulated in the same transformed coordinates:
//   A_g = sum_t w_t n_g c_g[idx_t],  B_g = sum_t w_t n_g rho_g kappa_g sigma_t,
//   out_g = ( FWHT(A_g) . s_had + FWHT(B_g) . s_qjl ) / sqrt(G)        (epilogue kernel)
// so no K/V vector is ever reconstructed.  "Virtual" coordinate order used below:
//   [c0: 64 | sigma0: 64 | c1: 64 | sigma1: 64] = 256 per (token, head).
//
// The reference has no kernel for this (vllm/hooks.py:297-345 decodes every block and
// calls dense SDPA); this is a scalar first version: warp per (seq, kv head, part), lane
// l owns dims 2l, 2l+1 of each of the four segments.
// ---------------------------------------------------------------------------
__device__ int g_hybrid_window_status;   // 1: hybrid_attn_mma_kernel found its shared window taken and returned

struct HybridAttnArgs {
  const uint8_t* k_cache; const uint8_t* v_cache;
  int64_t k_sb, k_sp, k_sh, v_sb, v_sp, v_sh;   // bytes
  const void* block_tables; int bt_dtype; int64_t bt_stride;
  const void* context_lens; int cl_dtype;
  int num_q_heads, num_kv_heads, block_size, max_blocks_per_seq;
  int64_t num_blocks;
  int blocks_per_split, num_parts;
  const float* qprime;     // [S][QH][256], scale*log2e and kappa folded in
  const float* centroids;  // [2][8]
  float* part_acc;         // [S][QH][NP][256]
  float* part_ml;          // [S][QH][NP][2]
};

constexpr int HA_WARPS = 4;

struct HyVals { float c0a, c0b, s0a, s0b, c1a, c1b, s1a, s1b, n0, r0, n1, r1; };

__device__ __forceinline__ HyVals hy_load(const uint8_t* rec, int lane, const float* cent) {
  HyVals v;
  // group 0 codes: 3 bits each, dims 2l and 2l+1 -> stream bits [6l, 6l+6)
  {
    const int pos = 6 * lane, byte = pos >> 3, off = pos & 7;
    const int hi = rec[byte], lo = (byte + 1 < 24) ? rec[byte + 1] : 0;
    const int six = (((hi << 8) | lo) >> (10 - off)) & 63;
    v.c0a = cent[six >> 3];
    v.c0b = cent[six & 7];
  }
  {
    const int two = (rec[24 + (lane >> 2)] >> (6 - 2 * (lane & 3))) & 3;
    v.s0a = (two & 2) ? 1.f : -1.f;
    v.s0b = (two & 1) ? 1.f : -1.f;
  }
  {
    const int four = (rec[36 + (lane >> 1)] >> (4 - 4 * (lane & 1))) & 15;
    v.c1a = cent[8 + (four >> 2)];
    v.c1b = cent[8 + (four & 3)];
  }
  {
    const int two = (rec[52 + (lane >> 2)] >> (6 - 2 * (lane & 3))) & 3;
    v.s1a = (two & 2) ? 1.f : -1.f;
    v.s1b = (two & 1) ? 1.f : -1.f;
  }
  const __half2 n0 = *reinterpret_cast<const __half2*>(rec + 32);
  const __half2 n1 = *reinterpret_cast<const __half2*>(rec + 60);
  v.n0 = __low2float(n0); v.r0 = __high2float(n0);
  v.n1 = __low2float(n1); v.r1 = __high2float(n1);
  return v;
}

__global__ void __launch_bounds__(HA_WARPS * 32)
hybrid_attn_kernel(HybridAttnArgs a) {
  const int split = blockIdx.x, h = blockIdx.y, seq = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int G = a.num_q_heads / a.num_kv_heads;
  const int64_t ctx = load_ctx(a.context_lens, a.cl_dtype, seq, (int64_t)a.max_blocks_per_seq * a.block_size);
  const int bs = a.block_size;
  const int64_t nblk = (ctx + bs - 1) / bs;
  const int64_t blk_begin = (int64_t)split * a.blocks_per_split;
  if (blk_begin >= nblk) return;
  const int64_t blk_end = (blk_begin + a.blocks_per_split < nblk) ? blk_begin + a.blocks_per_split : nblk;
  __shared__ float cent[16];
  if (threadIdx.x < 16) cent[threadIdx.x] = a.centroids[threadIdx.x];
  __syncthreads();
  const int part = split * HA_WARPS + warp;

  for (int g0 = 0; g0 < G; g0 += 4) {
    const int ng = (G - g0 < 4) ? G - g0 : 4;
    float q[4][8], acc[4][8], m[4], l[4];
#pragma unroll
    for (int gi = 0; gi < 4; ++gi) {
      m[gi] = -CUDART_INF_F; l[gi] = 0.f;
      const float* qp = a.qprime + ((int64_t)seq * a.num_q_heads + h * G + g0 + (gi < ng ? gi : 0)) * 256;
#pragma unroll
      for (int s = 0; s < 4; ++s) {
        q[gi][2 * s] = (gi < ng) ? qp[64 * s + 2 * lane] : 0.f;
        q[gi][2 * s + 1] = (gi < ng) ? qp[64 * s + 2 * lane + 1] : 0.f;
      }
#pragma unroll
      for (int k = 0; k < 8; ++k) acc[gi][k] = 0.f;
    }
    for (int64_t blk = blk_begin + warp; blk < blk_end; blk += HA_WARPS) {
      int64_t pb = load_index(a.block_tables, a.bt_dtype, (int64_t)seq * a.bt_stride + blk);
      if (pb < 0) pb = 0;
      if (pb >= a.num_blocks) pb = a.num_blocks - 1;
      const int ntok = (int)((ctx - blk * bs < bs) ? ctx - blk * bs : bs);
      for (int t = 0; t < ntok; ++t) {
        const HyVals k = hy_load(a.k_cache + pb * a.k_sb + t * a.k_sp + h * a.k_sh, lane, cent);
        const HyVals v = hy_load(a.v_cache + pb * a.v_sb + t * a.v_sp + h * a.v_sh, lane, cent);
        const float kw0 = k.n0, kw1 = k.n0 * k.r0, kw2 = k.n1, kw3 = k.n1 * k.r1;
        const float vw0 = v.n0, vw1 = v.n0 * v.r0, vw2 = v.n1, vw3 = v.n1 * v.r1;
        const float vv[8] = {v.c0a * vw0, v.c0b * vw0, v.s0a * vw1, v.s0b * vw1,
                             v.c1a * vw2, v.c1b * vw2, v.s1a * vw3, v.s1b * vw3};
#pragma unroll
        for (int gi = 0; gi < 4; ++gi) {
          if (gi >= ng) continue;
          float d = kw0 * (q[gi][0] * k.c0a + q[gi][1] * k.c0b) + kw1 * (q[gi][2] * k.s0a + q[gi][3] * k.s0b) +
                    kw2 * (q[gi][4] * k.c1a + q[gi][5] * k.c1b) + kw3 * (q[gi][6] * k.s1a + q[gi][7] * k.s1b);
#pragma unroll
          for (int o = 16; o > 0; o >>= 1) d += __shfl_xor_sync(0xffffffffu, d, o);
          const float mn = fmaxf(m[gi], d);
          const float alpha = exp2f(m[gi] - mn);
          const float p = exp2f(d - mn);
          l[gi] = l[gi] * alpha + p;
#pragma unroll
          for (int kk = 0; kk < 8; ++kk) acc[gi][kk] = __fmaf_rn(p, vv[kk], acc[gi][kk] * alpha);
          m[gi] = mn;
        }
      }
    }
    for (int gi = 0; gi < ng; ++gi) {
      const int64_t row = (int64_t)seq * a.num_q_heads + h * G + g0 + gi;
      float* pa = a.part_acc + (row * a.num_parts + part) * 256;
#pragma unroll
      for (int s = 0; s < 4; ++s) {
        pa[64 * s + 2 * lane] = acc[gi][2 * s];
        pa[64 * s + 2 * lane + 1] = acc[gi][2 * s + 1];
      }
      if (lane == 0) {
        a.part_ml[(row * a.num_parts + part) * 2] = m[gi];
        a.part_ml[(row * a.num_parts + part) * 2 + 1] = l[gi];
      }
    }
  }
}

// ---------------------------------------------------------------------------
// The same computation for tq25 records (44 bytes: group 0 = 32 coordinates with 2-bit codes, group 1 = 96
// coordinates with 1-bit codes, a sign bit per coordinate in both).  The 256 virtual coordinates are
//   [0, 32) group-0 centroids, [32, 64) group-0 signs, [64, 160) group-1 centroids, [160, 256) group-1 signs;
// a lane holds coordinate `lane` of the first two segments and `lane`, `lane + 32`, `lane + 64` of the others.
// ---------------------------------------------------------------------------
struct Hy25Vals { float c0, s0, c1[3], s1[3], n0, r0, n1, r1; };

__device__ __forceinline__ Hy25Vals hy25_load(const uint8_t* rec, int lane, const float* cent) {
  Hy25Vals v;
  v.c0 = cent[(rec[lane >> 2] >> (6 - 2 * (lane & 3))) & 3];
  v.s0 = ((rec[8 + (lane >> 3)] >> (7 - (lane & 7))) & 1) ? 1.f : -1.f;
#pragma unroll
  for (int j = 0; j < 3; ++j) {
    const int d = lane + 32 * j;
    v.c1[j] = cent[8 + ((rec[16 + (d >> 3)] >> (7 - (d & 7))) & 1)];
    v.s1[j] = ((rec[28 + (d >> 3)] >> (7 - (d & 7))) & 1) ? 1.f : -1.f;
  }
  const __half2 n0 = *reinterpret_cast<const __half2*>(rec + 12);
  const __half2 n1 = *reinterpret_cast<const __half2*>(rec + 40);
  v.n0 = __low2float(n0); v.r0 = __high2float(n0);
  v.n1 = __low2float(n1); v.r1 = __high2float(n1);
  return v;
}

// virtual coordinate of a lane's slot k (0..7)
__device__ __forceinline__ int hy25_coord(int k, int lane) {
  return k == 0 ? lane : k == 1 ? 32 + lane : k < 5 ? 64 + lane + 32 * (k - 2) : 160 + lane + 32 * (k - 5);
}

__global__ void __launch_bounds__(HA_WARPS * 32)
hybrid_attn25_kernel(HybridAttnArgs a) {
  const int split = blockIdx.x, h = blockIdx.y, seq = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int G = a.num_q_heads / a.num_kv_heads;
  const int64_t ctx = load_ctx(a.context_lens, a.cl_dtype, seq, (int64_t)a.max_blocks_per_seq * a.block_size);
  const int bs = a.block_size;
  const int64_t nblk = (ctx + bs - 1) / bs;
  const int64_t blk_begin = (int64_t)split * a.blocks_per_split;
  if (blk_begin >= nblk) return;
  const int64_t blk_end = (blk_begin + a.blocks_per_split < nblk) ? blk_begin + a.blocks_per_split : nblk;
  __shared__ float cent[16];
  if (threadIdx.x < 16) cent[threadIdx.x] = a.centroids[threadIdx.x];
  __syncthreads();
  const int part = split * HA_WARPS + warp;

  for (int g0 = 0; g0 < G; g0 += 4) {
    const int ng = (G - g0 < 4) ? G - g0 : 4;
    float q[4][8], acc[4][8], m[4], l[4];
#pragma unroll
    for (int gi = 0; gi < 4; ++gi) {
      m[gi] = -CUDART_INF_F; l[gi] = 0.f;
      const float* qp = a.qprime + ((int64_t)seq * a.num_q_heads + h * G + g0 + (gi < ng ? gi : 0)) * 256;
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        q[gi][k] = (gi < ng) ? qp[hy25_coord(k, lane)] : 0.f;
        acc[gi][k] = 0.f;
      }
    }
    for (int64_t blk = blk_begin + warp; blk < blk_end; blk += HA_WARPS) {
      int64_t pb = load_index(a.block_tables, a.bt_dtype, (int64_t)seq * a.bt_stride + blk);
      if (pb < 0) pb = 0;
      if (pb >= a.num_blocks) pb = a.num_blocks - 1;
      const int ntok = (int)((ctx - blk * bs < bs) ? ctx - blk * bs : bs);
      for (int t = 0; t < ntok; ++t) {
        const Hy25Vals k = hy25_load(a.k_cache + pb * a.k_sb + t * a.k_sp + h * a.k_sh, lane, cent);
        const Hy25Vals v = hy25_load(a.v_cache + pb * a.v_sb + t * a.v_sp + h * a.v_sh, lane, cent);
        const float kw0 = k.n0, kw1 = k.n0 * k.r0, kw2 = k.n1, kw3 = k.n1 * k.r1;
        const float vw0 = v.n0, vw1 = v.n0 * v.r0, vw2 = v.n1, vw3 = v.n1 * v.r1;
        const float vv[8] = {v.c0 * vw0, v.s0 * vw1, v.c1[0] * vw2, v.c1[1] * vw2, v.c1[2] * vw2,
                             v.s1[0] * vw3, v.s1[1] * vw3, v.s1[2] * vw3};
#pragma unroll
        for (int gi = 0; gi < 4; ++gi) {
          if (gi >= ng) continue;
          float d = kw0 * (q[gi][0] * k.c0) + kw1 * (q[gi][1] * k.s0) +
                    kw2 * (q[gi][2] * k.c1[0] + q[gi][3] * k.c1[1] + q[gi][4] * k.c1[2]) +
                    kw3 * (q[gi][5] * k.s1[0] + q[gi][6] * k.s1[1] + q[gi][7] * k.s1[2]);
#pragma unroll
          for (int o = 16; o > 0; o >>= 1) d += __shfl_xor_sync(0xffffffffu, d, o);
          const float mn = fmaxf(m[gi], d);
          const float alpha = exp2f(m[gi] - mn);
          const float p = exp2f(d - mn);
          l[gi] = l[gi] * alpha + p;
#pragma unroll
          for (int kk = 0; kk < 8; ++kk) acc[gi][kk] = __fmaf_rn(p, vv[kk], acc[gi][kk] * alpha);
          m[gi] = mn;
        }
      }
    }
    for (int gi = 0; gi < ng; ++gi) {
      const int64_t row = (int64_t)seq * a.num_q_heads + h * G + g0 + gi;
      float* pa = a.part_acc + (row * a.num_parts + part) * 256;
#pragma unroll
      for (int k = 0; k < 8; ++k) pa[hy25_coord(k, lane)] = acc[gi][k];
      if (lane == 0) {
        a.part_ml[(row * a.num_parts + part) * 2] = m[gi];
        a.part_ml[(row * a.num_parts + part) * 2 + 1] = l[gi];
      }
    }
  }
}

// ---------------------------------------------------------------------------
// Tensor-core version of the same computation (same grid, same partials).
//
// A warp owns one part (one KV head, every HA_WARPS-th 16-token tile of the split) and all
// query heads of the head's GQA group (up to 8).  Per tile it copies the 16 K records and the
// 16 V records (2 KB) into its own double-buffered staging area with 16-byte cp.async (chunk
// q of token r is stored at chunk q ^ ((r >> 1) & 3), which spreads the fragment reads over
// the banks), then:
//   scores  S^T[16 tokens][8 q heads] = sum over the four segments of w_seg(token) * (A_seg q'_seg),
//           A_seg = 16 x 64 fp16 operand decoded from the record: centroid pairs through
//           per-lane lookup tables (3-bit: 6-bit pair index, 2-bit: whole byte -> 4 values),
//           sign nibbles through a 16-entry table of +-1 pairs; mma.sync m16n8k16, fp32 accumulate;
//   values  O^T[256 virtual dims][8 q heads] += V_seg^T (P . w_seg)^T with the softmax weights
//           scaled per segment and token, transposed by movmatrix.
// Thread (g, t) of the warp (g = lane / 4, t = lane % 4) decodes, for the scores, coordinates
// 16t..16t+15 of every segment of tokens g and g + 8; for the values, coordinates 8g..8g+7 of
// every segment of tokens 2t, 2t+1, 2t+8, 2t+9.
// ---------------------------------------------------------------------------
// Absolute shared-window addresses (a CTA's dynamic shared memory starts a little above 1 KB; the
// kernel checks).  Fixed addresses let every table lookup do without an address add: the 3-bit and
// the sign table are aligned to their size, so their base is OR-ed into the lane offset once, and
// the 2-bit table's base rides in the load instruction as an immediate.
constexpr uint32_t HM_LUT2 = 4096;               // 256 entries x 256 B: byte of four 2-bit codes -> 4 halves
constexpr uint32_t HM_LUT3 = 73728;              // 64 entries x 128 B (8 KB aligned): two 3-bit codes -> 2 halves
constexpr uint32_t HM_LUTS = 81920;              // 16 entries x 256 B (4 KB aligned): four sign bits -> 4 halves
constexpr uint32_t HM_STAGE = 86016;             // per warp: 2 buffers x (1 KB K + 1 KB V)
constexpr int HM_SMEM = HM_STAGE + HA_WARPS * 4096;   // 102400: covers every address above for any start >= 0

__device__ __forceinline__ uint32_t hm_lds32(uint32_t addr) {
  uint32_t v;
  asm volatile("ld.shared.u32 %0, [%1];\n" : "=r"(v) : "r"(addr));
  return v;
}
__device__ __forceinline__ uint32_t hm_lds16(uint32_t addr) {
  uint16_t v;
  asm volatile("ld.shared.u16 %0, [%1];\n" : "=h"(v) : "r"(addr));
  return v;
}
__device__ __forceinline__ uint32_t hm_lds8(uint32_t addr) {
  uint32_t v;
  asm volatile("ld.shared.u8 %0, [%1];\n" : "=r"(v) : "r"(addr));
  return v;
}
__device__ __forceinline__ uint2 hm_lds64(uint32_t addr) {
  uint2 v;
  asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];\n" : "=r"(v.x), "=r"(v.y) : "r"(addr));
  return v;
}
template <uint32_t C>
__device__ __forceinline__ uint32_t hm_lds32c(uint32_t r) {
  uint32_t v;
  asm volatile("ld.shared.u32 %0, [%1+%2];\n" : "=r"(v) : "r"(r), "n"(C));
  return v;
}
template <uint32_t C>
__device__ __forceinline__ uint32_t hm_lds16c(uint32_t r) {
  uint16_t v;
  asm volatile("ld.shared.u16 %0, [%1+%2];\n" : "=h"(v) : "r"(r), "n"(C));
  return v;
}
template <uint32_t C>
__device__ __forceinline__ uint32_t hm_lds8c(uint32_t r) {
  uint32_t v;
  asm volatile("ld.shared.u8 %0, [%1+%2];\n" : "=r"(v) : "r"(r), "n"(C));
  return v;
}
template <uint32_t C>
__device__ __forceinline__ uint2 hm_lds64c(uint32_t r) {
  uint2 v;
  asm volatile("ld.shared.v2.u32 {%0,%1}, [%2+%3];\n" : "=r"(v.x), "=r"(v.y) : "r"(r), "n"(C));
  return v;
}
__device__ __forceinline__ float2 hm_half2_bits(uint32_t u) {
  const __half2 h = *reinterpret_cast<const __half2*>(&u);
  return make_float2(__low2float(h), __high2float(h));
}
__device__ __forceinline__ void hm_mma(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                       uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t hm_trans(uint32_t x) {
  uint32_t y;
  asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;\n" : "=r"(y) : "r"(x));
  return y;
}
__device__ __forceinline__ uint32_t hm_pack(float lo, float hi) {
  __half2 h = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&h);
}
__device__ __forceinline__ float hm_ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// Pair P of an MSB-first 3-bit stream whose first 32 bits are B (P <= 4) -> half2 of two centroids.
template <int P>
__device__ __forceinline__ uint32_t hm_pair3(uint32_t lut3, uint32_t B, uint32_t lane4) {
  static_assert(6 * P <= 26, "pair must lie in the first word");
  return hm_lds32(lut3 + ((((B >> (26 - 6 * P)) & 63u) << 7) | lane4));
}
// Sign nibble (already shifted to bits 8..11 of x) -> two half2 of +-1.
__device__ __forceinline__ uint2 hm_signs(uint32_t luts, uint32_t x, uint32_t lane8) {
  return hm_lds64(luts + ((x & 0xF00u) | lane8));
}
// Byte K of w (four 2-bit codes) -> two half2 of centroids.
template <int K>
__device__ __forceinline__ uint2 hm_quad2(uint32_t w, uint32_t lane8) {
  return hm_lds64c<HM_LUT2>(__byte_perm(w, lane8, 0x7604 + (K << 4)));
}

// PAR (at most four query heads per KV head): the eight MMA columns of the value products are (query head, parity of
// the coordinate), so a table entry (two neighbouring coordinates of one token) is a complete A register and the
// accumulators halve; score columns 4..7 repeat heads 0..3 so that every column finds its weights.
template <bool PAR>
__global__ void __launch_bounds__(HA_WARPS * 32, 2)
hybrid_attn_mma_kernel(HybridAttnArgs a) {
  extern __shared__ __align__(16) unsigned char hm_smem[];
  const int split = blockIdx.x, h = blockIdx.y, seq = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int G = a.num_q_heads / a.num_kv_heads;
  const int64_t ctx = load_ctx(a.context_lens, a.cl_dtype, seq, (int64_t)a.max_blocks_per_seq * a.block_size);
  const int tpb = a.block_size / 16;
  const int64_t tiles_total = (ctx + 15) / 16;
  const int64_t tile_begin = (int64_t)split * a.blocks_per_split * tpb;
  if (tile_begin >= tiles_total) return;   // uniform for the CTA
  int64_t tile_end = tile_begin + (int64_t)a.blocks_per_split * tpb;
  if (tile_end > tiles_total) tile_end = tiles_total;

  const uint32_t dyn0 = (uint32_t)__cvta_generic_to_shared(hm_smem);
  if (dyn0 > HM_LUT2) {        // the window below the tables is taken (static + system-reserved bytes)
    if (threadIdx.x == 0) g_hybrid_window_status = 1;   // the host checks the window before launching
    return;
  }
  unsigned char* const abs0 = hm_smem - dyn0;     // generic pointer to shared-window address 0
  // ---- lookup tables, one copy per lane ----
  const float* c0 = a.centroids;        // 8 centroids of group 0 (3-bit)
  const float* c1 = a.centroids + 8;    // 4 centroids of group 1 (2-bit)
  for (int i = threadIdx.x; i < 256 * 32; i += blockDim.x) {
    const int e = i >> 5, l = i & 31;
    *reinterpret_cast<uint2*>(abs0 + HM_LUT2 + e * 256 + l * 8) =
        make_uint2(hm_pack(c1[e >> 6], c1[(e >> 4) & 3]), hm_pack(c1[(e >> 2) & 3], c1[e & 3]));
  }
  for (int i = threadIdx.x; i < 64 * 32; i += blockDim.x) {
    const int e = i >> 5, l = i & 31;
    *reinterpret_cast<uint32_t*>(abs0 + HM_LUT3 + e * 128 + l * 4) = hm_pack(c0[e >> 3], c0[e & 7]);
  }
  for (int i = threadIdx.x; i < 16 * 32; i += blockDim.x) {
    const int e = i >> 5, l = i & 31;
    *reinterpret_cast<uint2*>(abs0 + HM_LUTS + e * 256 + l * 8) =
        make_uint2(hm_pack((e & 8) ? 1.f : -1.f, (e & 4) ? 1.f : -1.f),
                   hm_pack((e & 2) ? 1.f : -1.f, (e & 1) ? 1.f : -1.f));
  }
  __syncthreads();

  constexpr uint32_t lut3 = 0, luts = 0;           // bases are folded into the lane offsets below
  const uint32_t stage_s = HM_STAGE + warp * 4096;
  const uint32_t lane4 = HM_LUT3 | (lane * 4);     // 3-bit table lookups: (pair << 7) | lane4
  const uint32_t lane8s = HM_LUTS | (lane * 8);    // sign table lookups: (nibble << 8) | lane8s
  const uint32_t lane8 = lane * 8;                 // 2-bit table lookups: base as load immediate

  // ---- query fragments: thread (g, t) holds q'[q head g][segment][16t .. 16t+15] ----
  uint32_t bq[4][4][2];
  {
    const int qcol = PAR ? (g & 3) : g;        // query head of score column g
    const float* qp = a.qprime + ((int64_t)seq * a.num_q_heads + h * G + (qcol < G ? qcol : 0)) * 256 + 16 * t;
#pragma unroll
    for (int sg = 0; sg < 4; ++sg)
#pragma unroll
      for (int kk = 0; kk < 4; ++kk) {
        float4 f = *reinterpret_cast<const float4*>(qp + 64 * sg + 4 * kk);
        if (qcol >= G) f = make_float4(0.f, 0.f, 0.f, 0.f);
        bq[sg][kk][0] = hm_pack(f.x, f.y);
        bq[sg][kk][1] = hm_pack(f.z, f.w);
      }
  }

  // ---- per-thread byte offsets inside a staged record ----
  // logical byte b of token r lives at r*64 + (((b >> 4) ^ ((r >> 1) & 3)) << 4) + (b & 15)
  const uint32_t sK = (g >> 1) & 3;     // tokens g, g + 8
  const uint32_t sV = t;                // tokens 2t, 2t+1, 2t+8, 2t+9
  auto swz = [](uint32_t b, uint32_t sw) { return (((b >> 4) ^ sw) << 4) | (b & 15u); };
  const uint32_t kRow = g * 64;
  const uint32_t kw0 = 4 * ((6 * t) >> 2);
  const uint32_t oK0a = kRow + swz(kw0, sK), oK0b = kRow + swz(kw0 + 4, sK);
  const uint32_t oKs0 = kRow + swz(24 + 2 * t, sK), oKn0 = kRow + swz(32, sK);
  const uint32_t oKc1 = kRow + swz(36 + 4 * t, sK), oKs1 = kRow + swz(52 + 2 * t, sK), oKn1 = kRow + swz(60, sK);
  // 48 stream bits start at byte 6t: at byte 0 (t even) or byte 2 (t odd) of the two words read
  const uint32_t selK0 = (t & 1) ? 0x2345u : 0x0123u, selK1 = (t & 1) ? 0x6700u : 0x4500u;
  const uint32_t vRow = 1024 + 2 * t * 64;
  const uint32_t vw0 = 4 * ((3 * g) >> 2), vo = (3 * g) & 3;
  const uint32_t oV0a = vRow + swz(vw0, sV), oV0b = vRow + swz(vw0 + 4, sV);
  const uint32_t oVs0 = vRow + swz(24 + g, sV), oVc1 = vRow + swz(36 + 2 * g, sV), oVs1 = vRow + swz(52 + g, sV);
  const uint32_t selV0 = (vo << 12) | ((vo + 1) << 8) | ((vo + 2) << 4) | (vo + 3);

  constexpr int NT = PAR ? 2 : 4;        // accumulator tiles per segment
  float o[4][NT][4];
#pragma unroll
  for (int sg = 0; sg < 4; ++sg)
#pragma unroll
    for (int j = 0; j < NT; ++j) { o[sg][j][0] = o[sg][j][1] = o[sg][j][2] = o[sg][j][3] = 0.f; }
  // PAR: B operand of a value product from the transposed weights x = (P[token 2t], P[token 2t+1]) of column g's head:
  // the weight goes into the half that matches the column's parity, the other half is zero
  const uint32_t selA = (g >> 2) ? 0x1044u : 0x4410u, selB = (g >> 2) ? 0x3244u : 0x4432u;
  auto value_mmas = [&](float (&acc)[NT][4], const uint32_t (&n)[4][4], uint32_t pa_, uint32_t pb_) {
    if constexpr (PAR) {
      // rows g / g+8 of tile mt are coordinate pairs 4g + 2mt / 4g + 2mt + 1; k-step 0 holds tokens 2t, 2t+1, k-step 1 tokens 2t+8, 2t+9
#pragma unroll
      for (int mt = 0; mt < 2; ++mt) {
        hm_mma(acc[mt], n[0][2 * mt], n[0][2 * mt + 1], n[1][2 * mt], n[1][2 * mt + 1],
               __byte_perm(pa_, 0u, selA), __byte_perm(pa_, 0u, selB));
        hm_mma(acc[mt], n[2][2 * mt], n[2][2 * mt + 1], n[3][2 * mt], n[3][2 * mt + 1],
               __byte_perm(pb_, 0u, selA), __byte_perm(pb_, 0u, selB));
      }
    } else {
      // M-tile j pairs the same coordinate of two tokens: rows g / g+8 of the tile are coordinates 8g+2j / 8g+2j+1
#pragma unroll
      for (int j = 0; j < 4; ++j)
        hm_mma(acc[j], __byte_perm(n[0][j], n[1][j], 0x5410), __byte_perm(n[0][j], n[1][j], 0x7632),
               __byte_perm(n[2][j], n[3][j], 0x5410), __byte_perm(n[2][j], n[3][j], 0x7632), pa_, pb_);
    }
  };
  float m0 = -CUDART_INF_F, m1 = -CUDART_INF_F, l0 = 0.f, l1 = 0.f;

  const int64_t first = tile_begin + warp;
  const int n_tiles = first < tile_end ? (int)((tile_end - first + HA_WARPS - 1) / HA_WARPS) : 0;

  auto issue = [&](int i) {     // copy tile i of this warp into buffer i & 1
    const int64_t tile = first + (int64_t)i * HA_WARPS;
    int64_t pb = load_index(a.block_tables, a.bt_dtype, (int64_t)seq * a.bt_stride + tile / tpb);
    if (pb < 0) pb = 0;
    if (pb >= a.num_blocks) pb = a.num_blocks - 1;
    const int pos0 = (int)(tile % tpb) * 16;
    const uint32_t dst0 = stage_s + (uint32_t)(i & 1) * 2048;
#pragma unroll
    for (int r2 = 0; r2 < 2; ++r2) {
      const int c = lane + 32 * r2, tok = c >> 2, q = c & 3;
      const uint32_t d = dst0 + tok * 64 + ((q ^ ((tok >> 1) & 3)) << 4);
      const uint8_t* ks = a.k_cache + pb * a.k_sb + (int64_t)(pos0 + tok) * a.k_sp + h * a.k_sh + q * 16;
      const uint8_t* vs = a.v_cache + pb * a.v_sb + (int64_t)(pos0 + tok) * a.v_sp + h * a.v_sh + q * 16;
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" :: "r"(d), "l"(ks) : "memory");
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" :: "r"(d + 1024), "l"(vs) : "memory");
    }
  };

  if (n_tiles > 0) issue(0);
  asm volatile("cp.async.commit_group;\n" ::: "memory");
#pragma unroll 1
  for (int i = 0; i < n_tiles; ++i) {
    if (i + 1 < n_tiles) issue(i + 1);
    asm volatile("cp.async.commit_group;\n" ::: "memory");
    asm volatile("cp.async.wait_group 1;\n" ::: "memory");
    __syncwarp();
    const uint32_t buf = stage_s + (uint32_t)(i & 1) * 2048;
    // this tile's load bases; every further displacement is an immediate of the load
    const uint32_t pK0a = buf + oK0a, pK0b = buf + oK0b, pKs0 = buf + oKs0, pKs1 = buf + oKs1;
    const uint32_t pKn0 = buf + oKn0, pKn1 = buf + oKn1, pKc1 = buf + oKc1;
    const uint32_t pV0a = buf + oV0a, pV0b = buf + oV0b, pVs0 = buf + oVs0, pVs1 = buf + oVs1, pVc1 = buf + oVc1;
    const int64_t tile = first + (int64_t)i * HA_WARPS;
    const int64_t rem = ctx - tile * 16;
    const int n_valid = rem < 16 ? (int)rem : 16;

    // ================= scores =================
    float sc[4][4];
#pragma unroll
    for (int sg = 0; sg < 4; ++sg) sc[sg][0] = sc[sg][1] = sc[sg][2] = sc[sg][3] = 0.f;
    {   // segment 0: 3-bit codes
      const uint32_t a0 = hm_lds32c<0>(pK0a), a1 = hm_lds32c<0>(pK0b);
      const uint32_t b0 = hm_lds32c<512>(pK0a), b1 = hm_lds32c<512>(pK0b);
      const uint32_t A0 = __byte_perm(a0, a1, selK0), A1 = __byte_perm(a0, a1, selK1);
      const uint32_t B0 = __byte_perm(b0, b1, selK0), B1 = __byte_perm(b0, b1, selK1);
      uint32_t na[8], nb[8];
      na[0] = hm_pair3<0>(lut3, A0, lane4); na[1] = hm_pair3<1>(lut3, A0, lane4);
      na[2] = hm_pair3<2>(lut3, A0, lane4); na[3] = hm_pair3<3>(lut3, A0, lane4);
      na[4] = hm_pair3<4>(lut3, A0, lane4);
      nb[0] = hm_pair3<0>(lut3, B0, lane4); nb[1] = hm_pair3<1>(lut3, B0, lane4);
      nb[2] = hm_pair3<2>(lut3, B0, lane4); nb[3] = hm_pair3<3>(lut3, B0, lane4);
      nb[4] = hm_pair3<4>(lut3, B0, lane4);
      // pair 5 = stream bits 30..35 straddles the words; pairs 6, 7 sit in the second word
      na[5] = hm_lds32(lut3 + (((__funnelshift_l(A1, A0, 4) & 63u) << 7) | lane4));
      nb[5] = hm_lds32(lut3 + (((__funnelshift_l(B1, B0, 4) & 63u) << 7) | lane4));
      na[6] = hm_lds32(lut3 + ((((A1 >> 22) & 63u) << 7) | lane4));
      nb[6] = hm_lds32(lut3 + ((((B1 >> 22) & 63u) << 7) | lane4));
      na[7] = hm_lds32(lut3 + ((((A1 >> 16) & 63u) << 7) | lane4));
      nb[7] = hm_lds32(lut3 + ((((B1 >> 16) & 63u) << 7) | lane4));
#pragma unroll
      for (int kk = 0; kk < 4; ++kk)
        hm_mma(sc[0], na[2 * kk], nb[2 * kk], na[2 * kk + 1], nb[2 * kk + 1], bq[0][kk][0], bq[0][kk][1]);
    }
#pragma unroll
    for (int sgn = 0; sgn < 2; ++sgn) {   // segments 1 and 3: sign bits
      const uint32_t va = hm_lds16c<0>(sgn ? pKs1 : pKs0), vb = hm_lds16c<512>(sgn ? pKs1 : pKs0);
      const uint2 a0 = hm_signs(luts, va << 4, lane8s), a1 = hm_signs(luts, va << 8, lane8s);
      const uint2 a2 = hm_signs(luts, va >> 4, lane8s), a3 = hm_signs(luts, va, lane8s);
      const uint2 b0 = hm_signs(luts, vb << 4, lane8s), b1 = hm_signs(luts, vb << 8, lane8s);
      const uint2 b2 = hm_signs(luts, vb >> 4, lane8s), b3 = hm_signs(luts, vb, lane8s);
      const int sg = 1 + 2 * sgn;
      hm_mma(sc[sg], a0.x, b0.x, a0.y, b0.y, bq[sg][0][0], bq[sg][0][1]);
      hm_mma(sc[sg], a1.x, b1.x, a1.y, b1.y, bq[sg][1][0], bq[sg][1][1]);
      hm_mma(sc[sg], a2.x, b2.x, a2.y, b2.y, bq[sg][2][0], bq[sg][2][1]);
      hm_mma(sc[sg], a3.x, b3.x, a3.y, b3.y, bq[sg][3][0], bq[sg][3][1]);
    }
    {   // segment 2: 2-bit codes, one byte per k-tile
      const uint32_t wa = hm_lds32c<0>(pKc1), wb = hm_lds32c<512>(pKc1);
      const uint2 a0 = hm_quad2<0>(wa, lane8), a1 = hm_quad2<1>(wa, lane8);
      const uint2 a2 = hm_quad2<2>(wa, lane8), a3 = hm_quad2<3>(wa, lane8);
      const uint2 b0 = hm_quad2<0>(wb, lane8), b1 = hm_quad2<1>(wb, lane8);
      const uint2 b2 = hm_quad2<2>(wb, lane8), b3 = hm_quad2<3>(wb, lane8);
      hm_mma(sc[2], a0.x, b0.x, a0.y, b0.y, bq[2][0][0], bq[2][0][1]);
      hm_mma(sc[2], a1.x, b1.x, a1.y, b1.y, bq[2][1][0], bq[2][1][1]);
      hm_mma(sc[2], a2.x, b2.x, a2.y, b2.y, bq[2][2][0], bq[2][2][1]);
      hm_mma(sc[2], a3.x, b3.x, a3.y, b3.y, bq[2][3][0], bq[2][3][1]);
    }
    float s0, s1, s2, s3;
    {
      const float2 kA0 = hm_half2_bits(hm_lds32c<0>(pKn0)), kA1 = hm_half2_bits(hm_lds32c<0>(pKn1));
      const float2 kB0 = hm_half2_bits(hm_lds32c<512>(pKn0)), kB1 = hm_half2_bits(hm_lds32c<512>(pKn1));
      const float nA0 = kA0.x, rA0 = nA0 * kA0.y;
      const float nA1 = kA1.x, rA1 = nA1 * kA1.y;
      const float nB0 = kB0.x, rB0 = nB0 * kB0.y;
      const float nB1 = kB1.x, rB1 = nB1 * kB1.y;
      s0 = nA0 * sc[0][0] + rA0 * sc[1][0] + nA1 * sc[2][0] + rA1 * sc[3][0];
      s1 = nA0 * sc[0][1] + rA0 * sc[1][1] + nA1 * sc[2][1] + rA1 * sc[3][1];
      s2 = nB0 * sc[0][2] + rB0 * sc[1][2] + nB1 * sc[2][2] + rB1 * sc[3][2];
      s3 = nB0 * sc[0][3] + rB0 * sc[1][3] + nB1 * sc[2][3] + rB1 * sc[3][3];
    }
    // value-side segment weights of tokens g and g + 8 (same staged layout, V half)
    float wA[4], wB[4];
    {
      const float2 vA0 = hm_half2_bits(hm_lds32c<1024>(pKn0)), vA1 = hm_half2_bits(hm_lds32c<1024>(pKn1));
      const float2 vB0 = hm_half2_bits(hm_lds32c<1536>(pKn0)), vB1 = hm_half2_bits(hm_lds32c<1536>(pKn1));
      wA[0] = vA0.x; wA[1] = wA[0] * vA0.y;
      wA[2] = vA1.x; wA[3] = wA[2] * vA1.y;
      wB[0] = vB0.x; wB[1] = wB[0] * vB0.y;
      wB[2] = vB1.x; wB[3] = wB[2] * vB1.y;
    }
    if (n_valid < 16) {   // warp-uniform: only the last tile of a sequence
      if (g >= n_valid) { s0 = -CUDART_INF_F; s1 = -CUDART_INF_F; wA[0] = wA[1] = wA[2] = wA[3] = 0.f; }
      if (g + 8 >= n_valid) { s2 = -CUDART_INF_F; s3 = -CUDART_INF_F; wB[0] = wB[1] = wB[2] = wB[3] = 0.f; }
    }

    // ================= online softmax (log2 units) =================
    float mx0 = fmaxf(s0, s2), mx1 = fmaxf(s1, s3);
#pragma unroll
    for (int off = 4; off < 32; off <<= 1) {
      mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, off));
      mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, off));
    }
    const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
    if (__any_sync(0xffffffffu, (mn0 != m0) | (mn1 != m1))) {
      const float al0 = hm_ex2(m0 - mn0), al1 = hm_ex2(m1 - mn1);
      l0 *= al0; l1 *= al1;
#pragma unroll
      for (int sg = 0; sg < 4; ++sg)
#pragma unroll
        for (int j = 0; j < NT; ++j) { o[sg][j][0] *= al0; o[sg][j][1] *= al1; o[sg][j][2] *= al0; o[sg][j][3] *= al1; }
      m0 = mn0; m1 = mn1;
    }
    const float p0 = hm_ex2(s0 - mn0), p1 = hm_ex2(s1 - mn1), p2 = hm_ex2(s2 - mn0), p3 = hm_ex2(s3 - mn1);
    l0 += p0 + p2;
    l1 += p1 + p3;
    uint32_t pbA[4], pbB[4];
#pragma unroll
    for (int sg = 0; sg < 4; ++sg) {
      pbA[sg] = hm_trans(hm_pack(p0 * wA[sg], p1 * wA[sg]));
      pbB[sg] = hm_trans(hm_pack(p2 * wB[sg], p3 * wB[sg]));
    }

    // ================= values =================
    // n[tok][j] = half2(coordinate 8g+2j, 8g+2j+1) of token tok; M-tile j pairs the same
    // coordinate of two tokens: rows g / g+8 of the tile are coordinates 8g+2j / 8g+2j+1.
    // token k of the thread's four (2t, 2t+1, 2t+8, 2t+9) sits RO bytes after the first one
#define HM_FOUR_TOKENS(F) F(0, 0) F(1, 64) F(2, 512) F(3, 576)
    {   // segment 0
      uint32_t n[4][4];
#define HM_V0(K, RO)                                                                                  \
      {                                                                                               \
        const uint32_t B = __byte_perm(hm_lds32c<RO>(pV0a), hm_lds32c<RO>(pV0b), selV0);              \
        n[K][0] = hm_pair3<0>(lut3, B, lane4); n[K][1] = hm_pair3<1>(lut3, B, lane4);                 \
        n[K][2] = hm_pair3<2>(lut3, B, lane4); n[K][3] = hm_pair3<3>(lut3, B, lane4);                 \
      }
      HM_FOUR_TOKENS(HM_V0)
#undef HM_V0
      value_mmas(o[0], n, pbA[0], pbB[0]);
    }
#pragma unroll
    for (int sgn = 0; sgn < 2; ++sgn) {   // segments 1 and 3
      const int sg = 1 + 2 * sgn;
      const uint32_t pVs = sgn ? pVs1 : pVs0;
      uint32_t n[4][4];
#define HM_VS(K, RO)                                                                                  \
      {                                                                                               \
        const uint32_t v = hm_lds8c<RO>(pVs);                                                         \
        const uint2 hi = hm_signs(luts, v << 4, lane8s), lo = hm_signs(luts, v << 8, lane8s);         \
        n[K][0] = hi.x; n[K][1] = hi.y; n[K][2] = lo.x; n[K][3] = lo.y;                               \
      }
      HM_FOUR_TOKENS(HM_VS)
#undef HM_VS
      value_mmas(o[sg], n, pbA[sg], pbB[sg]);
    }
    {   // segment 2
      uint32_t n[4][4];
#define HM_V2(K, RO)                                                                                  \
      {                                                                                               \
        const uint32_t v = hm_lds16c<RO>(pVc1);                                                       \
        const uint2 q0 = hm_quad2<0>(v, lane8), q1 = hm_quad2<1>(v, lane8);                           \
        n[K][0] = q0.x; n[K][1] = q0.y; n[K][2] = q1.x; n[K][3] = q1.y;                               \
      }
      HM_FOUR_TOKENS(HM_V2)
#undef HM_V2
#undef HM_FOUR_TOKENS
      value_mmas(o[2], n, pbA[2], pbB[2]);
    }
    __syncwarp();   // every lane is done with this buffer before the copy after next lands in it
  }
  asm volatile("cp.async.wait_group 0;\n" ::: "memory");

  // ---- this warp's partial ----
#pragma unroll
  for (int offs = 4; offs < 32; offs <<= 1) {
    l0 += __shfl_xor_sync(0xffffffffu, l0, offs);
    l1 += __shfl_xor_sync(0xffffffffu, l1, offs);
  }
  const int part = split * HA_WARPS + warp;
  if constexpr (PAR) {
    // accumulator columns 2t, 2t+1 are query heads 2 (t & 1), 2 (t & 1) + 1 at coordinate parity t >> 1
    const int par = t >> 1;
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      const int qg = 2 * (t & 1) + e;
      if (qg >= G) continue;
      const int64_t row = (int64_t)seq * a.num_q_heads + h * G + qg;
      float* pa = a.part_acc + (row * a.num_parts + part) * 256;
#pragma unroll
      for (int sg = 0; sg < 4; ++sg)
#pragma unroll
        for (int mt = 0; mt < 2; ++mt) {
          pa[64 * sg + 8 * g + 4 * mt + par] = o[sg][mt][e];
          pa[64 * sg + 8 * g + 4 * mt + 2 + par] = o[sg][mt][2 + e];
        }
      if (g == 0 && t < 2) {
        a.part_ml[(row * a.num_parts + part) * 2] = e ? m1 : m0;
        a.part_ml[(row * a.num_parts + part) * 2 + 1] = e ? l1 : l0;
      }
    }
    return;
  }
#pragma unroll
  for (int e = 0; e < 2; ++e) {
    const int qg = 2 * t + e;
    if (qg >= G) continue;
    const int64_t row = (int64_t)seq * a.num_q_heads + h * G + qg;
    float* pa = a.part_acc + (row * a.num_parts + part) * 256;
#pragma unroll
    for (int sg = 0; sg < 4; ++sg)
#pragma unroll
      for (int j = 0; j < NT; ++j)
        *reinterpret_cast<float2*>(pa + 64 * sg + 8 * g + 2 * j) = make_float2(o[sg][j][e], o[sg][j][2 + e]);
    if (g == 0) {
      a.part_ml[(row * a.num_parts + part) * 2] = e ? m1 : m0;
      a.part_ml[(row * a.num_parts + part) * 2 + 1] = e ? l1 : l0;
    }
  }
}

// q'[s][qh] = [FWHT(q_g0.s_had0)/8 | kappa0 FWHT(q_g0.s_qjl0)/8 | same for g1] * premul.
// One warp per (seq, q head); 64-point transforms via shared memory.
__device__ __forceinline__ void fwht64_smem(float* w, int lane) {
  for (int h = 1; h < 64; h <<= 1) {
    __syncwarp();
    const int j = ((lane & ~(h - 1)) << 1) | (lane & (h - 1));   // lower index of the lane's butterfly
    const float a = w[j], b = w[j + h];
    __syncwarp();
    w[j] = a + b;
    w[j + h] = a - b;
  }
  __syncwarp();
}

__device__ __forceinline__ void hybrid_qprime_row(const void* __restrict__ q, int q_dtype, int64_t q_ss, int64_t q_sh,
                                                  int num_q_heads, const HybridTables& t, float premul,
                                                  float* __restrict__ qprime, int row, int lane, float (*w)[64]) {
  const int seq = row / num_q_heads, qh = row % num_q_heads;
  for (int k = lane; k < 64; k += 32) {
    const float a = load_as_float(q, q_dtype, seq * q_ss + qh * q_sh + t.group_index[k]);
    const float b = load_as_float(q, q_dtype, seq * q_ss + qh * q_sh + t.group_index[64 + k]);
    w[0][k] = a * t.had_signs[k];
    w[1][k] = a * t.qjl_signs[k];
    w[2][k] = b * t.had_signs[64 + k];
    w[3][k] = b * t.qjl_signs[64 + k];
  }
  for (int s = 0; s < 4; ++s) fwht64_smem(w[s], lane);
  for (int k = lane; k < 64; k += 32) {
    float* o = qprime + (int64_t)row * 256;
    o[k] = w[0][k] * 0.125f * premul;
    o[64 + k] = w[1][k] * 0.125f * premul * t.qjl_scale0;
    o[128 + k] = w[2][k] * 0.125f * premul;
    o[192 + k] = w[3][k] * 0.125f * premul * t.qjl_scale1;
  }
}

__global__ void __launch_bounds__(32)
hybrid_qprime_kernel(const void* __restrict__ q, int q_dtype, int64_t q_ss, int64_t q_sh, int num_q_heads,
                     HybridTables t, float premul, float* __restrict__ qprime) {
  __shared__ float w[4][64];
  hybrid_qprime_row(q, q_dtype, q_ss, q_sh, num_q_heads, t, premul, qprime, blockIdx.x, threadIdx.x, w);
}

// In-place Walsh-Hadamard transform of n = 32 or 64 shared floats by one warp (stages h = 1, 2, 4, ...).
__device__ __forceinline__ void fwht_warp_smem(float* w, int n, int lane) {
  for (int h = 1; h < n; h <<= 1) {
    __syncwarp();
    for (int l = lane; l < n / 2; l += 32) {
      const int j = ((l & ~(h - 1)) << 1) | (l & (h - 1));
      const float x = w[j], y = w[j + h];
      w[j] = x + y;
      w[j + h] = x - y;
    }
  }
  __syncwarp();
}

// The transforms of the 256 virtual coordinates of tq25: blocks of 32, 32, 64 + 32 (the 96-coordinate group is
// block diagonal, hybrid_quantizer.py:130-193) and again 64 + 32.
__device__ __forceinline__ void hy25_transforms(float* w, int warp, int nwarps, int lane) {
  const int off[6] = {0, 32, 64, 128, 160, 224}, len[6] = {32, 32, 64, 32, 64, 32};
  for (int b = warp; b < 6; b += nwarps) fwht_warp_smem(w + off[b], len[b], lane);
}

// Query side of tq25 attention: q'(virtual) = transform(q gathered by group, times the sign vectors) / sqrt(group size),
// scale * log2(e) and the sketch factor kappa folded in.  One warp per (sequence, query head).
__global__ void __launch_bounds__(32)
hybrid_qprime25_kernel(const void* __restrict__ q, int q_dtype, int64_t q_ss, int64_t q_sh, int num_q_heads,
                       HybridTables t, float premul, float* __restrict__ qprime) {
  __shared__ float w[256];
  const int row = blockIdx.x, lane = threadIdx.x;
  const int seq = row / num_q_heads, qh = row % num_q_heads;
  {
    const float a = load_as_float(q, q_dtype, seq * q_ss + qh * q_sh + t.group_index[lane]);
    w[lane] = a * t.had_signs[lane];
    w[32 + lane] = a * t.qjl_signs[lane];
  }
  for (int k = lane; k < 96; k += 32) {
    const float b = load_as_float(q, q_dtype, seq * q_ss + qh * q_sh + t.group_index[32 + k]);
    w[64 + k] = b * t.had_signs[32 + k];
    w[160 + k] = b * t.qjl_signs[32 + k];
  }
  __syncwarp();
  hy25_transforms(w, 0, 1, lane);
  const float r0 = 0.17677669529663687f * premul, r1 = 0.10206207261596577f * premul;     // 1/sqrt(32), 1/sqrt(96)
  float* o = qprime + (int64_t)row * 256;
  o[lane] = w[lane] * r0;
  o[32 + lane] = w[32 + lane] * r0 * t.qjl_scale0;
  for (int k = lane; k < 96; k += 32) {
    o[64 + k] = w[64 + k] * r1;
    o[160 + k] = w[160 + k] * r1 * t.qjl_scale1;
  }
}

// The new token's K and V vectors of a serving step (16-bit, rows readable in 16-byte pieces), written
// into the paged record cache by extra blocks of the query-transform launch.
struct HyStepWrite {
  const uint16_t* xk; const uint16_t* xv;
  HyRowMap mk, mv;
  uint8_t* ck; uint8_t* cv;
  int64_t n_rows;          // vectors per side (tokens x KV heads); 0: nothing to write
};

// First launch of a serving step: blocks [0, q_blocks) transform four query rows each (one warp per
// row), the blocks after them encode 32 K vectors each, then 32 V vectors each.
template <bool BF16>
__global__ void __launch_bounds__(HC_THREADS, 4)
hybrid_step_prologue_kernel(const void* __restrict__ q, int q_dtype, int64_t q_ss, int64_t q_sh, int num_q_heads,
                            HybridTables t, float premul, float* __restrict__ qprime, int rows, int q_blocks,
                            HyStepWrite wr) {
  __shared__ __align__(16) uint32_t xs[32 * HC_ROW_WORDS];
  __shared__ float s_had[128], s_qjl[128], s_cent[16], s_bnd[16];
  __shared__ int s_idx[128];
  if ((int)blockIdx.x >= q_blocks) {
    const int e = (int)blockIdx.x - q_blocks, nb = (int)((wr.n_rows + 31) / 32);
    const bool is_v = e >= nb;
    hc_encode35_rows<BF16>(is_v ? wr.xv : wr.xk, wr.n_rows, (int64_t)(is_v ? e - nb : e) * 32, is_v ? wr.mv : wr.mk, t,
                           is_v ? wr.cv : wr.ck, xs, s_had, s_qjl, s_cent, s_bnd, s_idx);
    return;
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row = (int)blockIdx.x * 4 + warp;
  float (*w)[64] = reinterpret_cast<float (*)[64]>(reinterpret_cast<float*>(xs) + warp * 256);   // 4 x 64 floats per warp
  if (row < rows) hybrid_qprime_row(q, q_dtype, q_ss, q_sh, num_q_heads, t, premul, qprime, row, lane, w);
}

// LSE merge of the 256-coordinate partials and the inverse transforms of the epilogue.
// One CTA of 256 threads per (sequence, query head): thread c owns coordinate c, so every
// read of a partial is one coalesced 1 KB row; the weights 2^(m_p - M) are computed once
// per part (256 parts at a time) and shared.
__device__ __forceinline__ float block_reduce_256(float v, bool is_max, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float u = __shfl_xor_sync(0xffffffffu, v, o);
    v = is_max ? fmaxf(v, u) : v + u;
  }
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float r = scratch[0];
#pragma unroll
  for (int k = 1; k < 8; ++k) r = is_max ? fmaxf(r, scratch[k]) : r + scratch[k];
  return r;
}

template <int MODE>       // 35: four 64-coordinate segments; 25: segments of 32, 32, 96, 96
__global__ void __launch_bounds__(256)
hybrid_merge_kernel(const float* __restrict__ part_acc, const float* __restrict__ part_ml, int num_parts,
                    const void* context_lens, int cl_dtype, int tokens_per_split, int num_q_heads,
                    HybridTables t, void* __restrict__ out, int out_dtype, int64_t out_ss, int64_t out_sh) {
  __shared__ float w[4][64];
  __shared__ float wgt[256];
  __shared__ float scratch[8];
  const int row = blockIdx.x, seq = row / num_q_heads, qh = row % num_q_heads, tid = threadIdx.x;
  const int64_t ctx = load_index(context_lens, cl_dtype, seq);
  int64_t nv = (ctx + tokens_per_split - 1) / tokens_per_split * HA_WARPS;
  const int np = (int)(nv < num_parts ? nv : num_parts);
  const float* ml = part_ml + (int64_t)row * num_parts * 2;
  float mx = -CUDART_INF_F;
  for (int p = tid; p < np; p += 256) if (ml[2 * p + 1] > 0.f) mx = fmaxf(mx, ml[2 * p]);
  const float M = block_reduce_256(mx, true, scratch);
  float ls = 0.f, acc = 0.f;
  const float* pa = part_acc + (int64_t)row * num_parts * 256 + tid;
  for (int p0 = 0; p0 < np; p0 += 256) {
    __syncthreads();
    {
      const int p = p0 + tid;
      float wv = 0.f;
      if (p < np && ml[2 * p + 1] > 0.f) { wv = exp2f(ml[2 * p] - M); ls += ml[2 * p + 1] * wv; }
      wgt[tid] = wv;
    }
    __syncthreads();
    const int cnt = np - p0 < 256 ? np - p0 : 256;
    for (int q = 0; q < cnt; q += 16) {     // 16 loads in flight per round, the last round masked
      float v[16];
#pragma unroll
      for (int k = 0; k < 16; ++k) v[k] = (q + k < cnt) ? pa[(int64_t)(p0 + q + k) * 256] : 0.f;
#pragma unroll
      for (int k = 0; k < 16; ++k) {
        const float wv = (q + k < cnt) ? wgt[q + k] : 0.f;
        acc = (wv > 0.f) ? __fmaf_rn(v[k], wv, acc) : acc;                   // weight 0: part never written
      }
    }
  }
  const float L = block_reduce_256(ls, false, scratch);
  const float inv = L > 0.f ? 1.f / L : 0.f;
  w[tid >> 6][tid & 63] = acc * inv;
  if (MODE == 25) {
    float* wf = &w[0][0];
    __syncthreads();
    hy25_transforms(wf, tid >> 5, 8, tid & 31);
    __syncthreads();
    if (tid < 128) {
      float o;
      if (tid < 32) {
        o = (wf[tid] * t.had_signs[tid] + wf[32 + tid] * t.qjl_scale0 * t.qjl_signs[tid]) * 0.17677669529663687f;
      } else {
        const int k = tid - 32;
        o = (wf[64 + k] * t.had_signs[tid] + wf[160 + k] * t.qjl_scale1 * t.qjl_signs[tid]) * 0.10206207261596577f;
      }
      store_from_float(out, out_dtype, seq * out_ss + qh * out_sh + t.group_index[tid], o);
    }
  } else {
    // four 64-point transforms: 128 butterflies per stage, one per thread of the first half
    for (int h = 1; h < 64; h <<= 1) {
      __syncthreads();
      if (tid < 128) {
        const int sg = tid >> 5, l = tid & 31;
        const int j = ((l & ~(h - 1)) << 1) | (l & (h - 1));
        const float a = w[sg][j], b = w[sg][j + h];
        w[sg][j] = a + b;
        w[sg][j + h] = a - b;
      }
    }
    __syncthreads();
    if (tid < 128) {
      const int grp = tid >> 6, k = tid & 63;
      const float o = (w[2 * grp][k] * t.had_signs[64 * grp + k] +
                       w[2 * grp + 1][k] * (grp ? t.qjl_scale1 : t.qjl_scale0) * t.qjl_signs[64 * grp + k]) * 0.125f;
      store_from_float(out, out_dtype, seq * out_ss + qh * out_sh + t.group_index[64 * grp + k], o);
    }
  }
}

static int mode_from(int head_dim, int packed_dim) {
  if (head_dim == 128 && packed_dim == 64) return 35;
  if (head_dim == 128 && packed_dim == 44) return 25;
  return 0;
}

}  // namespace akv

using namespace akv;

// Mirror of akv_hybrid_tables in include/akv_b200.h.
struct akv_hybrid_tables {
  int head_dim, packed_dim;
  const int* group_index; int num_index_heads;
  const float* had_signs; const float* qjl_signs;
  const float* centroids; const float* boundaries;
  float qjl_scale0, qjl_scale1;
};

static int tables_from(const akv_hybrid_tables* t, HybridTables* o, int* mode) {
  if (!t) return fail(AKV_ERR_ARG, "null hybrid tables");
  *mode = mode_from(t->head_dim, t->packed_dim);
  if (*mode == 0)
    return fail(AKV_ERR_UNSUPPORTED, "hybrid codec: head_dim %d / packed_dim %d is not tq35 or tq25 at 128",
                t->head_dim, t->packed_dim);
  if (!t->group_index || !t->had_signs || !t->qjl_signs || !t->centroids || !t->boundaries || t->num_index_heads < 1)
    return fail(AKV_ERR_ARG, "hybrid tables: null pointer");
  o->group_index = t->group_index; o->num_index_heads = t->num_index_heads;
  o->had_signs = t->had_signs; o->qjl_signs = t->qjl_signs;
  o->centroids = t->centroids; o->boundaries = t->boundaries;
  o->qjl_scale0 = t->qjl_scale0; o->qjl_scale1 = t->qjl_scale1;
  return AKV_OK;
}

// Encode n_rows vectors through `map` (contiguous rows or the paged scatter) with the kernel that fits
// the input type and alignment.
static int hybrid_encode_rows(const void* x, int x_dtype, int64_t n_rows, const HyRowMap& map, const HybridTables& t,
                              int mode, uint8_t* out, cudaStream_t st) {
  const bool paged = map.slot_mapping != nullptr;
  if (x_dtype != AKV_F32) {
    static const bool no_coop = getenv("AKV_HYBRID_NO_COOP") != nullptr;
    const int64_t xs = paged ? (map.x_stride_tok | map.x_stride_head) : map.x_stride_row;
    const int64_t os = paged ? (map.p_stride_blk | map.p_stride_pos | map.p_stride_head) : map.out_stride_row;
    const bool rows16 = (reinterpret_cast<uintptr_t>(x) & 15) == 0 && (xs & 7) == 0 &&
                        (reinterpret_cast<uintptr_t>(out) & 3) == 0 && (os & 3) == 0;
    if (mode == 35 && rows16 && !no_coop) return launch_hybrid_encode35_coop(x, x_dtype, n_rows, map, t, out, st);
    if (mode == 35) return launch_hybrid_encode16<64, 3, 64, 2>(x, x_dtype, n_rows, map, t, out, st);
    return launch_hybrid_encode16<32, 2, 96, 1>(x, x_dtype, n_rows, map, t, out, st);
  }
  const int grid = (int)((n_rows + HY_THREADS - 1) / HY_THREADS);
  if (mode == 35)
    hybrid_encode_kernel<64, 3, 64, 2><<<grid, HY_THREADS, 0, st>>>(x, x_dtype, n_rows, map, t, out);
  else
    hybrid_encode_kernel<32, 2, 96, 1><<<grid, HY_THREADS, 0, st>>>(x, x_dtype, n_rows, map, t, out);
  return check_launch("hybrid_encode_kernel");
}

AKV_EXPORT int akv_hybrid_encode(const void* x, int x_dtype, int64_t n_rows, int64_t x_row_stride,
                                 const akv_hybrid_tables* tables, uint8_t* packed,
                                 int64_t packed_row_stride, void* stream) {
  HybridTables t; int mode;
  if (int rc = tables_from(tables, &t, &mode)) return rc;
  if (n_rows < 0) return fail(AKV_ERR_ARG, "n_rows < 0");
  if (n_rows == 0) return AKV_OK;
  if (!x || !packed) return fail(AKV_ERR_ARG, "akv_hybrid_encode: null pointer");
  if (x_dtype < AKV_F16 || x_dtype > AKV_F32) return fail(AKV_ERR_ARG, "bad x_dtype %d", x_dtype);
  return hybrid_encode_rows(x, x_dtype, n_rows, hy_contiguous(x_row_stride, packed_row_stride), t, mode, packed,
                            (cudaStream_t)stream);
}

static int hybrid_paged_map(HyRowMap* m, int64_t num_tokens, int num_kv_heads, int64_t x_stride_tok,
                            int64_t x_stride_head, const int64_t* slot_mapping, int64_t c_stride_blk,
                            int64_t c_stride_pos, int64_t c_stride_head, int block_size, int64_t max_blocks) {
  if (num_tokens < 0 || num_kv_heads <= 0 || block_size <= 0 || max_blocks <= 0)
    return fail(AKV_ERR_ARG, "hybrid paged write: bad sizes");
  *m = HyRowMap{};
  m->slot_mapping = slot_mapping; m->num_heads = num_kv_heads; m->block_size = block_size; m->max_blocks = max_blocks;
  m->x_stride_tok = x_stride_tok; m->x_stride_head = x_stride_head;
  m->p_stride_blk = c_stride_blk; m->p_stride_pos = c_stride_pos; m->p_stride_head = c_stride_head;
  return AKV_OK;
}

// Paged write of hybrid records: x [num_tokens, num_kv_heads, 128] is encoded and record (token, head) is
// stored at cache[slot / block_size][slot % block_size][head]; tokens whose slot is negative or whose block is
// >= max_blocks are skipped.
AKV_EXPORT int akv_hybrid_kv_update(const void* x, int x_dtype, int64_t num_tokens, int num_kv_heads,
                                    int64_t x_stride_tok, int64_t x_stride_head, const int64_t* slot_mapping,
                                    const akv_hybrid_tables* tables, uint8_t* cache, int64_t c_stride_blk,
                                    int64_t c_stride_pos, int64_t c_stride_head, int block_size,
                                    int64_t max_blocks, void* stream) {
  HybridTables t; int mode;
  if (int rc = tables_from(tables, &t, &mode)) return rc;
  HyRowMap m;
  if (int rc = hybrid_paged_map(&m, num_tokens, num_kv_heads, x_stride_tok, x_stride_head, slot_mapping, c_stride_blk,
                                c_stride_pos, c_stride_head, block_size, max_blocks)) return rc;
  if (num_tokens == 0) return AKV_OK;
  if (!x || !cache || !slot_mapping) return fail(AKV_ERR_ARG, "akv_hybrid_kv_update: null pointer");
  if (x_dtype < AKV_F16 || x_dtype > AKV_F32) return fail(AKV_ERR_ARG, "bad x_dtype %d", x_dtype);
  return hybrid_encode_rows(x, x_dtype, num_tokens * num_kv_heads, m, t, mode, cache, (cudaStream_t)stream);
}

AKV_EXPORT int akv_hybrid_decode(const uint8_t* packed, int64_t packed_row_stride, int64_t n_rows,
                                 const akv_hybrid_tables* tables, void* out, int out_dtype, void* stream) {
  HybridTables t; int mode;
  if (int rc = tables_from(tables, &t, &mode)) return rc;
  if (n_rows < 0) return fail(AKV_ERR_ARG, "n_rows < 0");
  if (n_rows == 0) return AKV_OK;
  if (!packed || !out) return fail(AKV_ERR_ARG, "akv_hybrid_decode: null pointer");
  if (out_dtype < AKV_F16 || out_dtype > AKV_F32) return fail(AKV_ERR_ARG, "bad out_dtype %d", out_dtype);
  cudaStream_t st = (cudaStream_t)stream;
  static const bool no_coop = getenv("AKV_HYBRID_NO_COOP") != nullptr;
  if (mode == 35 && !no_coop && (reinterpret_cast<uintptr_t>(packed) & 15) == 0 && (packed_row_stride & 15) == 0 &&
      (reinterpret_cast<uintptr_t>(out) & 15) == 0) {
    hybrid_decode35_coop_kernel<<<(int)((n_rows + 31) / 32), HC_THREADS, 0, st>>>(packed, packed_row_stride, n_rows, t,
                                                                                   out, out_dtype);
    return check_launch("hybrid_decode35_coop_kernel");
  }
  const int grid = (int)((n_rows + HY_THREADS - 1) / HY_THREADS);
  if (mode == 35)
    hybrid_decode_kernel<64, 3, 64, 2><<<grid, HY_THREADS, 0, st>>>(packed, packed_row_stride, n_rows, t, out, out_dtype);
  else
    hybrid_decode_kernel<32, 2, 96, 1><<<grid, HY_THREADS, 0, st>>>(packed, packed_row_stride, n_rows, t, out, out_dtype);
  return check_launch("hybrid_decode_kernel");
}

// ---------------------------------------------------------------------------
// Pre-pass of the staged chunked-prefill kernel for tq35 caches (tq_prefill_tc.cu): every 128-key tile of every
// sequence and KV head is decoded once - exactly as hybrid_decode35_coop_kernel decodes, four lanes per record - and
// written as the fp16 operand images the tensor-core attention kernel copies into shared memory (layout: PFI_* in
// tq_prefill_args.cuh).  The decoded vectors are in the original domain: that attention runs without rotations.
// The reference decodes the active blocks to bf16 and calls vLLM's unified attention (vllm/hooks.py:726-850).
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(HC_THREADS, 2)
hybrid_prefill_stage35_kernel(PrefillArgs a, HybridTables t) {
  extern __shared__ __align__(16) uint8_t hp_image[];            // PFI_BYTES
  __shared__ uint32_t recs[32 * 17];
  __shared__ __align__(16) float outs[32 * HD_ROW];
  __shared__ float s_had[128], s_qjl[128], s_cent[16];
  __shared__ int s_idx[128];
  const int tid = threadIdx.x;
  const int s = blockIdx.y, kvh = blockIdx.z, tile = blockIdx.x;
  const int64_t max_ctx = (int64_t)a.max_blocks_per_seq * a.block_size;
  const int seq_len = (int)load_ctx(a.seq_lens, a.sl_dtype, s, max_ctx);
  int n_tiles = (seq_len + PFI_KEYS - 1) / PFI_KEYS;
  if (n_tiles > a.tiles_per_seq) n_tiles = a.tiles_per_seq;
  if (tile >= n_tiles) return;
  const int* gsrc = t.group_index + (t.num_index_heads > 1 ? (kvh % t.num_index_heads) * 128 : 0);
  if (tid < 128) { s_had[tid] = t.had_signs[tid]; s_qjl[tid] = t.qjl_signs[tid]; s_idx[tid] = gsrc[tid]; }
  if (tid < 16) s_cent[tid] = t.centroids[tid];
  const int bs = a.block_size;
  for (int side = 0; side < 2; ++side) {
    const uint8_t* cache = side ? a.v_packed : a.k_packed;
    const int64_t sb = side ? a.vp_sb : a.kp_sb, sp = side ? a.vp_sp : a.kp_sp, sh = side ? a.vp_sh : a.kp_sh;
    for (int pass = 0; pass < PFI_KEYS / 32; ++pass) {
      __syncthreads();                 // tables staged; the previous pass's rows have been read
      {   // 32 records x 16 words, one 16-byte piece per thread
        const int r = tid >> 2, c = tid & 3;
        const int key = PFI_KEYS * tile + 32 * pass + r;
        int blk = key / bs;
        if (blk >= a.max_blocks_per_seq) blk = a.max_blocks_per_seq - 1;
        int64_t pb = load_index(a.block_tables, a.bt_dtype, (int64_t)s * a.bt_stride + blk);
        pb = pb < 0 ? 0 : (pb >= a.num_blocks ? a.num_blocks - 1 : pb);
        const uint4 v = *reinterpret_cast<const uint4*>(cache + pb * sb + (int64_t)(key - (key / bs) * bs) * sp + (int64_t)kvh * sh + c * 16);
        uint32_t* d = recs + r * 17 + 4 * c;
        d[0] = v.x; d[1] = v.y; d[2] = v.z; d[3] = v.w;
      }
      __syncthreads();
      const int vec = tid >> 2, q = tid & 3;
      hc_decode_group<3>(recs + vec * 17, s_idx, s_had, s_qjl, s_cent, t.qjl_scale0, q, outs + vec * HD_ROW);
      hc_decode_group<2>(recs + vec * 17 + 9, s_idx + 64, s_had + 64, s_qjl + 64, s_cent + 8, t.qjl_scale1, q,
                         outs + vec * HD_ROW);
      __syncthreads();
      const int key0 = PFI_KEYS * tile + 32 * pass;
      if (side == 0) {
        // K image: 32 rows x 16 chunks of 8 dims
        for (int e = tid; e < 32 * 16; e += HC_THREADS) {
          const int r = e >> 4, c = e & 15;
          const bool live = key0 + r < seq_len;
          const float4 x = *reinterpret_cast<const float4*>(outs + r * HD_ROW + 8 * c);
          const float4 y = *reinterpret_cast<const float4*>(outs + r * HD_ROW + 8 * c + 4);
          __half2 h[4] = {__floats2half2_rn(x.x, x.y), __floats2half2_rn(x.z, x.w), __floats2half2_rn(y.x, y.y), __floats2half2_rn(y.z, y.w)};
          uint4 w = *reinterpret_cast<uint4*>(h);
          if (!live) w = make_uint4(0u, 0u, 0u, 0u);
          const int row = 32 * pass + r;
          *reinterpret_cast<uint4*>(hp_image + (c >> 3) * PFI_KHALF + row * 128 + (((c & 7) ^ (row & 7)) << 4)) = w;
        }
      } else {
        // transposed V image: 4 key groups of 8 keys x 128 dims
        for (int e = tid; e < 4 * 128; e += HC_THREADS) {
          const int gl = e >> 7, d = e & 127;
          float v[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) v[i] = key0 + 8 * gl + i < seq_len ? outs[(8 * gl + i) * HD_ROW + d] : 0.f;
          __half2 h[4] = {__floats2half2_rn(v[0], v[1]), __floats2half2_rn(v[2], v[3]), __floats2half2_rn(v[4], v[5]), __floats2half2_rn(v[6], v[7])};
          const int g = 4 * pass + gl;
          *reinterpret_cast<uint4*>(hp_image + PFI_VOFF + (g >> 3) * PFI_VHALF + d * 128 + (((g & 7) ^ (d & 7)) << 4)) =
              *reinterpret_cast<uint4*>(h);
        }
      }
    }
  }
  __syncthreads();
  uint4* dst = reinterpret_cast<uint4*>(a.staged + (((int64_t)s * a.tiles_per_seq + tile) * a.num_kv_heads + kvh) * PFI_BYTES);
  for (int i = tid; i < PFI_BYTES / 16; i += HC_THREADS) dst[i] = reinterpret_cast<const uint4*>(hp_image)[i];
}

// The same for any dim split (tq25: 32 + 96 dims, 44-byte records): one thread per record, the decode of
// hybrid_decode_kernel, 64 records per pass.
template <int G0, int B0, int G1, int B1>
__global__ void __launch_bounds__(HY_THREADS)
hybrid_prefill_stage_kernel(PrefillArgs a, HybridTables t) {
  constexpr int D = G0 + G1;
  static_assert(D == 128, "head_dim 128");
  constexpr int BYTES0 = (G0 * B0 + 7) / 8 + (G0 + 7) / 8 + 4;
  constexpr int BYTES1 = (G1 * B1 + 7) / 8 + (G1 + 7) / 8 + 4;
  extern __shared__ __align__(16) uint8_t hp_image[];            // PFI_BYTES
  __shared__ float xs[HY_THREADS * HY_LD];
  __shared__ float s_had[D], s_qjl[D], s_cent[16];
  __shared__ int s_idx[D];
  const int tid = threadIdx.x;
  const int s = blockIdx.y, kvh = blockIdx.z, tile = blockIdx.x;
  const int64_t max_ctx = (int64_t)a.max_blocks_per_seq * a.block_size;
  const int seq_len = (int)load_ctx(a.seq_lens, a.sl_dtype, s, max_ctx);
  int n_tiles = (seq_len + PFI_KEYS - 1) / PFI_KEYS;
  if (n_tiles > a.tiles_per_seq) n_tiles = a.tiles_per_seq;
  if (tile >= n_tiles) return;
  const int* gsrc = t.group_index + (t.num_index_heads > 1 ? (kvh % t.num_index_heads) * D : 0);
  for (int i = tid; i < D; i += HY_THREADS) { s_had[i] = t.had_signs[i]; s_qjl[i] = t.qjl_signs[i]; s_idx[i] = gsrc[i]; }
  if (tid < 16) s_cent[tid] = t.centroids[tid];
  const int bs = a.block_size;
  for (int side = 0; side < 2; ++side) {
    const uint8_t* cache = side ? a.v_packed : a.k_packed;
    const int64_t sb = side ? a.vp_sb : a.kp_sb, sp = side ? a.vp_sp : a.kp_sp, sh = side ? a.vp_sh : a.kp_sh;
    for (int pass = 0; pass < PFI_KEYS / HY_THREADS; ++pass) {
      __syncthreads();                 // tables staged; the previous pass's rows have been read
      const int key0 = PFI_KEYS * tile + HY_THREADS * pass;
      {
        const int key = key0 + tid;
        int blk = key / bs;
        if (blk >= a.max_blocks_per_seq) blk = a.max_blocks_per_seq - 1;
        int64_t pb = load_index(a.block_tables, a.bt_dtype, (int64_t)s * a.bt_stride + blk);
        pb = pb < 0 ? 0 : (pb >= a.num_blocks ? a.num_blocks - 1 : pb);
        const uint8_t* src = cache + pb * sb + (int64_t)(key - (key / bs) * bs) * sp + (int64_t)kvh * sh;
        uint8_t rec[BYTES0 + BYTES1];
#pragma unroll
        for (int wd = 0; wd < (BYTES0 + BYTES1) / 4; ++wd) {      // records are 4-byte aligned (checked by the host)
          const uint32_t v = reinterpret_cast<const uint32_t*>(src)[wd];
          rec[4 * wd] = (uint8_t)v; rec[4 * wd + 1] = (uint8_t)(v >> 8);
          rec[4 * wd + 2] = (uint8_t)(v >> 16); rec[4 * wd + 3] = (uint8_t)(v >> 24);
        }
        decode_group<G0, B0>(rec, s_idx, s_had, s_qjl, s_cent, t.qjl_scale0, xs + tid * HY_LD);
        decode_group<G1, B1>(rec + BYTES0, s_idx + G0, s_had + G0, s_qjl + G0, s_cent + 8, t.qjl_scale1, xs + tid * HY_LD);
      }
      __syncthreads();
      if (side == 0) {
        for (int e = tid; e < HY_THREADS * 16; e += HY_THREADS) {
          const int r = e >> 4, c = e & 15;
          const bool live = key0 + r < seq_len;
          const float* x = xs + r * HY_LD + 8 * c;
          __half2 h[4] = {__floats2half2_rn(x[0], x[1]), __floats2half2_rn(x[2], x[3]), __floats2half2_rn(x[4], x[5]), __floats2half2_rn(x[6], x[7])};
          uint4 w = *reinterpret_cast<uint4*>(h);
          if (!live) w = make_uint4(0u, 0u, 0u, 0u);
          const int row = HY_THREADS * pass + r;
          *reinterpret_cast<uint4*>(hp_image + (c >> 3) * PFI_KHALF + row * 128 + (((c & 7) ^ (row & 7)) << 4)) = w;
        }
      } else {
        for (int e = tid; e < (HY_THREADS / 8) * 128; e += HY_THREADS) {
          const int gl = e >> 7, d = e & 127;
          float v[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) v[i] = key0 + 8 * gl + i < seq_len ? xs[(8 * gl + i) * HY_LD + d] : 0.f;
          __half2 h[4] = {__floats2half2_rn(v[0], v[1]), __floats2half2_rn(v[2], v[3]), __floats2half2_rn(v[4], v[5]), __floats2half2_rn(v[6], v[7])};
          const int g = (HY_THREADS / 8) * pass + gl;
          *reinterpret_cast<uint4*>(hp_image + PFI_VOFF + (g >> 3) * PFI_VHALF + d * 128 + (((g & 7) ^ (d & 7)) << 4)) =
              *reinterpret_cast<uint4*>(h);
        }
      }
    }
  }
  __syncthreads();
  uint4* dst = reinterpret_cast<uint4*>(a.staged + (((int64_t)s * a.tiles_per_seq + tile) * a.num_kv_heads + kvh) * PFI_BYTES);
  for (int i = tid; i < PFI_BYTES / 16; i += HY_THREADS) dst[i] = reinterpret_cast<const uint4*>(hp_image)[i];
}

int akv::launch_hybrid_prefill_stage(const PrefillArgs& a, cudaStream_t st) {
  HybridTables t; int mode;
  if (int rc = tables_from(reinterpret_cast<const akv_hybrid_tables*>(a.hybrid_tables), &t, &mode)) return rc;
  const uintptr_t al = reinterpret_cast<uintptr_t>(a.k_packed) | reinterpret_cast<uintptr_t>(a.v_packed) | (uintptr_t)a.kp_sb |
                       (uintptr_t)a.kp_sp | (uintptr_t)a.kp_sh | (uintptr_t)a.vp_sb | (uintptr_t)a.vp_sp | (uintptr_t)a.vp_sh;
  if (mode != 35 || (al & 15) != 0) {      // tq25, or tq35 records that cannot be read in 16-byte pieces
    if ((al & 3) != 0) return fail(AKV_ERR_UNSUPPORTED, "staged prefill attention needs records readable in 4-byte pieces");
    dim3 grid(a.tiles_per_seq, a.num_seqs, a.num_kv_heads);
    cudaError_t e;
    if (mode == 35) {
      e = cudaFuncSetAttribute(hybrid_prefill_stage_kernel<64, 3, 64, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, PFI_BYTES);
      if (e == cudaSuccess) hybrid_prefill_stage_kernel<64, 3, 64, 2><<<grid, HY_THREADS, PFI_BYTES, st>>>(a, t);
    } else {
      e = cudaFuncSetAttribute(hybrid_prefill_stage_kernel<32, 2, 96, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, PFI_BYTES);
      if (e == cudaSuccess) hybrid_prefill_stage_kernel<32, 2, 96, 1><<<grid, HY_THREADS, PFI_BYTES, st>>>(a, t);
    }
    if (e != cudaSuccess) return fail((int)e, "prefill attention: smem attribute: %s", cudaGetErrorString(e));
    return check_launch("hybrid_prefill_stage_kernel");
  }
  cudaError_t e = cudaFuncSetAttribute(hybrid_prefill_stage35_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, PFI_BYTES);
  if (e != cudaSuccess) return fail((int)e, "prefill attention: smem attribute: %s", cudaGetErrorString(e));
  dim3 grid(a.tiles_per_seq, a.num_seqs, a.num_kv_heads);
  hybrid_prefill_stage35_kernel<<<grid, HC_THREADS, PFI_BYTES, st>>>(a, t);
  return check_launch("hybrid_prefill_stage35_kernel");
}

// Mirror of akv_hybrid_attn_params in include/akv_b200.h.
struct akv_hybrid_attn_params {
  const void* query; int q_dtype; int64_t q_stride_seq, q_stride_head;
  const uint8_t* k_cache; int64_t k_stride_blk, k_stride_pos, k_stride_head;
  const uint8_t* v_cache; int64_t v_stride_blk, v_stride_pos, v_stride_head;
  const void* block_tables; int bt_dtype; int64_t bt_stride_seq;
  const void* context_lens; int cl_dtype;
  int num_seqs, num_q_heads, num_kv_heads, block_size, max_blocks_per_seq;
  int64_t num_blocks;
  const akv_hybrid_tables* tables;
  float scale;
  void* out; int out_dtype; int64_t out_stride_seq, out_stride_head;
  void* workspace; size_t workspace_bytes;
  int blocks_per_split;
  void* stream;
};

static void hybrid_plan(int num_seqs, int num_q_heads, int block_size, int max_blocks, int bps_in, int* bps,
                        int* parts, size_t* off_acc, size_t* off_ml, size_t* total) {
  int b = bps_in > 0 ? bps_in : (2048 + block_size - 1) / block_size;   // ~2048 tokens per split
  if (b > max_blocks) b = max_blocks > 0 ? max_blocks : 1;
  const int splits = max_blocks > 0 ? (max_blocks + b - 1) / b : 1;
  *bps = b;
  *parts = splits * HA_WARPS;
  const size_t rows = (size_t)num_seqs * num_q_heads;
  auto al = [](size_t v) { return (v + 255) & ~(size_t)255; };
  *off_acc = al(rows * 256 * sizeof(float));
  *off_ml = *off_acc + al(rows * (size_t)*parts * 256 * sizeof(float));
  *total = *off_ml + al(rows * (size_t)*parts * 2 * sizeof(float));
}

namespace akv {
int hybrid_window_status(int* host_out, int reset) {
  cudaError_t e = cudaMemcpyFromSymbol(host_out, g_hybrid_window_status, sizeof(int));
  if (e == cudaSuccess && reset) { const int z = 0; e = cudaMemcpyToSymbol(g_hybrid_window_status, &z, sizeof(int)); }
  return e == cudaSuccess ? AKV_OK : fail((int)e, "hybrid status: %s", cudaGetErrorString(e));
}
}  // namespace akv

AKV_EXPORT size_t akv_hybrid_paged_attn_workspace_bytes(int num_seqs, int num_q_heads, int block_size,
                                                        int max_blocks_per_seq, int blocks_per_split) {
  if (num_seqs <= 0 || num_q_heads <= 0 || block_size <= 0) return 0;
  int bps, parts; size_t a, m, total;
  hybrid_plan(num_seqs, num_q_heads, block_size, max_blocks_per_seq, blocks_per_split, &bps, &parts, &a, &m, &total);
  return total;
}

static int run_hybrid_attn(const akv_hybrid_attn_params* p, const HyStepWrite* wr, bool wr_bf16) {
  if (!p) return fail(AKV_ERR_ARG, "null params");
  HybridTables t; int mode;
  if (int rc = tables_from(p->tables, &t, &mode)) return rc;
  if (mode == 25 && wr != nullptr && wr->n_rows > 0)
    return fail(AKV_ERR_UNSUPPORTED, "hybrid paged attention: the fused record write is built for tq35");
  if (t.num_index_heads != 1)
    return fail(AKV_ERR_UNSUPPORTED, "hybrid paged attention needs one dim split shared by all heads");
  if (p->num_seqs < 0 || p->num_q_heads <= 0 || p->num_kv_heads <= 0 || p->num_q_heads % p->num_kv_heads ||
      p->block_size <= 0 || p->max_blocks_per_seq < 0 || p->num_blocks <= 0)
    return fail(AKV_ERR_ARG, "hybrid paged attention: bad sizes");
  if (p->num_seqs == 0) return AKV_OK;
  if (!p->query || !p->k_cache || !p->v_cache || !p->block_tables || !p->context_lens || !p->out)
    return fail(AKV_ERR_ARG, "hybrid paged attention: null pointer");
  if ((reinterpret_cast<uintptr_t>(p->k_cache) | reinterpret_cast<uintptr_t>(p->v_cache) | p->k_stride_blk |
       p->k_stride_pos | p->k_stride_head | p->v_stride_blk | p->v_stride_pos | p->v_stride_head) & 3)
    return fail(AKV_ERR_UNSUPPORTED, "hybrid cache records must be 4-byte aligned");
  int bps, parts; size_t off_acc, off_ml, total;
  hybrid_plan(p->num_seqs, p->num_q_heads, p->block_size, p->max_blocks_per_seq, p->blocks_per_split, &bps,
              &parts, &off_acc, &off_ml, &total);
  if (!p->workspace || p->workspace_bytes < total)
    return fail(AKV_ERR_WORKSPACE, "workspace too small: need %zu bytes, got %zu", total, p->workspace_bytes);
  char* ws = reinterpret_cast<char*>(p->workspace);
  float* qprime = reinterpret_cast<float*>(ws);
  float* part_acc = reinterpret_cast<float*>(ws + off_acc);
  float* part_ml = reinterpret_cast<float*>(ws + off_ml);
  cudaStream_t st = (cudaStream_t)p->stream;
  const int rows = p->num_seqs * p->num_q_heads;
  if (wr != nullptr && wr->n_rows > 0) {
    const int q_blocks = (rows + 3) / 4;
    const unsigned grid0 = (unsigned)(q_blocks + 2 * ((wr->n_rows + 31) / 32));
    if (wr_bf16)
      hybrid_step_prologue_kernel<true><<<grid0, HC_THREADS, 0, st>>>(p->query, p->q_dtype, p->q_stride_seq,
          p->q_stride_head, p->num_q_heads, t, p->scale * 1.4426950408889634f, qprime, rows, q_blocks, *wr);
    else
      hybrid_step_prologue_kernel<false><<<grid0, HC_THREADS, 0, st>>>(p->query, p->q_dtype, p->q_stride_seq,
          p->q_stride_head, p->num_q_heads, t, p->scale * 1.4426950408889634f, qprime, rows, q_blocks, *wr);
    if (int rc = check_launch("hybrid_step_prologue_kernel")) return rc;
  } else if (mode == 25) {
    hybrid_qprime25_kernel<<<rows, 32, 0, st>>>(p->query, p->q_dtype, p->q_stride_seq, p->q_stride_head,
                                                p->num_q_heads, t, p->scale * 1.4426950408889634f, qprime);
    if (int rc = check_launch("hybrid_qprime25_kernel")) return rc;
  } else {
    hybrid_qprime_kernel<<<rows, 32, 0, st>>>(p->query, p->q_dtype, p->q_stride_seq, p->q_stride_head,
                                              p->num_q_heads, t, p->scale * 1.4426950408889634f, qprime);
    if (int rc = check_launch("hybrid_qprime_kernel")) return rc;
  }
  if (p->max_blocks_per_seq > 0) {
    HybridAttnArgs a{};
    a.k_cache = p->k_cache; a.v_cache = p->v_cache;
    a.k_sb = p->k_stride_blk; a.k_sp = p->k_stride_pos; a.k_sh = p->k_stride_head;
    a.v_sb = p->v_stride_blk; a.v_sp = p->v_stride_pos; a.v_sh = p->v_stride_head;
    a.block_tables = p->block_tables; a.bt_dtype = p->bt_dtype; a.bt_stride = p->bt_stride_seq;
    a.context_lens = p->context_lens; a.cl_dtype = p->cl_dtype;
    a.num_q_heads = p->num_q_heads; a.num_kv_heads = p->num_kv_heads; a.block_size = p->block_size;
    a.max_blocks_per_seq = p->max_blocks_per_seq;
    a.num_blocks = p->num_blocks; a.blocks_per_split = bps; a.num_parts = parts;
    a.qprime = qprime; a.centroids = t.centroids; a.part_acc = part_acc; a.part_ml = part_ml;
    dim3 grid(parts / HA_WARPS, p->num_kv_heads, p->num_seqs);
    // tensor-core kernel: 16-token tiles, GQA groups of up to 8, records readable in 16-byte pieces
    static const bool force_scalar = getenv("AKV_HYBRID_SCALAR") != nullptr;
    const bool aligned16 = ((reinterpret_cast<uintptr_t>(p->k_cache) | reinterpret_cast<uintptr_t>(p->v_cache) |
                             p->k_stride_blk | p->k_stride_pos | p->k_stride_head | p->v_stride_blk |
                             p->v_stride_pos | p->v_stride_head) & 15) == 0;
    // the tensor-core kernel keeps its tables at fixed shared addresses: its dynamic window must start below them
    static const bool window_ok = dyn_smem_window_start(reinterpret_cast<const void*>(hybrid_attn_mma_kernel<false>)) <= HM_LUT2 &&
        dyn_smem_window_start(reinterpret_cast<const void*>(hybrid_attn_mma_kernel<true>)) <= HM_LUT2;
    if (mode == 25) {
      hybrid_attn25_kernel<<<grid, HA_WARPS * 32, 0, st>>>(a);
      if (int rc = check_launch("hybrid_attn25_kernel")) return rc;
    } else if (!force_scalar && window_ok && aligned16 && p->block_size % 16 == 0 && p->num_q_heads / p->num_kv_heads <= 8) {
      static const bool no_par = getenv("AKV_HYBRID_NO_PAR") != nullptr;
      auto kern = (p->num_q_heads / p->num_kv_heads <= 4 && !no_par) ? hybrid_attn_mma_kernel<true> : hybrid_attn_mma_kernel<false>;
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, HM_SMEM);
      if (e != cudaSuccess) return fail((int)e, "hybrid attention: smem attribute: %s", cudaGetErrorString(e));
      kern<<<grid, HA_WARPS * 32, HM_SMEM, st>>>(a);
      if (int rc = check_launch("hybrid_attn_mma_kernel")) return rc;
    } else {
      hybrid_attn_kernel<<<grid, HA_WARPS * 32, 0, st>>>(a);
      if (int rc = check_launch("hybrid_attn_kernel")) return rc;
    }
  }
  if (mode == 25)
    hybrid_merge_kernel<25><<<rows, 256, 0, st>>>(part_acc, part_ml, p->max_blocks_per_seq > 0 ? parts : 0,
                                                 p->context_lens, p->cl_dtype, bps * p->block_size, p->num_q_heads, t,
                                                 p->out, p->out_dtype, p->out_stride_seq, p->out_stride_head);
  else
    hybrid_merge_kernel<35><<<rows, 256, 0, st>>>(part_acc, part_ml, p->max_blocks_per_seq > 0 ? parts : 0,
                                                 p->context_lens, p->cl_dtype, bps * p->block_size, p->num_q_heads, t,
                                                 p->out, p->out_dtype, p->out_stride_seq, p->out_stride_head);
  return check_launch("hybrid_merge_kernel");
}

AKV_EXPORT int akv_hybrid_paged_attn(const akv_hybrid_attn_params* p) { return run_hybrid_attn(p, nullptr, false); }

// Mirror of akv_hybrid_decode_step_params in include/akv_b200.h.
struct akv_hybrid_decode_step_params {
  const void* key; const void* value; int kv_dtype;
  int64_t num_tokens;
  int64_t k_stride_tok, k_stride_head, v_stride_tok, v_stride_head;
  const int64_t* slot_mapping;
  int64_t max_blocks;
  akv_hybrid_attn_params attn;
};

// One serving step in one call: encode the new tokens' K and V records into the paged cache, then attend.
// With 16-bit K/V rows readable in 16-byte pieces (the serving case) the records are written by extra
// blocks of the query-transform launch: three launches in all (transform + write, attention, merge).
AKV_EXPORT int akv_hybrid_decode_step(const akv_hybrid_decode_step_params* p) {
  if (!p) return fail(AKV_ERR_ARG, "null params");
  const akv_hybrid_attn_params& a = p->attn;
  if (p->num_tokens <= 0) return run_hybrid_attn(&p->attn, nullptr, false);
  if (!p->key || !p->value || !p->slot_mapping || !a.k_cache || !a.v_cache)
    return fail(AKV_ERR_ARG, "akv_hybrid_decode_step: null pointer");
  HybridTables t; int mode;
  if (int rc = tables_from(a.tables, &t, &mode)) return rc;
  HyRowMap mk, mv;
  if (int rc = hybrid_paged_map(&mk, p->num_tokens, a.num_kv_heads, p->k_stride_tok, p->k_stride_head, p->slot_mapping,
                                a.k_stride_blk, a.k_stride_pos, a.k_stride_head, a.block_size, p->max_blocks)) return rc;
  if (int rc = hybrid_paged_map(&mv, p->num_tokens, a.num_kv_heads, p->v_stride_tok, p->v_stride_head, p->slot_mapping,
                                a.v_stride_blk, a.v_stride_pos, a.v_stride_head, a.block_size, p->max_blocks)) return rc;
  const int64_t rows = p->num_tokens * (int64_t)a.num_kv_heads;
  uint8_t* ck = const_cast<uint8_t*>(a.k_cache);
  uint8_t* cv = const_cast<uint8_t*>(a.v_cache);
  const bool x16 = p->kv_dtype == AKV_F16 || p->kv_dtype == AKV_BF16;
  const bool aligned = ((reinterpret_cast<uintptr_t>(p->key) | reinterpret_cast<uintptr_t>(p->value)) & 15) == 0 &&
                       ((p->k_stride_tok | p->k_stride_head | p->v_stride_tok | p->v_stride_head) & 7) == 0 &&
                       ((reinterpret_cast<uintptr_t>(ck) | reinterpret_cast<uintptr_t>(cv) | a.k_stride_blk | a.k_stride_pos |
                         a.k_stride_head | a.v_stride_blk | a.v_stride_pos | a.v_stride_head) & 3) == 0;
  if (mode == 35 && x16 && aligned && a.num_seqs > 0 && rows < (1 << 20)) {
    HyStepWrite wr{};
    wr.xk = reinterpret_cast<const uint16_t*>(p->key); wr.xv = reinterpret_cast<const uint16_t*>(p->value);
    wr.mk = mk; wr.mv = mv; wr.ck = ck; wr.cv = cv; wr.n_rows = rows;
    return run_hybrid_attn(&p->attn, &wr, p->kv_dtype == AKV_BF16);
  }
  if (p->kv_dtype < AKV_F16 || p->kv_dtype > AKV_F32) return fail(AKV_ERR_ARG, "bad kv_dtype %d", p->kv_dtype);
  cudaStream_t st = (cudaStream_t)a.stream;
  if (int rc = hybrid_encode_rows(p->key, p->kv_dtype, rows, mk, t, mode, ck, st)) return rc;
  if (int rc = hybrid_encode_rows(p->value, p->kv_dtype, rows, mv, t, mode, cv, st)) return rc;
  return run_hybrid_attn(&p->attn, nullptr, false);
}
