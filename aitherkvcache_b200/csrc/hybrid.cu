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
#include <math_constants.h>

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
hybrid_encode_kernel(const void* __restrict__ x, int x_dtype, int64_t n_rows, int64_t x_row_stride,
                     HybridTables t, uint8_t* __restrict__ out, int64_t out_row_stride) {
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
    xs[r * HY_LD + c] = (n < n_rows) ? load_as_float(x, x_dtype, n * x_row_stride + c) : 0.f;
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
  uint8_t rec[BYTES0 + BYTES1];
  encode_group<G0, B0>(xs + tid * HY_LD, gidx, s_had, s_qjl, s_cent, s_bnd, rec);
  encode_group<G1, B1>(xs + tid * HY_LD, gidx + G0, s_had + G0, s_qjl + G0, s_cent + 8, s_bnd + 8,
                       rec + BYTES0);
  uint8_t* dst = out + n * out_row_stride;
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
hybrid_encode16_kernel(const uint16_t* __restrict__ x, int64_t n_rows, int64_t x_row_stride,
                       HybridTables t, uint8_t* __restrict__ out, int64_t out_row_stride) {
  constexpr int D = G0 + G1;
  static_assert(D == 128, "rows are staged as 16 chunks of 16 bytes");
  constexpr int GMAX = G0 > G1 ? G0 : G1;
  constexpr int W0 = G0 * B0 / 32 + G0 / 32 + 1, W1 = G1 * B1 / 32 + G1 / 32 + 1;
  extern __shared__ __align__(16) uint8_t he_smem[];
  uint32_t* xs = reinterpret_cast<uint32_t*>(he_smem);                 // [128 rows][64 words]
  float* us = reinterpret_cast<float*>(he_smem + HE_THREADS * 256);     // [GMAX][128]
  __shared__ float s_had[D], s_qjl[D], s_cent[16], s_bnd[16];
  __shared__ int s_idx[D];
  const int tid = threadIdx.x;
  if (tid < D) { s_had[tid] = t.had_signs[tid]; s_qjl[tid] = t.qjl_signs[tid]; s_idx[tid] = t.group_index[tid]; }
  if (tid < 16) { s_cent[tid] = t.centroids[tid]; s_bnd[tid] = t.boundaries[tid]; }
  const int64_t row0 = (int64_t)blockIdx.x * HE_THREADS;
  const bool vec = (reinterpret_cast<uintptr_t>(x) & 15) == 0 && (x_row_stride & 7) == 0;
#pragma unroll
  for (int i0 = 0; i0 < 16; i0 += 8) {
    uint4 v[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int e = (i0 + i) * HE_THREADS + tid, r = e >> 4, c = e & 15;
      const int64_t n = row0 + r;
      v[i] = make_uint4(0u, 0u, 0u, 0u);
      if (n < n_rows) {
        const uint16_t* src = x + n * x_row_stride + c * 8;
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
  uint8_t* dst = out + n * out_row_stride;
  if ((reinterpret_cast<uintptr_t>(dst) & 3) == 0) {
#pragma unroll
    for (int wd = 0; wd < W0 + W1; ++wd) reinterpret_cast<uint32_t*>(dst)[wd] = rec[wd];
  } else {
#pragma unroll
    for (int b = 0; b < 4 * (W0 + W1); ++b) dst[b] = (uint8_t)(rec[b >> 2] >> (8 * (b & 3)));
  }
}

template <int G0, int B0, int G1, int B1>
static int launch_hybrid_encode16(const void* x, int x_dtype, int64_t n_rows, int64_t x_row_stride,
                                  const HybridTables& t, uint8_t* out, int64_t out_row_stride, cudaStream_t st) {
  constexpr int GMAX = G0 > G1 ? G0 : G1;
  constexpr size_t SMEM = (size_t)HE_THREADS * 256 + (size_t)GMAX * HE_THREADS * 4;
  const int grid = (int)((n_rows + HE_THREADS - 1) / HE_THREADS);
  const uint16_t* xp = reinterpret_cast<const uint16_t*>(x);
  cudaError_t e;
  if (x_dtype == AKV_BF16) {
    auto kern = hybrid_encode16_kernel<G0, B0, G1, B1, true>;
    e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM);
    if (e == cudaSuccess) kern<<<grid, HE_THREADS, SMEM, st>>>(xp, n_rows, x_row_stride, t, out, out_row_stride);
  } else {
    auto kern = hybrid_encode16_kernel<G0, B0, G1, B1, false>;
    e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM);
    if (e == cudaSuccess) kern<<<grid, HE_THREADS, SMEM, st>>>(xp, n_rows, x_row_stride, t, out, out_row_stride);
  }
  if (e != cudaSuccess) return fail((int)e, "hybrid encode: smem attribute: %s", cudaGetErrorString(e));
  return check_launch("hybrid_encode16_kernel");
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
struct HybridAttnArgs {
  const uint8_t* k_cache; const uint8_t* v_cache;
  int64_t k_sb, k_sp, k_sh, v_sb, v_sp, v_sh;   // bytes
  const void* block_tables; int bt_dtype; int64_t bt_stride;
  const void* context_lens; int cl_dtype;
  int num_q_heads, num_kv_heads, block_size;
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
  const int64_t ctx = load_index(a.context_lens, a.cl_dtype, seq);
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

__global__ void __launch_bounds__(32)
hybrid_qprime_kernel(const void* __restrict__ q, int q_dtype, int64_t q_ss, int64_t q_sh, int num_q_heads,
                     HybridTables t, float premul, float* __restrict__ qprime) {
  __shared__ float w[4][64];
  const int row = blockIdx.x, seq = row / num_q_heads, qh = row % num_q_heads, lane = threadIdx.x;
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

// LSE merge of the 256-coordinate partials and the inverse transforms of the epilogue.
__global__ void __launch_bounds__(32)
hybrid_merge_kernel(const float* __restrict__ part_acc, const float* __restrict__ part_ml, int num_parts,
                    const void* context_lens, int cl_dtype, int tokens_per_split, int num_q_heads,
                    HybridTables t, void* __restrict__ out, int out_dtype, int64_t out_ss, int64_t out_sh) {
  __shared__ float w[4][64];
  const int row = blockIdx.x, seq = row / num_q_heads, qh = row % num_q_heads, lane = threadIdx.x;
  const int64_t ctx = load_index(context_lens, cl_dtype, seq);
  int64_t nv = (ctx + tokens_per_split - 1) / tokens_per_split * HA_WARPS;
  const int np = (int)(nv < num_parts ? nv : num_parts);
  const float* ml = part_ml + (int64_t)row * num_parts * 2;
  float M = -CUDART_INF_F, L = 0.f;
  for (int p = 0; p < np; ++p) if (ml[2 * p + 1] > 0.f) M = fmaxf(M, ml[2 * p]);
  for (int p = 0; p < np; ++p) if (ml[2 * p + 1] > 0.f) L += ml[2 * p + 1] * exp2f(ml[2 * p] - M);
  const float inv = L > 0.f ? 1.f / L : 0.f;
  for (int c = lane; c < 256; c += 32) {
    float o = 0.f;
    for (int p = 0; p < np; ++p)
      if (ml[2 * p + 1] > 0.f) o += part_acc[((int64_t)row * num_parts + p) * 256 + c] * exp2f(ml[2 * p] - M);
    w[c >> 6][c & 63] = o * inv;
  }
  for (int s = 0; s < 4; ++s) fwht64_smem(w[s], lane);
  for (int k = lane; k < 64; k += 32) {
    const float o0 = (w[0][k] * t.had_signs[k] + w[1][k] * t.qjl_scale0 * t.qjl_signs[k]) * 0.125f;
    const float o1 = (w[2][k] * t.had_signs[64 + k] + w[3][k] * t.qjl_scale1 * t.qjl_signs[64 + k]) * 0.125f;
    store_from_float(out, out_dtype, seq * out_ss + qh * out_sh + t.group_index[k], o0);
    store_from_float(out, out_dtype, seq * out_ss + qh * out_sh + t.group_index[64 + k], o1);
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

AKV_EXPORT int akv_hybrid_encode(const void* x, int x_dtype, int64_t n_rows, int64_t x_row_stride,
                                 const akv_hybrid_tables* tables, uint8_t* packed,
                                 int64_t packed_row_stride, void* stream) {
  HybridTables t; int mode;
  if (int rc = tables_from(tables, &t, &mode)) return rc;
  if (n_rows < 0) return fail(AKV_ERR_ARG, "n_rows < 0");
  if (n_rows == 0) return AKV_OK;
  if (!x || !packed) return fail(AKV_ERR_ARG, "akv_hybrid_encode: null pointer");
  if (x_dtype < AKV_F16 || x_dtype > AKV_F32) return fail(AKV_ERR_ARG, "bad x_dtype %d", x_dtype);
  cudaStream_t st = (cudaStream_t)stream;
  if (x_dtype != AKV_F32) {
    if (mode == 35)
      return launch_hybrid_encode16<64, 3, 64, 2>(x, x_dtype, n_rows, x_row_stride, t, packed, packed_row_stride, st);
    return launch_hybrid_encode16<32, 2, 96, 1>(x, x_dtype, n_rows, x_row_stride, t, packed, packed_row_stride, st);
  }
  const int grid = (int)((n_rows + HY_THREADS - 1) / HY_THREADS);
  if (mode == 35)
    hybrid_encode_kernel<64, 3, 64, 2><<<grid, HY_THREADS, 0, st>>>(x, x_dtype, n_rows, x_row_stride, t, packed, packed_row_stride);
  else
    hybrid_encode_kernel<32, 2, 96, 1><<<grid, HY_THREADS, 0, st>>>(x, x_dtype, n_rows, x_row_stride, t, packed, packed_row_stride);
  return check_launch("hybrid_encode_kernel");
}

AKV_EXPORT int akv_hybrid_decode(const uint8_t* packed, int64_t packed_row_stride, int64_t n_rows,
                                 const akv_hybrid_tables* tables, void* out, int out_dtype, void* stream) {
  HybridTables t; int mode;
  if (int rc = tables_from(tables, &t, &mode)) return rc;
  if (n_rows < 0) return fail(AKV_ERR_ARG, "n_rows < 0");
  if (n_rows == 0) return AKV_OK;
  if (!packed || !out) return fail(AKV_ERR_ARG, "akv_hybrid_decode: null pointer");
  if (out_dtype < AKV_F16 || out_dtype > AKV_F32) return fail(AKV_ERR_ARG, "bad out_dtype %d", out_dtype);
  const int grid = (int)((n_rows + HY_THREADS - 1) / HY_THREADS);
  cudaStream_t st = (cudaStream_t)stream;
  if (mode == 35)
    hybrid_decode_kernel<64, 3, 64, 2><<<grid, HY_THREADS, 0, st>>>(packed, packed_row_stride, n_rows, t, out, out_dtype);
  else
    hybrid_decode_kernel<32, 2, 96, 1><<<grid, HY_THREADS, 0, st>>>(packed, packed_row_stride, n_rows, t, out, out_dtype);
  return check_launch("hybrid_decode_kernel");
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
  int b = bps_in > 0 ? bps_in : (1024 + block_size - 1) / block_size;
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

AKV_EXPORT size_t akv_hybrid_paged_attn_workspace_bytes(int num_seqs, int num_q_heads, int block_size,
                                                        int max_blocks_per_seq, int blocks_per_split) {
  if (num_seqs <= 0 || num_q_heads <= 0 || block_size <= 0) return 0;
  int bps, parts; size_t a, m, total;
  hybrid_plan(num_seqs, num_q_heads, block_size, max_blocks_per_seq, blocks_per_split, &bps, &parts, &a, &m, &total);
  return total;
}

AKV_EXPORT int akv_hybrid_paged_attn(const akv_hybrid_attn_params* p) {
  if (!p) return fail(AKV_ERR_ARG, "null params");
  HybridTables t; int mode;
  if (int rc = tables_from(p->tables, &t, &mode)) return rc;
  if (mode != 35) return fail(AKV_ERR_UNSUPPORTED, "hybrid paged attention is built for tq35 (64-byte records)");
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
  hybrid_qprime_kernel<<<rows, 32, 0, st>>>(p->query, p->q_dtype, p->q_stride_seq, p->q_stride_head,
                                            p->num_q_heads, t, p->scale * 1.4426950408889634f, qprime);
  if (int rc = check_launch("hybrid_qprime_kernel")) return rc;
  if (p->max_blocks_per_seq > 0) {
    HybridAttnArgs a{};
    a.k_cache = p->k_cache; a.v_cache = p->v_cache;
    a.k_sb = p->k_stride_blk; a.k_sp = p->k_stride_pos; a.k_sh = p->k_stride_head;
    a.v_sb = p->v_stride_blk; a.v_sp = p->v_stride_pos; a.v_sh = p->v_stride_head;
    a.block_tables = p->block_tables; a.bt_dtype = p->bt_dtype; a.bt_stride = p->bt_stride_seq;
    a.context_lens = p->context_lens; a.cl_dtype = p->cl_dtype;
    a.num_q_heads = p->num_q_heads; a.num_kv_heads = p->num_kv_heads; a.block_size = p->block_size;
    a.num_blocks = p->num_blocks; a.blocks_per_split = bps; a.num_parts = parts;
    a.qprime = qprime; a.centroids = t.centroids; a.part_acc = part_acc; a.part_ml = part_ml;
    dim3 grid(parts / HA_WARPS, p->num_kv_heads, p->num_seqs);
    hybrid_attn_kernel<<<grid, HA_WARPS * 32, 0, st>>>(a);
    if (int rc = check_launch("hybrid_attn_kernel")) return rc;
  }
  hybrid_merge_kernel<<<rows, 32, 0, st>>>(part_acc, part_ml, p->max_blocks_per_seq > 0 ? parts : 0,
                                           p->context_lens, p->cl_dtype, bps * p->block_size, p->num_q_heads, t,
                                           p->out, p->out_dtype, p->out_stride_seq, p->out_stride_head);
  return check_launch("hybrid_merge_kernel");
}
