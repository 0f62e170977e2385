// Uniform TurboQuant codec kernels: fused encode (contiguous or paged scatter
// write) and decode.
//
// Semantics follow the reference's torch path
//   aither_kvcache/quantizer.py:122-212        (encode / decode)
//   aither_kvcache/fused_kv_update.py:220-293  (paged write, slot_mapping rules)
//   aither_kvcache/packing.py:13-98            (MSB-first byte format)
// with these bit-level rules:
//   * norm = sqrtf of eight strided float32 partial sums of squares, squares and
//     adds rounded separately, lanes folded 0..7 (this is the rounding order of
//     the CPU reduction the reference calls, so norms come out bit-equal);
//   * u = x / (norm + 1e-10f) with IEEE division;
//   * y_i = sum_j R[i][j] * u_j accumulated with float32 FMA in the order j = 0..D-1;
//   * code = number of boundaries strictly below y (searchsorted "left").
#include "common.cuh"
#include "tq_rowmap.cuh"
#include "tq_encode_generic.cuh"
#include <stdlib.h>

namespace akv {

__device__ __forceinline__ int quantize(float y, const float* bnd, int nb) {
  int c = 0;
  for (int k = 0; k < nb; ++k) c += (bnd[k] < y) ? 1 : 0;
  return c;
}

// Store 8 consecutive codes (a multiple-of-8 offset `o8` into the row).
template <int BITS>
__device__ __forceinline__ void store_codes8(uint8_t* row, int o8, const int* c) {
  if (BITS == 4) {
    uint32_t w = 0;
#pragma unroll
    for (int k = 0; k < 4; ++k) w |= (uint32_t)((c[2 * k] << 4) | c[2 * k + 1]) << (8 * k);
    uint8_t* p = row + o8 / 2;
    if ((reinterpret_cast<uintptr_t>(p) & 3) == 0) {
      *reinterpret_cast<uint32_t*>(p) = w;
    } else {
#pragma unroll
      for (int k = 0; k < 4; ++k) p[k] = (uint8_t)(w >> (8 * k));
    }
  } else if (BITS == 2) {
    uint8_t* p = row + o8 / 4;
    p[0] = (uint8_t)((c[0] << 6) | (c[1] << 4) | (c[2] << 2) | c[3]);
    p[1] = (uint8_t)((c[4] << 6) | (c[5] << 4) | (c[6] << 2) | c[7]);
  } else {
    uint32_t w = 0;
#pragma unroll
    for (int k = 0; k < 8; ++k) w |= (uint32_t)(c[k] & 7) << (21 - 3 * k);
    uint8_t* p = row + (o8 / 8) * 3;
    p[0] = (uint8_t)(w >> 16);
    p[1] = (uint8_t)(w >> 8);
    p[2] = (uint8_t)w;
  }
}

// ---------------------------------------------------------------------------
// Tiled kernels for D in {64, 128}: the whole D x D matrix lives in shared
// memory (64 KB at D = 128) and a persistent CTA walks tiles of TV vectors.
// 256 threads; thread (ty, tx) owns 4 vectors x 8 consecutive outputs.
// ---------------------------------------------------------------------------
template <int D>
struct Tile {
  static constexpr int TX = D / 8;          // threads across outputs
  static constexpr int TY = 256 / TX;       // thread rows
  static constexpr int TV = TY * 4;         // vectors per tile
  static constexpr int LDX = D + 4;         // padded row of the vector tile
  static constexpr size_t SMEM = (size_t)(D * D + TV * LDX + 64) * sizeof(float);
};

// Column o of the matrix is kept at this position of a shared-memory row so that
// a thread's outputs tx*8 .. tx*8+7 are two float4 reads that are contiguous
// across the threads of a warp (no bank conflicts).
template <int D>
__device__ __forceinline__ int smem_col(int o) {
  int tx = o >> 3, b = o & 7;
  return (b < 4) ? (tx * 4 + b) : (D / 2 + tx * 4 + (b - 4));
}

template <int D>
__device__ __forceinline__ void tile_gemm(const float* __restrict__ Bs, const float* __restrict__ xs,
                                          int ty, int tx, float (&acc)[4][8]) {
  using T = Tile<D>;
#pragma unroll
  for (int a = 0; a < 4; ++a)
#pragma unroll
    for (int b = 0; b < 8; ++b) acc[a][b] = 0.f;
  for (int j4 = 0; j4 < D; j4 += 4) {
    float4 u[4];
#pragma unroll
    for (int a = 0; a < 4; ++a)
      u[a] = *reinterpret_cast<const float4*>(xs + (ty * 4 + a) * T::LDX + j4);
#pragma unroll
    for (int jj = 0; jj < 4; ++jj) {
      const float* brow = Bs + (j4 + jj) * D;
      float4 b0 = *reinterpret_cast<const float4*>(brow + tx * 4);
      float4 b1 = *reinterpret_cast<const float4*>(brow + D / 2 + tx * 4);
      float bv[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
#pragma unroll
      for (int a = 0; a < 4; ++a) {
        float ua = jj == 0 ? u[a].x : jj == 1 ? u[a].y : jj == 2 ? u[a].z : u[a].w;
#pragma unroll
        for (int b = 0; b < 8; ++b) acc[a][b] = __fmaf_rn(ua, bv[b], acc[a][b]);
      }
    }
  }
}

// rot_t: the rotation transposed, rot_t[j*D + i] = R[i][j].
template <int D, int BITS>
__global__ void __launch_bounds__(256, 2)
tq_encode_tiled_kernel(RowMap m, int64_t n_rows, const float* __restrict__ rot_t,
                       const float* __restrict__ boundaries) {
  using T = Tile<D>;
  extern __shared__ __align__(16) float smem_f[];
  float* Bs = smem_f;                 // [D][D] permuted columns
  float* xs = Bs + D * D;             // [TV][LDX]
  float* bnd = xs + T::TV * T::LDX;   // [<=15] boundaries, then +inf padding
  constexpr int NB = (1 << BITS) - 1;

  const int tid = threadIdx.x;
  for (int e = tid; e < D * D; e += 256) {
    int j = e / D, o = e % D;
    Bs[j * D + smem_col<D>(o)] = rot_t[e];
  }
  if (tid < NB) bnd[tid] = boundaries[tid];
  __syncthreads();

  const int tx = tid % T::TX, ty = tid / T::TX;
  const int64_t num_tiles = (n_rows + T::TV - 1) / T::TV;
  for (int64_t tile = blockIdx.x; tile < num_tiles; tile += gridDim.x) {
    const int64_t row0 = tile * T::TV;
    // 1) load the tile as float32
    constexpr int TPR = D / 8;  // threads per row, 8 elements each
    for (int r = tid / TPR; r < T::TV; r += 256 / TPR) {
      int64_t n = row0 + r;
      float* dst = xs + r * T::LDX + (tid % TPR) * 8;
      if (n < n_rows) {
        RowAddr a = map_row(m, n);
        int64_t off = a.src_off + (tid % TPR) * 8;
#pragma unroll
        for (int k = 0; k < 8; ++k) dst[k] = load_as_float(a.src_base, m.x_dtype, off + k);
      } else {
#pragma unroll
        for (int k = 0; k < 8; ++k) dst[k] = 0.f;
      }
    }
    __syncthreads();
    // 2) norms (8 lanes per row) and normalisation
    for (int r = tid / 8; r < T::TV; r += 32) {
      float* row = xs + r * T::LDX;
      float tot = sumsq_8lane(row, D, tid & 7, 0xffffffffu);
      float nrm = __fsqrt_rn(tot);
      float den = __fadd_rn(nrm, 1e-10f);
      for (int i = (tid & 7); i < D; i += 8) row[i] = __fdiv_rn(row[i], den);
      if ((tid & 7) == 0) {
        int64_t n = row0 + r;
        if (n < n_rows) {
          RowAddr a = map_row(m, n);
          if (a.dst_norm) *a.dst_norm = nrm;
        }
      }
    }
    __syncthreads();
    // 3) rotate, quantise, pack
    float acc[4][8];
    tile_gemm<D>(Bs, xs, ty, tx, acc);
#pragma unroll
    for (int a = 0; a < 4; ++a) {
      int64_t n = row0 + ty * 4 + a;
      if (n >= n_rows) continue;
      RowAddr ra = map_row(m, n);
      if (ra.dst == nullptr) continue;
      int c[8];
#pragma unroll
      for (int b = 0; b < 8; ++b) c[b] = quantize(acc[a][b], bnd, NB);
      store_codes8<BITS>(ra.dst, tx * 8, c);
    }
    __syncthreads();
  }
}

// rot: R row-major (x_hat_j = sum_i y_hat_i R[i][j]).
template <int D, int BITS>
__global__ void __launch_bounds__(256, 2)
tq_decode_tiled_kernel(const uint8_t* __restrict__ packed, int64_t p_stride_row,
                       const float* __restrict__ norms, int64_t n_rows,
                       const float* __restrict__ rot, const float* __restrict__ centroids,
                       void* out, int out_dtype) {
  using T = Tile<D>;
  extern __shared__ __align__(16) float smem_f[];
  float* Bs = smem_f;
  float* xs = Bs + D * D;
  float* cent = xs + T::TV * T::LDX;
  constexpr int PD = D * BITS / 8;

  const int tid = threadIdx.x;
  for (int e = tid; e < D * D; e += 256) {
    int i = e / D, j = e % D;
    Bs[i * D + smem_col<D>(j)] = rot[e];
  }
  if (tid < (1 << BITS)) cent[tid] = centroids[tid];
  __syncthreads();

  const int tx = tid % T::TX, ty = tid / T::TX;
  const int64_t num_tiles = (n_rows + T::TV - 1) / T::TV;
  for (int64_t tile = blockIdx.x; tile < num_tiles; tile += gridDim.x) {
    const int64_t row0 = tile * T::TV;
    for (int e = tid; e < T::TV * D; e += 256) {
      int r = e / D, k = e % D;
      int64_t n = row0 + r;
      float v = 0.f;
      if (n < n_rows) v = cent[extract_code(packed + n * p_stride_row, k, BITS, PD)];
      xs[r * T::LDX + k] = v;
    }
    __syncthreads();
    float acc[4][8];
    tile_gemm<D>(Bs, xs, ty, tx, acc);
#pragma unroll
    for (int a = 0; a < 4; ++a) {
      int64_t n = row0 + ty * 4 + a;
      if (n >= n_rows) continue;
      float nrm = norms[n];
      int64_t o = n * D + tx * 8;
      if (out_dtype == AKV_F16) {
        __align__(16) __half h[8];
#pragma unroll
        for (int b = 0; b < 8; ++b) h[b] = __float2half_rn(__fmul_rn(acc[a][b], nrm));
        *reinterpret_cast<uint4*>(reinterpret_cast<__half*>(out) + o) = *reinterpret_cast<uint4*>(h);
      } else {
#pragma unroll
        for (int b = 0; b < 8; ++b) store_from_float(out, out_dtype, o + b, __fmul_rn(acc[a][b], nrm));
      }
    }
    __syncthreads();
  }
}

// ---------------------------------------------------------------------------
// Any power-of-two head_dim up to 1024: one warp per vector, the matrix is read
// through L2.  Slow path for shapes outside {64, 128}.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(128)
tq_encode_generic_kernel(RowMap m, int64_t n_rows, int D, int bits, const float* __restrict__ rot_t,
                         const float* __restrict__ boundaries) {
  encode_generic_rows(m, blockIdx.x, gridDim.x, n_rows, D, bits, rot_t, boundaries);
}

// The K and the V vectors of a decode step in one launch: blockIdx.y picks the tensor.
__global__ void __launch_bounds__(128)
tq_encode_generic_pair_kernel(RowMap mk, RowMap mv, int64_t n_rows, int D, int bits,
                              const float* __restrict__ rot_t, const float* __restrict__ boundaries) {
  encode_generic_rows(blockIdx.y ? mv : mk, blockIdx.x, gridDim.x, n_rows, D, bits, rot_t, boundaries);
}

__global__ void __launch_bounds__(128)
tq_decode_generic_kernel(const uint8_t* __restrict__ packed, int64_t p_stride_row,
                         const float* __restrict__ norms, int64_t n_rows, int D, int bits,
                         const float* __restrict__ rot, const float* __restrict__ centroids,
                         void* out, int out_dtype) {
  extern __shared__ __align__(16) float smem_f[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float* yh = smem_f + warp * D;
  const int pd = D * bits / 8;
  for (int64_t n = (int64_t)blockIdx.x * 4 + warp; n < n_rows; n += (int64_t)gridDim.x * 4) {
    const uint8_t* row = packed + n * p_stride_row;
    for (int k = lane; k < D; k += 32) yh[k] = centroids[extract_code(row, k, bits, pd)];
    __syncwarp();
    float nrm = norms[n];
    for (int j = lane; j < D; j += 32) {
      float x = 0.f;
      for (int i0 = 0; i0 < D; i0 += 8) {
        float r[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) r[k] = rot[(int64_t)(i0 + k) * D + j];
#pragma unroll
        for (int k = 0; k < 8; ++k) x = __fmaf_rn(yh[i0 + k], r[k], x);
      }
      store_from_float(out, out_dtype, n * D + j, __fmul_rn(x, nrm));
    }
    __syncwarp();
  }
}

// ---------------------------------------------------------------------------
// Tensor-core encode for 16-bit inputs, D in {64, 128}.
//
// The rotation is float32; a 16-bit input times a float32 matrix is computed on
// the tensor cores by splitting every matrix entry into 16-bit terms whose sum
// carries it to 2^-22 or better (fp16 input: two fp16 terms, the second scaled by
// 2^11 into its own accumulator; bf16 input: three bf16 terms, one accumulator).
// The products are exact, the accumulation is float32.  The vector is rotated
// before it is normalised (y = (R x) * (1 / (norm + 1e-10f))), so y differs from
// the scalar kernels' value by a few float32 ulps: codes can differ only for a
// coordinate that lies within ~2e-7 of a boundary.  Norms are bit-equal (same
// eight-lane summation).
//
// 8 warps per CTA, one CTA per SM, no CTA barrier in the main loop: each warp
// owns tiles of 32 vectors, stages them in its own 32 x D 16-bit buffer
// (16-byte chunks XOR-swizzled by row), and reuses the buffer for the codes.
// ---------------------------------------------------------------------------
template <int D, bool BF16>
struct MmaEnc {
  static constexpr int TERMS = BF16 ? 3 : 2;
  static constexpr int ROWB = D * 2;
  static constexpr int TERM_BYTES = D * ROWB;
  static constexpr int STAGE_BYTES = 32 * ROWB;
  static constexpr int CELLS = 256;
  static constexpr size_t SMEM = (size_t)TERMS * TERM_BYTES + 8 * STAGE_BYTES + CELLS * 8 + 64;
  static constexpr int CODE_STRIDE = D + 4;   // bytes per row of the code staging (odd word count)
};

__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t (&r)[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}

template <bool BF16>
__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  if (BF16) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  } else {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  }
}

template <bool BF16>
__device__ __forceinline__ float half_bits_to_float(uint32_t h) {
  if (BF16) return __uint_as_float(h << 16);
  return __half2float(__ushort_as_half((unsigned short)h));
}

template <int D, int BITS, bool BF16>
__global__ void __launch_bounds__(256, 1)
tq_encode_mma_kernel(RowMap m, int64_t n_rows, const float* __restrict__ rot_t,
                     const float* __restrict__ boundaries) {
  using E = MmaEnc<D, BF16>;
  constexpr int TERMS = E::TERMS, ROWB = E::ROWB, CH = D / 8, KK = D / 16, NB = (1 << BITS) - 1;
  constexpr int CELLS = E::CELLS, PD = D * BITS / 8;
  extern __shared__ __align__(128) uint8_t smem_b[];
  uint8_t* terms = smem_b;
  uint8_t* stage_all = terms + TERMS * E::TERM_BYTES;
  float2* lut = reinterpret_cast<float2*>(stage_all + 8 * E::STAGE_BYTES);
  float* bnd = reinterpret_cast<float*>(lut + CELLS);
  __shared__ int s_simple;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  // ---- one-time setup: split matrix, boundaries, cell table ----
  if (tid == 0) s_simple = 1;
  if (tid < 16) bnd[tid] = tid < NB ? boundaries[tid] : __int_as_float(0x7f800000);
  for (int e = tid; e < D * D; e += 256) {
    int j = e / D, i = e % D;          // rot_t[j][i] = R[i][j]
    float r = rot_t[e];
    uint32_t off = (uint32_t)(i * ROWB + ((((j >> 3) ^ (i & 7)) << 4) | ((j & 7) << 1)));
    if (BF16) {
      __nv_bfloat16 t1 = __float2bfloat16_rn(r);
      float e1 = r - __bfloat162float(t1);
      __nv_bfloat16 t2 = __float2bfloat16_rn(e1);
      float e2 = e1 - __bfloat162float(t2);
      __nv_bfloat16 t3 = __float2bfloat16_rn(e2);
      *reinterpret_cast<__nv_bfloat16*>(terms + off) = t1;
      *reinterpret_cast<__nv_bfloat16*>(terms + E::TERM_BYTES + off) = t2;
      *reinterpret_cast<__nv_bfloat16*>(terms + 2 * E::TERM_BYTES + off) = t3;
    } else {
      __half t1 = __float2half_rn(r);
      float e1 = (r - __half2float(t1)) * 2048.f;
      *reinterpret_cast<__half*>(terms + off) = t1;
      *reinterpret_cast<__half*>(terms + E::TERM_BYTES + off) = __float2half_rn(e1);
    }
  }
  __syncthreads();
  // Cell table over [b_first - 4w, b_last + 4w): cell c answers for y in cells c-1..c+1
  // (the cell index is computed in float32 and may be off by one).
  const float b_first = bnd[0], b_last = bnd[NB - 1];
  const float cw = (b_last - b_first) / (float)(CELLS - 8);
  const float inv_cw = 1.0f / cw;
  const float cell_off = 4.0f - b_first * inv_cw;
  {
    int c = tid;
    float lo_edge = b_first + (float)(c - 4 - 1) * cw;
    float hi_edge = b_first + (float)(c - 4 + 2) * cw;
    int base = 0, cnt = 0;
    for (int k = 0; k < NB; ++k) {
      bool below = (c > 0) && (bnd[k] < lo_edge);
      bool above = (c < CELLS - 1) && (bnd[k] >= hi_edge);
      base += below ? 1 : 0;
      cnt += (!below && !above) ? 1 : 0;
    }
    lut[c] = make_float2(cnt > 0 ? bnd[base] : __int_as_float(0x7f800000), __int_as_float(base));
    if (cnt > 1 || !(cw > 0.f) || !(inv_cw < 3.0e38f)) s_simple = 0;
  }
  __syncthreads();
  const bool simple = s_simple != 0;

  uint8_t* stage = stage_all + warp * E::STAGE_BYTES;
  const uint32_t stage_s = (uint32_t)__cvta_generic_to_shared(stage);
  const uint32_t terms_s = (uint32_t)__cvta_generic_to_shared(terms);
  const int g = lane >> 2, t = lane & 3, q = lane >> 3, l7 = lane & 7;
  // ldmatrix lane addresses: A (rows of the vector tile) and B (rows of the matrix)
  const uint32_t a_base = stage_s + (uint32_t)(((q & 1) * 8 + l7) * ROWB);
  const uint32_t a_x = (uint32_t)(((q >> 1) ^ l7) << 4);
  const uint32_t b_base = terms_s + (uint32_t)(((q >> 1) * 8 + l7) * ROWB);
  const uint32_t b_x = (uint32_t)(((q & 1) ^ l7) << 4);

  const int64_t num_tiles = (n_rows + 31) >> 5;
  for (int64_t tile = (int64_t)blockIdx.x * 8 + warp; tile < num_tiles; tile += (int64_t)gridDim.x * 8) {
    const int64_t row0 = tile << 5;
    // lane <-> row mapping for loads of the row address, the norm and the stores
    const int64_t n_mine = row0 + lane;
    const bool valid = n_mine < n_rows;
    RowAddr ra = map_row(m, valid ? n_mine : n_rows - 1);
    // ---- stage the tile: coalesced 16-byte loads, swizzled stores ----
    constexpr int RPI = 32 / CH;        // rows covered by one warp-wide load
    constexpr int ITERS = 32 / RPI;
    const int sub = lane / CH, c16 = lane % CH;
#pragma unroll
    for (int i0 = 0; i0 < ITERS; i0 += 8) {
      uint4 v[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        int row = (i0 + i) * RPI + sub;
        int64_t off = __shfl_sync(0xffffffffu, ra.src_off, row);
        bool ok = __shfl_sync(0xffffffffu, (int)valid, row) != 0;
        v[i] = make_uint4(0u, 0u, 0u, 0u);
        if (ok) v[i] = *reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(m.x) + off + c16 * 8);
      }
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        int row = (i0 + i) * RPI + sub;
        *reinterpret_cast<uint4*>(stage + row * ROWB + ((c16 ^ (row & 7)) << 4)) = v[i];
      }
    }
    __syncwarp();
    // ---- norm of row `lane`, in the reference's summation order ----
    float s8[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) s8[j] = 0.f;
#pragma unroll
    for (int c = 0; c < CH; ++c) {
      uint4 w = *reinterpret_cast<const uint4*>(stage + lane * ROWB + ((c ^ l7) << 4));
      uint32_t ww[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        float lo = half_bits_to_float<BF16>(ww[k] & 0xffffu);
        float hi = half_bits_to_float<BF16>(ww[k] >> 16);
        s8[2 * k] = __fadd_rn(s8[2 * k], __fmul_rn(lo, lo));
        s8[2 * k + 1] = __fadd_rn(s8[2 * k + 1], __fmul_rn(hi, hi));
      }
    }
    float tot = s8[0];
#pragma unroll
    for (int j = 1; j < 8; ++j) tot = __fadd_rn(tot, s8[j]);
    const float nrm = __fsqrt_rn(tot);
    const float rinv = __frcp_rn(__fadd_rn(nrm, 1e-10f));
    float rinv_r[2][2];
#pragma unroll
    for (int mt = 0; mt < 2; ++mt)
#pragma unroll
      for (int h = 0; h < 2; ++h) rinv_r[mt][h] = __shfl_sync(0xffffffffu, rinv, mt * 16 + h * 8 + g);
    // ---- A fragments of both 16-row halves ----
    uint32_t af[2][KK][4];
#pragma unroll
    for (int mt = 0; mt < 2; ++mt)
#pragma unroll
      for (int kk = 0; kk < KK; ++kk)
        ldsm_x4(a_base + (uint32_t)(mt * 16 * ROWB) + (((uint32_t)kk << 5) ^ a_x), af[mt][kk]);
    __syncwarp();
    // ---- rotate 32 outputs at a time, quantise, park the codes in the stage buffer ----
    uint8_t* codes = stage;
#pragma unroll 1
    for (int nc = 0; nc < D / 32; ++nc) {
      constexpr int NACC = BF16 ? 1 : 2;
      float acc[NACC][2][4][4];
#pragma unroll
      for (int a = 0; a < NACC; ++a)
#pragma unroll
        for (int mt = 0; mt < 2; ++mt)
#pragma unroll
          for (int nq = 0; nq < 4; ++nq)
#pragma unroll
            for (int k = 0; k < 4; ++k) acc[a][mt][nq][k] = 0.f;
#pragma unroll
      for (int kk = 0; kk < KK; ++kk) {
#pragma unroll
        for (int p = 0; p < 2; ++p) {
#pragma unroll
          for (int tm = 0; tm < TERMS; ++tm) {
            uint32_t bf[4];
            ldsm_x4(b_base + (uint32_t)(tm * E::TERM_BYTES + (nc * 4 + 2 * p) * 8 * ROWB) +
                        (((uint32_t)kk << 5) ^ b_x), bf);
            constexpr int dummy = 0; (void)dummy;
            const int a = BF16 ? 0 : tm;
#pragma unroll
            for (int mt = 0; mt < 2; ++mt) {
              mma16816<BF16>(acc[a][mt][2 * p], af[mt][kk], bf[0], bf[1]);
              mma16816<BF16>(acc[a][mt][2 * p + 1], af[mt][kk], bf[2], bf[3]);
            }
          }
        }
      }
#pragma unroll
      for (int mt = 0; mt < 2; ++mt)
#pragma unroll
        for (int nq = 0; nq < 4; ++nq)
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            int cc[2];
#pragma unroll
            for (int k = 0; k < 2; ++k) {
              float v = acc[0][mt][nq][2 * h + k];
              if (!BF16) v = __fmaf_rn(acc[NACC - 1][mt][nq][2 * h + k], 1.0f / 2048.f, v);
              float y = __fmul_rn(v, rinv_r[mt][h]);
              int c;
              if (simple) {
                int ci = __float2int_rd(__fmaf_rn(y, inv_cw, cell_off));
                ci = min(max(ci, 0), CELLS - 1);
                float2 e = lut[ci];
                c = __float_as_int(e.y) + ((e.x < y) ? 1 : 0);
              } else {
                c = quantize(y, bnd, NB);
              }
              cc[k] = c;
            }
            int row = mt * 16 + h * 8 + g;
            int col = (nc * 4 + nq) * 8 + 2 * t;
            *reinterpret_cast<uint16_t*>(codes + row * E::CODE_STRIDE + col) = (uint16_t)(cc[0] | (cc[1] << 8));
          }
    }
    __syncwarp();
    // ---- pack row `lane` and store ----
    if (valid && ra.dst != nullptr) {
      uint32_t pw[PD / 4];
#pragma unroll
      for (int k = 0; k < PD / 4; ++k) pw[k] = 0u;
      const uint32_t* crow = reinterpret_cast<const uint32_t*>(codes + lane * E::CODE_STRIDE);
      if (BITS == 4) {
#pragma unroll
        for (int k = 0; k < PD / 4; ++k) {
          uint32_t w0 = crow[2 * k], w1 = crow[2 * k + 1];
          uint32_t v0 = (w0 << 4) | (w0 >> 8), v1 = (w1 << 4) | (w1 >> 8);
          pw[k] = __byte_perm(v0, v1, 0x6420);
        }
      } else if (BITS == 2) {
#pragma unroll
        for (int b = 0; b < PD; ++b) {
          uint32_t w = crow[b];
          uint32_t byte = ((w & 3u) << 6) | (((w >> 8) & 3u) << 4) | (((w >> 16) & 3u) << 2) | ((w >> 24) & 3u);
          pw[b >> 2] |= byte << (8 * (b & 3));
        }
      } else {
#pragma unroll
        for (int g8 = 0; g8 < D / 8; ++g8) {
          uint32_t w0 = crow[2 * g8], w1 = crow[2 * g8 + 1];
          uint32_t v = ((w0 & 7u) << 21) | (((w0 >> 8) & 7u) << 18) | (((w0 >> 16) & 7u) << 15) |
                       (((w0 >> 24) & 7u) << 12) | ((w1 & 7u) << 9) | (((w1 >> 8) & 7u) << 6) |
                       (((w1 >> 16) & 7u) << 3) | ((w1 >> 24) & 7u);
#pragma unroll
          for (int k = 0; k < 3; ++k) {
            int b = 3 * g8 + k;
            pw[b >> 2] |= ((v >> (16 - 8 * k)) & 0xffu) << (8 * (b & 3));
          }
        }
      }
      uintptr_t dp = reinterpret_cast<uintptr_t>(ra.dst);
      if (PD % 16 == 0 && (dp & 15) == 0) {
#pragma unroll
        for (int k = 0; k < PD / 16; ++k)
          reinterpret_cast<uint4*>(ra.dst)[k] = make_uint4(pw[4 * k], pw[4 * k + 1], pw[4 * k + 2], pw[4 * k + 3]);
      } else if ((dp & 3) == 0) {
#pragma unroll
        for (int k = 0; k < PD / 4; ++k) reinterpret_cast<uint32_t*>(ra.dst)[k] = pw[k];
      } else {
#pragma unroll
        for (int b = 0; b < PD; ++b) ra.dst[b] = (uint8_t)(pw[b >> 2] >> (8 * (b & 3)));
      }
      *ra.dst_norm = nrm;
    }
    __syncwarp();
  }
}

template <int D, int BITS, bool BF16>
int launch_encode_mma(const RowMap& m, int64_t n_rows, const float* rot_t, const float* bnd,
                      cudaStream_t st) {
  using E = MmaEnc<D, BF16>;
  auto kern = tq_encode_mma_kernel<D, BITS, BF16>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)E::SMEM);
  if (e != cudaSuccess) return fail((int)e, "encode: smem attribute: %s", cudaGetErrorString(e));
  int64_t ctas = (n_rows + 255) / 256;
  int grid = (int)(ctas < sm_count() ? ctas : sm_count());
  kern<<<grid, 256, E::SMEM, st>>>(m, n_rows, rot_t, bnd);
  return check_launch("tq_encode_mma_kernel");
}

template <int D, int BITS>
int launch_encode_tiled(const RowMap& m, int64_t n_rows, const float* rot_t, const float* bnd,
                        cudaStream_t st) {
  using T = Tile<D>;
  auto kern = tq_encode_tiled_kernel<D, BITS>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)T::SMEM);
  if (e != cudaSuccess) return fail((int)e, "encode: smem attribute: %s", cudaGetErrorString(e));
  int64_t tiles = (n_rows + T::TV - 1) / T::TV;
  int grid = (int)(tiles < 2 * sm_count() ? tiles : 2 * sm_count());
  kern<<<grid, 256, T::SMEM, st>>>(m, n_rows, rot_t, bnd);
  return check_launch("tq_encode_tiled_kernel");
}

template <int D, int BITS>
int launch_decode_tiled(const uint8_t* packed, int64_t ps, const float* norms, int64_t n_rows,
                        const float* rot, const float* cent, void* out, int out_dtype, cudaStream_t st) {
  using T = Tile<D>;
  auto kern = tq_decode_tiled_kernel<D, BITS>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)T::SMEM);
  if (e != cudaSuccess) return fail((int)e, "decode: smem attribute: %s", cudaGetErrorString(e));
  int64_t tiles = (n_rows + T::TV - 1) / T::TV;
  int grid = (int)(tiles < 2 * sm_count() ? tiles : 2 * sm_count());
  kern<<<grid, 256, T::SMEM, st>>>(packed, ps, norms, n_rows, rot, cent, out, out_dtype);
  return check_launch("tq_decode_tiled_kernel");
}

static int encode_dispatch(const RowMap& m, int64_t n_rows, int D, int bits, const float* rot_t,
                           const float* bnd, cudaStream_t st) {
  if (n_rows == 0) return AKV_OK;
  // 16-bit inputs whose rows can be read in 16-byte pieces go to the tensor-core kernel
  const bool half_in = m.x_dtype == AKV_F16 || m.x_dtype == AKV_BF16;
  bool vec_ok = half_in && (reinterpret_cast<uintptr_t>(m.x) & 15) == 0;
  if (m.slot_mapping == nullptr) vec_ok = vec_ok && (m.x_stride_row % 8 == 0);
  else vec_ok = vec_ok && (m.x_stride_tok % 8 == 0) && (m.x_stride_head % 8 == 0);
  static const bool no_mma = getenv("AKV_NO_MMA_ENCODE") != nullptr;
  static const bool no_tc = getenv("AKV_NO_TC_ENCODE") != nullptr;
  if (vec_ok && !no_tc && D == 128 && n_rows >= 2048)
    return launch_encode_tc(m, n_rows, bits, m.x_dtype == AKV_BF16, rot_t, bnd, st);
  if (vec_ok && !no_mma && n_rows >= 2048) {
#define AKV_ENCM(DD, BB)                                                                      \
  if (D == DD && bits == BB)                                                                  \
    return m.x_dtype == AKV_BF16 ? launch_encode_mma<DD, BB, true>(m, n_rows, rot_t, bnd, st) \
                                 : launch_encode_mma<DD, BB, false>(m, n_rows, rot_t, bnd, st);
    AKV_ENCM(128, 4) AKV_ENCM(128, 3) AKV_ENCM(128, 2) AKV_ENCM(64, 4) AKV_ENCM(64, 3) AKV_ENCM(64, 2)
#undef AKV_ENCM
  }
  // small batches (a decode step) are not worth filling 64 KB of shared memory per CTA
#define AKV_ENC(DD, BB) \
  if (D == DD && bits == BB && n_rows >= 2048) return launch_encode_tiled<DD, BB>(m, n_rows, rot_t, bnd, st);
  AKV_ENC(128, 4) AKV_ENC(128, 3) AKV_ENC(128, 2) AKV_ENC(64, 4) AKV_ENC(64, 3) AKV_ENC(64, 2)
#undef AKV_ENC
  size_t smem = (size_t)(D + D / 4 + 16) * sizeof(float);
  int grid = (int)(n_rows < 16 * sm_count() ? n_rows : 16 * sm_count());
  tq_encode_generic_kernel<<<grid, 128, smem, st>>>(m, n_rows, D, bits, rot_t, bnd);
  return check_launch("tq_encode_generic_kernel");
}

// Two small paged writes (the new token's K and V) as one launch of the generic kernel.
int launch_encode_generic_pair(const RowMap& mk, const RowMap& mv, int64_t n_rows, int D, int bits,
                               const float* rot_t, const float* bnd, cudaStream_t st) {
  if (n_rows == 0) return AKV_OK;
  size_t smem = (size_t)(D + D / 4 + 16) * sizeof(float);
  dim3 grid((unsigned)(n_rows < 8 * sm_count() ? n_rows : 8 * sm_count()), 2);
  tq_encode_generic_pair_kernel<<<grid, 128, smem, st>>>(mk, mv, n_rows, D, bits, rot_t, bnd);
  return check_launch("tq_encode_generic_pair_kernel");
}

static int check_codec_args(int head_dim, int bits) {
  if (bits != 2 && bits != 3 && bits != 4)
    return fail(AKV_ERR_ARG, "Supported bit-widths: 2, 3, 4. Got %d", bits);
  if (!is_pow2(head_dim) || head_dim < 8 || head_dim > 1024)
    return fail(AKV_ERR_ARG, "head_dim must be a power of 2 in [8, 1024], got %d", head_dim);
  return AKV_OK;
}

}  // namespace akv

using namespace akv;

AKV_EXPORT int akv_tq_encode(const void* x, int x_dtype, int64_t n_rows, int64_t x_row_stride,
                             int head_dim, int bits, const float* rotation_t,
                             const float* boundaries, uint8_t* packed, int64_t packed_row_stride,
                             float* norms, void* stream) {
  if (int rc = check_codec_args(head_dim, bits)) return rc;
  if (n_rows < 0) return fail(AKV_ERR_ARG, "n_rows < 0");
  if (n_rows > 0 && (!x || !rotation_t || !boundaries || !packed || !norms))
    return fail(AKV_ERR_ARG, "akv_tq_encode: null pointer");
  if (x_dtype < AKV_F16 || x_dtype > AKV_F32) return fail(AKV_ERR_ARG, "bad x_dtype %d", x_dtype);
  RowMap m{};
  m.x = x; m.x_dtype = x_dtype; m.x_stride_row = x_row_stride;
  m.packed = packed; m.norms = norms; m.p_stride_row = packed_row_stride;
  m.slot_mapping = nullptr;
  return encode_dispatch(m, n_rows, head_dim, bits, rotation_t, boundaries, (cudaStream_t)stream);
}

AKV_EXPORT int akv_tq_decode(const uint8_t* packed, int64_t packed_row_stride, const float* norms,
                             int64_t n_rows, int head_dim, int bits, const float* rotation,
                             const float* centroids, void* out, int out_dtype, void* stream) {
  if (int rc = check_codec_args(head_dim, bits)) return rc;
  if (n_rows < 0) return fail(AKV_ERR_ARG, "n_rows < 0");
  if (n_rows == 0) return AKV_OK;
  if (!packed || !norms || !rotation || !centroids || !out)
    return fail(AKV_ERR_ARG, "akv_tq_decode: null pointer");
  if (out_dtype < AKV_F16 || out_dtype > AKV_F32) return fail(AKV_ERR_ARG, "bad out_dtype %d", out_dtype);
  cudaStream_t st = (cudaStream_t)stream;
  const int D = head_dim;
  static const bool no_tc = getenv("AKV_NO_TC_DECODE") != nullptr;
  if (D == 128 && n_rows >= 2048 && !no_tc && (packed_row_stride & 3) == 0 &&
      (reinterpret_cast<uintptr_t>(packed) & 3) == 0 && (reinterpret_cast<uintptr_t>(out) & 15) == 0)
    return launch_decode_tc(packed, packed_row_stride, norms, n_rows, bits, rotation, centroids, out, out_dtype, st);
#define AKV_DEC(DD, BB)            \
  if (D == DD && bits == BB)       \
    return launch_decode_tiled<DD, BB>(packed, packed_row_stride, norms, n_rows, rotation, centroids, out, out_dtype, st);
  AKV_DEC(128, 4) AKV_DEC(128, 3) AKV_DEC(128, 2) AKV_DEC(64, 4) AKV_DEC(64, 3) AKV_DEC(64, 2)
#undef AKV_DEC
  size_t smem = 4 * (size_t)D * sizeof(float);
  int64_t blocks = (n_rows + 3) / 4;
  int grid = (int)(blocks < 8 * sm_count() ? blocks : 8 * sm_count());
  tq_decode_generic_kernel<<<grid, 128, smem, st>>>(packed, packed_row_stride, norms, n_rows, D, bits,
                                                    rotation, centroids, out, out_dtype);
  return check_launch("tq_decode_generic_kernel");
}

AKV_EXPORT int akv_tq_kv_update(const void* x, int x_dtype, int64_t num_tokens, int num_kv_heads,
                                int head_dim, int64_t x_stride_tok, int64_t x_stride_head,
                                const int64_t* slot_mapping, uint8_t* out_packed,
                                int64_t p_stride_blk, int64_t p_stride_pos, int64_t p_stride_head,
                                float* out_norms, int64_t n_stride_blk, int64_t n_stride_pos,
                                int64_t n_stride_head, int bits, const float* rotation_t,
                                const float* boundaries, int block_size, int64_t max_blocks,
                                void* stream) {
  if (int rc = check_codec_args(head_dim, bits)) return rc;
  if (num_tokens < 0 || num_kv_heads <= 0 || block_size <= 0 || max_blocks < 0)
    return fail(AKV_ERR_ARG, "akv_tq_kv_update: bad sizes");
  if (num_tokens == 0 || max_blocks == 0) return AKV_OK;
  if (!x || !slot_mapping || !out_packed || !out_norms || !rotation_t || !boundaries)
    return fail(AKV_ERR_ARG, "akv_tq_kv_update: null pointer");
  if (x_dtype < AKV_F16 || x_dtype > AKV_F32) return fail(AKV_ERR_ARG, "bad x_dtype %d", x_dtype);
  RowMap m{};
  m.x = x; m.x_dtype = x_dtype; m.x_stride_tok = x_stride_tok; m.x_stride_head = x_stride_head;
  m.packed = out_packed; m.norms = out_norms;
  m.slot_mapping = slot_mapping; m.num_heads = num_kv_heads; m.block_size = block_size;
  m.max_blocks = max_blocks;
  m.p_stride_blk = p_stride_blk; m.p_stride_pos = p_stride_pos; m.p_stride_head = p_stride_head;
  m.n_stride_blk = n_stride_blk; m.n_stride_pos = n_stride_pos; m.n_stride_head = n_stride_head;
  return encode_dispatch(m, num_tokens * num_kv_heads, head_dim, bits, rotation_t, boundaries,
                         (cudaStream_t)stream);
}
