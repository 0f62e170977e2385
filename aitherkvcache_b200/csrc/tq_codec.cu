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

namespace akv {

// ---------------------------------------------------------------------------
// Row addressing shared by the contiguous and the paged variants.
// ---------------------------------------------------------------------------
struct RowMap {
  // input
  const void* x;
  int x_dtype;
  int64_t x_stride_row;   // contiguous mode: elements between rows
  int64_t x_stride_tok;   // paged mode: elements between tokens
  int64_t x_stride_head;  // paged mode: elements between heads
  // output
  uint8_t* packed;
  float* norms;
  int64_t p_stride_row;   // contiguous mode: bytes between packed rows
  // paged mode
  const int64_t* slot_mapping;  // nullptr => contiguous mode
  int num_heads;
  int block_size;
  int64_t max_blocks;
  int64_t p_stride_blk, p_stride_pos, p_stride_head;  // bytes
  int64_t n_stride_blk, n_stride_pos, n_stride_head;  // floats
};

struct RowAddr {
  const void* src_base;
  int64_t src_off;   // element offset of the row
  uint8_t* dst;      // nullptr => skip the store
  float* dst_norm;
};

__device__ __forceinline__ RowAddr map_row(const RowMap& m, int64_t n) {
  RowAddr a;
  a.src_base = m.x;
  if (m.slot_mapping == nullptr) {
    a.src_off = n * m.x_stride_row;
    a.dst = m.packed + n * m.p_stride_row;
    a.dst_norm = m.norms + n;
    return a;
  }
  int64_t t = n / m.num_heads;
  int h = (int)(n - t * m.num_heads);
  a.src_off = t * m.x_stride_tok + h * m.x_stride_head;
  int64_t slot = m.slot_mapping[t];
  a.dst = nullptr;
  a.dst_norm = nullptr;
  if (slot >= 0) {
    int64_t blk = slot / m.block_size;
    int pos = (int)(slot - blk * m.block_size);
    if (blk < m.max_blocks) {
      a.dst = m.packed + blk * m.p_stride_blk + pos * m.p_stride_pos + h * m.p_stride_head;
      a.dst_norm = m.norms + blk * m.n_stride_blk + pos * m.n_stride_pos + h * m.n_stride_head;
    }
  }
  return a;
}

// Sum of squares of `d` floats spaced `stride` apart, in the reference's order.
// Called by 8 consecutive lanes (j = lane & 7); every one of them returns the total.
__device__ __forceinline__ float sumsq_8lane(const float* row, int d, int j, unsigned mask) {
  float s = 0.f;
  for (int i = j; i < d; i += 8) s = __fadd_rn(s, __fmul_rn(row[i], row[i]));
  int base = (threadIdx.x & 31) & ~7;
  float tot = __shfl_sync(mask, s, base);
#pragma unroll
  for (int k = 1; k < 8; ++k) tot = __fadd_rn(tot, __shfl_sync(mask, s, base + k));
  return tot;
}

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
  // one CTA per vector: thread o produces outputs o, o+128, ...
  extern __shared__ __align__(16) float smem_f[];
  float* u = smem_f;                                        // [D]
  uint8_t* codes = reinterpret_cast<uint8_t*>(u + D);       // [D]
  __shared__ float s_nrm;
  const int tid = threadIdx.x;
  const int nb = (1 << bits) - 1;
  const int pd = D * bits / 8;
  for (int64_t n = blockIdx.x; n < n_rows; n += gridDim.x) {
    RowAddr a = map_row(m, n);
    for (int i = tid; i < D; i += 128) u[i] = load_as_float(a.src_base, m.x_dtype, a.src_off + i);
    __syncthreads();
    if (tid < 32) {
      float tot = sumsq_8lane(u, D, tid & 7, 0xffffffffu);
      if (tid == 0) s_nrm = __fsqrt_rn(tot);
    }
    __syncthreads();
    const float nrm = s_nrm;
    const float den = __fadd_rn(nrm, 1e-10f);
    for (int i = tid; i < D; i += 128) u[i] = __fdiv_rn(u[i], den);
    __syncthreads();
    for (int o = tid; o < D; o += 128) {
      float y = 0.f;      // one chain in the order j = 0..D-1 (bit-identical to the tiled kernel)
      for (int j0 = 0; j0 < D; j0 += 8) {    // 8 loads in flight per round (D is a multiple of 8)
        float r[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) r[k] = rot_t[(int64_t)(j0 + k) * D + o];
#pragma unroll
        for (int k = 0; k < 8; ++k) y = __fmaf_rn(u[j0 + k], r[k], y);
      }
      int c = 0;
      for (int k = 0; k < nb; ++k) c += (boundaries[k] < y) ? 1 : 0;
      codes[o] = (uint8_t)c;
    }
    __syncthreads();
    if (a.dst != nullptr) {
      for (int bi = tid; bi < pd; bi += 128) {
        int val = 0;
        for (int bit = 0; bit < 8; ++bit) {
          int pos = bi * 8 + bit;
          int k = pos / bits, off = pos - k * bits;
          val = (val << 1) | ((codes[k] >> (bits - 1 - off)) & 1);
        }
        a.dst[bi] = (uint8_t)val;
      }
      if (tid == 0) *a.dst_norm = nrm;
    }
    __syncthreads();
  }
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
