// Rotation of many rows at once: out[r][j] = scale * sum_i (src[r][i] * inv_r) * M[i][j], head_dim 128.
//
// The decode path rotates a handful of query rows and partial results per step (akv_qrot128_kernel, akv_merge128_kernel:
// one row per warp, the matrix staged per CTA).  Chunked prefill rotates tens of thousands of rows - the queries of a
// chunk (M = R^T: q_rot = R q, reference fused_attention.py:600-612) and its attention results (M = R, inv_r = 1 / l_r:
// out = R^T (acc / l), fused_attention.py:513-531) - which is a [rows, 128] x [128, 128] GEMM.  It runs on mma.sync
// m16n8k16 with float32 accuracy: the matrix is split into two fp16 terms of 1024 M (the factor keeps the second term
// out of fp16's subnormal range), a float32 source row into two fp16 terms as well, and the product is accumulated as
// a1 M1 + a1 M2 + a2 M1 in float32 (the dropped a2 M2 term is 2^-22 of the result).  A 16-bit source needs one term.
// CTA = 8 warps = a tile of 128 rows (16 per warp), persistent over the tiles; both operands come from shared memory
// (rows padded to 272 bytes: conflict-free 4-byte fragment loads).  With few row tiles the 128 output columns are
// split over 2 or 4 CTAs (gridDim.y), each staging and using only its columns of the matrix, so that a call of a
// few thousand rows still spreads over the GPU.
#include "common.cuh"

namespace akv {
namespace {

constexpr int RR_THREADS = 256;
constexpr int RR_LD = 136;                                   // halves per padded row
constexpr int RR_MAT = 128 * RR_LD * 2;                      // one fp16 term of a 128 x 128 operand
// M1, M2 (as [j][i], the CTA's 8 NJ columns), A1, A2 (as [row][i]); a column-split CTA leaves room for a second one per SM
constexpr int rr_smem(int nj) { return 2 * (8 * nj) * RR_LD * 2 + 2 * RR_MAT; }

struct RotRowsArgs {
  const void* src; int src_dtype; int64_t src_outer, src_inner; int inner;   // row r = (r / inner, r % inner); strides in elements
  const float* inv_l; int64_t inv_stride;                    // optional: row r is divided by inv_l[r * inv_stride] (0 -> zero row)
  const float* mat;                                          // [128][128] row-major
  float scale;
  void* out; int out_dtype; int64_t out_outer, out_inner;
  int64_t rows;
};

__device__ __forceinline__ void rr_mma(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

template <int NJ>        // n-tiles (8 columns each) of this CTA: 16, 8 or 4
__global__ void __launch_bounds__(RR_THREADS, NJ == 16 ? 1 : 2)
akv_rot_rows_kernel(RotRowsArgs a) {
  extern __shared__ __align__(16) unsigned char rr_smem_raw[];
  __half* m1 = reinterpret_cast<__half*>(rr_smem_raw);
  __half* m2 = m1 + 8 * NJ * RR_LD;
  __half* a1 = m2 + 8 * NJ * RR_LD;
  __half* a2 = a1 + 128 * RR_LD;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
  const int j0 = blockIdx.y * (8 * NJ);          // first column of this CTA

  // B operand: element (k = i, n = j) is M[i][j]; stored as [j][i] so that a fragment register is two neighbouring i
  // (128 x 8 NJ values as 16-byte loads, up to eight per thread in flight at a time; local column jl = j - j0)
  constexpr int QUADS = 128 * 8 * NJ / 4, PER = QUADS / RR_THREADS;       // 16, 8 or 4 loads per thread
#pragma unroll 1
  for (int b = 0; b < PER; b += 8) {
    float4 x[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      if (b + u < PER) {
        const int qd = (b + u) * RR_THREADS + tid, i = qd / (2 * NJ), jl = (qd % (2 * NJ)) * 4;
        x[u] = __ldg(reinterpret_cast<const float4*>(a.mat + i * 128 + j0 + jl));
      }
    }
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      if (b + u < PER) {
        const int qd = (b + u) * RR_THREADS + tid, i = qd / (2 * NJ), jl = (qd % (2 * NJ)) * 4;
        const float v[4] = {x[u].x * 1024.0f, x[u].y * 1024.0f, x[u].z * 1024.0f, x[u].w * 1024.0f};
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const __half h = __float2half_rn(v[q]);
          m1[(jl + q) * RR_LD + i] = h;
          m2[(jl + q) * RR_LD + i] = __float2half_rn(v[q] - __half2float(h));
        }
      }
    }
  }
  const bool two_terms = a.src_dtype == AKV_F32;
  const float out_scale = a.scale * (1.0f / 1024.0f);
  const int64_t tiles = (a.rows + 127) >> 7;
  for (int64_t tile = blockIdx.x; tile < tiles; tile += gridDim.x) {
    __syncthreads();                    // the matrix is in place; the previous tile's fragments have been read
    // ---- A operand: 128 rows x 128, eight elements per thread and pass (eight passes, unrolled: loads in flight together) ----
#pragma unroll
    for (int e = tid; e < 128 * 16; e += RR_THREADS) {
      const int r = e >> 4, c = e & 15;
      const int64_t row = tile * 128 + r;
      float v[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) v[i] = 0.f;
      if (row < a.rows) {
        const int64_t off = (row / a.inner) * a.src_outer + (row % a.inner) * a.src_inner + 8 * c;
        if (a.src_dtype == AKV_F32) {
          const float4* p = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(a.src) + off);
          const float4 x = p[0], y = p[1];
          v[0] = x.x; v[1] = x.y; v[2] = x.z; v[3] = x.w; v[4] = y.x; v[5] = y.y; v[6] = y.z; v[7] = y.w;
        } else {
          const uint4 x = *reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(a.src) + off);
          const uint32_t w[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            if (a.src_dtype == AKV_F16) {
              const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
              v[2 * i] = f.x; v[2 * i + 1] = f.y;
            } else {
              const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w[i]));
              v[2 * i] = f.x; v[2 * i + 1] = f.y;
            }
          }
        }
        if (a.inv_l != nullptr) {
          const float l = a.inv_l[row * a.inv_stride];       // l = 0: a row nobody wrote, whatever the scratch holds
          const float inv = 1.0f / l;
#pragma unroll
          for (int i = 0; i < 8; ++i) v[i] = l > 0.f ? v[i] * inv : 0.f;
        }
      }
      uint32_t hi[4], lo[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const __half2 h = __floats2half2_rn(v[2 * i], v[2 * i + 1]);
        const float2 hf = __half22float2(h);
        const __half2 l2 = __floats2half2_rn(v[2 * i] - hf.x, v[2 * i + 1] - hf.y);
        hi[i] = *reinterpret_cast<const uint32_t*>(&h);
        lo[i] = *reinterpret_cast<const uint32_t*>(&l2);
      }
      *reinterpret_cast<uint4*>(a1 + r * RR_LD + 8 * c) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
      if (two_terms) *reinterpret_cast<uint4*>(a2 + r * RR_LD + 8 * c) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
    }
    __syncthreads();
    // ---- warp: rows 16 warp .. 16 warp + 15, all 128 columns ----
    float acc[NJ][4];
#pragma unroll
    for (int j = 0; j < NJ; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;
    const __half* ra1 = a1 + (16 * warp + g) * RR_LD + 2 * t;
    const __half* ra2 = a2 + (16 * warp + g) * RR_LD + 2 * t;
#pragma unroll
    for (int kk = 0; kk < 8; ++kk) {
      const uint32_t x0 = *reinterpret_cast<const uint32_t*>(ra1 + 16 * kk), x1 = *reinterpret_cast<const uint32_t*>(ra1 + 8 * RR_LD + 16 * kk);
      const uint32_t x2 = *reinterpret_cast<const uint32_t*>(ra1 + 16 * kk + 8), x3 = *reinterpret_cast<const uint32_t*>(ra1 + 8 * RR_LD + 16 * kk + 8);
      uint32_t y0 = 0, y1 = 0, y2 = 0, y3 = 0;
      if (two_terms) {
        y0 = *reinterpret_cast<const uint32_t*>(ra2 + 16 * kk); y1 = *reinterpret_cast<const uint32_t*>(ra2 + 8 * RR_LD + 16 * kk);
        y2 = *reinterpret_cast<const uint32_t*>(ra2 + 16 * kk + 8); y3 = *reinterpret_cast<const uint32_t*>(ra2 + 8 * RR_LD + 16 * kk + 8);
      }
#pragma unroll
      for (int j = 0; j < NJ; ++j) {
        const __half* rb1 = m1 + (8 * j + g) * RR_LD + 16 * kk + 2 * t;
        const __half* rb2 = m2 + (8 * j + g) * RR_LD + 16 * kk + 2 * t;
        const uint32_t b0 = *reinterpret_cast<const uint32_t*>(rb1), b1 = *reinterpret_cast<const uint32_t*>(rb1 + 8);
        const uint32_t c0 = *reinterpret_cast<const uint32_t*>(rb2), c1 = *reinterpret_cast<const uint32_t*>(rb2 + 8);
        rr_mma(acc[j], x0, x1, x2, x3, b0, b1);
        rr_mma(acc[j], x0, x1, x2, x3, c0, c1);
        if (two_terms) rr_mma(acc[j], y0, y1, y2, y3, b0, b1);
      }
    }
    // ---- results: thread holds rows g, g + 8 of the warp's 16, columns 8 j + 2 t, + 1 ----
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int64_t row = tile * 128 + 16 * warp + g + 8 * half;
      if (row >= a.rows) continue;
      const int64_t off = (row / a.inner) * a.out_outer + (row % a.inner) * a.out_inner + j0 + 2 * t;
#pragma unroll
      for (int j = 0; j < NJ; ++j) {
        const float lo = acc[j][2 * half] * out_scale, hi = acc[j][2 * half + 1] * out_scale;
        if (a.out_dtype == AKV_F32) {
          *reinterpret_cast<float2*>(reinterpret_cast<float*>(a.out) + off + 8 * j) = make_float2(lo, hi);
        } else if (a.out_dtype == AKV_F16) {
          *reinterpret_cast<__half2*>(reinterpret_cast<__half*>(a.out) + off + 8 * j) = __floats2half2_rn(lo, hi);
        } else {
          *reinterpret_cast<__nv_bfloat162*>(reinterpret_cast<__nv_bfloat16*>(a.out) + off + 8 * j) = __floats2bfloat162_rn(lo, hi);
        }
      }
    }
  }
}

}  // namespace

// True when the strides and pointers allow the vector accesses of the kernel (16-byte source pieces, 4- or 8-byte stores).
bool rot_rows_ok(const void* src, int src_dtype, int64_t src_outer, int64_t src_inner, const void* out, int out_dtype,
                 int64_t out_outer, int64_t out_inner) {
  const int64_t se = src_dtype == AKV_F32 ? 4 : 2, oe = out_dtype == AKV_F32 ? 4 : 2;
  const bool s_ok = ((reinterpret_cast<uintptr_t>(src) | (uintptr_t)(src_outer * se) | (uintptr_t)(src_inner * se)) & 15) == 0;
  const bool o_ok = ((reinterpret_cast<uintptr_t>(out) | (uintptr_t)(out_outer * oe) | (uintptr_t)(out_inner * oe)) & (2 * oe - 1)) == 0;
  return s_ok && o_ok;
}

int launch_rot_rows(const void* src, int src_dtype, int64_t src_outer, int64_t src_inner, int inner, const float* inv_l,
                    int64_t inv_stride, const float* mat, float scale, void* out, int out_dtype, int64_t out_outer,
                    int64_t out_inner, int64_t rows, cudaStream_t st) {
  if (rows <= 0) return AKV_OK;
  RotRowsArgs a{};
  a.src = src; a.src_dtype = src_dtype; a.src_outer = src_outer; a.src_inner = src_inner; a.inner = inner;
  a.inv_l = inv_l; a.inv_stride = inv_stride; a.mat = mat; a.scale = scale;
  a.out = out; a.out_dtype = out_dtype; a.out_outer = out_outer; a.out_inner = out_inner; a.rows = rows;
  const int64_t tiles = (rows + 127) / 128;
  // column split 4, 2 or 1: the largest that keeps the CTAs within what the GPU holds at once (two split CTAs per SM)
  const int64_t room = 2 * (int64_t)sm_count();
  const int split = 4 * tiles <= room ? 4 : (2 * tiles <= room ? 2 : 1);
  const int64_t per = split == 1 ? sm_count() : room / split;
  dim3 grid((unsigned)(tiles < per ? tiles : per), split);
  cudaError_t e;
  if (split == 4) {
    e = cudaFuncSetAttribute(akv_rot_rows_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, rr_smem(4));
    if (e == cudaSuccess) akv_rot_rows_kernel<4><<<grid, RR_THREADS, rr_smem(4), st>>>(a);
  } else if (split == 2) {
    e = cudaFuncSetAttribute(akv_rot_rows_kernel<8>, cudaFuncAttributeMaxDynamicSharedMemorySize, rr_smem(8));
    if (e == cudaSuccess) akv_rot_rows_kernel<8><<<grid, RR_THREADS, rr_smem(8), st>>>(a);
  } else {
    e = cudaFuncSetAttribute(akv_rot_rows_kernel<16>, cudaFuncAttributeMaxDynamicSharedMemorySize, rr_smem(16));
    if (e == cudaSuccess) akv_rot_rows_kernel<16><<<grid, RR_THREADS, rr_smem(16), st>>>(a);
  }
  if (e != cudaSuccess) return fail((int)e, "row rotation: smem attribute: %s", cudaGetErrorString(e));
  return check_launch("akv_rot_rows_kernel");
}

}  // namespace akv
