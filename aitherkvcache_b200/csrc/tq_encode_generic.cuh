// The one-vector-per-CTA TurboQuant encoder (any power-of-two head_dim up to 1024), as a device
// function so that a small batch - the new token of a decode step - can ride in another kernel's launch.
// Any block size that is a multiple of 32; dynamic shared memory (D + D/4 + 16) floats.  Same arithmetic, in the same order, as the
// tiled encoders (reference semantics: aither_kvcache/quantizer.py:90-125).
#pragma once

#include "tq_rowmap.cuh"

namespace akv {

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

__device__ __forceinline__ void encode_generic_rows(const RowMap& m, int64_t first, int64_t step, int64_t n_rows, int D,
                                                    int bits,
                                                    const float* __restrict__ rot_t,
                                                    const float* __restrict__ boundaries) {
  // one CTA per vector: thread o produces outputs o, o+128, ...
  extern __shared__ __align__(16) float smem_f[];
  float* u = smem_f;                                        // [D]
  uint8_t* codes = reinterpret_cast<uint8_t*>(u + D);       // [D]
  __shared__ float s_nrm;
  const int tid = threadIdx.x, nthr = blockDim.x;
  const int nb = (1 << bits) - 1;
  const int pd = D * bits / 8;
  for (int64_t n = first; n < n_rows; n += step) {
    RowAddr a = map_row(m, n);
    for (int i = tid; i < D; i += nthr) u[i] = load_as_float(a.src_base, m.x_dtype, a.src_off + i);
    __syncthreads();
    if (tid < 32) {
      float tot = sumsq_8lane(u, D, tid & 7, 0xffffffffu);
      if (tid == 0) s_nrm = __fsqrt_rn(tot);
    }
    __syncthreads();
    const float nrm = s_nrm;
    const float den = __fadd_rn(nrm, 1e-10f);
    for (int i = tid; i < D; i += nthr) u[i] = __fdiv_rn(u[i], den);
    __syncthreads();
    for (int o = tid; o < D; o += nthr) {
      float y = 0.f;      // one chain in the order j = 0..D-1 (bit-identical to the tiled kernel)
      int j0 = 0;
      for (; j0 + 32 <= D; j0 += 32) {       // 32 loads in flight per round: the matrix comes from L2
        float r[32];
#pragma unroll
        for (int k = 0; k < 32; ++k) r[k] = rot_t[(int64_t)(j0 + k) * D + o];
#pragma unroll
        for (int k = 0; k < 32; ++k) y = __fmaf_rn(u[j0 + k], r[k], y);
      }
      for (; j0 < D; j0 += 8) {              // D is a multiple of 8
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
      for (int bi = tid; bi < pd; bi += nthr) {
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

}  // namespace akv
