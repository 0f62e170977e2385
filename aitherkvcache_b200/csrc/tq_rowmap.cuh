// Row addressing of the TurboQuant encode kernels: contiguous rows, or the paged
// scatter write driven by a slot mapping (fused_kv_update.py:220-293 in the reference).
#pragma once

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

// Tensor-core encode for head_dim 128 and 16-bit inputs (tq_encode_tc.cu).
int launch_encode_tc(const RowMap& m, int64_t n_rows, int bits, bool bf16, const float* rot_t,
                     const float* boundaries, cudaStream_t st);

// The K and V paged writes of a decode step (few rows) as one launch of the generic kernel (tq_codec.cu).
int launch_encode_generic_pair(const RowMap& mk, const RowMap& mv, int64_t n_rows, int D, int bits,
                               const float* rot_t, const float* boundaries, cudaStream_t st);

// Tensor-core decode for head_dim 128 (tq_decode_tc.cu).
int launch_decode_tc(const uint8_t* packed, int64_t packed_row_stride, const float* norms, int64_t n_rows,
                     int bits, const float* rot, const float* centroids, void* out, int out_dtype,
                     cudaStream_t st);

}  // namespace akv
