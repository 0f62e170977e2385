// Shared helpers for the sm_100a kernels behind the C ABI in include/akv_b200.h.
#pragma once

#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include <stdio.h>
#include <stdarg.h>

#define AKV_EXPORT extern "C" __attribute__((visibility("default")))

// Element types accepted for float inputs/outputs (akv_dtype in the header).
enum { AKV_F16 = 0, AKV_BF16 = 1, AKV_F32 = 2 };
// Integer index types for block tables / context lengths.
enum { AKV_I32 = 0, AKV_I64 = 1 };

// Error codes returned by every entry point (0 = success, >0 = cudaError_t).
enum {
  AKV_OK = 0,
  AKV_ERR_ARG = -1,        // bad argument (message in akv_last_error)
  AKV_ERR_UNSUPPORTED = -2,
  AKV_ERR_WORKSPACE = -3,  // workspace too small
};

namespace akv {

char* error_buffer();  // thread-local, 512 bytes (defined in api.cu)

inline int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(error_buffer(), 512, fmt, ap);
  va_end(ap);
  return code;
}

// Launch bookkeeping (api.cu): every kernel launch of the library passes through check_launch, which
// counts it and remembers the kernel's name (per host thread).
void note_launch(const char* what);

inline int check_launch(const char* what) {
  note_launch(what);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    return fail((int)e, "%s: %s", what, cudaGetErrorString(e));
  }
  return AKV_OK;
}

inline bool is_pow2(int v) { return v > 0 && (v & (v - 1)) == 0; }

inline int packed_bytes(int head_dim, int bits) { return head_dim * bits / 8; }

inline int sm_count() {
  static int n = 0;
  if (n == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    if (n <= 0) n = 148;
  }
  return n;
}

// Shared-window address at which `kernel`'s dynamic shared memory will start on the current
// device: the bytes the system reserves per CTA plus the kernel's static shared memory, rounded
// up to the 128-byte alignment the kernels declare for their dynamic array.  Kernels that place
// tables at fixed shared addresses are only launched when this is at or below their first
// fixed address.  0xffffffff if the attributes cannot be read.
inline uint32_t dyn_smem_window_start(const void* kernel) {
  cudaFuncAttributes fa{};
  int dev = 0, reserved = 0;
  if (cudaFuncGetAttributes(&fa, kernel) != cudaSuccess || cudaGetDevice(&dev) != cudaSuccess ||
      cudaDeviceGetAttribute(&reserved, cudaDevAttrReservedSharedMemoryPerBlock, dev) != cudaSuccess) {
    cudaGetLastError();
    return 0xffffffffu;
  }
  return (uint32_t)(((size_t)reserved + fa.sharedSizeBytes + 127) / 128 * 128);
}

// Device-side status words, one per group of kernels (0 = nothing happened):
//   tc_encode / tc_decode : 1 = a bounded wait on the MMA barrier gave up (rows of the tile were not
//                           written), 2 = and the CTA could not confirm its MMAs had drained, so it kept
//                           its tensor-memory columns
//   attn_window / hybrid_window : 1 = a kernel found its dynamic shared memory starting above its first
//                           fixed table address and returned without writing partials
int tc_encode_status(int* host_out, int reset);
int tc_decode_status(int* host_out, int reset);
int attn_window_status(int* host_out, int reset);
int tri_status(int* host_out, int reset);
// rot_rows.cu: out[r] = scale * (src[r] / l_r) M for many rows at once (tensor cores, float32 accuracy); row r = (r / inner, r % inner)
bool rot_rows_ok(const void* src, int src_dtype, int64_t src_outer, int64_t src_inner, const void* out, int out_dtype,
                 int64_t out_outer, int64_t out_inner);
int launch_rot_rows(const void* src, int src_dtype, int64_t src_outer, int64_t src_inner, int inner, const float* inv_l,
                    int64_t inv_stride, const float* mat, float scale, void* out, int out_dtype, int64_t out_outer,
                    int64_t out_inner, int64_t rows, cudaStream_t st);
int prefill_tc_status(int* host_out, int reset);
int prefill_tc_withhold(int tile);
int hybrid_window_status(int* host_out, int reset);
int tc_encode_withhold(int tile);
int tc_decode_withhold(int tile);

__device__ __forceinline__ float load_as_float(const void* p, int dtype, int64_t i) {
  if (dtype == AKV_F16) return __half2float(reinterpret_cast<const __half*>(p)[i]);
  if (dtype == AKV_BF16) return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i]);
  return reinterpret_cast<const float*>(p)[i];
}

__device__ __forceinline__ void store_from_float(void* p, int dtype, int64_t i, float v) {
  if (dtype == AKV_F16) reinterpret_cast<__half*>(p)[i] = __float2half_rn(v);
  else if (dtype == AKV_BF16) reinterpret_cast<__nv_bfloat16*>(p)[i] = __float2bfloat16_rn(v);
  else reinterpret_cast<float*>(p)[i] = v;
}

__device__ __forceinline__ int64_t load_index(const void* p, int itype, int64_t i) {
  return itype == AKV_I64 ? reinterpret_cast<const int64_t*>(p)[i]
                          : (int64_t)reinterpret_cast<const int32_t*>(p)[i];
}

// Context length of one sequence, clamped to [0, limit]: `limit` is what the sequence's
// block-table row can address (max_blocks_per_seq * block_size), so a stale, padded or
// negative entry can never index past the row.
__device__ __forceinline__ int64_t load_ctx(const void* p, int itype, int64_t seq, int64_t limit) {
  const int64_t c = load_index(p, itype, seq);
  return c < 0 ? 0 : (c > limit ? limit : c);
}

// Code k (0-based) of an MSB-first packed row with `bits` bits per code
// (byte format of packing.py:13-98 in the reference).
__device__ __forceinline__ int extract_code(const uint8_t* row, int k, int bits, int row_bytes) {
  int bit = k * bits;
  int byte = bit >> 3;
  int hi = row[byte];
  int lo = (byte + 1 < row_bytes) ? row[byte + 1] : 0;
  int w = (hi << 8) | lo;
  return (w >> (16 - bits - (bit & 7))) & ((1 << bits) - 1);
}

// LSE merge of split partials (kernel and launcher live in tq_attention.cu).
enum { MERGE_ROTATE = 0, MERGE_NORMALIZE = 1, MERGE_RAW = 2 };

struct MergeArgs {
  int mode;
  const float* acc; int64_t acc_row, acc_part;
  const float* ml; int64_t ml_row, ml_part;
  int np;
  const void* context_lens; int cl_dtype; int num_q_heads;
  int tokens_per_split, warps_per_head;   // used when context_lens != nullptr
  int D;
  const float* rot;              // R row-major (MERGE_ROTATE only)
  void* out; int out_dtype; int64_t out_ss, out_sh;
  void* out2;                    // optional second destination (MERGE_ROTATE): dense [rows][D] rows of out_dtype, same values
  float* raw_out;
  const int* part_counts;       // optional [num_seqs]: number of valid parts of each sequence
  // optional: the partials live in one of two halves of a double buffer; *half_select (a device word
  // written earlier in the stream) says which, half_stride floats apart
  const unsigned int* half_select;
  int64_t half_stride;
  // optional float32 [rows][128] scratch: with it, MERGE_ROTATE of 2048+ rows normalises into the scratch and rotates
  // all rows as one tensor-core product (rot_rows.cu) instead of one matrix-vector product per row
  float* gemm_scratch;
};

__device__ __forceinline__ int64_t merge_half_offset(const MergeArgs& a) {
  return a.half_select != nullptr ? (int64_t)(*a.half_select) * a.half_stride : 0;
}

int p2p_status(int* host_out, int reset);

int launch_merge(const MergeArgs& a, int rows, cudaStream_t st, bool pdl = false);

}  // namespace akv
