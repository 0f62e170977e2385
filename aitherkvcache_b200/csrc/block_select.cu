// Block selection for sparse paged decode attention (reference: aither_kvcache/block_selector.py).
//
// The reference keeps, per physical cache block and KV head, the mean of the norm-weighted
// rotated-domain key vectors ("representative"), scores every block of a sequence against the
// GQA-averaged rotated query, forces the first and last few blocks in, takes the top-k by score,
// sorts the chosen logical blocks and gathers their physical ids into a shorter block table
// (block_selector.py:65-101 update, :128-172 score_blocks, :175-228 select_blocks).  All of that is
// torch op chains there; here it is four kernels and no host synchronisation:
//
//   bs_update_kernel    codes + norm of newly written tokens -> atomic adds into acc[block][head][dim]
//   bs_finalize_kernel  rep = acc / count for the blocks those tokens touched
//   bs_score_kernel     q_mean = mean over the GQA group of R q;  score[s][j] = sum_h q_mean[h] . rep[bt[s][j]][h]
//   bs_select_kernel    one CTA per sequence: exact k-th largest score by a radix select on the
//                       order-preserving integer image of the floats, then an ordered compaction, so the
//                       chosen blocks come out in logical order without a sort
#include "common.cuh"
#include <math_constants.h>

namespace akv {

constexpr int BS_D = 128;

// acc [max_blocks][H][128] float, counts [max_blocks][H] int.  One CTA per (token, head), thread per dim.
__global__ void __launch_bounds__(BS_D)
bs_update_kernel(const int64_t* __restrict__ block_idx, const uint8_t* __restrict__ k_packed, int64_t kp_st, int64_t kp_sh,
                 const float* __restrict__ k_norms, int64_t kn_st, int64_t kn_sh, const float* __restrict__ centroids,
                 int bits, int H, int64_t max_blocks, float* __restrict__ acc, int* __restrict__ counts) {
  const int tok = blockIdx.x, h = blockIdx.y, d = threadIdx.x;
  const int64_t blk = block_idx[tok];
  if (blk < 0 || blk >= max_blocks) return;
  const uint8_t* row = k_packed + tok * kp_st + h * kp_sh;
  const int code = extract_code(row, d, bits, BS_D * bits / 8);
  const float v = centroids[code] * k_norms[tok * kn_st + h * kn_sh];
  atomicAdd(acc + (blk * H + h) * BS_D + d, v);
  if (d == 0) atomicAdd(counts + blk * H + h, 1);
}

__global__ void __launch_bounds__(BS_D)
bs_finalize_kernel(const int64_t* __restrict__ block_idx, int H, int64_t max_blocks, const float* __restrict__ acc,
                   const int* __restrict__ counts, float* __restrict__ rep) {
  const int64_t blk = block_idx[blockIdx.x];
  if (blk < 0 || blk >= max_blocks) return;
  const int64_t o = (blk * H + blockIdx.y) * BS_D + threadIdx.x;
  const int c = counts[blk * H + blockIdx.y];
  rep[o] = acc[o] / (float)(c > 0 ? c : 1);
}

__global__ void __launch_bounds__(BS_D)
bs_clear_kernel(const int64_t* __restrict__ block_idx, int H, int64_t max_blocks, float* __restrict__ acc,
                int* __restrict__ counts, float* __restrict__ rep) {
  const int64_t blk = block_idx[blockIdx.x];
  if (blk < 0 || blk >= max_blocks) return;
  const int64_t o = (blk * H + blockIdx.y) * BS_D + threadIdx.x;
  acc[o] = 0.f;
  rep[o] = 0.f;
  if (threadIdx.x == 0) counts[blk * H + blockIdx.y] = 0;
}

// q_mean[s][h][i] = sum_j R[i][j] * mean_g q[s][h*G+g][j]   (rot_t[j*128+i] = R[i][j]); one CTA per (s, h).
__global__ void __launch_bounds__(BS_D)
bs_qmean_kernel(const void* __restrict__ q, int q_dtype, int64_t q_ss, int64_t q_sh, int G,
                const float* __restrict__ rot_t, float* __restrict__ qmean, int H) {
  __shared__ float m[BS_D];
  const int s = blockIdx.x, h = blockIdx.y, i = threadIdx.x;
  float v = 0.f;
  for (int gq = 0; gq < G; ++gq) v += load_as_float(q, q_dtype, s * q_ss + (int64_t)(h * G + gq) * q_sh + i);
  m[i] = v / (float)G;
  __syncthreads();
  float a0 = 0.f, a1 = 0.f;
  for (int j = 0; j < BS_D; j += 2) {
    a0 = __fmaf_rn(rot_t[j * BS_D + i], m[j], a0);
    a1 = __fmaf_rn(rot_t[(j + 1) * BS_D + i], m[j + 1], a1);
  }
  qmean[((int64_t)s * H + h) * BS_D + i] = a0 + a1;
}

// scores[s][j] for j < max_bps: one warp per block; -inf for blocks past the context.
__global__ void __launch_bounds__(256)
bs_score_kernel(const float* __restrict__ qmean, const float* __restrict__ rep, const void* __restrict__ block_tables,
                int bt_dtype, int64_t bt_stride, const void* __restrict__ context_lens, int cl_dtype, int H,
                int block_size, int max_bps, int64_t max_blocks, float* __restrict__ scores) {
  extern __shared__ float qs[];          // [H][128]
  const int s = blockIdx.y;
  for (int i = threadIdx.x; i < H * BS_D; i += 256) qs[i] = qmean[(int64_t)s * H * BS_D + i];
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int j = blockIdx.x * 8 + warp;
  if (j >= max_bps) return;
  const int64_t ctx = load_ctx(context_lens, cl_dtype, s, (int64_t)max_bps * block_size);
  const int64_t nb = (ctx + block_size - 1) / block_size;
  float sc = -CUDART_INF_F;
  if (j < nb) {
    int64_t blk = load_index(block_tables, bt_dtype, (int64_t)s * bt_stride + j);
    blk = blk < 0 ? 0 : (blk >= max_blocks ? max_blocks - 1 : blk);
    const float4* r = reinterpret_cast<const float4*>(rep + blk * H * BS_D);
    const float4* qv = reinterpret_cast<const float4*>(qs);
    float a = 0.f;
    for (int i = lane; i < H * BS_D / 4; i += 32) {
      const float4 x = r[i], y = qv[i];
      a += x.x * y.x + x.y * y.y + x.z * y.z + x.w * y.w;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) a += __shfl_xor_sync(0xffffffffu, a, o);
    sc = a;
  }
  if (lane == 0) scores[(int64_t)s * max_bps + j] = sc;
}

__device__ __forceinline__ uint32_t bs_key(float f) {          // larger float <=> larger unsigned key
  const uint32_t u = __float_as_uint(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

// One CTA per sequence.  keys: valid mandatory blocks +inf, other valid blocks their score, invalid -inf.
// Chooses the k = min(max_selected, max_bps) largest keys (ties: lowest logical index first), writes their
// physical ids in logical order, pads the row with block 0, and writes the adjusted context length.
__global__ void __launch_bounds__(256)
bs_select_kernel(const float* __restrict__ scores, const void* __restrict__ block_tables, int bt_dtype, int64_t bt_stride,
                 const void* __restrict__ context_lens, int cl_dtype, int block_size, int max_bps, int max_selected,
                 int num_sink, int num_recent, int exact_tail, int* __restrict__ out_bt, int* __restrict__ out_cl) {
  __shared__ int s_cnt[256];
  __shared__ int s_scan[256];
  __shared__ uint32_t s_prefix;
  __shared__ int s_need;
  const int s = blockIdx.x, tid = threadIdx.x;
  const int64_t ctx = load_ctx(context_lens, cl_dtype, s, (int64_t)max_bps * block_size);
  const int nb = (int)((ctx + block_size - 1) / block_size);
  const int k = max_selected < max_bps ? max_selected : max_bps;
  const float* row = scores + (int64_t)s * max_bps;
  auto key_of = [&](int j) -> uint32_t {
    if (j >= nb) return bs_key(-CUDART_INF_F);
    if (j < num_sink || j >= nb - num_recent) return bs_key(CUDART_INF_F);
    return bs_key(row[j]);
  };
  // radix select, 8 bits at a time from the top: after each pass `prefix` fixes the high bits of the
  // k-th largest key and `need` counts how many keys equal to the prefix so far are still wanted
  if (tid == 0) { s_prefix = 0u; s_need = k; }
  __syncthreads();
  for (int shift = 24; shift >= 0; shift -= 8) {
    s_cnt[tid] = 0;
    __syncthreads();
    const uint32_t prefix = s_prefix;
    const uint32_t himask = shift == 24 ? 0u : (0xffffffffu << (shift + 8));
    for (int j = tid; j < max_bps; j += 256) {
      const uint32_t key = key_of(j);
      if ((key & himask) == prefix) atomicAdd(&s_cnt[(key >> shift) & 255u], 1);
    }
    __syncthreads();
    if (tid == 0) {
      int need = s_need, b = 255;
      for (; b > 0; --b) {
        if (s_cnt[b] >= need) break;
        need -= s_cnt[b];
      }
      s_prefix = prefix | ((uint32_t)b << shift);
      s_need = need;
    }
    __syncthreads();
  }
  const uint32_t kth = s_prefix;     // the k-th largest key; s_need of the keys equal to it are taken (lowest index first)
  const int need_eq = s_need;
  // ordered compaction in chunks of 256 logical blocks
  __shared__ int s_base, s_eq_base;
  if (tid == 0) { s_base = 0; s_eq_base = 0; }
  __syncthreads();
  int* out = out_bt + (int64_t)s * max_selected;
  for (int j0 = 0; j0 < max_bps; j0 += 256) {
    const int j = j0 + tid;
    const uint32_t key = j < max_bps ? key_of(j) : 0u;
    const int gt = (j < max_bps && key > kth) ? 1 : 0, eq = (j < max_bps && key == kth) ? 1 : 0;
    // inclusive scans of gt and eq over the chunk (two passes of a simple shared-memory scan)
    s_cnt[tid] = gt; s_scan[tid] = eq;
    __syncthreads();
    for (int o = 1; o < 256; o <<= 1) {
      const int a = tid >= o ? s_cnt[tid - o] : 0, b2 = tid >= o ? s_scan[tid - o] : 0;
      __syncthreads();
      s_cnt[tid] += a; s_scan[tid] += b2;
      __syncthreads();
    }
    const int eq_before = s_eq_base + s_scan[tid] - eq;            // equal keys with a lower logical index
    const int take = gt | (eq && eq_before < need_eq ? 1 : 0);
    // position = selected before this chunk + selected before this element inside the chunk
    const int eq_taken_incl = min(s_eq_base + s_scan[tid], need_eq) - min(s_eq_base, need_eq);
    const int pos = s_base + (s_cnt[tid] - gt) + (eq_taken_incl - (eq && eq_before < need_eq ? 1 : 0));
    if (take && pos < max_selected) {
      int64_t blk = load_index(block_tables, bt_dtype, (int64_t)s * bt_stride + j);
      out[pos] = (int)blk;
    }
    __syncthreads();
    if (tid == 255) {
      s_base += s_cnt[255] + (min(s_eq_base + s_scan[255], need_eq) - min(s_eq_base, need_eq));
      s_eq_base += s_scan[255];
    }
    __syncthreads();
  }
  for (int j = k + tid; j < max_selected; j += 256) out[j] = 0;
  if (tid == 0) {
    int64_t cl = ctx < (int64_t)k * block_size ? ctx : (int64_t)k * block_size;
    // more valid blocks than k: the last selected block is the sequence's last (it is mandatory) and may be
    // partial; exact_tail counts only its real tokens (the reference counts it as full)
    if (exact_tail && nb > k && num_recent > 0) cl = (int64_t)(k - 1) * block_size + (ctx - (int64_t)(nb - 1) * block_size);
    out_cl[s] = (int)cl;
  }
}

}  // namespace akv

using namespace akv;

// Scratch of one selector: acc and rep [max_blocks][H][128] float, counts [max_blocks][H] int - allocated
// and zeroed by the caller.
AKV_EXPORT int akv_block_select_update(const int64_t* block_idx, int64_t num_tokens, const uint8_t* k_packed,
                                       int64_t kp_stride_tok, int64_t kp_stride_head, const float* k_norms,
                                       int64_t kn_stride_tok, int64_t kn_stride_head, const float* centroids, int bits,
                                       int num_kv_heads, int head_dim, int64_t max_blocks, float* acc, int* counts,
                                       float* rep, void* stream) {
  if (head_dim != BS_D) return fail(AKV_ERR_UNSUPPORTED, "block selection is built for head_dim 128, got %d", head_dim);
  if (bits < 2 || bits > 4 || num_kv_heads <= 0 || max_blocks <= 0 || num_tokens < 0)
    return fail(AKV_ERR_ARG, "akv_block_select_update: bad sizes");
  if (num_tokens == 0) return AKV_OK;
  if (!block_idx || !k_packed || !k_norms || !centroids || !acc || !counts || !rep)
    return fail(AKV_ERR_ARG, "akv_block_select_update: null pointer");
  cudaStream_t st = (cudaStream_t)stream;
  dim3 grid((unsigned)num_tokens, num_kv_heads);
  bs_update_kernel<<<grid, BS_D, 0, st>>>(block_idx, k_packed, kp_stride_tok, kp_stride_head, k_norms, kn_stride_tok,
                                          kn_stride_head, centroids, bits, num_kv_heads, max_blocks, acc, counts);
  if (int rc = check_launch("bs_update_kernel")) return rc;
  bs_finalize_kernel<<<grid, BS_D, 0, st>>>(block_idx, num_kv_heads, max_blocks, acc, counts, rep);
  return check_launch("bs_finalize_kernel");
}

AKV_EXPORT int akv_block_select_clear(const int64_t* block_idx, int64_t num_blocks_to_clear, int num_kv_heads,
                                      int64_t max_blocks, float* acc, int* counts, float* rep, void* stream) {
  if (num_blocks_to_clear <= 0) return AKV_OK;
  if (!block_idx || !acc || !counts || !rep || num_kv_heads <= 0) return fail(AKV_ERR_ARG, "akv_block_select_clear: bad arguments");
  dim3 grid((unsigned)num_blocks_to_clear, num_kv_heads);
  bs_clear_kernel<<<grid, BS_D, 0, (cudaStream_t)stream>>>(block_idx, num_kv_heads, max_blocks, acc, counts, rep);
  return check_launch("bs_clear_kernel");
}

// Workspace: num_seqs * (num_kv_heads * 128 + max_blocks_per_seq) floats.
AKV_EXPORT size_t akv_block_select_workspace_bytes(int num_seqs, int num_kv_heads, int max_blocks_per_seq) {
  if (num_seqs <= 0 || num_kv_heads <= 0 || max_blocks_per_seq < 0) return 0;
  return ((size_t)num_seqs * ((size_t)num_kv_heads * BS_D + (size_t)max_blocks_per_seq) * sizeof(float) + 255) & ~(size_t)255;
}

AKV_EXPORT int akv_block_select(const void* query, int q_dtype, int64_t q_stride_seq, int64_t q_stride_head,
                                int num_seqs, int num_q_heads, int num_kv_heads, int head_dim, const float* rotation_t,
                                const float* rep, int64_t max_blocks, const void* block_tables, int bt_dtype,
                                int64_t bt_stride_seq, const void* context_lens, int cl_dtype, int block_size,
                                int max_blocks_per_seq, int max_selected, int num_sink_blocks, int num_recent_blocks,
                                int exact_tail, int* out_block_tables, int* out_context_lens, float* scores_out,
                                void* workspace, size_t workspace_bytes, void* stream) {
  if (head_dim != BS_D) return fail(AKV_ERR_UNSUPPORTED, "block selection is built for head_dim 128, got %d", head_dim);
  if (num_seqs < 0 || num_q_heads <= 0 || num_kv_heads <= 0 || num_q_heads % num_kv_heads || block_size <= 0 ||
      max_blocks_per_seq <= 0 || max_selected <= 0 || max_blocks <= 0 || num_sink_blocks < 0 || num_recent_blocks < 0)
    return fail(AKV_ERR_ARG, "akv_block_select: bad sizes");
  if (num_seqs == 0) return AKV_OK;
  if (!query || !rotation_t || !rep || !block_tables || !context_lens || !out_block_tables || !out_context_lens)
    return fail(AKV_ERR_ARG, "akv_block_select: null pointer");
  const size_t need = akv_block_select_workspace_bytes(num_seqs, num_kv_heads, max_blocks_per_seq);
  if (!workspace || workspace_bytes < need)
    return fail(AKV_ERR_WORKSPACE, "workspace too small: need %zu bytes, got %zu", need, workspace_bytes);
  cudaStream_t st = (cudaStream_t)stream;
  float* qmean = reinterpret_cast<float*>(workspace);
  float* scores = scores_out ? scores_out : qmean + (size_t)num_seqs * num_kv_heads * BS_D;
  bs_qmean_kernel<<<dim3(num_seqs, num_kv_heads), BS_D, 0, st>>>(query, q_dtype, q_stride_seq, q_stride_head,
                                                                  num_q_heads / num_kv_heads, rotation_t, qmean, num_kv_heads);
  if (int rc = check_launch("bs_qmean_kernel")) return rc;
  const size_t smem = (size_t)num_kv_heads * BS_D * sizeof(float);
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(bs_score_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return fail((int)e, "block select: smem attribute: %s", cudaGetErrorString(e));
  }
  bs_score_kernel<<<dim3((max_blocks_per_seq + 7) / 8, num_seqs), 256, smem, st>>>(
      qmean, rep, block_tables, bt_dtype, bt_stride_seq, context_lens, cl_dtype, num_kv_heads, block_size,
      max_blocks_per_seq, max_blocks, scores);
  if (int rc = check_launch("bs_score_kernel")) return rc;
  bs_select_kernel<<<num_seqs, 256, 0, st>>>(scores, block_tables, bt_dtype, bt_stride_seq, context_lens, cl_dtype,
                                             block_size, max_blocks_per_seq, max_selected, num_sink_blocks,
                                             num_recent_blocks, exact_tail, out_block_tables, out_context_lens);
  return check_launch("bs_select_kernel");
}
