// Arguments shared by the chunked-prefill attention kernels (tq_prefill.cuh: mma.sync, tq_prefill_tc.cu: tcgen05).
#pragma once

#include "common.cuh"

namespace akv {

struct PrefillArgs {
  const float* qrot;                   // [n_tokens * num_q_heads][128], scale * log2(e) folded in
  const uint8_t* k_packed; int64_t kp_sb, kp_sp, kp_sh;
  const float* k_norms; int64_t kn_sb, kn_sp, kn_sh;
  const uint8_t* v_packed; int64_t vp_sb, vp_sp, vp_sh;
  const float* v_norms; int64_t vn_sb, vn_sp, vn_sh;
  const void* block_tables; int bt_dtype; int64_t bt_stride;
  const void* seq_lens; int sl_dtype;              // [num_seqs] tokens of each sequence, the chunk's included
  const void* query_start_loc; int qs_dtype;       // [num_seqs + 1] first query row of each sequence
  int num_seqs, n_tokens, num_q_heads, num_kv_heads, block_size, max_blocks_per_seq;
  int64_t num_blocks;
  const float* centroids;
  float* part_acc;                     // [n_tokens * num_q_heads][splits][128]
  float* part_ml;                      // [n_tokens * num_q_heads][splits][2]
  // staged variant of the tensor-core kernel: [num_seqs][tiles_per_seq][num_kv_heads] operand images (512 B per key), or null
  uint8_t* staged;
  int tiles_per_seq;
  int bits;                            // 4; 3 or 2 only with staged images
  int byte_rows;                       // 4-bit rows that are not readable in 16-byte pieces: pre-pass by byte loads
  // tq35 records instead of TurboQuant codes (staged images only): host pointer to the akv_hybrid_tables of the call;
  // k_packed / v_packed are the 64-byte records, the norm arrays are unused
  const void* hybrid_tables;
  int splits;                          // tensor-core kernels: key-range splits = partials per row (1: part_acc [rows][128])
};

// Layout of a staged tile in global memory (what the pre-pass kernels write and tq_prefill_tc_kernel<G, true> copies):
// 128 keys of one KV head = the K operand [128 keys][128 dims] as two halves of 64 dims (128 rows x 128 B each, the
// 16-byte chunk c of row r at chunk c ^ (r & 7)), then the transposed V operand as two halves of 64 keys
// ([128 dims] rows x 128 B each, the chunk of key group g of dim d at chunk g ^ (d & 7)).
constexpr int PFI_KEYS = 128;
constexpr int PFI_KHALF = PFI_KEYS * 128;
constexpr int PFI_VOFF = 2 * PFI_KHALF;
constexpr int PFI_VHALF = 128 * 128;
constexpr int PFI_BYTES = PFI_VOFF + 2 * PFI_VHALF;

// hybrid.cu: the pre-pass for tq35 records
int launch_hybrid_prefill_stage(const PrefillArgs& a, cudaStream_t st);

// tcgen05 kernel (tq_prefill_tc.cu): one CTA per 128 (token, query head) rows and KV head.  Returns AKV_OK after
// the launch; AKV_ERR_UNSUPPORTED is never returned - the caller checks the shape (4-bit codes, head_dim 128,
// G in {1, 2, 4, 8}, block_size % 16 == 0, 16-byte readable caches) before calling.
// With a.staged set, a pre-pass (tq_prefill_stage_kernel) first writes every key tile's fp16 operand images there and the
// attention kernel is fed by bulk copies instead of decoding the codes itself.
int launch_prefill_tc(const PrefillArgs& a, int G, cudaStream_t st);
size_t prefill_staged_bytes(int num_seqs, int num_kv_heads, int max_seq_len);
int prefill_staged_tile_keys();
int prefill_tc_status(int* host_out, int reset);
int prefill_tc_withhold(int tile);

}  // namespace akv
