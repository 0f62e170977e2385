/*
 * C ABI of libakv_b200.so: sm_100a kernels for the compressed-KV hot path of
 * aither-kvcache (TurboQuant encode / decode / paged cache write / paged decode
 * attention, the hybrid tq35 codec, TriAttention's spectral codec).
 *
 * The reference has no C interface for this path: its callers reach Triton
 * kernels and torch op chains from Python.  Each entry point below names the
 * reference function it stands in for (paths inside the reference project).
 *
 * Conventions
 *   - Every pointer is a DEVICE pointer unless said otherwise; `stream` is a
 *     cudaStream_t (NULL = the legacy default stream).  Calls only enqueue
 *     work; nothing synchronises the host.
 *   - Sizes are element counts, strides are in elements of the pointed-to type
 *     (bytes for uint8_t), rows are row-major.
 *   - Return value: 0 on success, a positive cudaError_t if a launch failed,
 *     a negative AKV_ERR_* for rejected arguments.  akv_last_error() returns
 *     the message of the last failure on the calling thread.
 *   - Nothing here allocates device memory except where a function says so;
 *     scratch space is passed in as `workspace`.
 */
#ifndef AKV_B200_H
#define AKV_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* element types of floating-point tensors */
enum { AKV_F16 = 0, AKV_BF16 = 1, AKV_F32 = 2 };
/* element types of index tensors (block tables, context lengths) */
enum { AKV_I32 = 0, AKV_I64 = 1 };
/* negative return codes */
enum { AKV_OK = 0, AKV_ERR_ARG = -1, AKV_ERR_UNSUPPORTED = -2, AKV_ERR_WORKSPACE = -3 };

int akv_version(void);
const char* akv_last_error(void);
/* major*10+minor of the current device (100 on B200), negative if none */
int akv_device_arch(void);

/* Bookkeeping for benchmarks and tests (no counterpart in the reference): the number of kernels the
 * library has launched in this process (a launch recorded during stream capture counts once), and the
 * name of the split-K attention kernel the calling thread launched last ("" if none). */
long long akv_launch_count(void);
const char* akv_last_split_kernel(void);

/* Device-side status words of the current device (no counterpart in the reference: its Triton
 * kernels have no bounded waits).  Synchronises the device, then copies four words to the HOST
 * array out[0..3]; reset != 0 clears them.  0 = nothing happened.
 *   out[0] tensor-core encoder (akv_tq_encode / akv_tq_kv_update), out[1] tensor-core decoder
 *          (akv_tq_decode): 1 = a bounded wait on an MMA-completion barrier gave up and that CTA left
 *          its remaining tiles unwritten; 2 = it also could not confirm that its MMAs had drained and
 *          kept its tensor-memory columns.
 *   out[2] akv_tq_paged_attn / akv_tq_decode_step, out[3] akv_hybrid_paged_attn: 1 = a kernel that keeps
 *          tables at fixed shared-memory addresses found its window taken and returned without writing
 *          partials (the host checks the window before choosing such a kernel, so this stays 0); for the
 *          TMA-fed attention kernel 2 = a bounded wait on a copy barrier ran out.
 *   out[4] akv_p2p_lse_merge: 1 = the bounded wait for the peers' partials ran out (a peer is late or gone).
 * A diagnostic call for health checks and tests, not part of a serving step. */
int akv_device_status(int* out, int reset);

/* Test hook for those bounded waits: CTA 0 of later encoder (which = 0), decoder (which = 1) or
 * tensor-core prefill attention (which = 2: the score MMAs of key tile `tile`) launches issues neither
 * the MMAs nor the commit of its tile number `tile`, so the wait on that tile runs out with no tensor
 * work in flight and the CTA leaves through its give-up path.  tile < 0 (the default) switches the
 * hook off. */
int akv_debug_tc_withhold(int which, int tile);

/* ------------------------------------------------------------------------
 * Uniform TurboQuant codec
 * ---------------------------------------------------------------------- */

/* Replaces TurboQuant.encode (aither_kvcache/quantizer.py:122-166, with
 * _pytorch_encode :203-207 and the Triton kernels of triton_ops.py:26-57,92-126).
 *   x            [n_rows, head_dim], rows x_row_stride elements apart
 *   rotation_t   [head_dim, head_dim] float32, rotation_t[j][i] = R[i][j]
 *   boundaries   [2^bits - 1] float32, ascending
 *   packed       [n_rows, head_dim*bits/8] MSB-first codes (packing.py:13-98)
 *   norms        [n_rows] float32 L2 norms
 * bits in {2,3,4}; head_dim a power of two in [8, 1024]. */
int akv_tq_encode(const void* x, int x_dtype, int64_t n_rows, int64_t x_row_stride,
                  int head_dim, int bits, const float* rotation_t, const float* boundaries,
                  uint8_t* packed, int64_t packed_row_stride, float* norms, void* stream);

/* Replaces TurboQuant.decode (quantizer.py:168-197, _pytorch_decode :209-212,
 * triton_ops.py:59-86,128-159).  out is [n_rows, head_dim] contiguous of
 * out_dtype; rotation is R row-major; centroids has 2^bits entries. */
int akv_tq_decode(const uint8_t* packed, int64_t packed_row_stride, const float* norms,
                  int64_t n_rows, int head_dim, int bits, const float* rotation,
                  const float* centroids, void* out, int out_dtype, void* stream);

/* Replaces fused_tq4_kv_update (aither_kvcache/fused_kv_update.py:300-405; Triton
 * kernel :49-213; torch path :220-293) and, for 3/2-bit, encode + index-put
 * (vllm/hooks.py:487-497).  Token t, head h is written to
 * out_packed[slot/block_size][slot%block_size][h] where slot = slot_mapping[t];
 * tokens with slot < 0 or slot/block_size >= max_blocks are skipped. */
int akv_tq_kv_update(const void* x, int x_dtype, int64_t num_tokens, int num_kv_heads,
                     int head_dim, int64_t x_stride_tok, int64_t x_stride_head,
                     const int64_t* slot_mapping, uint8_t* out_packed, int64_t p_stride_blk,
                     int64_t p_stride_pos, int64_t p_stride_head, float* out_norms,
                     int64_t n_stride_blk, int64_t n_stride_pos, int64_t n_stride_head, int bits,
                     const float* rotation_t, const float* boundaries, int block_size,
                     int64_t max_blocks, void* stream);

/* Paged decode attention over the packed cache.  Replaces
 * TQPagedAttention.forward (aither_kvcache/fused_attention.py:594-748: the
 * pre-rotation sgemm, _tq_paged_attn_fused_4bit :204-356, _tq_splitk_phase1
 * :368-477, _tq_splitk_reduce :479-531 and the inverse-rotation sgemm), with the
 * semantics of TQPagedAttentionRef.forward (:91-185).
 *   query        [num_seqs, num_q_heads, head_dim]
 *   k/v_packed   [num_blocks, block_size, num_kv_heads, head_dim*bits/8] (strided views allowed)
 *   k/v_norms    [num_blocks, block_size, num_kv_heads] float32
 *   block_tables [num_seqs, max_blocks_per_seq]; context_lens [num_seqs]
 *   out          [num_seqs, num_q_heads, head_dim]; sequences with context 0 give zeros
 * If raw_out is non-NULL the call instead writes, per (seq, q head), the
 * un-normalised partial [m (log2 units), l, acc[head_dim]] in the rotated domain
 * (float32, [num_seqs*num_q_heads, head_dim+2]) for merging across devices with
 * akv_lse_merge; `out` and `rotation` may then be NULL. */
typedef struct akv_tq_attn_params {
  const void* query; int q_dtype; int64_t q_stride_seq, q_stride_head;
  const uint8_t* k_packed; int64_t kp_stride_blk, kp_stride_pos, kp_stride_head;
  const float* k_norms; int64_t kn_stride_blk, kn_stride_pos, kn_stride_head;
  const uint8_t* v_packed; int64_t vp_stride_blk, vp_stride_pos, vp_stride_head;
  const float* v_norms; int64_t vn_stride_blk, vn_stride_pos, vn_stride_head;
  const void* block_tables; int bt_dtype; int64_t bt_stride_seq;
  const void* context_lens; int cl_dtype;
  int num_seqs, num_q_heads, num_kv_heads, head_dim, block_size, max_blocks_per_seq;
  int64_t num_blocks;
  int bits;
  const float* rotation; const float* rotation_t; const float* centroids;
  float scale;
  void* out; int out_dtype; int64_t out_stride_seq, out_stride_head;
  float* raw_out;
  void* workspace; size_t workspace_bytes;
  int blocks_per_split;   /* KV blocks per split-K work item; 0 = library default */
  void* stream;
  void* ev_kernel_start;  /* optional cudaEvent_t pair recorded around the split-K kernel, */
  void* ev_kernel_stop;   /* so a caller can time that kernel alone; NULL = off */
  void* out_copy;         /* optional second destination of the result: dense [num_seqs, num_q_heads, head_dim] of
                           * out_dtype, written by the same kernel as `out` (the reference's op mutates `output` and
                           * returns a copy of it, vllm/hooks.py:129-205); NULL = off; ignored with raw_out */
} akv_tq_attn_params;

size_t akv_tq_paged_attn_workspace_bytes(int num_seqs, int num_q_heads, int num_kv_heads,
                                         int head_dim, int bits, int block_size,
                                         int max_blocks_per_seq, int blocks_per_split);
int akv_tq_paged_attn(const akv_tq_attn_params* params);

/* Chunked-prefill attention over the packed cache: replaces the prefill body of the reference's backend,
 * which decompresses every active block to bf16 and calls vLLM's unified attention
 * (vllm/backend.py:1093-1244, vllm/hooks.py:726-850).  Query token i of sequence s (rows
 * query_start_loc[s] .. query_start_loc[s+1]-1 of `query`, the last tokens of the sequence) attends causally
 * over the first seq_lens[s] - (query_len_s - 1 - i) cached tokens; the chunk's own K/V must already be in the
 * cache.  The query tokens of a sequence share one pass over its blocks.
 *   query [num_tokens, num_q_heads, 128]; caches, block tables as for akv_tq_paged_attn (4-bit codes);
 *   seq_lens [num_seqs], query_start_loc [num_seqs + 1] int32 (dtype 0) or int64 (1);
 *   out [num_tokens, num_q_heads, 128]; rows beyond query_start_loc[num_seqs] come out as zeros.
 * Built for head_dim 128, 1 / 2 / 4 / 8 query heads per KV head, block_size % 16 == 0 and 4-bit code rows that
 * are readable in 16-byte pieces; 3- and 2-bit caches and 4-bit rows of any alignment (68-byte records with the
 * norm inside) are served when max_seq_len and the staged workspace are given and the chunk fills 128-row tiles.  Anything else returns AKV_ERR_UNSUPPORTED before any launch (attend
 * row by row with akv_tq_paged_attn then). */
typedef struct akv_tq_prefill_params {
  const void* query; int q_dtype; int64_t q_stride_tok, q_stride_head;
  const uint8_t* k_packed; int64_t kp_stride_blk, kp_stride_pos, kp_stride_head;
  const float* k_norms; int64_t kn_stride_blk, kn_stride_pos, kn_stride_head;
  const uint8_t* v_packed; int64_t vp_stride_blk, vp_stride_pos, vp_stride_head;
  const float* v_norms; int64_t vn_stride_blk, vn_stride_pos, vn_stride_head;
  const void* block_tables; int bt_dtype; int64_t bt_stride_seq;
  const void* seq_lens; int sl_dtype;
  const void* query_start_loc; int qs_dtype;
  int num_seqs, num_tokens, num_q_heads, num_kv_heads, head_dim, block_size, max_blocks_per_seq;
  int64_t num_blocks;
  int bits;
  const float* rotation; const float* rotation_t; const float* centroids;
  float scale;
  void* out; int out_dtype; int64_t out_stride_tok, out_stride_head;
  void* workspace; size_t workspace_bytes;   /* akv_tq_prefill_attn_workspace_bytes(num_tokens, num_q_heads) */
  void* stream;
  int max_seq_len;   /* longest entry of seq_lens if the host knows it (vLLM's metadata does), else 0 */
  /* NULL, or the tables of a tq35 / tq25 cache (HOST pointer, see akv_hybrid_tables below): k_packed / v_packed are then
   * the 64- / 44-byte records [num_blocks, block_size, num_kv_heads, packed_dim], the norm arrays, bits and centroids are ignored, and
   * the attention runs in the original domain - pass identity matrices as rotation and rotation_t.  Staged kernel
   * only (max_seq_len and the staged workspace).  Replaces the decompress-then-attend prefill of the hybrid modes
   * (vllm/hooks.py:726-850). */
  const struct akv_hybrid_tables* hybrid_tables;
} akv_tq_prefill_params;

/* Workspace: the first function gives what every call needs.  With max_seq_len set and a workspace of at least
 * akv_tq_prefill_attn_workspace_bytes_staged(...) bytes (32 KB per 64 keys, sequence and KV head more), chunks large
 * enough for the tensor-core kernel are served by its staged variant: one pre-pass turns the codes of every key
 * tile into fp16 operand images in the workspace, and the attention kernel pulls them in with bulk copies instead
 * of decoding them once per 128 query rows. */
size_t akv_tq_prefill_attn_workspace_bytes(int num_tokens, int num_q_heads);
size_t akv_tq_prefill_attn_workspace_bytes_staged(int num_tokens, int num_q_heads, int num_kv_heads, int num_seqs,
                                                  int max_seq_len);
int akv_tq_prefill_attn(const akv_tq_prefill_params* params);

/* One decode step of the serving path in a single call: encode the new tokens'
 * key and value ([num_tokens, num_kv_heads, head_dim], one dtype) into the packed
 * cache named by attn.k_packed / k_norms / v_packed / v_norms (akv_tq_kv_update
 * twice, with attn.bits, attn.rotation_t, attn.block_size), then run
 * akv_tq_paged_attn(&attn) over the updated cache.  Replaces the body of the
 * reference's tq::decode_step op (aither_kvcache/vllm/hooks.py:150-195:
 * encode + index-put of K and V, then TQPagedAttention.forward).  max_blocks
 * bounds the slots that are written (0 is not allowed: pass the number of cache
 * blocks).  Nothing is allocated and nothing synchronises.  With fewer than 2048
 * vectors to write and head_dim 128 or 256 the vectors are encoded by extra
 * blocks of the attention's first launch; in that case a call whose attention
 * arguments are rejected returns the error without having written the cache. */
typedef struct akv_tq_decode_step_params {
  const void* key; const void* value; int kv_dtype;
  int64_t num_tokens;
  int64_t k_stride_tok, k_stride_head, v_stride_tok, v_stride_head;
  const int64_t* slot_mapping;
  const float* boundaries;
  int64_t max_blocks;
  akv_tq_attn_params attn;
} akv_tq_decode_step_params;
int akv_tq_decode_step(const akv_tq_decode_step_params* params);

/* akv_tq_paged_attn without a caller-supplied workspace and without any device
 * allocation.  It has no counterpart in the reference.  It is for callers that
 * cannot allocate around the call - an engine whose memory is fully committed to
 * its KV-cache pool, a plugin that must stay out of the host program's
 * allocator.  The scratch is a fixed array inside the library image
 * (akv_tq_paged_attn_static_scratch_bytes(), 8 MiB per GPU, held until exit);
 * params->workspace / workspace_bytes are ignored.  With blocks_per_split == 0
 * the split size is grown until the partials fit; problems that still do not fit
 * return AKV_ERR_WORKSPACE.  The first call on each device resolves the array's
 * address and should happen before any stream capture.  Calls on one device share
 * the array: calls that can overlap on the GPU race and must be serialised. */
size_t akv_tq_paged_attn_static_scratch_bytes(void);
int akv_tq_paged_attn_static(const akv_tq_attn_params* params);

/* Log-sum-exp merge of partial attention results, the arithmetic of
 * _tq_splitk_reduce (fused_attention.py:479-531) applied across devices.
 *   parts [num_parts, num_seqs*num_q_heads, head_dim+2] float32 as written to raw_out
 * out = R^T (acc / l) when rotation is given, acc / l when it is NULL. */
int akv_lse_merge(const float* parts, int num_parts, int num_seqs, int num_q_heads, int head_dim,
                  const float* rotation, void* out, int out_dtype, int64_t out_stride_seq,
                  int64_t out_stride_head, void* stream);

/* ------------------------------------------------------------------------
 * Block selection for sparse decode attention (head_dim 128)
 * ---------------------------------------------------------------------- */

/* Replaces BlockRepresentativeCache.update + finalize (aither_kvcache/block_selector.py:65-113): for
 * every newly written token t and head h, centroid[code] * norm is added to acc[block_idx[t]][h][:] and
 * counts[block][h] is incremented, then rep = acc / count for the touched blocks.  acc / rep
 * [max_blocks][num_kv_heads][128] float32 and counts [max_blocks][num_kv_heads] int32 are the caller's
 * (zero-initialised) tensors.  Strides in elements. */
int akv_block_select_update(const int64_t* block_idx, int64_t num_tokens, const uint8_t* k_packed,
                            int64_t kp_stride_tok, int64_t kp_stride_head, const float* k_norms,
                            int64_t kn_stride_tok, int64_t kn_stride_head, const float* centroids, int bits,
                            int num_kv_heads, int head_dim, int64_t max_blocks, float* acc, int* counts,
                            float* rep, void* stream);

/* Replaces BlockRepresentativeCache.clear_blocks (block_selector.py:115-121). */
int akv_block_select_clear(const int64_t* block_idx, int64_t num_blocks_to_clear, int num_kv_heads,
                           int64_t max_blocks, float* acc, int* counts, float* rep, void* stream);

/* Replaces score_blocks + select_blocks (block_selector.py:128-228): scores every block of every sequence
 * against the rotated, GQA-averaged query, keeps the first num_sink_blocks and last num_recent_blocks
 * valid blocks, takes the max_selected best (ties: lower logical index) and writes their physical ids in
 * logical order to out_block_tables int32 [num_seqs][max_selected] (rows padded with 0) and the adjusted
 * context lengths to out_context_lens int32 [num_seqs].  exact_tail != 0 counts only the real tokens of a
 * kept partial last block (the reference counts it as full).  scores_out (optional) float32
 * [num_seqs][max_blocks_per_seq] receives the raw scores (-inf past the context). */
size_t akv_block_select_workspace_bytes(int num_seqs, int num_kv_heads, int max_blocks_per_seq);
int akv_block_select(const void* query, int q_dtype, int64_t q_stride_seq, int64_t q_stride_head,
                     int num_seqs, int num_q_heads, int num_kv_heads, int head_dim, const float* rotation_t,
                     const float* rep, int64_t max_blocks, const void* block_tables, int bt_dtype,
                     int64_t bt_stride_seq, const void* context_lens, int cl_dtype, int block_size,
                     int max_blocks_per_seq, int max_selected, int num_sink_blocks, int num_recent_blocks,
                     int exact_tail, int* out_block_tables, int* out_context_lens, float* scores_out,
                     void* workspace, size_t workspace_bytes, void* stream);

/* ------------------------------------------------------------------------
 * Hybrid split-group codec (tq35 / tq25, head_dim 128)
 * ---------------------------------------------------------------------- */

/* Tables of one HybridTurboQuant instance (aither_kvcache/hybrid_quantizer.py:486-547,
 * calibrate/calibrate_uniform :553-603).  All arrays live on the device.
 *   group_index [num_index_heads][head_dim] int32: the dims of group 0, then of group 1
 *   had_signs / qjl_signs [head_dim]: +-1, group 0 then group 1
 *   centroids / boundaries [16]: group 0 in [0..8), group 1 in [8..16) (unused tail ignored)
 * packed_dim selects the mode: 64 = tq35, 44 = tq25. */
typedef struct akv_hybrid_tables {
  int head_dim, packed_dim;
  const int* group_index; int num_index_heads;
  const float* had_signs; const float* qjl_signs;
  const float* centroids; const float* boundaries;
  float qjl_scale0, qjl_scale1;
} akv_hybrid_tables;

/* Replaces HybridTurboQuant.encode (hybrid_quantizer.py:616-779): x [n_rows, 128] ->
 * packed [n_rows, packed_dim] (codes | residual sign bits | fp16 norm | fp16 residual norm,
 * per group).  Row n uses index head n % num_index_heads. */
int akv_hybrid_encode(const void* x, int x_dtype, int64_t n_rows, int64_t x_row_stride,
                      const akv_hybrid_tables* tables, uint8_t* packed, int64_t packed_row_stride,
                      void* stream);

/* Replaces HybridTurboQuant.decode (hybrid_quantizer.py:785-933): out [n_rows, 128] contiguous. */
int akv_hybrid_decode(const uint8_t* packed, int64_t packed_row_stride, int64_t n_rows,
                      const akv_hybrid_tables* tables, void* out, int out_dtype, void* stream);

/* Paged decode attention over tq35 records without reconstructing K/V.  Replaces the
 * decompress-then-SDPA body of tq::hybrid_decode_step (vllm/hooks.py:297-345).
 *   k_cache / v_cache [num_blocks, block_size, num_kv_heads, 64] uint8 (strided views allowed) */
typedef struct akv_hybrid_attn_params {
  const void* query; int q_dtype; int64_t q_stride_seq, q_stride_head;
  const uint8_t* k_cache; int64_t k_stride_blk, k_stride_pos, k_stride_head;
  const uint8_t* v_cache; int64_t v_stride_blk, v_stride_pos, v_stride_head;
  const void* block_tables; int bt_dtype; int64_t bt_stride_seq;
  const void* context_lens; int cl_dtype;
  int num_seqs, num_q_heads, num_kv_heads, block_size, max_blocks_per_seq;
  int64_t num_blocks;
  const akv_hybrid_tables* tables;   /* HOST pointer to the struct; its arrays are device arrays */
  float scale;
  void* out; int out_dtype; int64_t out_stride_seq, out_stride_head;
  void* workspace; size_t workspace_bytes;
  int blocks_per_split;
  void* stream;
} akv_hybrid_attn_params;

size_t akv_hybrid_paged_attn_workspace_bytes(int num_seqs, int num_q_heads, int block_size,
                                             int max_blocks_per_seq, int blocks_per_split);
int akv_hybrid_paged_attn(const akv_hybrid_attn_params* params);

/* Paged write of hybrid records.  Replaces the encode + index-put of tq::hybrid_decode_step
 * (vllm/hooks.py:259-296): x [num_tokens, num_kv_heads, 128] (strides in elements) is encoded and the
 * record of (token, head) is stored at cache[slot / block_size][slot % block_size][head] (strides in
 * bytes), slot = slot_mapping[token].  Tokens with a negative slot, or whose block is >= max_blocks, are
 * skipped (the reference's index-put would wrap a negative slot to the last block). */
int akv_hybrid_kv_update(const void* x, int x_dtype, int64_t num_tokens, int num_kv_heads,
                         int64_t x_stride_tok, int64_t x_stride_head, const int64_t* slot_mapping,
                         const akv_hybrid_tables* tables, uint8_t* cache, int64_t c_stride_blk,
                         int64_t c_stride_pos, int64_t c_stride_head, int block_size, int64_t max_blocks,
                         void* stream);

/* One serving step in one call: body of tq::hybrid_decode_step (vllm/hooks.py:240-355).  The new
 * tokens' K and V records go into attn.k_cache / attn.v_cache at slot_mapping (as akv_hybrid_kv_update),
 * then the attention of akv_hybrid_paged_attn runs over the updated cache.  With fp16 / bf16 K and V
 * whose rows start on 16-byte boundaries the records are written by extra blocks of the attention's
 * first launch (three kernel launches per step); other inputs take two write launches first. */
typedef struct akv_hybrid_decode_step_params {
  const void* key; const void* value; int kv_dtype;   /* [num_tokens, num_kv_heads, 128] */
  int64_t num_tokens;
  int64_t k_stride_tok, k_stride_head, v_stride_tok, v_stride_head;
  const int64_t* slot_mapping;                        /* [num_tokens] */
  int64_t max_blocks;
  akv_hybrid_attn_params attn;
} akv_hybrid_decode_step_params;
int akv_hybrid_decode_step(const akv_hybrid_decode_step_params* params);

/* ------------------------------------------------------------------------
 * TriAttention spectral codec (head_dim 128, int4 coefficients, pre-RoPE keys)
 * ---------------------------------------------------------------------- */

/* Replaces SpectralKVEncoder.encode (aither_kvcache/triattention/encoder.py:73-149, coeff_bits 4;
 * called twice by TriAttention.encode_kv, attention.py:96-112).  Per vector: the num_freqs
 * (8, 12 or 16) RoPE pairs of largest energy in ascending order, their two coefficients
 * quantised to 4 bits against the largest magnitude, and that magnitude as fp16.
 *   indices, packed [n_rows, num_freqs] uint8; scales [n_rows] fp16. */
int akv_tri_encode(const void* x, int x_dtype, int64_t n_rows, int64_t x_row_stride, int head_dim,
                   int num_freqs, uint8_t* indices, uint8_t* packed, void* scales_f16, void* stream);
/* The same with the encoder's other coefficient formats (encoder.py:104-147): coeff_bits 8 stores the
 * two components of a pair as bytes, packed [n_rows, 2 * num_freqs] uint8 (q = round((v / scale + 1) * 127.5));
 * coeff_bits 16 stores them as fp16, packed [n_rows, num_freqs, 2], scales all 1; coeff_bits 4 as above. */
int akv_tri_encode_bits(const void* x, int x_dtype, int64_t n_rows, int64_t x_row_stride, int head_dim,
                        int num_freqs, int coeff_bits, uint8_t* indices, void* packed, void* scales_f16, void* stream);

/* Replaces TriAttention.decode_step (attention.py:186-280) = TrigSeriesScorer.score
 * (scorer.py:115-208) + softmax + _accumulate_values.
 *   query [batch, num_q_heads, 128]; k_ / v_ indices, packed [batch, seq_len, num_kv_heads, F] uint8,
 *   scales [batch, seq_len, num_kv_heads] fp16; theta [64] float32 RoPE frequencies.
 *   key_positions [batch, seq_len] int64 or NULL (position = key_pos_start + index);
 *   query_pos [batch] int64 or NULL (query_pos_default).
 * out is float32 [batch, num_q_heads, 128].  With raw_out the un-normalised partial
 * (m in log2 units, l, acc[128]) per (batch, q head) is written instead, so that key ranges held
 * by different devices can be merged with akv_lse_merge(rotation = NULL). */
typedef struct akv_tri_decode_params {
  const void* query; int q_dtype; int64_t q_stride_batch, q_stride_head;
  const uint8_t* k_indices; const uint8_t* k_packed; const void* k_scales;
  const uint8_t* v_indices; const uint8_t* v_packed; const void* v_scales;
  int batch, seq_len, num_kv_heads, num_q_heads, head_dim, num_freqs;
  const int64_t* key_positions; int64_t key_pos_start;
  const int64_t* query_pos; int64_t query_pos_default;
  const float* theta;
  float scale;
  float* out;
  float* raw_out;
  void* workspace; size_t workspace_bytes;
  int tokens_per_split;   /* 0 = library default */
  void* stream;
  void* ev_kernel_start; void* ev_kernel_stop;   /* optional cudaEvent_t pair around the main kernel */
  float* scores_out;      /* optional [batch, num_q_heads, seq_len] float32: the pre-softmax scores
                             (what TrigSeriesScorer.score returns); NULL = not written */
  /* Paged records (SpectralKVCache, triattention/cache.py:48-110): with block_tables the six arrays are
   * [num_blocks, block_size, num_kv_heads, ...] and token s of batch element b is slot s % block_size of
   * block block_tables[b][s / block_size]; seq_len = table width x block_size; key_positions must be NULL.
   * context_lens (optional, also without block_tables) [batch]: tokens of each batch element, clamped to
   * [0, seq_len]; an element of length 0 gives zeros.  Index arrays are int32 (dtype 0) or int64 (1). */
  const void* block_tables; int bt_dtype; int64_t bt_stride_batch;
  int block_size; int64_t num_blocks;
  const void* context_lens; int cl_dtype;
  /* Coefficient format of the packed arrays (SpectralKVEncoder, encoder.py:97-147; scorer.py:94-113):
   * 0 or 4: one byte per pair, [.., F]; 8: two bytes per pair (even, odd), [.., 2F]; 16: two fp16 per pair,
   * [.., F, 2], scales ignored.  post_rope != 0: keys were encoded after RoPE, scores are the plain sparse
   * dot product (scorer.py:201-203) and positions are not used. */
  int coeff_bits, post_rope;
} akv_tri_decode_params;

size_t akv_tri_decode_workspace_bytes(int batch, int num_q_heads, int seq_len, int tokens_per_split);
int akv_tri_decode_step(const akv_tri_decode_params* params);

/* ------------------------------------------------------------------------
 * Cross-GPU merge of split-K partials over NVLink peer memory (no counterpart in the reference, which
 * has no multi-device path; the merge arithmetic is that of fused_attention.py:513-527)
 * ---------------------------------------------------------------------- */

/* Every rank calls this with its partial local_raw [num_seqs*num_q_heads][head_dim+2] (m in log2 units, l,
 * acc - the raw_out of akv_tq_paged_attn / akv_tri_decode_step).  The call copies the partial into slot
 * `rank` of every rank's exchange buffer with peer stores, raises a flag word on every rank, waits
 * (bounded, about a second) until all ranks' partials of this step have arrived locally, and merges them:
 * out = R^T (acc / l) with `rotation`, acc / l without.  Three kernel launches, no collective library, no
 * multimem; capturable in a CUDA graph (step counter and buffer half live in `state`).
 *   peer_buffers  HOST array [world]: device pointer of each rank's exchange buffer of
 *                 akv_p2p_exchange_bytes() bytes, 16-byte aligned, mapped on this device (entry `rank`
 *                 is this rank's own buffer) - e.g. torch symmetric memory
 *   peer_flags    HOST array [world]: device pointer of each rank's flag array, `world` uint32 words,
 *                 zero before the first step
 *   state         two local uint32 device words, zero before the first step
 * All ranks must make the same sequence of calls.  A wait that runs out sets status word 4 of
 * akv_device_status and the merge proceeds on whatever has arrived. */
typedef struct akv_p2p_merge_params {
  const float* local_raw;
  int num_seqs, num_q_heads, head_dim;
  int world, rank;
  void* const* peer_buffers;
  void* const* peer_flags;
  unsigned int* state;
  const float* rotation;             /* optional R, row-major */
  void* out; int out_dtype; int64_t out_stride_seq, out_stride_head;
  void* stream;
} akv_p2p_merge_params;
size_t akv_p2p_exchange_bytes(int world, int num_seqs, int num_q_heads, int head_dim);
int akv_p2p_lse_merge(const akv_p2p_merge_params* params);

#ifdef __cplusplus
}
#endif
#endif /* AKV_B200_H */
