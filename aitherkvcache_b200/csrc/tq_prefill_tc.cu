// Chunked-prefill attention over the packed 4-bit cache on the 5th-generation tensor cores (tcgen05 / TMEM).
//
// Same operation as tq_prefill_attn_kernel (tq_prefill.cuh); the reference decompresses every active block to
// bf16 and calls vLLM's unified attention (vllm/backend.py:1093-1244, vllm/hooks.py:726-850).  A CTA owns 128
// (token, query head) rows of one sequence and one KV head - 128 / G consecutive query tokens, G = query heads per
// KV head - and walks over the causal key range in tiles of 64 keys.  Both products of a tile are tcgen05 MMAs with
// float32 accumulators in tensor memory:
//   S[128 rows][64 keys]  = Q K^T   A = the rotated queries (fp16, shared memory, written once),
//                                   B = the tile's keys, codes -> fp16 centroids times the key norm;
//   O[128 rows][144]      += P V    A = the probabilities (fp16, shared memory), B = the tile's values transposed,
//                                   codes -> fp16 centroids times the value norm, plus a row of ones: column 128 of
//                                   O is the row sum of the probabilities as the tensor cores saw them.
// (Norms are folded in as fp16 factors: a key or value norm below 1e-2 loses bits to fp16's subnormal range.)
// All operands are K-major in the 128-byte-swizzled layout of umma.cuh.  Thirteen warps, no CTA-wide barrier in the loop:
//   warps 0-3   softmax: thread = row (staged variant: warps 0-7, two threads per row with 64 keys of the tile each).  S out of tensor memory (tcgen05.ld), causal limit, running reference maximum
//               (the accumulator O is rescaled only when the maximum grows by more than 2^8: tcgen05.ld / st of the
//               thread's own lane), exp2, fp16 probabilities into the P operand.
//   warps 4-11  decode: packed bytes and norms from global memory two tiles ahead in registers (block-table entries
//               three tiles ahead), byte -> half2 by a per-lane lookup table; a thread writes 16-byte pieces of the K
//               operand (32 dims of one key) and of the transposed V operand (8 keys of 4 dims).
//   warp 12     one lane issues the MMAs: S of tile j+1 before P V of tile j, so the tensor cores compute the next
//               scores while the softmax warps work on the current ones.
// Hand-overs are mbarriers (tile j uses stage j % 2 of every operand and accumulator S):
//   k_full / v_full  8 decode-warp arrivals: the operand stage is written          -> MMA warp
//   s_full           tcgen05.commit after S: scores ready                          -> softmax warps; K stage free -> decode warps
//   s_free           4 softmax-warp arrivals: S is in registers                    -> MMA warp may overwrite it
//   p_full           4 arrivals: P written, O rescaled if need be                  -> MMA warp
//   pv_done          tcgen05.commit after P V                                      -> V stage and P buffer free, O readable
// Every wait is bounded; a wait that gives up sets g_prefill_tc_status and a shared flag that ends all loops; the
// CTA then leaves after releasing its tensor memory, its rows unwritten (they come out as zeros).
//
// Three kernels live here: tq_prefill_tc_kernel<G, false> as described above (codes decoded in the kernel),
// tq_prefill_tc_kernel<G, true> (operand images staged in global memory by a pre-pass, tiles of 128 keys, Q and P as
// tensor-memory operands, all softmax warps on one tile) and tq_prefill_pp_kernel<G> (staged images, two softmax groups
// in ping-pong over the key tiles: the default whenever images are staged; its own description is above it).
#include "tq_prefill_args.cuh"
#include "umma.cuh"
#include <math_constants.h>

namespace akv {
namespace {

__device__ int g_prefill_tc_status;          // 1: a bounded wait gave up, 2: tensor-memory columns were kept
__device__ int g_prefill_tc_withhold = -1;   // test hook: CTAs (0, 0, z) issue neither the score MMAs nor the commit of this tile of their share

constexpr int PT_VHALF = 144 * 128;                  // 64 keys of a value operand: 128 dims + the row of ones (+ 15 zero rows)

// Shared-memory layout and warp roles of the two variants: codes decoded in the kernel (13 warps, tiles of 64 keys, two
// operand stages, the lookup table) or operand images staged in global memory by tq_prefill_stage_kernel (10 warps, tiles
// of 128 keys - half as many MMA instructions per key -, two softmax threads per row, three stages fed by bulk copies).
template <bool STAGED> struct PtL {
  static constexpr int KT = STAGED ? 128 : 64;        // keys per tile
  static constexpr int NST = STAGED ? 3 : 2;          // K / V operand stages (the barrier block has room for four)
  static_assert(NST <= 4, "barrier slots");
  static constexpr int SW = STAGED ? 8 : 4;           // softmax warps: 4 = a thread per row, 8 = two threads per row (64 keys each)
  static constexpr int WARPS = STAGED ? 10 : 13;
  static constexpr int THREADS = WARPS * 32;
  static constexpr int MMA_WARP = STAGED ? 8 : 12;
  static constexpr int LOAD_WARP = 9;                 // staged: the lane that issues the bulk copies
  static_assert(KT / (SW / 4) == 64, "a softmax thread handles 64 keys of a tile");
  static constexpr int KHALF = KT * 128;              // 64 dims of a key operand: KT rows x 128 B
  static constexpr int KSTAGE = 2 * KHALF;            // B of S: [KT keys][128 dims], two halves of 64 dims
  static constexpr int VSTAGE = (KT / 64) * PT_VHALF; // B of PV: [144 rows][KT keys], one half per 64 keys
  static constexpr int K = 0;
  static constexpr int V = K + NST * KSTAGE;
  static constexpr int LUT = V + NST * VSTAGE;        // byte -> half2, one copy per lane (256 x 128 B); not staged only
  static constexpr int BAR = LUT + (STAGED ? 0 : 32768);      // mbarriers, tensor-memory slot, failed flag
  static constexpr int SMEM = BAR + 512 + 1024;       // + slack for the 1024-byte alignment
  // tensor memory (512 columns): S stage s at column KT s - its first KT / 2 columns are reused for the fp16 P of the same
  // tile -, O at 2 KT (144 columns, column 128 = row sum), Q (64 columns of fp16 pairs) behind it
  static constexpr int T_O = 2 * KT, T_Q = 2 * KT + 160;
  static_assert(T_Q + 64 <= 512, "tensor memory");
};
constexpr int PS_KT = PtL<true>::KT;                 // keys per staged tile
constexpr int PT_IMAGE = PS_KT * 512;                // a staged tile in global memory: K operand image, then V operand halves
static_assert(PS_KT == PFI_KEYS && PT_IMAGE == PFI_BYTES && PtL<true>::KHALF == PFI_KHALF && PtL<true>::KSTAGE == PFI_VOFF,
              "image layout shared with the other pre-pass kernels");
// barrier slots (8 bytes each; up to four operand stages)
constexpr uint32_t B_KFULL = 0, B_VFULL = 32, B_SFULL = 64, B_PFULL = 96, B_PVDONE = 112,
                   B_VFREE = 160, B_DRAIN = 192, B_TMEM = 200, B_FAILED = 204,
                   B_MX = 256;          // 4 row quadrants x 2 tile parities: both half-row warps have published their maxima
constexpr int PT_TMEM_COLS = 512;
constexpr float PT_RESCALE = 8.0f;                   // log2 units the row maximum may grow before O is rescaled

__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
      "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
      :: "r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]),
         "r"(v[8]), "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]),
         "r"(v[16]), "r"(v[17]), "r"(v[18]), "r"(v[19]), "r"(v[20]), "r"(v[21]), "r"(v[22]), "r"(v[23]),
         "r"(v[24]), "r"(v[25]), "r"(v[26]), "r"(v[27]), "r"(v[28]), "r"(v[29]), "r"(v[30]), "r"(v[31])
      : "memory");
}

// MMA with the A operand in tensor memory: row i of A is lane i, its K elements are packed two per 32-bit column
// (a 16-element K step = 8 columns) - the layout a thread's tcgen05.st of packed half2 registers produces.
__device__ __forceinline__ void umma_f16_ta(uint32_t tmem_d, uint32_t tmem_a, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}\n"
      :: "r"(tmem_d), "r"(tmem_a), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}

__device__ __forceinline__ void pt_sts128(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" :: "r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}
__device__ __forceinline__ uint32_t pt_pack_half2(float lo, float hi) {
  __half2 h = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&h);
}
__device__ __forceinline__ float pt_ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ void pt_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" :: "r"(bar) : "memory");
}

// K operand rows: thread (key kr, chunk kc) turns its 16 packed bytes (32 dims) into four 16-byte pieces of row kr, times
// the key norm.  Words 2, 3 first for the upper chunks: the eight threads of a quarter warp then store to eight
// different bank groups.  `stage` is the shared address of a [keys][128 dims] operand: two halves of 64 dims,
// `half_stride` bytes apart; the key is row row0 + kr.
__device__ __forceinline__ void pt_decode_k(uint32_t stage, uint32_t half_stride, int row0, uint32_t lut, int kr, int kc,
                                            const uint4& kw, float kn) {
  const uint32_t hi = (uint32_t)(kc >> 1);
  const __half2 knh = __float2half2_rn(kn);
  const uint32_t ws[4] = {hi ? kw.z : kw.x, hi ? kw.w : kw.y, hi ? kw.x : kw.z, hi ? kw.y : kw.w};
  const uint32_t row = stage + hi * half_stride + (uint32_t)(row0 + kr) * 128u;     // row0 is a multiple of 8
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    uint32_t h[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const uint32_t x = lds_u32(lut + (((ws[i] >> (8 * e)) & 0xffu) << 7));
      const __half2 y = __hmul2(*reinterpret_cast<const __half2*>(&x), knh);
      h[e] = *reinterpret_cast<const uint32_t*>(&y);
    }
    const uint32_t chunk = (uint32_t)(4 * (kc & 1)) + ((uint32_t)i ^ (hi << 1));
    pt_sts128(row + ((chunk ^ (uint32_t)(kr & 7)) << 4), h[0], h[1], h[2], h[3]);
  }
}

// Transposed V operand: thread (key group kg, bytes vbyte, vbyte + 1) turns two bytes of each of the keys 8 kg .. 8 kg + 7
// into the 16-byte pieces (8 keys) of the four dim rows 2 vbyte .. 2 vbyte + 3, times the value norms.
__device__ __forceinline__ void pt_decode_v(uint32_t stage, uint32_t lut, int kg, int vbyte, const uint32_t (&vw)[8],
                                            const float (&vn)[8]) {
  uint32_t e0[8], e1[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const __half2 nh = __float2half2_rn(vn[i]);
    const uint32_t x0 = lds_u32(lut + ((vw[i] & 0xffu) << 7)), x1 = lds_u32(lut + (((vw[i] >> 8) & 0xffu) << 7));
    const __half2 y0 = __hmul2(*reinterpret_cast<const __half2*>(&x0), nh), y1 = __hmul2(*reinterpret_cast<const __half2*>(&x1), nh);
    e0[i] = *reinterpret_cast<const uint32_t*>(&y0);
    e1[i] = *reinterpret_cast<const uint32_t*>(&y1);
  }
  const int r0 = 2 * vbyte;            // dims 2 vbyte, + 1 (first byte), + 2, + 3 (second byte)
  auto put = [&](int row, const uint32_t (&e)[8], uint32_t sel) {
    pt_sts128(stage + (uint32_t)row * 128u + (((uint32_t)kg ^ (uint32_t)(row & 7)) << 4),
              __byte_perm(e[0], e[1], sel), __byte_perm(e[2], e[3], sel), __byte_perm(e[4], e[5], sel), __byte_perm(e[6], e[7], sel));
  };
  put(r0, e0, 0x5410u);
  put(r0 + 1, e0, 0x7632u);
  put(r0 + 2, e1, 0x5410u);
  put(r0 + 3, e1, 0x7632u);
}

__device__ __forceinline__ void pt_fill_lut(uint8_t* lut, const float* centroids, int tid, int threads) {
  // byte -> half2(centroid[high nibble], centroid[low nibble]) = coordinates 2b, 2b+1; one copy per lane
  __shared__ float s_cent[16];
  if (tid < 16) s_cent[tid] = centroids[tid];
  __syncthreads();
  for (int i = tid; i < 256 * 8; i += threads) {
    const int e = i >> 3, q4 = i & 7;
    const uint32_t v = pt_pack_half2(s_cent[e >> 4], s_cent[e & 15]);
    *reinterpret_cast<uint4*>(lut + e * 128 + q4 * 16) = make_uint4(v, v, v, v);
  }
}

template <int G, bool STAGED>
__global__ void __launch_bounds__(PtL<STAGED>::THREADS, 1)
tq_prefill_tc_kernel(PrefillArgs a) {
  using L = PtL<STAGED>;
  constexpr int PT_THREADS = L::THREADS, PT_K = L::K, PT_V = L::V, PT_LUT = L::LUT, PT_BAR = L::BAR;
  constexpr int NST = L::NST, PT_KT = L::KT, PT_STAGE = L::KSTAGE, PT_VSTAGE = L::VSTAGE;
  static_assert(G == 1 || G == 2 || G == 4 || G == 8, "query heads per KV head");
  constexpr int TT = 128 / G;           // query tokens of a CTA
  extern __shared__ uint8_t pt_smem_raw[];
  const uint32_t raw_s = smem_u32(pt_smem_raw);
  const uint32_t base_s = (raw_s + 1023u) & ~1023u;
  uint8_t* base = pt_smem_raw + (base_s - raw_s);
  const uint32_t bar_s = base_s + PT_BAR, failed_s = bar_s + B_FAILED;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int kvh = blockIdx.y;

  // ---- which sequence and which of its query tiles (uniform for the CTA) ----
  int tile = blockIdx.x, s = 0, q0 = 0, qlen = 0;
  bool found = false;
  for (s = 0; s < a.num_seqs; ++s) {
    q0 = (int)load_index(a.query_start_loc, a.qs_dtype, s);
    const int q1 = (int)load_index(a.query_start_loc, a.qs_dtype, s + 1);
    qlen = q1 - q0;
    if (qlen < 0) qlen = 0;
    const int tiles = (qlen + TT - 1) / TT;
    if (tile < tiles) { found = true; break; }
    tile -= tiles;
  }
  if (!found) return;
  const int64_t max_ctx = (int64_t)a.max_blocks_per_seq * a.block_size;
  const int seq_len = (int)load_ctx(a.seq_lens, a.sl_dtype, s, max_ctx);
  int past = seq_len - qlen;            // keys before the chunk
  if (past < 0) past = 0;
  const int tok_lo = tile * TT;
  const int tok_hi = (tok_lo + TT < qlen) ? tok_lo + TT : qlen;
  int kend = past + tok_hi;             // keys any row of this CTA may see
  if (kend > seq_len) kend = seq_len;
  int n_all = (kend + PT_KT - 1) / PT_KT;
  if (STAGED && n_all > a.tiles_per_seq) n_all = a.tiles_per_seq;      // a caller that understated max_seq_len: no read past the images
  // split z of gridDim.z takes an even share of the CTA's key tiles and writes partial z of its rows (short chunks on
  // long contexts: more CTAs than row tiles); tile indices below are local to the share, jbase + j is the tile itself
  const int jbase = (int)((int64_t)n_all * blockIdx.z / gridDim.z);
  const int n_ktiles = (int)((int64_t)n_all * (blockIdx.z + 1) / gridDim.z) - jbase;
  if (n_ktiles <= 0) return;            // nothing to attend to: the partial keeps l = 0

  // ---------------- one-time setup ----------------
  if (tid == 0) {
    for (int i = 0; i < NST; ++i) {
      // decoded in the kernel: 8 decode-warp arrivals; staged: the producer's arrive.expect_tx + the copy's bytes
      asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" :: "r"(bar_s + B_KFULL + 8 * i), "r"(STAGED ? 1 : 8));
      asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" :: "r"(bar_s + B_VFULL + 8 * i), "r"(STAGED ? 1 : 8));
      asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" :: "r"(bar_s + B_VFREE + 8 * i));
    }
    for (int i = 0; i < 2; ++i) {
      asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" :: "r"(bar_s + B_SFULL + 8 * i));
      asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" :: "r"(bar_s + B_PFULL + 8 * i), "r"(L::SW));
      asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" :: "r"(bar_s + B_PVDONE + 8 * i));
    }
    for (int i = 0; i < 8; ++i) asm volatile("mbarrier.init.shared::cta.b64 [%0], 2;" :: "r"(bar_s + B_MX + 8 * i));
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" :: "r"(bar_s + B_DRAIN));
    asm volatile("st.shared.u32 [%0], %1;" :: "r"(failed_s), "r"(0u) : "memory");
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncwarp();
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" :: "r"(bar_s + B_TMEM), "n"(PT_TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  if constexpr (!STAGED) pt_fill_lut(base + PT_LUT, a.centroids, tid, PT_THREADS);
  // rows 128..143 of both value stages: a row of ones (output column 128 becomes the row sum of P) and zero rows
  for (int e = tid; e < NST * (PT_KT / 64) * 16 * 8; e += PT_THREADS) {
    const int half = e >> 7, r = (e >> 3) & 15, c = e & 7;         // the halves of all stages lie back to back
    const uint32_t v = r == 0 ? 0x3C003C00u : 0u;
    *reinterpret_cast<uint4*>(base + PT_V + half * PT_VHALF + (128 + r) * 128 + c * 16) = make_uint4(v, v, v, v);
  }
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = lds_u32(bar_s + B_TMEM);
  const uint32_t tmem_o = tmem_base + L::T_O, tmem_q = tmem_base + L::T_Q;
  // A operand of S: the CTA's query rows, row r = (token tok_lo + r / G, head r % G), zeros for rows without a token;
  // thread r of the softmax warps writes its row into its lane of tensor memory
  if (warp < 4) {
    const int r = tid, tok = tok_lo + r / G;
    const bool have = tok < qlen && q0 + tok < a.n_tokens;
    const float4* src = reinterpret_cast<const float4*>(a.qrot + ((int64_t)(q0 + (have ? tok : 0)) * a.num_q_heads + kvh * G + r % G) * 128);
#pragma unroll 1
    for (int c = 0; c < 2; ++c) {
      uint32_t w[32];
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        const float4 f = have ? src[16 * c + i] : make_float4(0.f, 0.f, 0.f, 0.f);
        w[2 * i] = pt_pack_half2(f.x, f.y);
        w[2 * i + 1] = pt_pack_half2(f.z, f.w);
      }
      tmem_st32(tmem_q + (((uint32_t)(warp * 32)) << 16) + 32 * c, w);
    }
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");

  // Bounded wait.  Fast path: one try_wait (the hardware parks the thread for a while if the phase has not flipped).  Only
  // a wait that comes back empty goes into the counted loop; once one wait of the CTA has run out, the others return
  // at once.
  auto wait = [&](uint32_t bar, uint32_t parity) -> bool {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}\n"
        : "=r"(done) : "r"(bar), "r"(parity) : "memory");
    if (done) return true;
    if (lds_u32(failed_s) != 0u) return false;
    if (mbar_wait(bar, parity)) return true;
    g_prefill_tc_status = 1;
    asm volatile("st.shared.u32 [%0], %1;" :: "r"(failed_s), "r"(1u) : "memory");
    return false;
  };
  auto wait_warp = [&](uint32_t bar, uint32_t parity) -> bool { return __all_sync(0xffffffffu, wait(bar, parity)); };
  auto par2 = [](int j) -> uint32_t { return (uint32_t)((j >> 1) & 1); };      // phase parity of tile j on a two-stage barrier
  auto kst = [](int j) -> uint32_t { return (uint32_t)(j % NST); };             // operand stage of tile j ...
  auto kpar = [](int j) -> uint32_t { return (uint32_t)((j / NST) & 1); };      // ... and its phase parity

  if (warp == L::MMA_WARP) {
    // ================= MMA warp =================
    if (lane == 0) {
      // D = f32, A / B = f16, B K-major; N = keys per tile (scores) or 144 (values), M = 128
      constexpr uint32_t IDESC_S = (1u << 4) | (((uint32_t)PT_KT >> 3) << 17) | ((128u >> 4) << 24);
      constexpr uint32_t IDESC_O = (1u << 4) | ((144u >> 3) << 17) | ((128u >> 4) << 24);
      const int withhold = (blockIdx.x | blockIdx.y) == 0 ? g_prefill_tc_withhold : -1;
      // Descriptors differ only in their 14-bit address field: one constant upper half, lower halves by 32-bit adds.
      const uint64_t d_hi = umma_desc(0u) & 0xffffffff00000000ull;
      const uint32_t d_lo = (uint32_t)umma_desc(0u);
      auto desc = [&](uint32_t saddr) -> uint64_t { return d_hi | (uint64_t)(d_lo + ((saddr & 0x3FFFFu) >> 4)); };
      const uint32_t k_lo = base_s + PT_K, v_lo = base_s + PT_V;
      // S buffer (j & 1) was last read by the softmax warps for tile j-2, whose p_full this lane has waited for before
      // it issued P V of tile j-2: no separate "scores read" barrier is needed.
      auto issue_s = [&](int j) -> bool {
        const uint32_t st = (uint32_t)(j & 1), ks = kst(j);
        if (!wait(bar_s + B_KFULL + 8 * ks, kpar(j))) return false;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        if (j == withhold) return true;
        const uint32_t kb = k_lo + ks * PT_STAGE;
#pragma unroll
        for (int kk = 0; kk < 8; ++kk)
          umma_f16_ta(tmem_base + st * PT_KT, tmem_q + (uint32_t)(kk * 8), desc(kb + (uint32_t)((kk >> 2) * L::KHALF + (kk & 3) * 32)),
                      IDESC_S, (uint32_t)(kk != 0));
        umma_commit(bar_s + B_SFULL + 8 * st);
        return true;
      };
      auto issue_pv = [&](int j) -> bool {
        const uint32_t st = (uint32_t)(j & 1), ks = kst(j);
        if (!wait(bar_s + B_PFULL + 8 * st, par2(j))) return false;
        if constexpr (!STAGED) {       // staged: the value image arrived on the same barrier as the key image
          if (!wait(bar_s + B_VFULL + 8 * ks, kpar(j))) return false;
        }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t vb = v_lo + ks * PT_VSTAGE;
#pragma unroll
        for (int kk = 0; kk < PT_KT / 16; ++kk)      // P of the tile: fp16 pairs in the first columns of its S stage
          umma_f16_ta(tmem_o, tmem_base + st * PT_KT + (uint32_t)(kk * 8), desc(vb + (uint32_t)((kk >> 2) * PT_VHALF + (kk & 3) * 32)),
                      IDESC_O, (uint32_t)((j | kk) != 0));
        umma_commit(bar_s + B_PVDONE + 8 * st);
        if constexpr (STAGED) umma_commit(bar_s + B_VFREE + 8 * ks);
        return true;
      };
      if (issue_s(0)) {
        for (int j = 0; j < n_ktiles; ++j) {
          if (j + 1 < n_ktiles && !issue_s(j + 1)) break;
          if (!issue_pv(j)) break;
        }
      }
    }
    __syncwarp();
  } else if (STAGED && warp == L::LOAD_WARP) {
    // ================= producer: operand images of tile j by two bulk copies =================
    if (lane == 0) {
      const uint8_t* src = a.staged + (((int64_t)s * a.tiles_per_seq + jbase) * a.num_kv_heads + kvh) * PT_IMAGE;
      const int64_t step = (int64_t)a.num_kv_heads * PT_IMAGE;
      int issued = 0;
      for (int j = 0; j < n_ktiles; ++j) {
        const uint32_t ks = kst(j);
        // P V of tile j - NST complete: its value stage is free, and so is its key stage (the scores came first)
        if (j >= NST && !wait(bar_s + B_VFREE + 8 * ks, kpar(j - NST))) break;
        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" :: "r"(bar_s + B_KFULL + 8 * ks), "r"(PT_IMAGE) : "memory");
        asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                     :: "r"(base_s + PT_K + ks * PT_STAGE), "l"(src + j * step), "r"(PT_STAGE), "r"(bar_s + B_KFULL + 8 * ks) : "memory");
#pragma unroll
        for (int h = 0; h < PT_KT / 64; ++h)       // the value halves leave room for their rows of ones in shared memory
          asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                       :: "r"(base_s + PT_V + ks * PT_VSTAGE + h * PT_VHALF), "l"(src + j * step + PT_STAGE + h * 16384), "r"(16384),
                          "r"(bar_s + B_KFULL + 8 * ks) : "memory");
        issued = j + 1;
      }
      // a CTA that gives up must not leave while copies into its shared memory are in flight: the last copies of every
      // stage are waited for here (bounded); in the regular flow the MMA warp has consumed them all already
      if (lds_u32(failed_s) != 0u)
        for (int j = issued - NST < 0 ? 0 : issued - NST; j < issued; ++j) mbar_wait(bar_s + B_KFULL + 8 * kst(j), kpar(j));
    }
    __syncwarp();
  } else if (!STAGED && warp >= 4) {
    // ================= decode warps =================
    const int d = tid - 128;
    const int kr = d >> 2, kc = d & 3;                          // K: 16 bytes (32 dims) of key kr
    const int kg = d & 7, vbyte = 4 * (d >> 4) + 2 * ((d >> 3) & 1);     // V: bytes vbyte, vbyte + 1 of keys 8 kg .. 8 kg + 7
    const uint32_t lut = base_s + PT_LUT + lane * 4;
    const int n_table = a.max_blocks_per_seq, bs = a.block_size;
    // Addressing without divisions or 64-bit products in the loop: (block index, position in block) of the thread's K key
    // and of its first V key advance by one tile per step; a block-table entry is read two tiles ahead of its use.
    // the entry comes back as loaded (nothing waits for it here); phys() turns it into a block number at its use
    const bool bt64 = a.bt_dtype == AKV_I64;
    const char* bt_row = reinterpret_cast<const char*>(a.block_tables) + (int64_t)s * a.bt_stride * (bt64 ? 8 : 4);
    auto entry = [&](int blk) -> uint64_t {
      if (blk >= n_table) blk = n_table - 1;
      if (blk < 0) blk = 0;
      if (n_table <= 0) return 0ull;
      return bt64 ? (uint64_t)__ldg(reinterpret_cast<const long long*>(bt_row) + blk)
                  : (uint64_t)(uint32_t)__ldg(reinterpret_cast<const int*>(bt_row) + blk);
    };
    auto phys = [&](uint64_t raw) -> int64_t {
      const int64_t pb = bt64 ? (int64_t)raw : (int64_t)(int32_t)(uint32_t)raw;
      return pb < 0 ? 0 : (pb >= a.num_blocks ? a.num_blocks - 1 : pb);
    };
    const int adv_blk = PT_KT / bs, adv_pos = PT_KT - adv_blk * bs;       // 64 keys = adv_blk blocks + adv_pos positions
    auto advance = [&](int& blk, int& pos) {
      blk += adv_blk;
      pos += adv_pos;
      if (pos >= bs) { pos -= bs; ++blk; }
    };
    const uint8_t* kbase = a.k_packed + (int64_t)kvh * a.kp_sh + kc * 16;
    const float* knbase = a.k_norms + (int64_t)kvh * a.kn_sh;
    const uint8_t* vbase = a.v_packed + (int64_t)kvh * a.vp_sh + vbyte;
    const float* vnbase = a.v_norms + (int64_t)kvh * a.vn_sh;
    const uint32_t kp_sp = (uint32_t)a.kp_sp, kn_sp = (uint32_t)a.kn_sp, vn_sp = (uint32_t)a.vn_sp;     // strides inside a block
    const int64_t vp_sp = a.vp_sp;
    // raw bytes and norms of three tiles: tile j is decoded out of set j % 3 while the loads of tiles j + 1 and j + 2 are
    // in flight (a load from a cold block takes longer than one tile's work)
    struct Raw { uint4 k; float kn; uint32_t v[8]; float vn[8]; };
    Raw R0, R1, R2;
    R0.k = R1.k = R2.k = make_uint4(0u, 0u, 0u, 0u);
    R0.kn = R1.kn = R2.kn = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) { R0.v[i] = R1.v[i] = R2.v[i] = 0u; R0.vn[i] = R1.vn[i] = R2.vn[i] = 0.f; }
    auto load = [&](int j, uint64_t rawk, int posk, uint64_t rawv, int posv, Raw& R) {
      uint4& k4 = R.k; float& knorm = R.kn; uint32_t (&v2)[8] = R.v; float (&vnorm)[8] = R.vn;
      if (j >= n_ktiles) return;
      const int64_t pbk = phys(rawk), pbv = phys(rawv);
      k4 = __ldg(reinterpret_cast<const uint4*>(kbase + pbk * a.kp_sb + (uint32_t)posk * kp_sp));
      knorm = __ldg(knbase + pbk * a.kn_sb + (uint32_t)posk * kn_sp);
      const uint8_t* vp = vbase + pbv * a.vp_sb + (int64_t)posv * vp_sp;
      const float* np = vnbase + pbv * a.vn_sb + (uint32_t)posv * vn_sp;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        v2[i] = (uint32_t)__ldg(reinterpret_cast<const unsigned short*>(vp));
        vnorm[i] = __ldg(np);
        vp += vp_sp;
        np += vn_sp;
      }
      if (j == n_ktiles - 1) {      // a key past the range carries any norm: its score is masked, its value row becomes zero
        const int key8 = PT_KT * (jbase + j) + 8 * kg;
#pragma unroll
        for (int i = 0; i < 8; ++i) vnorm[i] = key8 + i < kend ? vnorm[i] : 0.f;
        if (PT_KT * (jbase + j) + kr >= kend) knorm = 0.f;
      }
    };
    const int key_k0 = PT_KT * jbase + kr, key_v0 = PT_KT * jbase + 8 * kg;      // this thread's keys in the share's first tile
    int blk_k = key_k0 / bs, pos_k = key_k0 - blk_k * bs, blk_v = key_v0 / bs, pos_v = key_v0 - blk_v * bs;
    load(0, entry(blk_k), pos_k, entry(blk_v), pos_v, R0);
    advance(blk_k, pos_k);
    advance(blk_v, pos_v);
    load(1, entry(blk_k), pos_k, entry(blk_v), pos_v, R1);
    advance(blk_k, pos_k);
    advance(blk_v, pos_v);
    uint64_t pbk_nx = entry(blk_k), pbv_nx = entry(blk_v);      // tile 2
    int posk_nx = pos_k, posv_nx = pos_v;
    auto tile_step = [&](int j, Raw& cur, Raw& tgt) -> bool {
      const uint32_t st = (uint32_t)(j & 1);
      const uint4 kw = cur.k;
      const float kn = cur.kn;
      const uint32_t (&vw)[8] = cur.v;
      const float (&vn)[8] = cur.vn;
      load(j + 2, pbk_nx, posk_nx, pbv_nx, posv_nx, tgt);
      advance(blk_k, pos_k);
      advance(blk_v, pos_v);
      if (j + 3 < n_ktiles) { pbk_nx = entry(blk_k); pbv_nx = entry(blk_v); }       // tile j + 3
      posk_nx = pos_k;
      posv_nx = pos_v;
      // ---- K operand of tile j: free once the scores of tile j-2 are complete ----
      if (j >= 2 && !wait_warp(bar_s + B_SFULL + 8 * st, par2(j - 2))) return false;
      pt_decode_k(base_s + PT_K + st * PT_STAGE, L::KHALF, 0, lut, kr, kc, kw, kn);
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      __syncwarp();
      if (lane == 0) pt_arrive(bar_s + B_KFULL + 8 * st);
      // ---- transposed V operand of tile j: free once P V of tile j-2 is complete ----
      if (j >= 2 && !wait_warp(bar_s + B_PVDONE + 8 * st, par2(j - 2))) return false;
      pt_decode_v(base_s + PT_V + st * PT_VSTAGE, lut, kg, vbyte, vw, vn);
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      __syncwarp();
      if (lane == 0) pt_arrive(bar_s + B_VFULL + 8 * st);
      return true;
    };
    for (int j = 0; j < n_ktiles; j += 3) {
      if (!tile_step(j, R0, R2)) break;
      if (j + 1 < n_ktiles && !tile_step(j + 1, R1, R0)) break;
      if (j + 2 < n_ktiles && !tile_step(j + 2, R2, R1)) break;
    }
  } else if (warp < L::SW) {
    // ================= softmax warps: thread = 64 keys of a row =================
    // (warps 0-3: rows 32 warp .. + 31; with eight warps, warps 4-7 take the second 64 keys of the same rows - a warp
    // may only touch the 32 tensor-memory lanes of its index modulo 4)
    __shared__ float s_mx[2][2][128];             // [tile parity][half][row]: the half-row maxima of a tile
    constexpr int SPLIT = L::SW / 4;
    const int quad = warp & 3, hf = warp >> 2;
    const int r = quad * 32 + lane;
    const int tok = tok_lo + r / G;
    const bool live = tok < qlen && q0 + tok < a.n_tokens;
    int lim = live ? past + tok + 1 : 0;          // keys the row may see
    if (lim > seq_len) lim = seq_len;
    const uint32_t t_lane = ((uint32_t)(quad * 32)) << 16;
    float m_ref = -CUDART_INF_F;
    bool ok = true;
    for (int j = 0; j < n_ktiles && ok; ++j) {
      const uint32_t st = (uint32_t)(j & 1);
      if (!wait_warp(bar_s + B_SFULL + 8 * st, par2(j))) { ok = false; break; }
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      uint32_t v[64];
      tmem_ld32(tmem_base + t_lane + st * PT_KT + 64 * hf, *reinterpret_cast<uint32_t (*)[32]>(&v[0]));
      tmem_ld32(tmem_base + t_lane + st * PT_KT + 64 * hf + 32, *reinterpret_cast<uint32_t (*)[32]>(&v[32]));
      asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      // causal limit, maximum (the key norms are inside the K operand)
      const int vis = lim - PT_KT * (jbase + j) - 64 * hf;      // of this thread's 64 keys the row may see (<= 0: none, >= 64: all)
      if (vis < 64) {
#pragma unroll
        for (int i = 0; i < 64; ++i) v[i] = i < vis ? v[i] : 0xff800000u;
      }
      float mx = -CUDART_INF_F;
#pragma unroll
      for (int i = 0; i < 64; i += 2) mx = fmaxf(mx, fmaxf(__uint_as_float(v[i]), __uint_as_float(v[i + 1])));
      if constexpr (SPLIT == 2) {      // the other half of the row: maxima through shared memory, one mbarrier per quadrant and parity
        s_mx[j & 1][hf][r] = mx;
        __syncwarp();
        const uint32_t xb = bar_s + B_MX + 8 * (uint32_t)(2 * quad + (j & 1));
        if (lane == 0) pt_arrive(xb);
        if (!wait_warp(xb, par2(j))) { ok = false; break; }
        mx = fmaxf(mx, s_mx[j & 1][hf ^ 1][r]);
      }
      // the reference maximum moves only when the row maximum has grown by more than PT_RESCALE; tcgen05.ld / st are
      // warp-wide, so the rows of a warp rescale together (factor 1 for rows that keep their reference).  Column 128
      // of O is the row sum and is rescaled with the rest.  Two warps per row: each takes a share of the columns.
      const bool grow = mx > m_ref + PT_RESCALE;
      if (__any_sync(0xffffffffu, grow)) {
        const float alpha = grow ? pt_ex2(m_ref - mx) : 1.0f;      // m_ref = -inf: 0
        if (grow) m_ref = mx;
        if (j > 0) {
          if (!wait_warp(bar_s + B_PVDONE + 8 * (uint32_t)((j - 1) & 1), par2(j - 1))) { ok = false; break; }
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const int c_lo = SPLIT == 2 ? (hf ? 3 : 0) : 0, c_hi = SPLIT == 2 ? (hf ? 5 : 3) : 5;
#pragma unroll 1
          for (int c = c_lo; c < c_hi; ++c) {
            uint32_t o[32];
            tmem_ld32(tmem_o + t_lane + 32 * c, o);
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
            tmem_st32(tmem_o + t_lane + 32 * c, o);
          }
          asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
          asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        }
      }
      const float ref = m_ref == -CUDART_INF_F ? 0.f : m_ref;
      // probabilities as fp16 pairs (keys 2i, 2i + 1) into the first columns of the S stage they came from: the A
      // operand of P V.  P V of tile j-2, the last reader of these columns, was issued before the scores of tile j; the
      // tensor cores work in issue order, and this tile's s_full - a commit - completes only when everything issued
      // before it has.  With two warps per row, P of keys 64..127 lands on columns 32..63, which hold scores of the
      // other warp's keys: that warp loaded them before it arrived on the maxima barrier this warp has passed.
      {
        uint32_t ph[32];
#pragma unroll
        for (int i = 0; i < 32; ++i)
          ph[i] = pt_pack_half2(pt_ex2(__uint_as_float(v[2 * i]) - ref), pt_ex2(__uint_as_float(v[2 * i + 1]) - ref));
        tmem_st32(tmem_base + t_lane + st * PT_KT + 32 * hf, ph);
      }
      asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) pt_arrive(bar_s + B_PFULL + 8 * st);
    }
    // ---- un-normalised rows for the merge kernel ----
    if (ok && wait_warp(bar_s + B_PVDONE + 8 * (uint32_t)((n_ktiles - 1) & 1), par2(n_ktiles - 1))) {
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const int64_t row = ((int64_t)(q0 + tok) * a.num_q_heads + kvh * G + r % G) * gridDim.z + blockIdx.z;      // (row, partial)
      const int c_lo = SPLIT == 2 ? 2 * hf : 0, c_hi = SPLIT == 2 ? 2 * hf + 2 : 4;
#pragma unroll 1
      for (int c = c_lo; c < c_hi; ++c) {
        uint32_t o[32];
        tmem_ld32(tmem_o + t_lane + 32 * c, o);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        if (live) {
          float4* dst = reinterpret_cast<float4*>(a.part_acc + row * 128 + 32 * c);
#pragma unroll
          for (int i = 0; i < 8; ++i)
            dst[i] = make_float4(__uint_as_float(o[4 * i]), __uint_as_float(o[4 * i + 1]), __uint_as_float(o[4 * i + 2]),
                                 __uint_as_float(o[4 * i + 3]));
        }
      }
      if (hf == SPLIT - 1) {
        uint32_t o[32];
        tmem_ld32(tmem_o + t_lane + 128, o);      // column 128: the row sum of the fp16 probabilities
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        if (live) { a.part_ml[row * 2] = m_ref; a.part_ml[row * 2 + 1] = __uint_as_float(o[0]); }
      }
    }
  }

  // A CTA in which a wait gave up may still have MMAs in flight: before the columns go back, the issuing thread
  // commits once more on the drain barrier (it completes when every MMA that thread issued has) and waits, bounded.
  // Only if that wait gives up too are the columns kept (status 2).
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  int leak = 0;
  if (warp == L::MMA_WARP && lane == 0 && lds_u32(failed_s) != 0u) {
    umma_commit(bar_s + B_DRAIN);
    leak = mbar_wait(bar_s + B_DRAIN, 0u) ? 0 : 1;
    if (leak) g_prefill_tc_status = 2;
  }
  leak = __syncthreads_or(leak);
  if (warp == 0 && !leak) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" :: "r"(tmem_base), "n"(PT_TMEM_COLS) : "memory");
  }
}

// ---------------------------------------------------------------------------
// Staged variant with two softmax groups in ping-pong over the key tiles.
//
// In tq_prefill_tc_kernel<G, true> the eight softmax warps work on one tile together: their exponentials (the MUFU
// pipe, 1024 cycles per 128 x 128 tile) and everything else they do (loads from tensor memory, maxima, hand-overs)
// follow each other, about 2000 cycles per tile, and the tensor pipe waits.  Here warps 0-3 take the even tiles of the
// CTA's share and warps 4-7 the odd ones (thread = row, all 128 keys of a tile), so one group's exponentials run under
// the other group's loads and hand-overs.  What that needs:
//   * three score stages in tensor memory (tiles j and j+1 are in the softmax groups while S of tile j+2 is computed):
//     3 x 128 columns + O (128 columns) = 512.  Q moves to shared memory (A operand by descriptor), and the value
//     operand loses its row of ones: the row sums are accumulated by the softmax threads (float32, before rounding).
//   * the row's reference maximum is shared by the two threads that own the row (shared memory, one mbarrier per 32 rows
//     and tile parity): tile j+1's owner takes its decision after tile j's owner has published its own; only the
//     decision is serial (loads + maximum), the exponentials are not.  A thread keeps the row sum of its own tiles and
//     the reference it is relative to; the two are combined at the end.
//   * K operands are needed two tiles before the matching V operands and are released much earlier: two K slots fed by
//     one producer lane (slot free = scores of tile j-2 complete) and three V slots fed by another (value product of
//     tile j-3 complete).
// Barriers (index = tile modulo the ring size, phase parity = tile / ring size):
//   k_full[2], v_full[3]  bulk-copy bytes        s_full[3]   commit after S      p_full[3]  4 warp arrivals
//   pv_done[3]            commit after P V       ref[4][2]   the row quarter's reference of tile j is published
// ---------------------------------------------------------------------------
struct PpL {
  static constexpr int KT = 128, NKS = 3, NVS = 3, NSS = 3;
  static constexpr int WARPS = 11, THREADS = WARPS * 32, MMA_WARP = 8, K_WARP = 9, V_WARP = 10;
  static constexpr int KSLOT = 32768, VSLOT = 32768, VHALF = 16384;
  static constexpr int K = 0, V = K + NKS * KSLOT, Q = V + NVS * VSLOT, BAR = Q + 32768;
  static constexpr int SMEM = BAR + 1536 + 1024;      // barriers and the per-row words, + slack for the 1024-byte alignment
  static constexpr int T_O = 384;
};
static_assert(PpL::KSLOT == PFI_VOFF && PpL::VSLOT == 2 * PFI_VHALF && PpL::KSLOT + PpL::VSLOT == PFI_BYTES, "image layout");
constexpr uint32_t Q_KFULL = 0, Q_VFULL = 24, Q_SFULL = 48, Q_PFULL = 72, Q_PVDONE = 96, Q_REF = 120, Q_DRAIN = 184,
                   Q_TMEM = 192, Q_FAILED = 196, Q_SREF = 256, Q_SL = 768;      // s_ref [128] and s_l [128] floats

__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&v)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
      :: "r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]),
         "r"(v[8]), "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15])
      : "memory");
}
__device__ __forceinline__ float lds_f32(uint32_t addr) {
  float v;
  asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(addr) : "memory");
  return v;
}
__device__ __forceinline__ void sts_f32(uint32_t addr, float v) {
  asm volatile("st.shared.f32 [%0], %1;" :: "r"(addr), "f"(v) : "memory");
}

template <int G>
__global__ void __launch_bounds__(PpL::THREADS, 1)
tq_prefill_pp_kernel(PrefillArgs a) {
  using L = PpL;
  static_assert(G == 1 || G == 2 || G == 4 || G == 8, "query heads per KV head");
  constexpr int TT = 128 / G;
  extern __shared__ uint8_t pt_smem_raw[];
  const uint32_t raw_s = smem_u32(pt_smem_raw);
  const uint32_t base_s = (raw_s + 1023u) & ~1023u;
  uint8_t* base = pt_smem_raw + (base_s - raw_s);
  const uint32_t bar_s = base_s + L::BAR, failed_s = bar_s + Q_FAILED;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int kvh = blockIdx.y;

  int tile = blockIdx.x, s = 0, q0 = 0, qlen = 0;
  bool found = false;
  for (s = 0; s < a.num_seqs; ++s) {
    q0 = (int)load_index(a.query_start_loc, a.qs_dtype, s);
    const int q1 = (int)load_index(a.query_start_loc, a.qs_dtype, s + 1);
    qlen = q1 - q0;
    if (qlen < 0) qlen = 0;
    const int tiles = (qlen + TT - 1) / TT;
    if (tile < tiles) { found = true; break; }
    tile -= tiles;
  }
  if (!found) return;
  const int64_t max_ctx = (int64_t)a.max_blocks_per_seq * a.block_size;
  const int seq_len = (int)load_ctx(a.seq_lens, a.sl_dtype, s, max_ctx);
  int past = seq_len - qlen;
  if (past < 0) past = 0;
  const int tok_lo = tile * TT;
  const int tok_hi = (tok_lo + TT < qlen) ? tok_lo + TT : qlen;
  int kend = past + tok_hi;
  if (kend > seq_len) kend = seq_len;
  int n_all = (kend + L::KT - 1) / L::KT;
  if (n_all > a.tiles_per_seq) n_all = a.tiles_per_seq;
  const int jbase = (int)((int64_t)n_all * blockIdx.z / gridDim.z);
  const int n_ktiles = (int)((int64_t)n_all * (blockIdx.z + 1) / gridDim.z) - jbase;
  if (n_ktiles <= 0) return;

  if (tid == 0) {
    for (int i = 0; i < L::NKS; ++i) asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" :: "r"(bar_s + Q_KFULL + 8 * i));
    for (int i = 0; i < 3; ++i) {
      asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" :: "r"(bar_s + Q_VFULL + 8 * i));
      asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" :: "r"(bar_s + Q_SFULL + 8 * i));
      asm volatile("mbarrier.init.shared::cta.b64 [%0], 4;" :: "r"(bar_s + Q_PFULL + 8 * i));
      asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" :: "r"(bar_s + Q_PVDONE + 8 * i));
    }
    for (int i = 0; i < 8; ++i) asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" :: "r"(bar_s + Q_REF + 8 * i));
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" :: "r"(bar_s + Q_DRAIN));
    asm volatile("st.shared.u32 [%0], %1;" :: "r"(failed_s), "r"(0u) : "memory");
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncwarp();
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" :: "r"(bar_s + Q_TMEM), "n"(PT_TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  // A operand of S in shared memory: row r = (token tok_lo + r / G, head r % G), zeros for rows without a token
  if (warp < 4) {
    const int r = tid, tok = tok_lo + r / G;
    const bool have = tok < qlen && q0 + tok < a.n_tokens;
    const float4* src = reinterpret_cast<const float4*>(a.qrot + ((int64_t)(q0 + (have ? tok : 0)) * a.num_q_heads + kvh * G + r % G) * 128);
#pragma unroll 4
    for (int c = 0; c < 16; ++c) {           // 16-byte chunk c = dims 8c .. 8c + 7
      const float4 f0 = have ? src[2 * c] : make_float4(0.f, 0.f, 0.f, 0.f);
      const float4 f1 = have ? src[2 * c + 1] : make_float4(0.f, 0.f, 0.f, 0.f);
      pt_sts128(base_s + L::Q + (uint32_t)(c >> 3) * 16384u + (uint32_t)r * 128u + ((((uint32_t)c & 7u) ^ ((uint32_t)r & 7u)) << 4),
                pt_pack_half2(f0.x, f0.y), pt_pack_half2(f0.z, f0.w), pt_pack_half2(f1.x, f1.y), pt_pack_half2(f1.z, f1.w));
    }
    sts_f32(bar_s + Q_SREF + 4 * r, -CUDART_INF_F);
    sts_f32(bar_s + Q_SL + 4 * r, 0.f);
  }
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = lds_u32(bar_s + Q_TMEM);
  const uint32_t tmem_o = tmem_base + L::T_O;

  auto wait = [&](uint32_t bar, uint32_t parity) -> bool {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}\n"
        : "=r"(done) : "r"(bar), "r"(parity) : "memory");
    if (done) return true;
    if (lds_u32(failed_s) != 0u) return false;
    if (mbar_wait(bar, parity)) return true;
    g_prefill_tc_status = 1;
    asm volatile("st.shared.u32 [%0], %1;" :: "r"(failed_s), "r"(1u) : "memory");
    return false;
  };
  auto wait_warp = [&](uint32_t bar, uint32_t parity) -> bool { return __all_sync(0xffffffffu, wait(bar, parity)); };
  auto par = [](int j, int ring) -> uint32_t { return (uint32_t)((j / ring) & 1); };

  if (warp == L::MMA_WARP) {
    if (lane == 0) {
      constexpr uint32_t IDESC = (1u << 4) | ((128u >> 3) << 17) | ((128u >> 4) << 24);      // M 128, N 128, f16 -> f32, K-major
      const int withhold = (blockIdx.x | blockIdx.y) == 0 ? g_prefill_tc_withhold : -1;
      const uint64_t d_hi = umma_desc(0u) & 0xffffffff00000000ull;
      const uint32_t d_lo = (uint32_t)umma_desc(0u);
      auto desc = [&](uint32_t saddr) -> uint64_t { return d_hi | (uint64_t)(d_lo + ((saddr & 0x3FFFFu) >> 4)); };
      const uint32_t k_lo = base_s + L::K, v_lo = base_s + L::V, q_lo = base_s + L::Q;
      auto issue_s = [&](int j) -> bool {
        const uint32_t st = (uint32_t)(j % 3), ks = st;
        if (!wait(bar_s + Q_KFULL + 8 * ks, par(j, 3))) return false;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        if (j == withhold) return true;
        const uint32_t kb = k_lo + ks * L::KSLOT;
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          const uint32_t off = (uint32_t)((kk >> 2) * 16384 + (kk & 3) * 32);
          umma_f16(tmem_base + st * 128u, desc(q_lo + off), desc(kb + off), IDESC, (uint32_t)(kk != 0));
        }
        umma_commit(bar_s + Q_SFULL + 8 * st);
        return true;
      };
      auto issue_pv = [&](int j) -> bool {
        const uint32_t st = (uint32_t)(j % 3);
        if (!wait(bar_s + Q_PFULL + 8 * st, par(j, 3))) return false;
        if (!wait(bar_s + Q_VFULL + 8 * st, par(j, 3))) return false;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t vb = v_lo + st * L::VSLOT;
#pragma unroll
        for (int kk = 0; kk < 8; ++kk)
          umma_f16_ta(tmem_o, tmem_base + st * 128u + (uint32_t)(kk * 8), desc(vb + (uint32_t)((kk >> 2) * L::VHALF + (kk & 3) * 32)),
                      IDESC, (uint32_t)((j | kk) != 0));
        umma_commit(bar_s + Q_PVDONE + 8 * st);
        return true;
      };
      bool go = issue_s(0);
      if (go && n_ktiles > 1) go = issue_s(1);
      if (go) {
        for (int j = 0; j < n_ktiles; ++j) {
          if (j + 2 < n_ktiles && !issue_s(j + 2)) break;
          if (!issue_pv(j)) break;
        }
      }
    }
    __syncwarp();
  } else if (warp == L::K_WARP || warp == L::V_WARP) {
    if (lane == 0) {
      const bool isk = warp == L::K_WARP;
      constexpr int ring = 3;
      const uint8_t* src = a.staged + (((int64_t)s * a.tiles_per_seq + jbase) * a.num_kv_heads + kvh) * PT_IMAGE + (isk ? 0 : L::KSLOT);
      const int64_t step = (int64_t)a.num_kv_heads * PT_IMAGE;
      const uint32_t full0 = bar_s + (isk ? Q_KFULL : Q_VFULL), dst0 = base_s + (isk ? L::K : L::V);
      int issued = 0;
      for (int j = 0; j < n_ktiles; ++j) {
        const uint32_t slot = (uint32_t)(j % ring);
        if (j >= ring) {
          // K slot: the scores of tile j-3 are complete; V slot: the value product of tile j-3 is complete
          const int jj = j - ring;
          if (!wait(bar_s + (isk ? Q_SFULL : Q_PVDONE) + 8 * (uint32_t)(jj % 3), par(jj, 3))) break;
        }
        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" :: "r"(full0 + 8 * slot), "r"(32768) : "memory");
        asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                     :: "r"(dst0 + slot * 32768u), "l"(src + j * step), "r"(32768), "r"(full0 + 8 * slot) : "memory");
        issued = j + 1;
      }
      if (lds_u32(failed_s) != 0u)
        for (int j = issued - ring < 0 ? 0 : issued - ring; j < issued; ++j) mbar_wait(full0 + 8 * (uint32_t)(j % ring), par(j, ring));
    }
    __syncwarp();
  } else {
    // ================= softmax groups: warps 0-3 even tiles, warps 4-7 odd tiles; thread = row =================
    const int quad = warp & 3, grp = warp >> 2;
    const int r = quad * 32 + lane;
    const int tok = tok_lo + r / G;
    const bool live = tok < qlen && q0 + tok < a.n_tokens;
    int lim = live ? past + tok + 1 : 0;
    if (lim > seq_len) lim = seq_len;
    const uint32_t t_lane = ((uint32_t)(quad * 32)) << 16;
    const uint32_t sref_s = bar_s + Q_SREF + 4 * r, sl_s = bar_s + Q_SL + 4 * r;
    float l = 0.f, lref = -CUDART_INF_F;      // row sum of this thread's tiles and the reference it is relative to
    bool ok = true;
    for (int j = grp; j < n_ktiles && ok; j += 2) {
      const uint32_t st = (uint32_t)(j % 3);
      if (!wait_warp(bar_s + Q_SFULL + 8 * st, par(j, 3))) { ok = false; break; }
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const uint32_t s_addr = tmem_base + t_lane + st * 128u;
      const int vis = lim - L::KT * (jbase + j);      // keys of this tile the row may see (<= 0: none, >= 128: all)
      // ---- pass 1: the row maximum ----
      float mx = -CUDART_INF_F;
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t v[32];
        tmem_ld32(s_addr + 32 * c, v);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        if (vis < 32 * c + 32) {
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = 32 * c + i < vis ? v[i] : 0xff800000u;
        }
#pragma unroll
        for (int i = 0; i < 32; i += 2) mx = fmaxf(mx, fmaxf(__uint_as_float(v[i]), __uint_as_float(v[i + 1])));
      }
      // ---- the row's reference: after the owner of tile j-1 has published its decision ----
      if (j > 0 && !wait_warp(bar_s + Q_REF + 8 * (uint32_t)(2 * quad + ((j - 1) & 1)), par(j - 1, 2))) { ok = false; break; }
      float m_ref = lds_f32(sref_s);
      const bool grow = mx > m_ref + PT_RESCALE;
      const bool any = __any_sync(0xffffffffu, grow);
      const float alpha = grow ? pt_ex2(m_ref - mx) : 1.0f;      // m_ref = -inf: 0
      if (grow) { m_ref = mx; sts_f32(sref_s, mx); }
      __syncwarp();
      if (lane == 0) pt_arrive(bar_s + Q_REF + 8 * (uint32_t)(2 * quad + (j & 1)));
      if (lref != m_ref) {
        l = l > 0.f ? l * pt_ex2(lref - m_ref) : 0.f;
        lref = m_ref;
      }
      if (any && j > 0) {       // O holds the value products of tiles < j, all relative to the old reference
        if (!wait_warp(bar_s + Q_PVDONE + 8 * (uint32_t)((j - 1) % 3), par(j - 1, 3))) { ok = false; break; }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {
          uint32_t o[32];
          tmem_ld32(tmem_o + t_lane + 32 * c, o);
          asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
          tmem_st32(tmem_o + t_lane + 32 * c, o);
        }
        asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
      }
      // ---- pass 2: probabilities as fp16 pairs into the first 64 columns of the stage (chunk c lands on columns the
      // thread has consumed already), row sum in float32 ----
      const float ref = m_ref == -CUDART_INF_F ? 0.f : m_ref;
      float ls0 = 0.f, ls1 = 0.f;
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t v[32];
        tmem_ld32(s_addr + 32 * c, v);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        if (vis < 32 * c + 32) {
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = 32 * c + i < vis ? v[i] : 0xff800000u;
        }
        uint32_t ph[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const float p0 = pt_ex2(__uint_as_float(v[2 * i]) - ref), p1 = pt_ex2(__uint_as_float(v[2 * i + 1]) - ref);
          ls0 += p0;
          ls1 += p1;
          ph[i] = pt_pack_half2(p0, p1);
        }
        tmem_st16(s_addr + 16 * c, ph);
      }
      l += ls0 + ls1;
      asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) pt_arrive(bar_s + Q_PFULL + 8 * st);
    }
    // ---- the two owners of a row agree on its final reference and add their sums ----
    asm volatile("bar.sync 1, 256;" ::: "memory");
    const float fin = lds_f32(sref_s);
    if (lref != fin) l = l > 0.f ? l * pt_ex2(lref - fin) : 0.f;
    if (grp == 1) sts_f32(sl_s, l);
    asm volatile("bar.sync 1, 256;" ::: "memory");
    if (grp == 0) l += lds_f32(sl_s);
    if (ok && wait_warp(bar_s + Q_PVDONE + 8 * (uint32_t)((n_ktiles - 1) % 3), par(n_ktiles - 1, 3))) {
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const int64_t row = ((int64_t)(q0 + tok) * a.num_q_heads + kvh * G + r % G) * gridDim.z + blockIdx.z;
#pragma unroll 1
      for (int c = 2 * grp; c < 2 * grp + 2; ++c) {
        uint32_t o[32];
        tmem_ld32(tmem_o + t_lane + 32 * c, o);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        if (live) {
          float4* dst = reinterpret_cast<float4*>(a.part_acc + row * 128 + 32 * c);
#pragma unroll
          for (int i = 0; i < 8; ++i)
            dst[i] = make_float4(__uint_as_float(o[4 * i]), __uint_as_float(o[4 * i + 1]), __uint_as_float(o[4 * i + 2]),
                                 __uint_as_float(o[4 * i + 3]));
        }
      }
      if (grp == 0 && live) { a.part_ml[row * 2] = fin; a.part_ml[row * 2 + 1] = l; }
    }
  }

  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  int leak = 0;
  if (warp == L::MMA_WARP && lane == 0 && lds_u32(failed_s) != 0u) {
    umma_commit(bar_s + Q_DRAIN);
    leak = mbar_wait(bar_s + Q_DRAIN, 0u) ? 0 : 1;
    if (leak) g_prefill_tc_status = 2;
  }
  leak = __syncthreads_or(leak);
  if (warp == 0 && !leak) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" :: "r"(tmem_base), "n"(PT_TMEM_COLS) : "memory");
  }
}

// Pre-pass of the staged variant: every 128-key tile of every sequence and KV head becomes the 64 KB set of operand
// images (K rows, then the transposed V rows of its two 64-key halves; norms folded in, keys past the sequence zero)
// that tq_prefill_tc_kernel<G, true> pulls into shared memory with three bulk copies.  A CTA takes PS_TILES consecutive
// tiles of one (sequence, KV head) and decodes a tile in two passes of 64 keys.
constexpr int PS_THREADS = 256, PS_TILES = 2, PS_SMEM = 32768 + PT_IMAGE;

__global__ void __launch_bounds__(PS_THREADS, 2)
tq_prefill_stage_kernel(PrefillArgs a) {
  extern __shared__ __align__(128) uint8_t ps_smem[];
  const int tid = threadIdx.x, lane = tid & 31;
  const int s = blockIdx.y, kvh = blockIdx.z;
  const int64_t max_ctx = (int64_t)a.max_blocks_per_seq * a.block_size;
  const int seq_len = (int)load_ctx(a.seq_lens, a.sl_dtype, s, max_ctx);
  int n_tiles = (seq_len + PS_KT - 1) / PS_KT;
  if (n_tiles > a.tiles_per_seq) n_tiles = a.tiles_per_seq;
  const int t_begin = blockIdx.x * PS_TILES;
  if (t_begin >= n_tiles) return;
  const int t_end = t_begin + PS_TILES < n_tiles ? t_begin + PS_TILES : n_tiles;
  pt_fill_lut(ps_smem, a.centroids, tid, PS_THREADS);
  __syncthreads();
  const uint32_t lut = smem_u32(ps_smem) + lane * 4, img = smem_u32(ps_smem) + 32768;
  const int kr = tid >> 2, kc = tid & 3;
  const int kg = tid & 7, vbyte = 4 * (tid >> 4) + 2 * ((tid >> 3) & 1);
  const int bs = a.block_size;
  auto phys = [&](int key) -> int64_t {
    int blk = key / bs;
    if (blk >= a.max_blocks_per_seq) blk = a.max_blocks_per_seq - 1;
    const int64_t pb = load_index(a.block_tables, a.bt_dtype, (int64_t)s * a.bt_stride + blk);
    return pb < 0 ? 0 : (pb >= a.num_blocks ? a.num_blocks - 1 : pb);
  };
  for (int t = t_begin; t < t_end; ++t) {
#pragma unroll 1
    for (int u = 0; u < PS_KT / 64; ++u) {       // 64 keys at a time with the thread roles of the decode warps
      uint4 kw;
      float kn;
      uint32_t vw[8];
      float vn[8];
      {
        const int key = PS_KT * t + 64 * u + kr;
        const int64_t pb = phys(key);
        const int pos = key - (key / bs) * bs;
        kw = __ldg(reinterpret_cast<const uint4*>(a.k_packed + pb * a.kp_sb + (int64_t)pos * a.kp_sp + (int64_t)kvh * a.kp_sh + kc * 16));
        kn = key < seq_len ? __ldg(a.k_norms + pb * a.kn_sb + (int64_t)pos * a.kn_sp + (int64_t)kvh * a.kn_sh) : 0.f;
      }
      {
        const int key8 = PS_KT * t + 64 * u + 8 * kg;
        const int64_t pb = phys(key8);
        const int pos8 = key8 - (key8 / bs) * bs;
        const uint8_t* vp = a.v_packed + pb * a.vp_sb + (int64_t)pos8 * a.vp_sp + (int64_t)kvh * a.vp_sh + vbyte;
        const float* np = a.v_norms + pb * a.vn_sb + (int64_t)pos8 * a.vn_sp + (int64_t)kvh * a.vn_sh;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          vw[i] = (uint32_t)__ldg(reinterpret_cast<const unsigned short*>(vp + (int64_t)i * a.vp_sp));
          vn[i] = key8 + i < seq_len ? __ldg(np + (int64_t)i * a.vn_sp) : 0.f;
        }
      }
      pt_decode_k(img, PtL<true>::KHALF, 64 * u, lut, kr, kc, kw, kn);
      pt_decode_v(img + PtL<true>::KSTAGE + u * 16384, lut, kg, vbyte, vw, vn);
    }
    __syncthreads();
    uint4* dst = reinterpret_cast<uint4*>(a.staged + (((int64_t)s * a.tiles_per_seq + t) * a.num_kv_heads + kvh) * PT_IMAGE);
#pragma unroll
    for (int i = 0; i < PT_IMAGE / 16 / PS_THREADS; ++i) {
      const int idx = i * PS_THREADS + tid;
      uint4 v;
      asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(img + idx * 16));
      dst[idx] = v;
    }
    __syncthreads();
  }
}

// The same images from 3- and 2-bit codes (MSB-first streams of 48 / 32 bytes per key and head): nothing downstream
// depends on the code width.  Plain code - the pre-pass is a few percent of a call: a thread turns 8 dims of one key
// into one 16-byte piece of the K image, then 8 dims of 8 keys into eight pieces of the transposed V image.
template <int BITS>
__global__ void __launch_bounds__(PS_THREADS, 2)
tq_prefill_stage_bits_kernel(PrefillArgs a) {
  constexpr int CB = BITS;          // bytes per 8 codes
  extern __shared__ __align__(128) uint8_t ps_smem[];
  __shared__ float cent[1 << BITS];
  const int tid = threadIdx.x;
  const int s = blockIdx.y, kvh = blockIdx.z;
  const int64_t max_ctx = (int64_t)a.max_blocks_per_seq * a.block_size;
  const int seq_len = (int)load_ctx(a.seq_lens, a.sl_dtype, s, max_ctx);
  int n_tiles = (seq_len + PS_KT - 1) / PS_KT;
  if (n_tiles > a.tiles_per_seq) n_tiles = a.tiles_per_seq;
  const int t_begin = blockIdx.x * PS_TILES;
  if (t_begin >= n_tiles) return;
  const int t_end = t_begin + PS_TILES < n_tiles ? t_begin + PS_TILES : n_tiles;
  if (tid < (1 << BITS)) cent[tid] = a.centroids[tid];
  __syncthreads();
  const int bs = a.block_size;
  auto phys = [&](int key) -> int64_t {
    int blk = key / bs;
    if (blk >= a.max_blocks_per_seq) blk = a.max_blocks_per_seq - 1;
    const int64_t pb = load_index(a.block_tables, a.bt_dtype, (int64_t)s * a.bt_stride + blk);
    return pb < 0 ? 0 : (pb >= a.num_blocks ? a.num_blocks - 1 : pb);
  };
  // eight codes = CB whole bytes -> eight centroids times the norm
  auto decode8 = [&](const uint8_t* src, float norm, float (&out)[8]) {
    uint32_t w = 0;
#pragma unroll
    for (int i = 0; i < CB; ++i) w = (w << 8) | src[i];
#pragma unroll
    for (int i = 0; i < 8; ++i) out[i] = cent[(w >> (BITS * (7 - i))) & ((1u << BITS) - 1u)] * norm;
  };
  for (int t = t_begin; t < t_end; ++t) {
    // K image: [half = dims 0..63 | 64..127][key][128 B], 16-byte chunk c of key r at chunk c ^ (r & 7)
    for (int e = tid; e < PS_KT * 16; e += PS_THREADS) {
      const int r = e >> 4, c = e & 15;
      const int key = PS_KT * t + r;
      const int64_t pb = phys(key);
      const int pos = key - (key / bs) * bs;
      const float norm = key < seq_len ? a.k_norms[pb * a.kn_sb + (int64_t)pos * a.kn_sp + (int64_t)kvh * a.kn_sh] : 0.f;
      float v[8];
      decode8(a.k_packed + pb * a.kp_sb + (int64_t)pos * a.kp_sp + (int64_t)kvh * a.kp_sh + c * CB, norm, v);
      *reinterpret_cast<uint4*>(ps_smem + (c >> 3) * PtL<true>::KHALF + r * 128 + (((c & 7) ^ (r & 7)) << 4)) =
          make_uint4(pt_pack_half2(v[0], v[1]), pt_pack_half2(v[2], v[3]), pt_pack_half2(v[4], v[5]), pt_pack_half2(v[6], v[7]));
    }
    // V image: [half = keys 0..63 | 64..127][dim][128 B], the chunk of key group g (8 keys) of dim d at chunk g ^ (d & 7)
    for (int e = tid; e < (PS_KT / 8) * 16; e += PS_THREADS) {
      const int g = e >> 4, c = e & 15;              // keys 8 g .. 8 g + 7, dims 8 c .. 8 c + 7
      const int key8 = PS_KT * t + 8 * g;
      const int64_t pb = phys(key8);
      const int pos8 = key8 - (key8 / bs) * bs;
      float v[8][8];
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float norm = key8 + i < seq_len ? a.v_norms[pb * a.vn_sb + (int64_t)(pos8 + i) * a.vn_sp + (int64_t)kvh * a.vn_sh] : 0.f;
        decode8(a.v_packed + pb * a.vp_sb + (int64_t)(pos8 + i) * a.vp_sp + (int64_t)kvh * a.vp_sh + c * CB, norm, v[i]);
      }
#pragma unroll
      for (int dd = 0; dd < 8; ++dd) {
        const int d = 8 * c + dd;
        *reinterpret_cast<uint4*>(ps_smem + PtL<true>::KSTAGE + (g >> 3) * 16384 + d * 128 + ((((g & 7) ^ (d & 7))) << 4)) =
            make_uint4(pt_pack_half2(v[0][dd], v[1][dd]), pt_pack_half2(v[2][dd], v[3][dd]), pt_pack_half2(v[4][dd], v[5][dd]),
                       pt_pack_half2(v[6][dd], v[7][dd]));
      }
    }
    __syncthreads();
    uint4* dst = reinterpret_cast<uint4*>(a.staged + (((int64_t)s * a.tiles_per_seq + t) * a.num_kv_heads + kvh) * PT_IMAGE);
    for (int i = tid; i < PT_IMAGE / 16; i += PS_THREADS) dst[i] = reinterpret_cast<const uint4*>(ps_smem)[i];
    __syncthreads();
  }
}

}  // namespace

int prefill_tc_status(int* host_out, int reset) {
  cudaError_t e = cudaMemcpyFromSymbol(host_out, g_prefill_tc_status, sizeof(int));
  if (e == cudaSuccess && reset) { const int z = 0; e = cudaMemcpyToSymbol(g_prefill_tc_status, &z, sizeof(int)); }
  return e == cudaSuccess ? AKV_OK : fail((int)e, "prefill status: %s", cudaGetErrorString(e));
}

int prefill_tc_withhold(int tile) {
  cudaError_t e = cudaMemcpyToSymbol(g_prefill_tc_withhold, &tile, sizeof(int));
  return e == cudaSuccess ? AKV_OK : fail((int)e, "prefill test hook: %s", cudaGetErrorString(e));
}

int prefill_staged_tile_keys() { return PS_KT; }

int launch_prefill_tc(const PrefillArgs& a, int G, cudaStream_t st) {
  const int TT = 128 / G;
  dim3 grid((a.n_tokens + TT - 1) / TT + a.num_seqs, a.num_kv_heads, a.splits > 0 ? a.splits : 1);
  cudaError_t e = cudaSuccess;
  if (a.staged != nullptr) {
    // operand images first (ordered before the attention kernel by the stream), then the bulk-copy-fed kernel
    dim3 sgrid((a.tiles_per_seq + PS_TILES - 1) / PS_TILES, a.num_seqs, a.num_kv_heads);
    if (a.hybrid_tables != nullptr) {
      if (int rc = launch_hybrid_prefill_stage(a, st)) return rc;
    } else if (a.bits == 4 && !a.byte_rows) {
      e = cudaFuncSetAttribute(tq_prefill_stage_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, PS_SMEM);
      if (e == cudaSuccess) tq_prefill_stage_kernel<<<sgrid, PS_THREADS, PS_SMEM, st>>>(a);
    } else if (a.bits == 4) {
      e = cudaFuncSetAttribute(tq_prefill_stage_bits_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, PT_IMAGE);
      if (e == cudaSuccess) tq_prefill_stage_bits_kernel<4><<<sgrid, PS_THREADS, PT_IMAGE, st>>>(a);
    } else if (a.bits == 3) {
      e = cudaFuncSetAttribute(tq_prefill_stage_bits_kernel<3>, cudaFuncAttributeMaxDynamicSharedMemorySize, PT_IMAGE);
      if (e == cudaSuccess) tq_prefill_stage_bits_kernel<3><<<sgrid, PS_THREADS, PT_IMAGE, st>>>(a);
    } else {
      e = cudaFuncSetAttribute(tq_prefill_stage_bits_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, PT_IMAGE);
      if (e == cudaSuccess) tq_prefill_stage_bits_kernel<2><<<sgrid, PS_THREADS, PT_IMAGE, st>>>(a);
    }
    if (e != cudaSuccess) return fail((int)e, "prefill attention: smem attribute: %s", cudaGetErrorString(e));
    if (a.hybrid_tables == nullptr)
      if (int rc = check_launch("tq_prefill_stage_kernel")) return rc;
  }
#define AKV_PT(GG, ST)                                                                                                  \
  e = cudaFuncSetAttribute(tq_prefill_tc_kernel<GG, ST>, cudaFuncAttributeMaxDynamicSharedMemorySize, PtL<ST>::SMEM);     \
  if (e == cudaSuccess) tq_prefill_tc_kernel<GG, ST><<<grid, PtL<ST>::THREADS, PtL<ST>::SMEM, st>>>(a);
  const char* pp_env = getenv("AKV_PREFILL_PP");          // read per call; AKV_PREFILL_PP=0: the one-tile-at-a-time kernel
  const bool pingpong = pp_env == nullptr || atoi(pp_env) != 0;
#define AKV_PP(GG)                                                                                                       \
  e = cudaFuncSetAttribute(tq_prefill_pp_kernel<GG>, cudaFuncAttributeMaxDynamicSharedMemorySize, PpL::SMEM);             \
  if (e == cudaSuccess) tq_prefill_pp_kernel<GG><<<grid, PpL::THREADS, PpL::SMEM, st>>>(a);
  if (a.staged != nullptr && pingpong) {
    if (G == 1) { AKV_PP(1) } else if (G == 2) { AKV_PP(2) } else if (G == 4) { AKV_PP(4) } else { AKV_PP(8) }
  } else if (a.staged != nullptr) {
    if (G == 1) { AKV_PT(1, true) } else if (G == 2) { AKV_PT(2, true) } else if (G == 4) { AKV_PT(4, true) } else { AKV_PT(8, true) }
  } else {
    if (G == 1) { AKV_PT(1, false) } else if (G == 2) { AKV_PT(2, false) } else if (G == 4) { AKV_PT(4, false) } else { AKV_PT(8, false) }
  }
#undef AKV_PT
#undef AKV_PP
  if (e != cudaSuccess) return fail((int)e, "prefill attention: smem attribute: %s", cudaGetErrorString(e));
  return check_launch(a.staged == nullptr ? "tq_prefill_attn_tc_kernel"
                                          : (pingpong ? "tq_prefill_attn_tc_staged_kernel" : "tq_prefill_attn_tc_staged_onetile_kernel"));
}

size_t prefill_staged_bytes(int num_seqs, int num_kv_heads, int max_seq_len) {
  if (num_seqs <= 0 || num_kv_heads <= 0 || max_seq_len <= 0) return 0;
  return (size_t)num_seqs * (size_t)((max_seq_len + PS_KT - 1) / PS_KT) * (size_t)num_kv_heads * PT_IMAGE;
}

}  // namespace akv
