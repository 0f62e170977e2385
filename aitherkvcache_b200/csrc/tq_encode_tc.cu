// TurboQuant encode on the 5th-generation tensor cores (tcgen05 / TMEM), head_dim 128,
// fp16 or bf16 input.
//
// Same operation as the scalar kernels in tq_codec.cu (reference: quantizer.py:122-168,
// fused_kv_update.py:220-293): norm, rotate by the float32 matrix R, searchsorted against
// the Lloyd-Max boundaries, MSB-first pack.  The rotation of a tile of 128 vectors is one
// 128 x 128 x 128 GEMM, issued by a single thread as tcgen05.mma instructions that read both
// operands from shared memory and accumulate in tensor memory:
//
//   * R is float32 and the input is 16-bit, so R is split into 16-bit terms whose sum carries
//     it to 2^-22 or better: fp16 input -> two fp16 terms of 1024 R (the factor keeps the
//     second term out of fp16's subnormal range; it is divided out with the norm); bf16
//     input -> three bf16 terms.  All terms accumulate into the same 128 TMEM columns.
//     Products are exact, accumulation is float32.
//   * The vector is rotated before it is normalised, y = (R x) * (1 / (norm + 1e-10f)), so y
//     differs from the scalar kernels' value by a few float32 ulps; a code can differ only for
//     a coordinate within ~2e-7 of a boundary.  Norms are bit-equal (same eight-lane order).
//
// One persistent CTA per SM: 16 worker warps and one warp whose first lane issues the MMAs.  Worker warp w owns
// rows 8w .. 8w+7 of every tile on the input side: 16-byte cp.async copies bring them into a 32 KB operand buffer in the
// 128-byte-swizzled K-major layout the MMA descriptors name (AHEAD tiles ahead), and four of its threads per row
// compute the norm out of that buffer.  On the output side thread (row, quarter) quantises 32 consecutive coordinates
// of its row out of tensor memory (tcgen05.ld, so packing needs no exchange).  No CTA-wide barrier in the loop; the
// hand-overs are mbarriers:
//   full[b]        16 warp arrivals: the rows of operand buffer b have landed            -> the MMA warp may issue
//   norm_ready[i]  16 warp arrivals: norms, reciprocals and destinations of tile t's rows    -> quantisers of tile t
//                  (i = t % 4) stored
//   mma_done[s]    tcgen05.commit: the tile's MMAs are complete                           -> its operand buffer may be
//                                                                                            refilled, accumulator s read
//   acc_free[s]    16 warp arrivals: accumulator s has been loaded into registers         -> the MMA warp may reuse it
// Every wait is bounded; a wait that gives up sets g_tc_status and a shared flag that ends all loops, and the CTA
// leaves after releasing its tensor memory.
#include "tq_rowmap.cuh"
#include "umma.cuh"

namespace akv {
namespace {

constexpr int TC_CELLS = 128;
constexpr int TC_LUT_BYTES = TC_CELLS * 32 * 8;   // every cell replicated once per lane
constexpr int TC_THREADS = 17 * 32;                 // 16 worker warps + the MMA warp
constexpr int TC_TAIL_BYTES = TC_LUT_BYTES + 2 * 4 * 128 * 8 + 2 * 4 * 128 * 4 + 64 + 16 * 8 + 16 + 16;

struct TcRow {
  int64_t src_off;   // element offset of the vector; < 0: beyond the last row
  uint8_t* dst;      // nullptr: skipped slot
  float* dst_norm;
};

__device__ int g_tc_status;          // 1: a wait on the MMA barrier gave up
__device__ int g_tc_withhold = -1;   // test hook: CTA 0 issues neither the MMAs nor the commit of this tile

// Operand buffers of vector tiles in flight: what fits beside the matrix terms.
template <bool BF16> struct TcBuf { static constexpr int N = BF16 ? 2 : 3; };

template <bool BF16> constexpr size_t tc_smem_bytes() {
  return (size_t)(BF16 ? 3 : 2) * TC_OPER_BYTES + TcBuf<BF16>::N * TC_OPER_BYTES + TC_TAIL_BYTES + 1024;
}

template <bool BF16>
__device__ __forceinline__ float bits16_to_float(uint32_t h) {
  if (BF16) return __uint_as_float(h << 16);
  return __half2float(__ushort_as_half((unsigned short)h));
}

// Position of a row that a thread follows from tile to tile: rows advance by a fixed step, so the (token, head)
// split of the paged mode is kept by additions instead of a division per tile.
struct TcCursor {
  int64_t n, tok;
  int head;
};

__device__ __forceinline__ TcCursor cursor_at(const RowMap& m, int64_t n) {
  TcCursor c;
  c.n = n;
  if (m.slot_mapping == nullptr) { c.tok = n; c.head = 0; return c; }
  c.tok = n / m.num_heads;
  c.head = (int)(n - c.tok * m.num_heads);
  return c;
}

__device__ __forceinline__ void cursor_advance(const RowMap& m, TcCursor& c, int64_t step, int64_t step_tok, int step_head) {
  c.n += step;
  if (m.slot_mapping == nullptr) { c.tok = c.n; return; }
  c.tok += step_tok;
  c.head += step_head;
  if (c.head >= m.num_heads) { c.head -= m.num_heads; ++c.tok; }
}

// Element offset of the row's source vector; < 0: beyond the last row.
__device__ __forceinline__ int64_t cursor_src(const RowMap& m, const TcCursor& c, int64_t n_rows) {
  if (c.n >= n_rows) return -1;
  return m.slot_mapping == nullptr ? c.n * m.x_stride_row : c.tok * m.x_stride_tok + c.head * m.x_stride_head;
}

// Where the row's codes and norm go (nullptr: skipped slot or beyond the last row).
__device__ __forceinline__ TcRow cursor_dst(const RowMap& m, const TcCursor& c, int64_t n_rows) {
  TcRow r;
  r.src_off = -1; r.dst = nullptr; r.dst_norm = nullptr;
  if (c.n >= n_rows) return r;
  if (m.slot_mapping == nullptr) {
    r.dst = m.packed + c.n * m.p_stride_row;
    r.dst_norm = m.norms + c.n;
    return r;
  }
  const int64_t slot = m.slot_mapping[c.tok];
  if (slot < 0) return r;
  int64_t blk;
  if (slot < (1ll << 32)) blk = (int64_t)((uint32_t)slot / (uint32_t)m.block_size);     // no 64-bit division on the usual path
  else blk = slot / m.block_size;
  const int pos = (int)(slot - blk * m.block_size);
  if (blk < m.max_blocks) {
    r.dst = m.packed + blk * m.p_stride_blk + pos * m.p_stride_pos + c.head * m.p_stride_head;
    r.dst_norm = m.norms + blk * m.n_stride_blk + pos * m.n_stride_pos + c.head * m.n_stride_head;
  }
  return r;
}

template <int BITS, bool BF16>
__global__ void __launch_bounds__(TC_THREADS, 1)
tq_encode_tc_kernel(RowMap m, int64_t n_rows, const float* __restrict__ rot_t,
                    const float* __restrict__ boundaries) {
  constexpr int TERMS = BF16 ? 3 : 2;
  constexpr int ACC_COLS = 128;                // tensor-memory columns of one tile's accumulator
  constexpr float PRESCALE = BF16 ? 1.0f : 1024.0f;
  constexpr int NB = (1 << BITS) - 1;
  constexpr int CHUNK_BYTES = 32 * BITS / 8;   // packed bytes of 32 coordinates
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_s = smem_u32(smem_raw);
  const uint32_t base_s = (raw_s + 1023u) & ~1023u;
  uint8_t* base = smem_raw + (base_s - raw_s);
  uint8_t* terms = base;
  uint8_t* abuf = base + TERMS * TC_OPER_BYTES;
  constexpr int NBUF = TcBuf<BF16>::N;        // copies run NBUF - 1 tiles ahead of the MMAs
  constexpr int AHEAD = NBUF - 1;
  uint8_t* tail = abuf + NBUF * TC_OPER_BYTES;
  float2* lut = reinterpret_cast<float2*>(tail);                 // [cells][32 lanes]
  uint8_t** dstp_s = reinterpret_cast<uint8_t**>(tail + TC_LUT_BYTES);   // [4][128] where the codes of a row go
  float** dstn_s = reinterpret_cast<float**>(dstp_s + 4 * 128);          // [4][128] ... and its norm
  float* rinv_s = reinterpret_cast<float*>(dstn_s + 4 * 128);    // [4][128]
  float* nrm_s = rinv_s + 4 * 128;                               // [4][128]
  float* bnd = nrm_s + 4 * 128;                                  // [16]
  uint64_t* mbar = reinterpret_cast<uint64_t*>(bnd + 16);        // full[3], norm_ready[4], mma_done[2], acc_free[2], drain
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(mbar + 16);
  int* simple_flag = reinterpret_cast<int*>(tmem_slot + 1);
  uint32_t* failed_flag = tmem_slot + 2;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const uint32_t terms_s = base_s;
  const uint32_t abuf_s = base_s + TERMS * TC_OPER_BYTES;
  const uint32_t mbar_s = smem_u32(mbar);

  // ---------------- one-time setup ----------------
  if (tid == 0) {
    *simple_flag = 1;
    *failed_flag = 0u;
    for (int i = 0; i < 12; ++i) {     // full[0..2], norm_ready[0..3], mma_done[0..1], acc_free[0..1], drain
      const uint32_t count = (i == 7 || i == 8 || i == 11) ? 1u : 16u;
      asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" :: "r"(mbar_s + 8u * (uint32_t)i), "r"(count));
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  const int withhold = blockIdx.x == 0 ? g_tc_withhold : -1;
  if (tid < 16) bnd[tid] = tid < NB ? boundaries[tid] : __int_as_float(0x7f800000);
  __syncwarp();
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], 256;"
                 :: "r"(smem_u32(tmem_slot)) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  // Matrix terms.  rot_t[j][i] = R[i][j] is read with i fastest (coalesced) into a float32
  // staging copy (the operand buffers, not yet in use), then each operand row i is written
  // with j fastest; the XOR on the staging column keeps both passes free of bank conflicts.
  {
    float* stg = reinterpret_cast<float*>(abuf);
    for (int e = tid; e < 128 * 128; e += TC_THREADS) {
      int j = e >> 7, i = e & 127;
      stg[j * 128 + (i ^ (j & 31))] = rot_t[e];
    }
    __syncthreads();
    for (int e = tid; e < 128 * 128; e += TC_THREADS) {
      int i = e >> 7, j = e & 127;       // operand row i, K index j
      float r = stg[j * 128 + (i ^ (j & 31))] * PRESCALE;
      uint32_t off = (uint32_t)((j >> 6) * TC_HALF_BYTES + i * 128 + (((((j & 63) >> 3) ^ (i & 7)) << 4) | ((j & 7) << 1)));
      if (BF16) {
        __nv_bfloat16 t1 = __float2bfloat16_rn(r);
        float e1 = r - __bfloat162float(t1);
        __nv_bfloat16 t2 = __float2bfloat16_rn(e1);
        float e2 = e1 - __bfloat162float(t2);
        *reinterpret_cast<__nv_bfloat16*>(terms + off) = t1;
        *reinterpret_cast<__nv_bfloat16*>(terms + TC_OPER_BYTES + off) = t2;
        *reinterpret_cast<__nv_bfloat16*>(terms + 2 * TC_OPER_BYTES + off) = __float2bfloat16_rn(e2);
      } else {
        __half t1 = __float2half_rn(r);
        *reinterpret_cast<__half*>(terms + off) = t1;
        *reinterpret_cast<__half*>(terms + TC_OPER_BYTES + off) = __float2half_rn(r - __half2float(t1));
      }
    }
  }
  __syncthreads();
  // Cell table over [b_first - 4w, b_last + 4w): the entry of cell c answers for any y whose
  // cell index, computed in float32, comes out as c-1, c or c+1.
  const float b_first = bnd[0], b_last = bnd[NB - 1];
  const float cw = (b_last - b_first) / (float)(TC_CELLS - 8);
  const float inv_cw = 1.0f / cw;
  const float cell_off = 4.0f - b_first * inv_cw;
  {
    float2* cells = reinterpret_cast<float2*>(rinv_s);   // scratch until the main loop starts
    if (tid < TC_CELLS) {
      const int c = tid;
      const float lo_edge = b_first + (float)(c - 5) * cw;
      const float hi_edge = b_first + (float)(c - 2) * cw;
      int below_n = 0, cnt = 0;
      for (int k = 0; k < NB; ++k) {
        bool below = (c > 0) && (bnd[k] < lo_edge);
        bool above = (c < TC_CELLS - 1) && (bnd[k] >= hi_edge);
        below_n += below ? 1 : 0;
        cnt += (!below && !above) ? 1 : 0;
      }
      cells[c] = make_float2(cnt > 0 ? bnd[below_n] : __int_as_float(0x7f800000), __int_as_float(below_n));
      if (cnt > 1 || !(cw > 0.f) || !(inv_cw < 3.0e38f)) *simple_flag = 0;
    }
    __syncthreads();
    // one copy per lane, 8 bytes apart: a warp's 32 lookups never share a bank
    for (int e = tid; e < TC_CELLS * 32; e += TC_THREADS) lut[e] = cells[e >> 5];
  }
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_slot;
  const bool simple = *simple_flag != 0;

  // instruction descriptor: D = f32, A/B = f16 or bf16, both K-major, N = 128, M = 128
  constexpr uint32_t FMT = BF16 ? 1u : 0u;
  constexpr uint32_t IDESC = (1u << 4) | (FMT << 7) | (FMT << 10) | ((128u >> 3) << 17) | ((128u >> 4) << 24);

  const int64_t num_tiles = (n_rows + 127) >> 7;
  const int n_my = (int)((num_tiles - blockIdx.x + gridDim.x - 1) / gridDim.x);

  const uint32_t failed_s = smem_u32(failed_flag);
  const uint32_t full_s = mbar_s, nready_s = mbar_s + 24, done_s = mbar_s + 56, free_s = mbar_s + 72, drain_s = mbar_s + 88;
  // Bounded wait; once one wait of the CTA has run out, the others return at once.
  auto wait = [&](uint32_t bar, uint32_t parity) -> bool {
    if (lds_u32(failed_s) != 0u) return false;
    if (mbar_wait(bar, parity)) return true;
    g_tc_status = 1;
    asm volatile("st.shared.u32 [%0], %1;" :: "r"(failed_s), "r"(1u) : "memory");
    return false;
  };
  auto wait_warp = [&](uint32_t bar, uint32_t parity) -> bool { return __all_sync(0xffffffffu, wait(bar, parity)); };
  auto tile_row0 = [&](int t) { return ((int64_t)blockIdx.x + (int64_t)t * gridDim.x) * 128; };

  if (warp == 16) {
    // ---- MMA warp: the whole rotation of tile t, as soon as its rows are there and its accumulator is free ----
    if (lane == 0) {
      for (int t = 0; t < n_my; ++t) {
        const uint32_t b = (uint32_t)(t % NBUF), s = (uint32_t)(t & 1);
        if (!wait(full_s + 8u * b, (uint32_t)((t / NBUF) & 1))) break;
        if (t >= 2 && !wait(free_s + 8u * s, (uint32_t)(((t - 2) >> 1) & 1))) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        if (t == withhold) continue;
        const uint32_t a_s = abuf_s + b * TC_OPER_BYTES;
        const uint32_t d0 = tmem_base + s * ACC_COLS;
#pragma unroll
        for (int tm = 0; tm < TERMS; ++tm) {
#pragma unroll
          for (int kk = 0; kk < 8; ++kk) {
            const uint32_t koff = (uint32_t)((kk >> 2) * TC_HALF_BYTES + (kk & 3) * 32);
            umma_f16(d0, umma_desc(a_s + koff),
                     umma_desc(terms_s + (uint32_t)tm * TC_OPER_BYTES + koff), IDESC, (uint32_t)((tm | kk) != 0));
          }
        }
        umma_commit(done_s + 8u * s);
      }
    }
    __syncwarp();
  } else {
    // ---- worker warps ----
    // input side: row 8 warp + (lane >> 3) (+ 4), 16-byte piece lane & 7 of both K halves
    const int64_t step = (int64_t)gridDim.x * 128;
    const int64_t step_tok = m.slot_mapping ? step / m.num_heads : 0;
    const int step_head = m.slot_mapping ? (int)(step - step_tok * m.num_heads) : 0;
    TcCursor lc[2];         // the rows this thread loads, at the tile whose copies are issued next
    lc[0] = cursor_at(m, tile_row0(0) + 8 * warp + (lane >> 3));
    lc[1] = cursor_at(m, tile_row0(0) + 8 * warp + (lane >> 3) + 4);
    auto issue_loads = [&](int t) {         // called for t = 0, 1, 2, ... in order
      const uint32_t dst0 = abuf_s + (uint32_t)(t % NBUF) * TC_OPER_BYTES;
#pragma unroll
      for (int pass = 0; pass < 2; ++pass) {
        const int r = 8 * warp + (lane >> 3) + 4 * pass, c = lane & 7;
        const int64_t off = cursor_src(m, lc[pass], n_rows);
        cursor_advance(m, lc[pass], step, step_tok, step_head);
        const uint32_t nbytes = off >= 0 ? 16u : 0u;
        const uint16_t* src = reinterpret_cast<const uint16_t*>(m.x) + (off >= 0 ? off : 0) + c * 8;
        const uint32_t dst = dst0 + (uint32_t)(r * 128 + ((c ^ (r & 7)) << 4));
#pragma unroll
        for (int h = 0; h < 2; ++h)
          asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;"
                       :: "r"(dst + h * TC_HALF_BYTES), "l"(src + h * 64), "r"(nbytes) : "memory");
      }
    };
    // one commit group per tile slot, empty past the last tile, so that "all but the newest AHEAD - 1 groups"
    // always means "up to tile t"
    for (int t = 0; t < AHEAD; ++t) {
      if (t < n_my) issue_loads(t);
      asm volatile("cp.async.commit_group;" ::: "memory");
    }
    const int w4 = warp & 3, colq = warp >> 2;
    const int qrow = w4 * 32 + lane;                  // output side: this thread's row, coordinates 32 colq ..
    TcCursor nc = cursor_at(m, tile_row0(0) + (tid >> 2));      // the row whose norm this thread's quad computes
    for (int t = 0; t <= n_my; ++t) {
      const bool have = t < n_my;
      TcRow nrow;                                     // where that row goes: worked out early, its slot load has time
      nrow.src_off = -1; nrow.dst = nullptr; nrow.dst_norm = nullptr;
      if (have && (tid & 3) == 3) nrow = cursor_dst(m, nc, n_rows);
      if (have) cursor_advance(m, nc, step, step_tok, step_head);
      if (have) {
        // ---- tile t: this warp's rows have landed -> MMA warp ----
        asm volatile("cp.async.wait_group %0;" :: "n"(AHEAD - 1) : "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncwarp();
        if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" :: "r"(full_s + 8u * (uint32_t)(t % NBUF)) : "memory");
        // ---- tile t: norms, four threads per vector, in the reference's summation order ----
        const int row = tid >> 2, qs = tid & 3;
        const uint8_t* rp = abuf + (t % NBUF) * TC_OPER_BYTES + row * 128 + qs * 4;
        float s0 = 0.f, s1 = 0.f;          // partial sums of lanes 2 qs and 2 qs + 1
#pragma unroll
        for (int c = 0; c < 16; ++c) {
          uint32_t w = *reinterpret_cast<const uint32_t*>(rp + (c >> 3) * TC_HALF_BYTES + (((c & 7) ^ (row & 7)) << 4));
          float x0 = bits16_to_float<BF16>(w & 0xffffu), x1 = bits16_to_float<BF16>(w >> 16);
          if (BF16) {
            s0 = __fadd_rn(s0, __fmul_rn(x0, x0));
            s1 = __fadd_rn(s1, __fmul_rn(x1, x1));
          } else {     // the square of an fp16 value is exact in float32: one rounding either way
            s0 = __fmaf_rn(x0, x0, s0);
            s1 = __fmaf_rn(x1, x1, s1);
          }
        }
        float acc = __fadd_rn(s0, s1);     // right for qs == 0; the others chain on below
#pragma unroll
        for (int step = 1; step < 4; ++step) {
          float prev = __shfl_sync(0xffffffffu, acc, (lane & ~3) + step - 1);
          if (qs == step) acc = __fadd_rn(__fadd_rn(prev, s0), s1);
        }
        if (qs == 3) {
          float nrm = __fsqrt_rn(acc);
          nrm_s[(t & 3) * 128 + row] = nrm;
          rinv_s[(t & 3) * 128 + row] = __frcp_rn(__fadd_rn(nrm, 1e-10f)) * (1.0f / PRESCALE);
          dstp_s[(t & 3) * 128 + row] = nrow.dst;
          dstn_s[(t & 3) * 128 + row] = nrow.dst_norm;
        }
        __syncwarp();
        if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" :: "r"(nready_s + 8u * (uint32_t)(t & 3)) : "memory");
      }
      // ---- tile t-1: its MMAs are complete: its operand buffer takes the rows of tile t + AHEAD ----
      bool ok = true;
      if (t >= 1) ok = wait_warp(done_s + 8u * (uint32_t)((t - 1) & 1), (uint32_t)(((t - 1) >> 1) & 1));
      if (ok && t + AHEAD < n_my) issue_loads(t + AHEAD);
      asm volatile("cp.async.commit_group;" ::: "memory");
      if (!ok) break;
      // ---- tile t-1: quantise and pack out of tensor memory ----
      if (t >= 1) {
        const int p = (t - 1) & 1, pn = (t - 1) & 3;
        if (!wait_warp(nready_s + 8u * (uint32_t)pn, (uint32_t)(((t - 1) >> 2) & 1))) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        uint32_t v1[32];
        tmem_ld32(tmem_base + ((uint32_t)(w4 * 32) << 16) + (uint32_t)(p * ACC_COLS + colq * 32), v1);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncwarp();
        if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" :: "r"(free_s + 8u * (uint32_t)p) : "memory");
        const int row = qrow;
        uint8_t* const dst = dstp_s[pn * 128 + row];
        const float rinv = rinv_s[pn * 128 + row];
        const bool store = dst != nullptr;
        float y[32];
#pragma unroll
        for (int k = 0; k < 32; ++k) y[k] = __fmul_rn(__uint_as_float(v1[k]), rinv);
        // 32 codes -> MSB-first bit stream, 8 codes per 4*BITS-bit group
        uint32_t grp[4];
        if (simple) {
          const float2* my_lut = lut + lane;
#pragma unroll
          for (int g8 = 0; g8 < 4; ++g8) {
            uint32_t acc = 0;
#pragma unroll
            for (int k = 0; k < 8; ++k) {
              const float yy = y[g8 * 8 + k];
              unsigned ci = __float2uint_rd(__fmaf_rn(yy, inv_cw, cell_off));   // negative, NaN -> 0
              ci = min(ci, (unsigned)(TC_CELLS - 1));
              const float2 e = my_lut[ci * 32];
              // acc = (acc << BITS) + cell's count + (its boundary < y)
              asm("{\n\t.reg .pred p;\n\tsetp.lt.f32 p, %2, %3;\n\tmad.lo.u32 %0, %0, %4, %1;\n\t@p add.u32 %0, %0, 1;\n\t}"
                  : "+r"(acc) : "r"(__float_as_int(e.y)), "f"(e.x), "f"(yy), "n"(1 << BITS));
            }
            grp[g8] = acc;
          }
        } else {        // boundaries too close for the cell table: count them all
#pragma unroll
          for (int g8 = 0; g8 < 4; ++g8) {
            uint32_t acc = 0;
#pragma unroll
            for (int k = 0; k < 8; ++k) {
              const float yy = y[g8 * 8 + k];
              uint32_t c = 0;
#pragma unroll
              for (int b = 0; b < NB; ++b) c += (bnd[b] < yy) ? 1u : 0u;
              acc = (acc << BITS) | c;
            }
            grp[g8] = acc;
          }
        }
        uint32_t pw[CHUNK_BYTES / 4];
        if (BITS == 4) {
#pragma unroll
          for (int k = 0; k < 4; ++k) pw[k] = bswap32(grp[k]);
        } else if (BITS == 3) {   // four 24-bit groups -> 12 bytes
          pw[0] = bswap32((grp[0] << 8) | (grp[1] >> 16));
          pw[1] = bswap32((grp[1] << 16) | (grp[2] >> 8));
          pw[2] = bswap32((grp[2] << 24) | grp[3]);
        } else {                  // four 16-bit groups -> 8 bytes
          pw[0] = bswap32((grp[0] << 16) | grp[1]);
          pw[1] = bswap32((grp[2] << 16) | grp[3]);
        }
        if (store) {
          uint8_t* dp = dst + colq * CHUNK_BYTES;
          const uintptr_t da = reinterpret_cast<uintptr_t>(dp);
          if (BITS == 4 && (da & 15) == 0) {
            *reinterpret_cast<uint4*>(dp) = make_uint4(pw[0], pw[1], pw[2], pw[3]);
          } else if ((da & 3) == 0) {
#pragma unroll
            for (int k = 0; k < CHUNK_BYTES / 4; ++k) reinterpret_cast<uint32_t*>(dp)[k] = pw[k];
          } else {
#pragma unroll
            for (int b = 0; b < CHUNK_BYTES; ++b) dp[b] = (uint8_t)(pw[b >> 2] >> (8 * (b & 3)));
          }
          if (colq == 0) *dstn_s[pn * 128 + row] = nrm_s[pn * 128 + row];
        }
      }
    }
    asm volatile("cp.async.wait_all;" ::: "memory");      // nothing of this thread may still be landing when the CTA leaves
  }

  // A CTA in which a wait gave up may still have MMAs in flight: before the columns go back, the issuing thread
  // commits once more on the drain barrier (it completes when every MMA that thread issued has) and waits,
  // bounded.  Only if that wait gives up too are the columns kept (status 2): they are lost to this SM until the
  // context ends, which is better than freeing them under an MMA.
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  int leak = 0;
  if (warp == 16 && lane == 0 && lds_u32(failed_s) != 0u) {
    umma_commit(drain_s);
    leak = mbar_wait(drain_s, 0u) ? 0 : 1;
    if (leak) g_tc_status = 2;
  }
  leak = __syncthreads_or(leak);
  if (warp == 0 && !leak) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, 256;" :: "r"(tmem_base) : "memory");
  }
}

template <int BITS, bool BF16>
int launch_tc(const RowMap& m, int64_t n_rows, const float* rot_t, const float* bnd, cudaStream_t st) {
  auto kern = tq_encode_tc_kernel<BITS, BF16>;
  constexpr size_t SMEM = tc_smem_bytes<BF16>();
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM);
  if (e != cudaSuccess) return fail((int)e, "encode: smem attribute: %s", cudaGetErrorString(e));
  int64_t tiles = (n_rows + 127) / 128;
  int grid = (int)(tiles < sm_count() ? tiles : sm_count());
  kern<<<grid, TC_THREADS, SMEM, st>>>(m, n_rows, rot_t, bnd);
  return check_launch("tq_encode_tc_kernel");
}

}  // namespace

int tc_encode_status(int* host_out, int reset) {
  cudaError_t e = cudaMemcpyFromSymbol(host_out, g_tc_status, sizeof(int));
  if (e == cudaSuccess && reset) { const int z = 0; e = cudaMemcpyToSymbol(g_tc_status, &z, sizeof(int)); }
  return e == cudaSuccess ? AKV_OK : fail((int)e, "encode status: %s", cudaGetErrorString(e));
}

int tc_encode_withhold(int tile) {
  cudaError_t e = cudaMemcpyToSymbol(g_tc_withhold, &tile, sizeof(int));
  return e == cudaSuccess ? AKV_OK : fail((int)e, "encode test hook: %s", cudaGetErrorString(e));
}

int launch_encode_tc(const RowMap& m, int64_t n_rows, int bits, bool bf16, const float* rot_t,
                     const float* boundaries, cudaStream_t st) {
  if (bits == 4) return bf16 ? launch_tc<4, true>(m, n_rows, rot_t, boundaries, st)
                             : launch_tc<4, false>(m, n_rows, rot_t, boundaries, st);
  if (bits == 3) return bf16 ? launch_tc<3, true>(m, n_rows, rot_t, boundaries, st)
                             : launch_tc<3, false>(m, n_rows, rot_t, boundaries, st);
  if (bits == 2) return bf16 ? launch_tc<2, true>(m, n_rows, rot_t, boundaries, st)
                             : launch_tc<2, false>(m, n_rows, rot_t, boundaries, st);
  return fail(AKV_ERR_ARG, "launch_encode_tc: bits %d", bits);
}

}  // namespace akv
