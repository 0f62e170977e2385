// Cross-GPU exchange of split-K partials over NVLink peer memory, without a collective library.
//
// Long-context split-K leaves every GPU with one un-normalised partial (m, l, acc[D]) per (sequence,
// query head).  The NCCL route is all-gather + local merge; at these sizes (a few hundred KB) the
// all-gather is pure latency and dominates the step from four GPUs up.  Here every GPU owns an exchange
// buffer that its peers can write (symmetric memory, mapped by the caller):
//
//   push   every rank copies its partial into slot `rank` of EVERY rank's exchange buffer with plain
//          peer stores, then - after a system-scope fence - adds one to word `rank` of every rank's flag
//          array, once per CTA;
//   wait   one warp spins (bounded) until the local flag words of all ranks have reached this step's
//          target, publishes the step's buffer half and advances the step counter;
//   merge  the ordinary LSE merge kernel reads the world partials from local memory.
//
// Buffers are double-buffered by step parity; a rank can be at most one step ahead of its peers (its next
// wait needs their next push, which follows their merge of the current step in stream order), so two
// halves suffice.  The step counter and the parity word live in device memory, so the three launches can
// be captured in a CUDA graph and replayed.  No multimem / NVLS, no kernel on one GPU ever waits for
// another kernel of the same GPU.
#include "common.cuh"

namespace akv {

constexpr int P2P_MAX_WORLD = 16;
constexpr int P2P_PUSH_CTAS = 16;

__device__ int g_p2p_status;      // 1: a wait for the peers' partials ran out

struct P2PPeers {
  float* buf[P2P_MAX_WORLD];           // exchange buffers: [2 halves][world][row_floats] floats each
  unsigned int* flags[P2P_MAX_WORLD];  // flag words: [world] counters each
};

__global__ void __launch_bounds__(256)
p2p_push_kernel(const float* __restrict__ local, int64_t row_floats, int world, int rank, P2PPeers peers,
                const unsigned int* __restrict__ step_ctr) {
  const unsigned int step = *step_ctr;
  const int64_t half = (int64_t)(step & 1u) * world * row_floats;
  const int64_t n4 = row_floats / 4;
  const float4* src = reinterpret_cast<const float4*>(local);
  for (int p = 0; p < world; ++p) {
    float4* dst = reinterpret_cast<float4*>(peers.buf[p] + half + (int64_t)rank * row_floats);
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (int64_t)gridDim.x * blockDim.x)
      dst[i] = src[i];
  }
  __threadfence_system();
  __syncthreads();
  if ((int)threadIdx.x < world) atomicAdd_system(peers.flags[threadIdx.x] + rank, 1u);
}

// One warp: lane r watches rank r's word.  cur_half receives the buffer half of this step.
__global__ void __launch_bounds__(32)
p2p_wait_kernel(volatile unsigned int* flags, int world, unsigned int* step_ctr, unsigned int* cur_half) {
  const unsigned int step = *step_ctr;
  const unsigned int target = (step + 1u) * (unsigned int)P2P_PUSH_CTAS;
  const int lane = threadIdx.x;
  bool ok = true;
  if (lane < world) {
    const long long t0 = clock64();
    for (;;) {
      unsigned int v;
      asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(flags + lane) : "memory");
      if ((int)(v - target) >= 0) break;
      if (clock64() - t0 > (1ll << 31)) { ok = false; break; }       // about a second
    }
  }
  ok = __all_sync(0xffffffffu, ok);
  if (lane == 0) {
    if (!ok) g_p2p_status = 1;
    *cur_half = step & 1u;
    *step_ctr = step + 1u;
  }
}

int p2p_status(int* host_out, int reset) {
  cudaError_t e = cudaMemcpyFromSymbol(host_out, g_p2p_status, sizeof(int));
  if (e == cudaSuccess && reset) { const int z = 0; e = cudaMemcpyToSymbol(g_p2p_status, &z, sizeof(int)); }
  return e == cudaSuccess ? AKV_OK : fail((int)e, "p2p status: %s", cudaGetErrorString(e));
}

}  // namespace akv

using namespace akv;

// Mirror of akv_p2p_merge_params in include/akv_b200.h.
struct akv_p2p_merge_params {
  const float* local_raw;
  int num_seqs, num_q_heads, head_dim;
  int world, rank;
  void* const* peer_buffers;          // HOST array [world] of device pointers
  void* const* peer_flags;            // HOST array [world] of device pointers
  unsigned int* state;                // local device words: [0] step counter, [1] current half
  const float* rotation;
  void* out; int out_dtype; int64_t out_stride_seq, out_stride_head;
  void* stream;
};

AKV_EXPORT size_t akv_p2p_exchange_bytes(int world, int num_seqs, int num_q_heads, int head_dim) {
  if (world <= 0 || num_seqs <= 0 || num_q_heads <= 0 || head_dim <= 0) return 0;
  return (size_t)2 * world * num_seqs * num_q_heads * (head_dim + 2) * sizeof(float);
}

AKV_EXPORT int akv_p2p_lse_merge(const akv_p2p_merge_params* p) {
  if (!p) return fail(AKV_ERR_ARG, "null params");
  if (p->world <= 0 || p->world > P2P_MAX_WORLD || p->rank < 0 || p->rank >= p->world)
    return fail(AKV_ERR_ARG, "akv_p2p_lse_merge: world %d / rank %d (at most %d ranks)", p->world, p->rank, P2P_MAX_WORLD);
  if (p->num_seqs < 0 || p->num_q_heads <= 0 || p->head_dim <= 0 || p->head_dim > 1024 || (p->head_dim + 2) % 2 ||
      (p->rotation != nullptr && p->head_dim % 16 != 0))
    return fail(AKV_ERR_ARG, "akv_p2p_lse_merge: bad sizes");
  if (p->num_seqs == 0) return AKV_OK;
  if (!p->local_raw || !p->peer_buffers || !p->peer_flags || !p->state || !p->out)
    return fail(AKV_ERR_ARG, "akv_p2p_lse_merge: null pointer");
  const int rows = p->num_seqs * p->num_q_heads;
  const int64_t row_floats = (int64_t)rows * (p->head_dim + 2);
  if (row_floats % 4 != 0 || (reinterpret_cast<uintptr_t>(p->local_raw) & 15))
    return fail(AKV_ERR_UNSUPPORTED, "akv_p2p_lse_merge: the partial must be 16-byte aligned and a multiple of 16 bytes");
  P2PPeers peers{};
  for (int r = 0; r < p->world; ++r) {
    peers.buf[r] = reinterpret_cast<float*>(p->peer_buffers[r]);
    peers.flags[r] = reinterpret_cast<unsigned int*>(p->peer_flags[r]);
    if (!peers.buf[r] || !peers.flags[r] || (reinterpret_cast<uintptr_t>(peers.buf[r]) & 15))
      return fail(AKV_ERR_ARG, "akv_p2p_lse_merge: peer %d has a null or misaligned buffer", r);
  }
  cudaStream_t st = (cudaStream_t)p->stream;
  p2p_push_kernel<<<P2P_PUSH_CTAS, 256, 0, st>>>(p->local_raw, row_floats, p->world, p->rank, peers, p->state);
  if (int rc = check_launch("p2p_push_kernel")) return rc;
  p2p_wait_kernel<<<1, 32, 0, st>>>(peers.flags[p->rank], p->world, p->state, p->state + 1);
  if (int rc = check_launch("p2p_wait_kernel")) return rc;
  MergeArgs mg{};
  const float* parts = peers.buf[p->rank];
  mg.acc = parts + 2; mg.acc_row = p->head_dim + 2; mg.acc_part = row_floats;
  mg.ml = parts; mg.ml_row = p->head_dim + 2; mg.ml_part = row_floats;
  mg.np = p->world;
  mg.context_lens = nullptr; mg.num_q_heads = p->num_q_heads;
  mg.D = p->head_dim;
  mg.mode = p->rotation ? MERGE_ROTATE : MERGE_NORMALIZE;
  mg.rot = p->rotation;
  mg.out = p->out; mg.out_dtype = p->out_dtype; mg.out_ss = p->out_stride_seq; mg.out_sh = p->out_stride_head;
  mg.half_select = p->state + 1;
  mg.half_stride = (int64_t)p->world * row_floats;
  return launch_merge(mg, rows, st);
}
