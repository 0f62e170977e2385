// Library-wide entry points of the C ABI (version, last error text).
#include "common.cuh"

namespace akv {
char* error_buffer() {
  static thread_local char buf[512] = {0};
  return buf;
}

static long long g_launches = 0;                 // kernels launched by this process through the library
static thread_local const char* t_split_kernel = "";   // last split-K attention kernel of this thread

void note_launch(const char* what) {
  __atomic_add_fetch(&g_launches, 1, __ATOMIC_RELAXED);
  // the split-K kernels are the ones whose names contain "attn" or "tri_decode"; rotation, merge and
  // codec launches do not overwrite the record
  for (const char* c = what; *c; ++c)
    if ((c[0] == 'a' && c[1] == 't' && c[2] == 't' && c[3] == 'n') ||
        (c[0] == 't' && c[1] == 'r' && c[2] == 'i' && c[3] == '_' && c[4] == 'd')) { t_split_kernel = what; break; }
}
}  // namespace akv

AKV_EXPORT int akv_version(void) { return 101; }

// Number of kernels the library has launched in this process so far (launches recorded while a stream
// is being captured count once, at capture time).
AKV_EXPORT long long akv_launch_count(void) { return __atomic_load_n(&akv::g_launches, __ATOMIC_RELAXED); }

// Name of the split-K attention kernel most recently launched from the calling thread ("" if none).
AKV_EXPORT const char* akv_last_split_kernel(void) { return akv::t_split_kernel; }

AKV_EXPORT const char* akv_last_error(void) { return akv::error_buffer(); }

// Compute capability of the current device as major*10+minor (e.g. 100 on B200),
// or a negative value when no device is usable.
AKV_EXPORT int akv_device_arch(void) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return -1;
  int major = 0, minor = 0;
  if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess) return -1;
  cudaDeviceGetAttribute(&minor, cudaDevAttrComputeCapabilityMinor, dev);
  return major * 10 + minor;
}

// Device-side status words of the current device, copied to out[0..4] after everything queued on the
// device so far has finished (this call synchronises; it is a diagnostic, not part of a serving step):
//   out[0] tensor-core encoder, out[1] tensor-core decoder: 0 = fine, 1 = a bounded wait on an MMA barrier
//          gave up and the CTA left its tile unwritten, 2 = it also kept its tensor-memory columns
//   out[2] packed-cache attention, out[3] hybrid attention: 1 = a fixed-address kernel found its shared
//          window taken and returned without writing partials; out[2] = 2: a bounded wait for a bulk copy
//          ran out in a packed-cache attention kernel, in the TriAttention decode kernel or in the tensor-core
//          prefill kernel
//   out[4] akv_p2p_lse_merge: 1 = the bounded wait for the peers' partials ran out (a peer is late or gone)
// reset != 0 clears the words after reading them.
AKV_EXPORT int akv_device_status(int* out, int reset) {
  if (!out) return akv::fail(AKV_ERR_ARG, "akv_device_status: null pointer");
  cudaError_t e = cudaDeviceSynchronize();
  if (e != cudaSuccess) return akv::fail((int)e, "akv_device_status: %s", cudaGetErrorString(e));
  if (int rc = akv::tc_encode_status(out + 0, reset)) return rc;
  if (int rc = akv::tc_decode_status(out + 1, reset)) return rc;
  if (int rc = akv::attn_window_status(out + 2, reset)) return rc;
  int tri = 0;
  if (int rc = akv::tri_status(&tri, reset)) return rc;
  if (tri > out[2]) out[2] = tri;
  int pre = 0;
  if (int rc = akv::prefill_tc_status(&pre, reset)) return rc;
  if (pre != 0 && out[2] < 2) out[2] = 2;
  if (int rc = akv::hybrid_window_status(out + 3, reset)) return rc;
  return akv::p2p_status(out + 4, reset);
}

// Test hook for the bounded waits of the tensor-core codec kernels: CTA 0 of the next launches of the
// encoder (which = 0), decoder (which = 1) or prefill attention kernel (which = 2; CTA (0, 0), score MMAs of key tile
// `tile`) issues neither the MMAs nor the commit of its tile number
// `tile`, so the wait on that tile's barrier runs out with no tensor work in flight, the CTA leaves
// through its give-up path and akv_device_status reports 1.  tile < 0 switches the hook off (the default).
AKV_EXPORT int akv_debug_tc_withhold(int which, int tile) {
  if (which == 0) return akv::tc_encode_withhold(tile);
  if (which == 1) return akv::tc_decode_withhold(tile);
  if (which == 2) return akv::prefill_tc_withhold(tile);
  return akv::fail(AKV_ERR_ARG, "akv_debug_tc_withhold: which must be 0 (encode), 1 (decode) or 2 (prefill attention)");
}
