// Decode attention for callers that cannot hand the library a workspace.
//
// Some hosts of this library may not allocate device memory at the point where they call it: a
// serving loop whose device memory is owned and budgeted by the framework's pool (an extra
// cudaMalloc would bypass the accounting and can fail under fragmentation), or a latency-critical
// step where cudaMalloc's implicit device synchronisation is not acceptable.  For them the
// split-K partials of the tensor-core stream-K kernel live in a fixed
// array inside the library image instead of a caller-provided workspace.
//
// The array is per GPU (every device that loads the library holds kStaticScratchBytes until the
// process exits) and shared by all calls on that GPU: two calls that overlap on the device (two
// streams, two threads) would race on it — serialise them.  The kernel needs the part it uses
// zeroed and leaves it so; every call clears that part on the caller's stream all the same, so
// that a launch that ended in a time-out cannot leave anything behind for the next one.
#include <mutex>

#include "common.cuh"

namespace {

constexpr size_t kStaticScratchBytes = 8u << 20;   // 8 MiB: 444 CTAs x 2 partials x (5 x 128 + 16) tagged 8-byte words = 4.7 MB
constexpr int kMaxDevices = 64;

static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

std::mutex g_mu;
void* g_scratch_ptr[kMaxDevices] = {};   // device address of g_static_scratch, per device

// The array's name is only a host-side handle here: the device address has to be asked for, once
// per device, with that device current.
cudaError_t scratch_address(void** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev < 0 || dev >= kMaxDevices) return cudaErrorInvalidDevice;
  std::lock_guard<std::mutex> lock(g_mu);
  if (!g_scratch_ptr[dev]) {
    void* ptr = nullptr;
    e = cudaGetSymbolAddress(&ptr, g_static_scratch);
    if (e != cudaSuccess) return e;
    if (!ptr) return cudaErrorInvalidSymbol;
    g_scratch_ptr[dev] = ptr;
  }
  *out = g_scratch_ptr[dev];
  return cudaSuccess;
}

}  // namespace

extern "C" int b200attn_decode_static(const B200AttnShape* shape, const void* q, const void* k_cache,
                                      const void* v_cache, const float* k_scale, const float* v_scale,
                                      const int* seq_len, int seq_len_offset, float softmax_scale,
                                      int num_splits, void* out, int* status, void* stream) {
  // Every host-side check of b200attn_decode comes first, the size check among them: a call that is
  // going to be refused must not have touched the shared scratch, and an oversized request fails
  // before the array's address is even asked for.
  b200attn::Geometry g;
  int resolved = 0;
  size_t need = 0;
  int rc = b200attn::decode_precheck(shape, q, k_cache, v_cache, k_scale, v_scale, seq_len, out, false, status,
                                     B200ATTN_VARIANT_MMA, &num_splits, &g, &resolved, &need);
  if (rc) return rc;
  if (need > kStaticScratchBytes) return B200ATTN_ERR_TOO_LARGE;

  void* scratch = nullptr;
  cudaError_t e = scratch_address(&scratch);   // first call on a device: looks the address up
  if (e != cudaSuccess) return b200attn::record_cuda_error(e);
  e = cudaMemsetAsync(scratch, 0, need, (cudaStream_t)stream);
  if (e != cudaSuccess) return b200attn::record_cuda_error(e);
  return b200attn_decode(shape, q, k_cache, v_cache, k_scale, v_scale, seq_len, seq_len_offset, softmax_scale,
                         B200ATTN_VARIANT_MMA, num_splits, scratch, kStaticScratchBytes, out, status, stream);
}

extern "C" size_t b200attn_static_scratch_bytes(void) { return kStaticScratchBytes; }
