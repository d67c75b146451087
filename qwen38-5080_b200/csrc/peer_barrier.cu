// Cross-GPU arrive-and-wait for the fused output all-gather.
//
// After the attention kernel of rank r has stored its heads into every rank's output buffer, the
// ranks have to agree that all stores have landed before anyone reads the gathered tensor.  Each
// rank owns a small flag buffer that its peers can write (symmetric memory):
//   flags[0 .. world)  : arrival epoch written by rank i into slot i
//   flags[world]       : this rank's own epoch counter
//   flags[16 .. 19]    : two 64-bit %globaltimer stamps of the latest arrive-and-wait (arrival, end of the wait)
// One launch of one warp: bump the local epoch e, lane r stores e into slot `rank` of rank r (after a system-scope
// fence: the preceding kernel's peer stores are ordered before it), then waits until slot r of the own
// buffer has reached e (system-scope acquire).  The wait is bounded (1 s): on expiry the kernel sets
// B200ATTN_STATUS_WAIT_TIMEOUT and returns.  The epoch lives in device memory, so the same launch can
// be replayed from a CUDA graph.
#include "streamk.cuh"

namespace b200attn {

namespace {

struct PeerFlags { int* ptr[8]; };

__global__ void peer_barrier_kernel(PeerFlags f, int rank, int world, int* status) {
  warp_peer_barrier(f.ptr, rank, world, (int)threadIdx.x, status);
}

}  // namespace

cudaError_t launch_peer_barrier(int* const* flags, int rank, int world, int* status, cudaStream_t stream) {
  PeerFlags f;
  for (int r = 0; r < 8; ++r) f.ptr[r] = r < world ? flags[r] : nullptr;
  peer_barrier_kernel<<<1, 32, 0, stream>>>(f, rank, world, status);
  return cudaGetLastError();
}

}  // namespace b200attn
