// Cross-GPU arrive-and-wait for the fused output all-gather.
//
// After the attention kernel of rank r has stored its heads into every rank's output buffer, the
// ranks have to agree that all stores have landed before anyone reads the gathered tensor.  Each
// rank owns a small flag buffer that its peers can write (symmetric memory):
//   flags[0 .. world)  : arrival epoch written by rank i into slot i
//   flags[world]       : this rank's own epoch counter
// One launch: bump the local epoch e, store e into slot `rank` of every peer (system-scope release:
// the preceding kernel's peer stores are ordered before it), then wait until every slot of the own
// buffer has reached e (system-scope acquire).  The wait is bounded (1 s): on expiry the kernel sets
// B200ATTN_STATUS_WAIT_TIMEOUT and returns.  The epoch lives in device memory, so the same launch can
// be replayed from a CUDA graph.
#include "common.cuh"

namespace b200attn {

namespace {

struct PeerFlags { int* ptr[8]; };

__global__ void peer_barrier_kernel(PeerFlags f, int rank, int world, int* status) {
  int* mine = f.ptr[rank];
  const int t = threadIdx.x;
  __shared__ int epoch;
  if (t == 0) epoch = mine[world] + 1;
  __syncthreads();
  const int e = epoch;
  if (t < world) {
    __threadfence_system();
    asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(f.ptr[t] + rank), "r"(e) : "memory");
    unsigned long long t0;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t0));
    for (;;) {
      int v;
      asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(mine + t) : "memory");
      if (v - e >= 0) break;
      unsigned long long now;
      asm volatile("mov.u64 %0, %globaltimer;" : "=l"(now));
      if (now - t0 > 1000000000ull) { atomicOr(status, B200ATTN_STATUS_WAIT_TIMEOUT); break; }
    }
  }
  __syncthreads();
  if (t == 0) mine[world] = e;
}

}  // namespace

cudaError_t launch_peer_barrier(int* const* flags, int rank, int world, int* status, cudaStream_t stream) {
  PeerFlags f;
  for (int r = 0; r < 8; ++r) f.ptr[r] = r < world ? flags[r] : nullptr;
  peer_barrier_kernel<<<1, 32, 0, stream>>>(f, rank, world, status);
  return cudaGetLastError();
}

}  // namespace b200attn
