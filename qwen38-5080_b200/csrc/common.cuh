// Shared device helpers and the internal launcher interface of libb200attn.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/b200attn.h"

namespace b200attn {

// Index checks of the -DB200ATTN_BOUNDS=1 build: a violated condition sets B200ATTN_STATUS_BOUNDS in the status word
// (nothing traps); the regular build compiles them away.
#ifdef B200ATTN_BOUNDS
#define B200ATTN_CHECK(status, cond) do { if (!(cond)) atomicOr((status), B200ATTN_STATUS_BOUNDS); } while (0)
#else
#define B200ATTN_CHECK(status, cond) do { } while (0)
#endif

constexpr float kLog2e = 1.4426950408889634f;
constexpr float kE4m3Max = 448.0f;
constexpr int kMaxGroup = 8;  // query heads per KV head the kernels support (benchmark shape 40/8: 5, reference model 24/4: 6)

// Resolved geometry handed to the launchers (strides in bytes, always filled in).
struct Geometry {
  int n_layers, batch, h_q, h_kv, head_dim, capacity, scale_mode, group;
  long long k_layer_stride, v_layer_stride;
};

// ---- fp8 / bf16 conversion ---------------------------------------------------------------

// Two e4m3 bytes (low 16 bits of `pair`) -> two floats, exact.
__device__ __forceinline__ float2 e4m3x2_to_float2(uint32_t pair) {
  uint32_t h2;
  asm("{ .reg .b16 lo; cvt.u16.u32 lo, %1; cvt.rn.f16x2.e4m3x2 %0, lo; }" : "=r"(h2) : "r"(pair));
  return __half22float2(*reinterpret_cast<__half2*>(&h2));
}

// Two e4m3 bytes held in a 16-bit register -> packed f16x2 (exact).
__device__ __forceinline__ uint32_t e4m3x2_to_f16x2(uint16_t pair) {
  uint32_t h2;
  asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(h2) : "h"(pair));
  return h2;
}

// 16 e4m3 bytes -> 16 floats.
__device__ __forceinline__ void e4m3x16_to_float(const uint4& raw, float* out) {
  const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 a = e4m3x2_to_float2(w[i] & 0xFFFFu);
    float2 b = e4m3x2_to_float2(w[i] >> 16);
    out[4 * i + 0] = a.x; out[4 * i + 1] = a.y; out[4 * i + 2] = b.x; out[4 * i + 3] = b.y;
  }
}

// clamp(x / s, -448, 448) -> e4m3fn byte, round to nearest even.  IEEE division.  A NaN input
// keeps its sign and becomes 0x7F / 0xFF, as a float32 -> float8_e4m3fn cast of a clamped NaN
// does on the host (GPU arithmetic would canonicalise the sign away, so it is taken from x);
// a NaN produced by the division itself (inf/inf) becomes 0x7F.  A zero scale (an all-zero row or
// head: the formula's 0/0 has no frozen meaning) gives the zero byte, in both scale layouts.
__device__ __forceinline__ uint8_t quantize_e4m3(float x, float s) {
  if (s == 0.f) return 0;
  if (x != x) return (uint8_t)(0x7F | ((__float_as_uint(x) >> 31) << 7));
  float y = __fdiv_rn(x, s);
  if (y != y) return (uint8_t)0x7F;
  y = fminf(fmaxf(y, -kE4m3Max), kE4m3Max);
  return (uint8_t)__nv_cvt_float_to_fp8(y, __NV_SATFINITE, __NV_E4M3);
}

__device__ __forceinline__ float bf16_bits_to_float(uint32_t bits16) {
  return __uint_as_float(bits16 << 16);
}

// SMs of the current device (cached per device); 148, a B200, when no device can be asked.
int device_sms();

// Remember a failed CUDA call for b200attn_last_cuda_error() on this thread; returns B200ATTN_ERR_CUDA.
int record_cuda_error(cudaError_t e);

// Host-side argument checks of b200attn_decode short of the workspace (api.cu).
int decode_precheck(const B200AttnShape* shape, const void* q, const void* k_cache, const void* v_cache,
                    const float* k_scale, const float* v_scale, const int* seq_len, const void* out, bool has_peers,
                    const int* status, int variant, int* num_splits, Geometry* g, int* resolved, size_t* need);

// ---- launchers (defined in the .cu files; called by the C-ABI layer in api.cu) ------------

cudaError_t launch_append(const Geometry& g, int n_tokens, const void* k_new, const void* v_new,
                          void* k_cache, void* v_cache, float* k_scale, float* v_scale,
                          int* seq_pos, int advance_pos, int* status, cudaStream_t stream);

cudaError_t launch_advance_pos(const Geometry& g, int n_tokens, int* seq_pos, cudaStream_t stream);

cudaError_t launch_dequant_prefix(const Geometry& g, int n_tokens, const void* cache,
                                  long long layer_stride, const float* scale, void* out,
                                  cudaStream_t stream);

cudaError_t launch_calibrate(const Geometry& g, int n_tokens, const void* x, float* scale,
                             cudaStream_t stream);

// Producer side: q_norm / k_norm + rotary embedding + quantize-and-append (producer.cu).
cudaError_t launch_producer(const Geometry& g, int rotary_dim, float eps, const void* q_raw, const void* k_raw,
                            const void* v_new, const void* wq, const void* wk, const void* cosp, const void* sinp,
                            void* q_out, void* k_out, void* k_cache, void* v_cache, float* k_scale, float* v_scale,
                            int* seq_pos, int advance_pos, int* status, cudaStream_t stream);

struct DecodeArgs {
  const void* q;
  const void* k_cache;
  const void* v_cache;
  const float* k_scale;
  const float* v_scale;
  const int* seq_len;
  int seq_len_offset;
  float softmax_scale;
  int num_splits;
  void* workspace;
  size_t workspace_bytes;
  void* out;
  int* status;
  const void* gate;   // optional (tensor-core variants only)
  int n_out;          // peer mode (tensor-core variants only): number of rank buffers, 0 = local output
  int out_hq_total, out_head_base;
  void* out_peer[8];
  void* out_peer_alt[8] = {};    // double-buffered gathered output: the second tensor of every rank
  int* epoch = nullptr;          // and the step counter whose parity picks the tensor (null = out_peer always)
  const void* pkt_src = nullptr; // packet mode: this rank's staging buffer; out_peer / out_peer_alt are then this rank's slots
                                 // in the other ranks' staging buffers for even / odd steps, `out` its own gathered tensor
  // fused step (all-tcgen05 variant only): the new token of every pair is quantised into the cache by
  // the CTA that owns the pair's last tile, and the last CTA to finish advances the positions
  const void* k_new = nullptr;   // bf16 [n_layers][batch][h_kv][1][head_dim]; null = attention only
  const void* v_new = nullptr;
  int* seq_pos = nullptr;        // positions to advance (the same buffer as seq_len), or null
  // cross-GPU barrier done by the last CTA to finish (flag buffers as for launch_peer_barrier); 0 ranks = none
  int* bar_flags[8] = {};
  int bar_rank = 0, bar_world = 0;
};

// Cross-GPU arrive-and-wait on symmetric flag buffers (peer_barrier.cu).
cudaError_t launch_peer_barrier(int* const* flags, int rank, int world, int* status, cudaStream_t stream);

// SIMT variant: split-K partial kernel + combine kernel.
size_t simt_workspace_bytes(const Geometry& g, int num_splits);
int simt_pick_splits(const Geometry& g, int max_seq_len, int num_sms);
cudaError_t launch_decode_simt(const Geometry& g, const DecodeArgs& a, cudaStream_t stream);

// MMA variant: TMA-staged, tensor-core stream-K kernel with fused combine.
size_t mma_workspace_bytes(const Geometry& g, int num_ctas);
int mma_pick_ctas(const Geometry& g, int max_seq_len, int num_sms);
cudaError_t launch_decode_mma(const Geometry& g, const DecodeArgs& a, cudaStream_t stream);

// All-tcgen05 variant: both products on tcgen05.mma straight from the staged FP8 tiles.
bool umma2_supported(const Geometry& g);
int umma2_pick_ctas(const Geometry& g, int max_seq_len, int num_sms);
cudaError_t launch_decode_umma2(const Geometry& g, const DecodeArgs& a, cudaStream_t stream);

}  // namespace b200attn
