// Producer side of the attention block fused with the FP8 append: head-dim RMS norm of the query and
// key heads, rotary embedding, and quantize-and-append of the rotated key and of the value — the steps
// between the projections and the attention call in the model the reference runs (transformers'
// Qwen3.5 attention block: q_norm / k_norm, apply_rotary_pos_emb, cache update; the reference lists
// them as the elementwise work left around its fused attention,
// docs/journal/2026-10-23-phase2-r3-coordinator.md:147-150).
//
// One warp per head row, all layers in one launch.  Arithmetic follows the model's eager bf16 code:
//   y   = bf16( x * rsqrt(mean(x^2) + eps) * (1 + w) )                  fp32 inside, one rounding
//   out = bf16( bf16(y * cos) + bf16(rot(y) * sin) )  on the first rotary_dim dims, y elsewhere
// with rot(y)[i] = -y[i + r/2] for i < r/2 and y[i - r/2] above.  The key row is then quantised
// exactly as the append kernel does (per-head or per-token scales).  The fp32 sum of squares is a
// warp tree, not the model's CPU order, so y can differ from a CPU evaluation in the last bf16 bit.
#include "common.cuh"

namespace b200attn {

namespace {

__device__ __forceinline__ float bf16_round(float x) {
  return __bfloat162float(__float2bfloat16_rn(x));
}
__device__ __forceinline__ uint16_t bf16_bits(float x) {
  const __nv_bfloat16 b = __float2bfloat16_rn(x);
  return *reinterpret_cast<const uint16_t*>(&b);
}

template <int D>
__global__ void __launch_bounds__(256)
producer_kernel(Geometry g, int rotary_dim, float eps, const uint16_t* __restrict__ q_raw,
                const uint16_t* __restrict__ k_raw, const uint16_t* __restrict__ v_new,
                const uint16_t* __restrict__ wq, const uint16_t* __restrict__ wk, const uint16_t* __restrict__ cosp,
                const uint16_t* __restrict__ sinp, uint16_t* __restrict__ q_out, uint16_t* __restrict__ k_out,
                uint8_t* __restrict__ k_cache, uint8_t* __restrict__ v_cache, float* __restrict__ k_scale,
                float* __restrict__ v_scale, const int* __restrict__ seq_pos, int* __restrict__ status) {
  constexpr int EPL = D / 32;   // elements per lane, contiguous
  const int lane = threadIdx.x & 31;
  const long long row = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int per_lb = g.h_q + 2 * g.h_kv;
  const long long rows = (long long)g.n_layers * g.batch * per_lb;
  if (row >= rows) return;   // whole warps only: blockDim is a multiple of 32
  const long long lb = row / per_lb;
  const int r = (int)(row % per_lb);
  const int layer = (int)(lb / g.batch), b = (int)(lb % g.batch);
  const int kind = r < g.h_q ? 0 : (r < g.h_q + g.h_kv ? 1 : 2);   // query, key, value
  const int h = kind == 0 ? r : (kind == 1 ? r - g.h_q : r - g.h_q - g.h_kv);
  const uint16_t* src = kind == 0 ? q_raw + (lb * g.h_q + h) * D
                                  : (kind == 1 ? k_raw : v_new) + (lb * g.h_kv + h) * D;
  float x[EPL];
  {
    uint32_t w[EPL / 2];
    if (EPL == 4) {
      const uint2 raw = *reinterpret_cast<const uint2*>(src + lane * EPL);
      w[0] = raw.x; w[1] = raw.y;
    } else {
      const uint4 raw = *reinterpret_cast<const uint4*>(src + lane * EPL);
      w[0] = raw.x; w[1] = raw.y; w[EPL / 2 - 2] = raw.z; w[EPL / 2 - 1] = raw.w;
    }
#pragma unroll
    for (int i = 0; i < EPL / 2; ++i) {
      x[2 * i] = bf16_bits_to_float(w[i] & 0xFFFFu);
      x[2 * i + 1] = bf16_bits_to_float(w[i] >> 16);
    }
  }
  if (kind != 2) {
    // ---- RMS norm over the head dim, weight (1 + w) ----
    float ss = 0.f;
#pragma unroll
    for (int e = 0; e < EPL; ++e) ss += x[e] * x[e];
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, off);
    const float inv = __frsqrt_rn(ss * (1.f / D) + eps);
    const uint16_t* wn = (kind == 0 ? wq : wk) + (long long)layer * D + lane * EPL;
#pragma unroll
    for (int e = 0; e < EPL; ++e) x[e] = bf16_round((x[e] * inv) * (1.f + bf16_bits_to_float(wn[e])));
    // ---- rotary embedding on the first rotary_dim dims: the partner sits (r/2)/EPL lanes away ----
    const int half = rotary_dim >> 1, half_lanes = half / EPL;
    const int i0 = lane * EPL;
    const bool low = i0 < half;
    const int partner = low ? lane + half_lanes : lane - half_lanes;
#pragma unroll
    for (int e = 0; e < EPL; ++e) {
      const float other = __shfl_sync(0xffffffffu, x[e], partner & 31);
      if (i0 < rotary_dim) {
        const float c = bf16_bits_to_float(cosp[(long long)b * rotary_dim + i0 + e]);
        const float s = bf16_bits_to_float(sinp[(long long)b * rotary_dim + i0 + e]);
        x[e] = bf16_round(bf16_round(x[e] * c) + bf16_round((low ? -other : other) * s));
      }
    }
  }
  if (kind == 0 || (kind == 1 && k_out)) {
    uint16_t* dst = kind == 0 ? q_out + (lb * g.h_q + h) * D : k_out + (lb * g.h_kv + h) * D;
    uint32_t w[EPL / 2];
#pragma unroll
    for (int i = 0; i < EPL / 2; ++i) w[i] = (uint32_t)bf16_bits(x[2 * i]) | ((uint32_t)bf16_bits(x[2 * i + 1]) << 16);
    if (EPL == 4) *reinterpret_cast<uint2*>(dst + lane * EPL) = make_uint2(w[0], w[1]);
    else *reinterpret_cast<uint4*>(dst + lane * EPL) = make_uint4(w[0], w[1], w[EPL / 2 - 2], w[EPL / 2 - 1]);
  }
  if (kind == 0) return;
  // ---- quantize-and-append of the key / value row (same arithmetic as append_kernel) ----
  const int pos = seq_pos[b];
  const bool fits = pos >= 0 && pos < g.capacity;
  if (!fits && lane == 0 && h == 0 && layer == 0 && kind == 1) atomicOr(status, B200ATTN_STATUS_POS_AT_CAPACITY);
  float* scale = kind == 1 ? k_scale : v_scale;
  float s;
  if (g.scale_mode == B200ATTN_SCALE_PER_TOKEN) {
    float amax = 0.f;
#pragma unroll
    for (int e = 0; e < EPL; ++e) amax = fmaxf(amax, fabsf(x[e]));
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
    s = __fdiv_rn(amax, kE4m3Max);
    if (fits && lane == 0) scale[(((long long)layer * g.batch + b) * g.capacity + pos) * g.h_kv + h] = s;
  } else {
    s = scale[layer * g.h_kv + h];
  }
  if (!fits) return;
  uint32_t out[EPL / 4];
#pragma unroll
  for (int i = 0; i < EPL / 4; ++i) {
    out[i] = 0;
    if (!(g.scale_mode == B200ATTN_SCALE_PER_TOKEN && s == 0.f)) {   // all-zero row: bytes are defined as 0
#pragma unroll
      for (int j = 0; j < 4; ++j) out[i] |= (uint32_t)quantize_e4m3(x[4 * i + j], s) << (8 * j);
    }
  }
  uint8_t* cache = kind == 1 ? k_cache : v_cache;
  const long long lstride = kind == 1 ? g.k_layer_stride : g.v_layer_stride;
  uint8_t* dst = cache + (long long)layer * lstride + (((long long)b * g.h_kv + h) * g.capacity + pos) * D + lane * EPL;
  if (EPL == 4) *reinterpret_cast<uint32_t*>(dst) = out[0];
  else *reinterpret_cast<uint2*>(dst) = make_uint2(out[0], out[EPL / 4 - 1]);
}

}  // namespace

cudaError_t launch_producer(const Geometry& g, int rotary_dim, float eps, const void* q_raw, const void* k_raw,
                            const void* v_new, const void* wq, const void* wk, const void* cosp, const void* sinp,
                            void* q_out, void* k_out, void* k_cache, void* v_cache, float* k_scale, float* v_scale,
                            int* seq_pos, int advance_pos, int* status, cudaStream_t stream) {
  const long long rows = (long long)g.n_layers * g.batch * (g.h_q + 2 * g.h_kv);
  const int block = 256;
  const long long grid = (rows * 32 + block - 1) / block;
  if (grid > 0x7fffffffLL) return cudaErrorInvalidConfiguration;
  auto launch = [&](auto kernel) {
    kernel<<<(unsigned)grid, block, 0, stream>>>(g, rotary_dim, eps, (const uint16_t*)q_raw, (const uint16_t*)k_raw,
                                                 (const uint16_t*)v_new, (const uint16_t*)wq, (const uint16_t*)wk,
                                                 (const uint16_t*)cosp, (const uint16_t*)sinp, (uint16_t*)q_out,
                                                 (uint16_t*)k_out, (uint8_t*)k_cache, (uint8_t*)v_cache, k_scale,
                                                 v_scale, seq_pos, status);
  };
  if (g.head_dim == 128) launch(producer_kernel<128>); else launch(producer_kernel<256>);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return e;
  if (advance_pos) return launch_advance_pos(g, 1, seq_pos, stream);
  return cudaSuccess;
}

}  // namespace b200attn
