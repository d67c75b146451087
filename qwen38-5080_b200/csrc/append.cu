// FP8 K/V quantize-and-append, dequantised prefix view, and scale calibration.
//
// The append replaces the reference's StaticLayer.update / index_copy_ pair
// (runner/model/static_cache.py:69-77) with the frozen FP8 format
// (docs/journal/2026-10-23-phase2-r3-coordinator.md:43-49).  It is pure HBM / launch-latency
// bound: per step it reads n_layers*batch*h_kv*head_dim*2 bf16 values and writes half as many
// bytes, so the only design points are 16-byte vector accesses and one launch for all layers.
#include "common.cuh"

namespace b200attn {

namespace {

// One thread converts 8 consecutive bf16 values of one (layer, seq, head, token) row.
// blockDim.x threads; rows are K rows first, then V rows (`which`).
template <int D>
__global__ void __launch_bounds__(256)
append_kernel(Geometry g, int n_tokens, const uint4* __restrict__ k_new, const uint4* __restrict__ v_new,
              uint8_t* __restrict__ k_cache, uint8_t* __restrict__ v_cache,
              float* __restrict__ k_scale, float* __restrict__ v_scale,
              const int* __restrict__ seq_pos, int* __restrict__ status) {
  constexpr int TPR = D / 8;  // threads per row (16 or 32): a row never straddles a warp
  const long long rows = (long long)g.n_layers * g.batch * g.h_kv * n_tokens;
  const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long row2 = tid / TPR;            // [0, 2*rows)
  const int c = (int)(tid % TPR);
  const bool active = row2 < 2 * rows;
  const int which = active && row2 >= rows ? 1 : 0;
  const long long row = active ? row2 - (long long)which * rows : 0;
  // row = ((layer*batch + b)*h_kv + h)*n_tokens + t
  const int t = (int)(row % n_tokens);
  const long long r1 = row / n_tokens;
  const int h = (int)(r1 % g.h_kv);
  const long long r2 = r1 / g.h_kv;
  const int b = (int)(r2 % g.batch);
  const int layer = (int)(r2 / g.batch);

  const int pos = seq_pos[b] + t;
  const bool fits = pos >= 0 && pos < g.capacity;
  if (active && !fits && c == 0 && h == 0 && layer == 0 && which == 0)
    atomicOr(status, B200ATTN_STATUS_POS_AT_CAPACITY);

  float x[8];
  if (active) {
    const uint4 raw = (which ? v_new : k_new)[row * TPR + c];
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      x[2 * i] = bf16_bits_to_float(w[i] & 0xFFFFu);
      x[2 * i + 1] = bf16_bits_to_float(w[i] >> 16);
    }
  } else {
#pragma unroll
    for (int i = 0; i < 8; ++i) x[i] = 0.f;
  }

  float s;
  float* scale = which ? v_scale : k_scale;
  if (g.scale_mode == B200ATTN_SCALE_PER_TOKEN) {
    // s = amax|x| / 448 over the row; all TPR lanes of the row take part in the shuffles.
    float amax = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(x[i]));
#pragma unroll
    for (int off = TPR / 2; off > 0; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
    s = __fdiv_rn(amax, kE4m3Max);
    if (active && fits && c == 0)
      scale[(((long long)layer * g.batch + b) * g.capacity + pos) * g.h_kv + h] = s;
  } else {
    s = active ? scale[layer * g.h_kv + h] : 1.f;
  }
  if (!active || !fits) return;

  uint32_t lo = 0, hi = 0;   // a zero scale (all-zero row or head) gives zero bytes: quantize_e4m3
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    lo |= (uint32_t)quantize_e4m3(x[i], s) << (8 * i);
    hi |= (uint32_t)quantize_e4m3(x[4 + i], s) << (8 * i);
  }
  uint8_t* cache = which ? v_cache : k_cache;
  const long long lstride = which ? g.v_layer_stride : g.k_layer_stride;
  uint8_t* dst = cache + (long long)layer * lstride +
                 (((long long)b * g.h_kv + h) * g.capacity + pos) * D + c * 8;
  *reinterpret_cast<uint2*>(dst) = make_uint2(lo, hi);
}

__global__ void advance_pos_kernel(int batch, int capacity, int n_tokens, int* __restrict__ seq_pos) {
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b < batch) {
    const int p = seq_pos[b];
    if (p >= 0 && p + n_tokens <= capacity) seq_pos[b] = p + n_tokens;
  }
}

// One thread turns 16 cache bytes into 16 bf16 values: bf16(float(byte) * s).
template <int D>
__global__ void __launch_bounds__(256)
dequant_prefix_kernel(Geometry g, int n_tokens, const uint8_t* __restrict__ cache, long long layer_stride,
                      const float* __restrict__ scale, uint4* __restrict__ out) {
  constexpr int TPR = D / 16;
  const long long rows = (long long)g.n_layers * g.batch * g.h_kv * n_tokens;
  const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long row = tid / TPR;
  const int c = (int)(tid % TPR);
  if (row >= rows) return;
  const int t = (int)(row % n_tokens);
  const long long r1 = row / n_tokens;
  const int h = (int)(r1 % g.h_kv);
  const long long r2 = r1 / g.h_kv;
  const int b = (int)(r2 % g.batch);
  const int layer = (int)(r2 / g.batch);
  const float s = g.scale_mode == B200ATTN_SCALE_PER_TOKEN
                      ? scale[(((long long)layer * g.batch + b) * g.capacity + t) * g.h_kv + h]
                      : scale[layer * g.h_kv + h];
  const uint8_t* src = cache + (long long)layer * layer_stride +
                       (((long long)b * g.h_kv + h) * g.capacity + t) * D + c * 16;
  const uint4 raw = *reinterpret_cast<const uint4*>(src);
  float f[16];
  e4m3x16_to_float(raw, f);
  uint32_t o[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    __nv_bfloat162 p = __floats2bfloat162_rn(f[2 * i] * s, f[2 * i + 1] * s);
    o[i] = *reinterpret_cast<uint32_t*>(&p);
  }
  out[(row * TPR + c) * 2] = make_uint4(o[0], o[1], o[2], o[3]);
  out[(row * TPR + c) * 2 + 1] = make_uint4(o[4], o[5], o[6], o[7]);
}

// scale[layer][h] = amax over (batch, token, dim) / 448, and 1 for a head that is zero everywhere (a
// zero scale would make every later append of that head meaningless).  One CTA per (h, layer).
__global__ void __launch_bounds__(256)
calibrate_kernel(Geometry g, int n_tokens, const uint4* __restrict__ x, float* __restrict__ scale) {
  const int h = blockIdx.x, layer = blockIdx.y;
  const long long vec_per_head = (long long)n_tokens * g.head_dim / 8;
  float amax = 0.f;
  for (int b = 0; b < g.batch; ++b) {
    const uint4* base = x + (((long long)layer * g.batch + b) * g.h_kv + h) * vec_per_head;
    for (long long i = threadIdx.x; i < vec_per_head; i += blockDim.x) {
      const uint4 raw = base[i];
      const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        amax = fmaxf(amax, fabsf(bf16_bits_to_float(w[j] & 0xFFFFu)));
        amax = fmaxf(amax, fabsf(bf16_bits_to_float(w[j] >> 16)));
      }
    }
  }
  __shared__ float red[8];
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int i = 1; i < 8; ++i) amax = fmaxf(amax, red[i]);
    scale[layer * g.h_kv + h] = amax == 0.f ? 1.f : __fdiv_rn(amax, kE4m3Max);
  }
}

}  // namespace

cudaError_t launch_append(const Geometry& g, int n_tokens, const void* k_new, const void* v_new,
                          void* k_cache, void* v_cache, float* k_scale, float* v_scale,
                          int* seq_pos, int advance_pos, int* status, cudaStream_t stream) {
  const long long rows = (long long)g.n_layers * g.batch * g.h_kv * n_tokens;
  const long long threads = 2 * rows * (g.head_dim / 8);
  const int block = 256;
  const long long grid = (threads + block - 1) / block;
  if (grid > 0x7fffffffLL) return cudaErrorInvalidConfiguration;
  if (g.head_dim == 128)
    append_kernel<128><<<(unsigned)grid, block, 0, stream>>>(
        g, n_tokens, (const uint4*)k_new, (const uint4*)v_new, (uint8_t*)k_cache, (uint8_t*)v_cache,
        k_scale, v_scale, seq_pos, status);
  else
    append_kernel<256><<<(unsigned)grid, block, 0, stream>>>(
        g, n_tokens, (const uint4*)k_new, (const uint4*)v_new, (uint8_t*)k_cache, (uint8_t*)v_cache,
        k_scale, v_scale, seq_pos, status);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return e;
  if (advance_pos) return launch_advance_pos(g, n_tokens, seq_pos, stream);
  return cudaSuccess;
}

cudaError_t launch_advance_pos(const Geometry& g, int n_tokens, int* seq_pos, cudaStream_t stream) {
  advance_pos_kernel<<<(g.batch + 127) / 128, 128, 0, stream>>>(g.batch, g.capacity, n_tokens, seq_pos);
  return cudaGetLastError();
}

cudaError_t launch_dequant_prefix(const Geometry& g, int n_tokens, const void* cache,
                                  long long layer_stride, const float* scale, void* out,
                                  cudaStream_t stream) {
  const long long rows = (long long)g.n_layers * g.batch * g.h_kv * n_tokens;
  const long long threads = rows * (g.head_dim / 16);
  const int block = 256;
  const long long grid = (threads + block - 1) / block;
  if (grid == 0) return cudaSuccess;
  if (grid > 0x7fffffffLL) return cudaErrorInvalidConfiguration;
  if (g.head_dim == 128)
    dequant_prefix_kernel<128><<<(unsigned)grid, block, 0, stream>>>(g, n_tokens, (const uint8_t*)cache,
                                                                    layer_stride, scale, (uint4*)out);
  else
    dequant_prefix_kernel<256><<<(unsigned)grid, block, 0, stream>>>(g, n_tokens, (const uint8_t*)cache,
                                                                    layer_stride, scale, (uint4*)out);
  return cudaGetLastError();
}

cudaError_t launch_calibrate(const Geometry& g, int n_tokens, const void* x, float* scale,
                             cudaStream_t stream) {
  calibrate_kernel<<<dim3(g.h_kv, g.n_layers), 256, 0, stream>>>(g, n_tokens, (const uint4*)x, scale);
  return cudaGetLastError();
}

}  // namespace b200attn
