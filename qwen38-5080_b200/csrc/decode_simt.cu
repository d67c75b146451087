// SIMT variant of the decode attention: a CUDA-core split-K partial kernel and a separate
// log-sum-exp combine kernel.
//
// This is the direct restatement of the reference's fused kernel design ("one program = one
// (kv_head, split), covering all query heads that share the head; log2-domain online softmax;
// 2 kernels per layer", docs/journal/2026-10-23-phase2-r3-coordinator.md:137-141), extended to
// all layers and sequences in one launch.  Dequantisation happens in registers, QK^T is reduced
// with warp shuffles.  Each KV byte is read from HBM once and used for all G query heads.
// It is FMA/convert-issue bound on B200 (one convert and 2*G FMAs per cache byte), which is
// why the tensor-core variant exists; it stays as the independent second implementation the
// parity tests cross-check against.
//
// Layout of one CTA: 4 warps; a warp handles 32/LPT tokens at a time, LPT = D/16 lanes per token,
// each lane owning 16 consecutive dims (one 16-byte load per K row and per V row).
#include "common.cuh"

namespace b200attn {

namespace {

constexpr int kSimtWarps = 4;
constexpr int kSimtThreads = kSimtWarps * 32;

struct SimtParams {
  Geometry g;
  const uint16_t* q;      // bf16 bits [n_layers][batch][h_q][D]
  const uint8_t* k_cache;
  const uint8_t* v_cache;
  const float* k_scale;
  const float* v_scale;
  const int* seq_len;
  int seq_len_offset;
  float score_scale;      // softmax_scale * log2(e)
  int num_splits;
  float* part_acc;        // [pairs][splits][G][D]
  float* part_ml;         // [pairs][splits][2][kMaxGroup]
  uint16_t* out;          // bf16 bits [n_layers][batch][h_q][D]
  int* status;
};

__device__ __forceinline__ int clamp_len(int len, int capacity, int* status) {
  if (len < 0) {
    if (threadIdx.x == 0) atomicOr(status, B200ATTN_STATUS_LEN_NEGATIVE);
    return 0;
  }
  if (len > capacity) {
    if (threadIdx.x == 0) atomicOr(status, B200ATTN_STATUS_LEN_OVER_CAP);
    return capacity;
  }
  return len;
}

template <int D, int G>
__global__ void __launch_bounds__(kSimtThreads)
attn_splitk_simt_kernel(SimtParams p) {
  constexpr int LPT = D / 16;       // lanes per token
  constexpr int TPW = 32 / LPT;     // tokens per warp step
  constexpr int STEP = TPW * kSimtWarps;
  const Geometry& g = p.g;
  const int split = blockIdx.x, h = blockIdx.y;
  const int lb = blockIdx.z;        // layer*batch + b
  const int b = lb % g.batch, layer = lb / g.batch;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int grp = lane / LPT, lig = lane % LPT;

  const int len = clamp_len(p.seq_len[b] + p.seq_len_offset, g.capacity, p.status);
  // token range of this split: chunks are multiples of STEP
  int chunk = (len + p.num_splits - 1) / p.num_splits;
  chunk = (chunk + STEP - 1) / STEP * STEP;
  const int t0 = min(split * chunk, len), t1 = min(t0 + chunk, len);

  // q for the G heads of this KV head, this lane's 16 dims, as fp32
  float qf[G][16];
  {
    const uint16_t* qp = p.q + ((long long)lb * g.h_q + h * G) * D + lig * 16;
#pragma unroll
    for (int j = 0; j < G; ++j) {
      const uint4 a = *reinterpret_cast<const uint4*>(qp + j * D);
      const uint4 c = *reinterpret_cast<const uint4*>(qp + j * D + 8);
      const uint32_t w[8] = {a.x, a.y, a.z, a.w, c.x, c.y, c.z, c.w};
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        qf[j][2 * i] = bf16_bits_to_float(w[i] & 0xFFFFu);
        qf[j][2 * i + 1] = bf16_bits_to_float(w[i] >> 16);
      }
    }
  }
  const bool per_token = g.scale_mode == B200ATTN_SCALE_PER_TOKEN;
  const float ks_head = per_token ? 1.f : p.k_scale[layer * g.h_kv + h];
  const float vs_head = per_token ? 1.f : p.v_scale[layer * g.h_kv + h];
  const float* ks_tok = p.k_scale + (long long)lb * g.capacity * g.h_kv + h;  // + t*h_kv (per-token mode)
  const float* vs_tok = p.v_scale + (long long)lb * g.capacity * g.h_kv + h;

  const uint8_t* kbase = p.k_cache + (long long)layer * g.k_layer_stride +
                         ((long long)b * g.h_kv + h) * g.capacity * D + lig * 16;
  const uint8_t* vbase = p.v_cache + (long long)layer * g.v_layer_stride +
                         ((long long)b * g.h_kv + h) * g.capacity * D + lig * 16;

  float m[G], l[G], acc[G][16];
#pragma unroll
  for (int j = 0; j < G; ++j) {
    m[j] = -INFINITY;
    l[j] = 0.f;
#pragma unroll
    for (int i = 0; i < 16; ++i) acc[j][i] = 0.f;
  }

  int tok = t0 + warp * TPW + grp;
  uint4 kraw = make_uint4(0, 0, 0, 0), vraw = make_uint4(0, 0, 0, 0);
  if (tok < t1) {
    kraw = __ldg(reinterpret_cast<const uint4*>(kbase + (long long)tok * D));
    vraw = __ldg(reinterpret_cast<const uint4*>(vbase + (long long)tok * D));
  }
  for (int base = t0; base < t1; base += STEP) {   // uniform trip count for the whole CTA
    const int cur = tok;
    const uint4 kc = kraw, vc = vraw;
    tok += STEP;
    if (tok < t1) {  // prefetch the next step's rows
      kraw = __ldg(reinterpret_cast<const uint4*>(kbase + (long long)tok * D));
      vraw = __ldg(reinterpret_cast<const uint4*>(vbase + (long long)tok * D));
    }
    const bool valid = cur < t1;
    float kf[16];
    e4m3x16_to_float(kc, kf);
    float s[G];
#pragma unroll
    for (int j = 0; j < G; ++j) {
      float a = 0.f;
#pragma unroll
      for (int i = 0; i < 16; ++i) a = fmaf(qf[j][i], kf[i], a);
      s[j] = a;
    }
#pragma unroll
    for (int off = LPT / 2; off > 0; off >>= 1) {
#pragma unroll
      for (int j = 0; j < G; ++j) s[j] += __shfl_xor_sync(0xffffffffu, s[j], off);
    }
    if (valid) {
      const float kscale = (per_token ? ks_tok[(long long)cur * g.h_kv] : ks_head) * p.score_scale;
      const float vscale = per_token ? vs_tok[(long long)cur * g.h_kv] : 1.f;
      float vf[16];
      e4m3x16_to_float(vc, vf);
#pragma unroll
      for (int j = 0; j < G; ++j) {
        const float t = s[j] * kscale;
        if (t > m[j]) {
          const float alpha = exp2f(m[j] - t);   // m = -inf on first use -> 0
          l[j] *= alpha;
#pragma unroll
          for (int i = 0; i < 16; ++i) acc[j][i] *= alpha;
          m[j] = t;
        }
        const float pr = exp2f(t - m[j]);
        l[j] += pr;
        const float pv = pr * vscale;
#pragma unroll
        for (int i = 0; i < 16; ++i) acc[j][i] = fmaf(pv, vf[i], acc[j][i]);
      }
    }
  }

  // ---- merge the TPW token groups of the warp (lanes with equal lig) ----
#pragma unroll
  for (int j = 0; j < G; ++j) {
    float mm = m[j];
#pragma unroll
    for (int off = LPT; off < 32; off <<= 1) mm = fmaxf(mm, __shfl_xor_sync(0xffffffffu, mm, off));
    const float f = (m[j] == -INFINITY) ? 0.f : exp2f(m[j] - mm);
    float ll = l[j] * f;
#pragma unroll
    for (int off = LPT; off < 32; off <<= 1) ll += __shfl_xor_sync(0xffffffffu, ll, off);
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      float a = acc[j][i] * f;
#pragma unroll
      for (int off = LPT; off < 32; off <<= 1) a += __shfl_xor_sync(0xffffffffu, a, off);
      acc[j][i] = a;
    }
    m[j] = mm;
    l[j] = ll;
  }

  // ---- merge the warps through shared memory ----
  __shared__ float sm_m[kSimtWarps][kMaxGroup];
  __shared__ float sm_l[kSimtWarps][kMaxGroup];
  __shared__ float sm_acc[kSimtWarps][G][D];
  if (grp == 0) {
#pragma unroll
    for (int j = 0; j < G; ++j) {
      if (lig == 0) { sm_m[warp][j] = m[j]; sm_l[warp][j] = l[j]; }
#pragma unroll
      for (int i = 0; i < 16; ++i) sm_acc[warp][j][lig * 16 + i] = acc[j][i];
    }
  }
  __syncthreads();

  const long long pair = (long long)lb * g.h_kv + h;
  const bool direct = p.num_splits == 1;
  for (int idx = threadIdx.x; idx < G * D; idx += kSimtThreads) {
    const int j = idx / D, d = idx % D;
    float mm = sm_m[0][j];
#pragma unroll
    for (int w = 1; w < kSimtWarps; ++w) mm = fmaxf(mm, sm_m[w][j]);
    float a = 0.f, ll = 0.f;
#pragma unroll
    for (int w = 0; w < kSimtWarps; ++w) {
      const float f = (sm_m[w][j] == -INFINITY) ? 0.f : exp2f(sm_m[w][j] - mm);
      a += sm_acc[w][j][d] * f;
      ll += sm_l[w][j] * f;
    }
    if (direct) {
      const float o = ll > 0.f ? a * vs_head / ll : 0.f;
      __nv_bfloat16 ob = __float2bfloat16_rn(o);
      p.out[((long long)lb * g.h_q + h * G + j) * D + d] = *reinterpret_cast<uint16_t*>(&ob);
    } else {
      p.part_acc[((pair * p.num_splits + split) * G + j) * D + d] = a;
      if (d == 0) {
        float* ml = p.part_ml + (pair * p.num_splits + split) * 2 * kMaxGroup;
        ml[j] = mm;
        ml[kMaxGroup + j] = ll;
      }
    }
  }
}

// out[h][d] = sum_s acc_s * 2^(m_s - M) / sum_s l_s * 2^(m_s - M) * v_scale.  One CTA per pair.
template <int D, int G>
__global__ void __launch_bounds__(D)
combine_simt_kernel(SimtParams p) {
  const Geometry& g = p.g;
  const long long pair = blockIdx.x;
  const int h = (int)(pair % g.h_kv);
  const long long lb = pair / g.h_kv;
  const int layer = (int)(lb / g.batch);
  const int d = threadIdx.x;
  const float vs = g.scale_mode == B200ATTN_SCALE_PER_TOKEN ? 1.f : p.v_scale[layer * g.h_kv + h];
  const float* ml = p.part_ml + pair * p.num_splits * 2 * kMaxGroup;
  const float* pa = p.part_acc + pair * p.num_splits * G * D;
#pragma unroll
  for (int j = 0; j < G; ++j) {
    float mm = -INFINITY;
    for (int s = 0; s < p.num_splits; ++s) mm = fmaxf(mm, ml[s * 2 * kMaxGroup + j]);
    float a = 0.f, ll = 0.f;
    for (int s = 0; s < p.num_splits; ++s) {
      const float ms = ml[s * 2 * kMaxGroup + j];
      const float f = (ms == -INFINITY) ? 0.f : exp2f(ms - mm);
      ll += ml[s * 2 * kMaxGroup + kMaxGroup + j] * f;
      a += pa[(s * G + j) * D + d] * f;
    }
    const float o = ll > 0.f ? a * vs / ll : 0.f;
    __nv_bfloat16 ob = __float2bfloat16_rn(o);
    p.out[(lb * g.h_q + h * G + j) * D + d] = *reinterpret_cast<uint16_t*>(&ob);
  }
}

template <int D, int G>
cudaError_t launch_t(const SimtParams& p, cudaStream_t stream) {
  const Geometry& g = p.g;
  dim3 grid(p.num_splits, g.h_kv, g.n_layers * g.batch);
  attn_splitk_simt_kernel<D, G><<<grid, kSimtThreads, 0, stream>>>(p);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess || p.num_splits == 1) return e;
  combine_simt_kernel<D, G><<<(unsigned)((long long)g.n_layers * g.batch * g.h_kv), D, 0, stream>>>(p);
  return cudaGetLastError();
}

template <int D>
cudaError_t launch_d(const SimtParams& p, cudaStream_t stream) {
  switch (p.g.group) {
    case 1: return launch_t<D, 1>(p, stream);
    case 2: return launch_t<D, 2>(p, stream);
    case 3: return launch_t<D, 3>(p, stream);
    case 4: return launch_t<D, 4>(p, stream);
    case 5: return launch_t<D, 5>(p, stream);
    case 6: return launch_t<D, 6>(p, stream);
    case 7: return launch_t<D, 7>(p, stream);
    case 8: return launch_t<D, 8>(p, stream);
  }
  return cudaErrorInvalidValue;
}

}  // namespace

size_t simt_workspace_bytes(const Geometry& g, int num_splits) {
  const size_t pairs = (size_t)g.n_layers * g.batch * g.h_kv;
  return pairs * num_splits * ((size_t)g.group * g.head_dim + 2 * kMaxGroup) * sizeof(float);
}

int simt_pick_splits(const Geometry& g, int max_seq_len, int num_sms) {
  // enough CTAs for ~4 per SM, but at least 64 tokens per split
  const long long pairs = (long long)g.n_layers * g.batch * g.h_kv;
  long long want = (4LL * num_sms + pairs - 1) / pairs;
  long long max_by_len = max_seq_len / 64;
  if (max_by_len < 1) max_by_len = 1;
  if (want > max_by_len) want = max_by_len;
  if (want < 1) want = 1;
  if (want > 256) want = 256;
  return (int)want;
}

cudaError_t launch_decode_simt(const Geometry& g, const DecodeArgs& a, cudaStream_t stream) {
  SimtParams p;
  p.g = g;
  p.q = (const uint16_t*)a.q;
  p.k_cache = (const uint8_t*)a.k_cache;
  p.v_cache = (const uint8_t*)a.v_cache;
  p.k_scale = a.k_scale;
  p.v_scale = a.v_scale;
  p.seq_len = a.seq_len;
  p.seq_len_offset = a.seq_len_offset;
  p.score_scale = a.softmax_scale * kLog2e;
  p.num_splits = a.num_splits;
  const size_t pairs = (size_t)g.n_layers * g.batch * g.h_kv;
  p.part_acc = (float*)a.workspace;
  p.part_ml = p.part_acc + pairs * a.num_splits * g.group * g.head_dim;
  p.out = (uint16_t*)a.out;
  p.status = a.status;
  return g.head_dim == 128 ? launch_d<128>(p, stream) : launch_d<256>(p, stream);
}

}  // namespace b200attn
