// C-ABI layer of libb200attn: argument validation on the host, then kernel launches on the
// caller's stream.  Nothing here allocates, synchronises or reads device memory.
#include <atomic>

#include "common.cuh"

using namespace b200attn;

namespace {

thread_local int g_last_cuda_error = 0;

int cuda_fail(cudaError_t e) { return b200attn::record_cuda_error(e); }

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// Validate the shape and resolve strides.  Returns 0 or a B200ATTN_ERR_* code.
int resolve(const B200AttnShape* s, Geometry* g) {
  if (!s) return B200ATTN_ERR_NULL;
  if (s->n_layers < 1 || s->batch < 1 || s->h_q < 1 || s->h_kv < 1 || s->capacity < 1) return B200ATTN_ERR_SHAPE;
  if (s->head_dim != 128 && s->head_dim != 256) return B200ATTN_ERR_SHAPE;
  if (s->h_q % s->h_kv) return B200ATTN_ERR_SHAPE;
  const int group = s->h_q / s->h_kv;
  if (group < 1 || group > kMaxGroup) return B200ATTN_ERR_SHAPE;
  if (s->scale_mode != B200ATTN_SCALE_PER_HEAD && s->scale_mode != B200ATTN_SCALE_PER_TOKEN) return B200ATTN_ERR_SHAPE;
  if (s->reserved != 0) return B200ATTN_ERR_SHAPE;
  if ((long long)s->n_layers * s->batch > 65535) return B200ATTN_ERR_SHAPE;
  // token rows of one layer are a 32-bit TMA coordinate
  if ((long long)s->batch * s->h_kv * s->capacity > 0x7fffffffLL) return B200ATTN_ERR_SHAPE;
  const long long dense = (long long)s->batch * s->h_kv * s->capacity * s->head_dim;
  g->n_layers = s->n_layers; g->batch = s->batch; g->h_q = s->h_q; g->h_kv = s->h_kv;
  g->head_dim = s->head_dim; g->capacity = s->capacity; g->scale_mode = s->scale_mode; g->group = group;
  g->k_layer_stride = s->k_layer_stride ? s->k_layer_stride : dense;
  g->v_layer_stride = s->v_layer_stride ? s->v_layer_stride : dense;
  if (s->n_layers > 1 && (g->k_layer_stride < dense || g->v_layer_stride < dense)) return B200ATTN_ERR_SHAPE;
  if ((g->k_layer_stride & 15) || (g->v_layer_stride & 15)) return B200ATTN_ERR_ALIGN;
  return B200ATTN_OK;
}

// AUTO = a tensor-core stream-K kernel wherever one applies.  The all-tcgen05 kernel (one CTA per SM,
// 128-token tiles, ~19 us of fixed cost per launch) takes long caches and both scale layouts (each
// softmax thread owns one token and applies its two scales); the mma.sync kernel (three CTAs per SM,
// 64-token tiles, finer split, per-head scales only) takes short caches, where it measured faster
// (depth 512: 22 vs 25 us) — and small shards of long ones: below ~64 tiles per SM the fixed cost of the
// all-tcgen05 kernel outweighs its faster streaming (64 layers at depth 8192 with one KV head, 28 tiles per
// SM: 33.4 us against 32.3 us with the mma.sync kernel on two CTAs per SM; two KV heads, 57 tiles per SM:
// 53.2 against 51.8 us; from 110 tiles per SM the two are level, at 221 the all-tcgen05 kernel leads by 6 us).
// The lengths live on the device, so the cache capacity stands in for them: the all-tcgen05 kernel from 2048
// token slots and 64 tiles per SM at capacity (24 with per-token scales, which the mma.sync kernel does not
// take).  What is left (short caches with
// per-token scales, batches beyond 2048) goes to the CUDA-core kernel.
// An explicit request that cannot be met is an error.
int resolve_variant(int variant, const Geometry& g) {
  const bool mma_ok = g.scale_mode == B200ATTN_SCALE_PER_HEAD && g.batch <= 2048;
  const bool umma2_ok = g.batch <= 2048 && umma2_supported(g);
  if (variant == B200ATTN_VARIANT_AUTO && umma2_ok && g.capacity >= 2048) {
    const long long tiles = (long long)g.n_layers * g.batch * g.h_kv * ((g.capacity + 127) / 128);
    if (tiles >= (mma_ok ? 64LL : 24LL) * device_sms()) return B200ATTN_VARIANT_UMMA2;
  }
  if (variant == B200ATTN_VARIANT_AUTO) return mma_ok ? B200ATTN_VARIANT_MMA : B200ATTN_VARIANT_SIMT;
  if (variant == B200ATTN_VARIANT_SIMT) return variant;
  if (variant == B200ATTN_VARIANT_MMA) return mma_ok ? variant : B200ATTN_ERR_SHAPE;
  if (variant == B200ATTN_VARIANT_UMMA2) return umma2_ok ? variant : B200ATTN_ERR_SHAPE;
  return B200ATTN_ERR_VARIANT;
}

// Gathered-output description of a tensor-parallel call.
int check_peers(const B200AttnPeerOut* peers, const Geometry& g) {
  if (peers->n_peers < 1 || peers->n_peers > 8 || peers->rank < 0 || peers->rank >= peers->n_peers) return B200ATTN_ERR_SHAPE;
  if (peers->h_q_total != g.h_q * peers->n_peers) return B200ATTN_ERR_SHAPE;
  if (peers->mode < 0 || peers->mode > B200ATTN_GATHER_PACKETS) return B200ATTN_ERR_SHAPE;
  if (peers->mode == B200ATTN_GATHER_PACKETS) {
    if (!peers->out[peers->rank] || !peers->step) return B200ATTN_ERR_NULL;
    if (!aligned16(peers->out[peers->rank])) return B200ATTN_ERR_ALIGN;
    for (int r = 0; r < peers->n_peers; ++r) {
      if (!peers->staging[r]) return B200ATTN_ERR_NULL;
      if (!aligned16(peers->staging[r])) return B200ATTN_ERR_ALIGN;
    }
    return B200ATTN_OK;
  }
  for (int r = 0; r < peers->n_peers; ++r) {
    if (!peers->out[r]) return B200ATTN_ERR_NULL;
    if (!aligned16(peers->out[r])) return B200ATTN_ERR_ALIGN;
    if (peers->mode == B200ATTN_GATHER_STORES_2BUF) {
      if (!peers->out_alt[r]) return B200ATTN_ERR_NULL;
      if (!aligned16(peers->out_alt[r])) return B200ATTN_ERR_ALIGN;
    }
  }
  if (peers->mode == B200ATTN_GATHER_STORES_2BUF && !peers->step) return B200ATTN_ERR_NULL;
  return B200ATTN_OK;
}

size_t staging_slot_bytes(const Geometry& g) { return (size_t)g.n_layers * g.batch * g.h_q * g.head_dim / 2 * 8; }

int pick(const Geometry& g, int v, int max_seq_len, int num_sms) {
  if (v == B200ATTN_VARIANT_SIMT) return simt_pick_splits(g, max_seq_len, num_sms);
  if (v == B200ATTN_VARIANT_UMMA2) return umma2_pick_ctas(g, max_seq_len, num_sms);
  return mma_pick_ctas(g, max_seq_len, num_sms);
}

}  // namespace

// SMs of the current device (cached per device); 148, a B200, when no device can be asked (the
// pure host helpers also run where there is no GPU).
int b200attn::device_sms() {
  static std::atomic<int> cache[64];
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) { (void)cudaGetLastError(); return 148; }
  int n = cache[dev].load(std::memory_order_relaxed);
  if (n > 0) return n;
  if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n < 1) { (void)cudaGetLastError(); return 148; }
  cache[dev].store(n, std::memory_order_relaxed);
  return n;
}

namespace b200attn {
int record_cuda_error(cudaError_t e) {
  g_last_cuda_error = (int)e;
  return B200ATTN_ERR_CUDA;
}
}  // namespace b200attn

extern "C" {

int b200attn_version(void) { return B200ATTN_VERSION; }

int b200attn_bounds_checked(void) {
#ifdef B200ATTN_BOUNDS
  return 1;
#else
  return 0;
#endif
}

#ifndef B200ATTN_SOURCE_HASH
#define B200ATTN_SOURCE_HASH ""
#endif
const char* b200attn_source_hash(void) { return B200ATTN_SOURCE_HASH; }

const char* b200attn_error_string(int code) {
  switch (code) {
    case B200ATTN_OK: return "ok";
    case B200ATTN_ERR_NULL: return "a required pointer is NULL";
    case B200ATTN_ERR_SHAPE: return "unsupported shape (head_dim 128|256, h_q multiple of h_kv, group <= 8, sizes >= 1)";
    case B200ATTN_ERR_ALIGN: return "pointer or stride not 16-byte aligned";
    case B200ATTN_ERR_WORKSPACE: return "workspace too small";
    case B200ATTN_ERR_SPLITS: return "split count out of range";
    case B200ATTN_ERR_CUDA: return "CUDA call failed";
    case B200ATTN_ERR_CAPACITY: return "length exceeds capacity";
    case B200ATTN_ERR_VARIANT: return "unknown kernel variant";
    case B200ATTN_ERR_TOO_LARGE: return "request exceeds the fixed scratch of b200attn_decode_static (8 MiB)";
  }
  return "unknown error code";
}

int b200attn_last_cuda_error(void) { return g_last_cuda_error; }

int b200attn_pick_splits(const B200AttnShape* shape, int max_seq_len, int num_sms, int variant) {
  Geometry g;
  int rc = resolve(shape, &g);
  if (rc) return rc;
  if (max_seq_len < 0) return B200ATTN_ERR_CAPACITY;
  if (num_sms < 1) num_sms = device_sms();
  const int v = resolve_variant(variant, g);
  if (v < 0) return v;
  return pick(g, v, max_seq_len, num_sms);
}

int b200attn_resolve_variant(const B200AttnShape* shape, int variant) {
  Geometry g;
  int rc = resolve(shape, &g);
  if (rc) return rc;
  return resolve_variant(variant, g);
}

int b200attn_workspace_bytes(const B200AttnShape* shape, int num_splits, int variant, size_t* bytes) {
  Geometry g;
  int rc = resolve(shape, &g);
  if (rc) return rc;
  if (!bytes) return B200ATTN_ERR_NULL;
  if (num_splits < 1 || num_splits > 65535) return B200ATTN_ERR_SPLITS;
  const int v = resolve_variant(variant, g);
  if (v < 0) return v;
  *bytes = v == B200ATTN_VARIANT_SIMT ? simt_workspace_bytes(g, num_splits) : mma_workspace_bytes(g, num_splits);
  return B200ATTN_OK;
}

int b200attn_workspace_init(void* workspace, size_t workspace_bytes, void* stream) {
  if (!workspace) return B200ATTN_ERR_NULL;
  cudaError_t e = cudaMemsetAsync(workspace, 0, workspace_bytes, (cudaStream_t)stream);
  return e == cudaSuccess ? B200ATTN_OK : cuda_fail(e);
}

int b200attn_kv_quant_append_bulk(const B200AttnShape* shape, int n_tokens,
                                  const void* k_new, const void* v_new, void* k_cache, void* v_cache,
                                  float* k_scale, float* v_scale, int* seq_pos, int advance_pos,
                                  int* status, void* stream) {
  Geometry g;
  int rc = resolve(shape, &g);
  if (rc) return rc;
  if (!k_new || !v_new || !k_cache || !v_cache || !k_scale || !v_scale || !seq_pos || !status) return B200ATTN_ERR_NULL;
  if (n_tokens < 1 || n_tokens > g.capacity) return B200ATTN_ERR_CAPACITY;
  if (!aligned16(k_new) || !aligned16(v_new) || !aligned16(k_cache) || !aligned16(v_cache)) return B200ATTN_ERR_ALIGN;
  cudaError_t e = launch_append(g, n_tokens, k_new, v_new, k_cache, v_cache, k_scale, v_scale, seq_pos,
                                advance_pos, status, (cudaStream_t)stream);
  return e == cudaSuccess ? B200ATTN_OK : cuda_fail(e);
}

int b200attn_kv_quant_append(const B200AttnShape* shape, const void* k_new, const void* v_new,
                             void* k_cache, void* v_cache, float* k_scale, float* v_scale,
                             int* seq_pos, int advance_pos, int* status, void* stream) {
  return b200attn_kv_quant_append_bulk(shape, 1, k_new, v_new, k_cache, v_cache, k_scale, v_scale, seq_pos,
                                       advance_pos, status, stream);
}

// The fused step of the all-tcgen05 variant: new-token rows quantised into the cache and positions
// advanced by the attention launch itself.
struct FusedStep {
  const void* k_new;
  const void* v_new;
  int* seq_pos;               // null = do not advance
  void* const* barrier_flags; // null = no cross-GPU barrier at the end of the launch
};

}  // extern "C"

// The argument checks of b200attn_decode that need no workspace yet: shape, pointers, alignment, kernel
// choice and split count.  Fills in the geometry, the resolved kernel, the split count (0 = the
// default) and the workspace bytes that choice needs.  Shared with the entry point that brings its
// own scratch, which must know all of this before it touches that scratch.
int b200attn::decode_precheck(const B200AttnShape* shape, const void* q, const void* k_cache, const void* v_cache,
                              const float* k_scale, const float* v_scale, const int* seq_len, const void* out,
                              bool has_peers, const int* status, int variant, int* num_splits, Geometry* g,
                              int* resolved, size_t* need) {
  int rc = resolve(shape, g);
  if (rc) return rc;
  if (!q || !k_cache || !v_cache || !k_scale || !v_scale || !seq_len || (!out && !has_peers) || !status) return B200ATTN_ERR_NULL;
  if (!aligned16(q) || !aligned16(k_cache) || !aligned16(v_cache) || !aligned16(out)) return B200ATTN_ERR_ALIGN;
  const int v = resolve_variant(variant, *g);
  if (v < 0) return v;
  if (*num_splits == 0) *num_splits = pick(*g, v, g->capacity, device_sms());
  if (*num_splits < 1 || *num_splits > 65535) return B200ATTN_ERR_SPLITS;
  *resolved = v;
  *need = v == B200ATTN_VARIANT_SIMT ? simt_workspace_bytes(*g, *num_splits) : mma_workspace_bytes(*g, *num_splits);
  return B200ATTN_OK;
}

extern "C" {

static int decode_impl(const B200AttnShape* shape, const B200AttnPeerOut* peers, const void* q, const void* gate, const void* k_cache,
                       const void* v_cache, const float* k_scale, const float* v_scale, const int* seq_len,
                       int seq_len_offset, float softmax_scale, int variant, int num_splits, void* workspace,
                       size_t workspace_bytes, void* out, int* status, void* stream, const FusedStep* fused = nullptr) {
  Geometry g;
  int v = 0;
  size_t need = 0;
  int rc = decode_precheck(shape, q, k_cache, v_cache, k_scale, v_scale, seq_len, out, peers != nullptr, status, variant,
                           &num_splits, &g, &v, &need);
  if (rc) return rc;
  const bool needs_ws = !(v == B200ATTN_VARIANT_SIMT && num_splits == 1);
  if (needs_ws) {
    if (!workspace) return B200ATTN_ERR_NULL;
    if (!aligned16(workspace)) return B200ATTN_ERR_ALIGN;
    if (workspace_bytes < need) return B200ATTN_ERR_WORKSPACE;
  }
  if (gate && (v == B200ATTN_VARIANT_SIMT || !aligned16(gate))) return v == B200ATTN_VARIANT_SIMT ? B200ATTN_ERR_VARIANT : B200ATTN_ERR_ALIGN;
  DecodeArgs a{q, k_cache, v_cache, k_scale, v_scale, seq_len, seq_len_offset, softmax_scale,
               num_splits, workspace, workspace_bytes, out, status, gate, 0, 0, 0, {}};
  if (fused) {
    if (v != B200ATTN_VARIANT_UMMA2 && v != B200ATTN_VARIANT_MMA) return B200ATTN_ERR_VARIANT;
    a.k_new = fused->k_new;
    a.v_new = fused->v_new;
    a.seq_pos = fused->seq_pos;
    if (fused->barrier_flags) {
      if (!peers) return B200ATTN_ERR_NULL;
      for (int r = 0; r < peers->n_peers; ++r) {
        if (!fused->barrier_flags[r]) return B200ATTN_ERR_NULL;
        a.bar_flags[r] = (int*)fused->barrier_flags[r];
      }
      a.bar_rank = peers->rank;
      a.bar_world = peers->n_peers;
    }
  }
  if (peers) {
    if (v == B200ATTN_VARIANT_SIMT) return B200ATTN_ERR_VARIANT;
    a.n_out = peers->n_peers;
    a.out_hq_total = peers->h_q_total;
    a.out_head_base = peers->rank * g.h_q;
    rc = check_peers(peers, g);
    if (rc) return rc;
    if (peers->mode == B200ATTN_GATHER_PACKETS) {
      // this rank's slots in the other ranks' staging buffers ([2 parities][n_peers slots][slot]), its own staging
      // buffer to unpack from, its own gathered tensor
      if (fused && fused->barrier_flags) return B200ATTN_ERR_SHAPE;   // packets need no barrier and must not be mixed with one
      const size_t slot = staging_slot_bytes(g);
      if ((unsigned long long)peers->n_peers * (slot / 8) >= 0x7fffffffull) return B200ATTN_ERR_SHAPE;   // 32-bit packet indices
      for (int r = 0; r < peers->n_peers; ++r) {
        char* base = r == peers->rank ? nullptr : (char*)peers->staging[r] + (size_t)peers->rank * slot;
        a.out_peer[r] = base;
        a.out_peer_alt[r] = base ? base + (size_t)peers->n_peers * slot : nullptr;
      }
      a.pkt_src = peers->staging[peers->rank];
      a.out = peers->out[peers->rank];
      a.epoch = peers->step;
    } else {
      for (int r = 0; r < peers->n_peers; ++r) {
        a.out_peer[r] = peers->out[r];
        a.out_peer_alt[r] = peers->mode == B200ATTN_GATHER_STORES_2BUF ? peers->out_alt[r] : peers->out[r];
      }
      a.epoch = peers->mode == B200ATTN_GATHER_STORES_2BUF ? peers->step : nullptr;
    }
  }
  cudaError_t e = v == B200ATTN_VARIANT_SIMT ? launch_decode_simt(g, a, (cudaStream_t)stream)
                                             : v == B200ATTN_VARIANT_UMMA2 ? launch_decode_umma2(g, a, (cudaStream_t)stream)
                                             : launch_decode_mma(g, a, (cudaStream_t)stream);
  return e == cudaSuccess ? B200ATTN_OK : cuda_fail(e);
}

int b200attn_decode(const B200AttnShape* shape, const void* q, const void* k_cache, const void* v_cache,
                    const float* k_scale, const float* v_scale, const int* seq_len, int seq_len_offset,
                    float softmax_scale, int variant, int num_splits, void* workspace,
                    size_t workspace_bytes, void* out, int* status, void* stream) {
  return decode_impl(shape, nullptr, q, nullptr, k_cache, v_cache, k_scale, v_scale, seq_len, seq_len_offset, softmax_scale,
                     variant, num_splits, workspace, workspace_bytes, out, status, stream);
}

int b200attn_decode_gated(const B200AttnShape* shape, const void* q, const void* gate, const void* k_cache,
                          const void* v_cache, const float* k_scale, const float* v_scale, const int* seq_len,
                          int seq_len_offset, float softmax_scale, int variant, int num_splits, void* workspace,
                          size_t workspace_bytes, void* out, int* status, void* stream) {
  if (!gate) return B200ATTN_ERR_NULL;
  return decode_impl(shape, nullptr, q, gate, k_cache, v_cache, k_scale, v_scale, seq_len, seq_len_offset, softmax_scale,
                     variant, num_splits, workspace, workspace_bytes, out, status, stream);
}

int b200attn_decode_peers(const B200AttnShape* shape, const B200AttnPeerOut* peers, const void* q,
                          const void* k_cache, const void* v_cache, const float* k_scale, const float* v_scale,
                          const int* seq_len, int seq_len_offset, float softmax_scale, int variant, int num_splits,
                          void* workspace, size_t workspace_bytes, int* status, void* stream) {
  if (!peers) return B200ATTN_ERR_NULL;
  return decode_impl(shape, peers, q, nullptr, k_cache, v_cache, k_scale, v_scale, seq_len, seq_len_offset, softmax_scale,
                     variant, num_splits, workspace, workspace_bytes, nullptr, status, stream);
}

size_t b200attn_peer_staging_bytes(const B200AttnShape* shape, int n_peers) {
  Geometry g;
  if (resolve(shape, &g) || n_peers < 1 || n_peers > 8) return 0;
  return 2 * (size_t)n_peers * staging_slot_bytes(g);
}

int b200attn_peer_barrier(void* const* flags, int rank, int world, int* status, void* stream) {
  if (!flags || !status) return B200ATTN_ERR_NULL;
  if (world < 1 || world > 8 || rank < 0 || rank >= world) return B200ATTN_ERR_SHAPE;
  for (int r = 0; r < world; ++r) if (!flags[r]) return B200ATTN_ERR_NULL;
  cudaError_t e = launch_peer_barrier(reinterpret_cast<int* const*>(flags), rank, world, status, (cudaStream_t)stream);
  return e == cudaSuccess ? B200ATTN_OK : cuda_fail(e);
}

static int step_impl(const B200AttnShape* shape, const B200AttnPeerOut* peers, const void* q, const void* k_new, const void* v_new,
                     void* k_cache, void* v_cache, float* k_scale, float* v_scale, int* seq_pos,
                     int advance_pos, float softmax_scale, int variant, int num_splits,
                     void* workspace, size_t workspace_bytes, void* out, int* status, void* stream,
                     void* const* barrier_flags = nullptr) {
  // Validate everything before the first launch so that an argument error launches nothing.
  Geometry g;
  int rc = resolve(shape, &g);
  if (rc) return rc;
  if (!q || (!out && !peers) || !seq_pos || !status) return B200ATTN_ERR_NULL;
  if (peers) {
    rc = check_peers(peers, g);
    if (rc) return rc;
  }
  const int v = resolve_variant(variant, g);
  if (v < 0) return v;
  if (num_splits == 0)
    num_splits = pick(g, v, g.capacity, device_sms());
  if (num_splits < 1 || num_splits > 65535) return B200ATTN_ERR_SPLITS;
  const size_t need = v == B200ATTN_VARIANT_SIMT ? simt_workspace_bytes(g, num_splits) : mma_workspace_bytes(g, num_splits);
  if (!(v == B200ATTN_VARIANT_SIMT && num_splits == 1)) {
    if (!workspace) return B200ATTN_ERR_NULL;
    if (workspace_bytes < need) return B200ATTN_ERR_WORKSPACE;
  }
  if (!aligned16(q) || !aligned16(out) || !aligned16(workspace)) return B200ATTN_ERR_ALIGN;
  if (v == B200ATTN_VARIANT_UMMA2 || (v == B200ATTN_VARIANT_MMA && g.scale_mode == B200ATTN_SCALE_PER_HEAD)) {
    // one launch: the attention kernel appends the new rows (per-token layout: and computes their scales) and
    // advances the positions itself, and ends with the cross-GPU barrier when one is asked for
    if (!k_new || !v_new || !k_cache || !v_cache || !k_scale || !v_scale) return B200ATTN_ERR_NULL;
    if (!aligned16(k_new) || !aligned16(v_new) || !aligned16(k_cache) || !aligned16(v_cache)) return B200ATTN_ERR_ALIGN;
    const FusedStep fused{k_new, v_new, advance_pos ? seq_pos : nullptr, barrier_flags};
    return decode_impl(shape, peers, q, nullptr, k_cache, v_cache, k_scale, v_scale, seq_pos, 1, softmax_scale, v, num_splits,
                       workspace, workspace_bytes, out, status, stream, &fused);
  }
  if (peers && v == B200ATTN_VARIANT_SIMT) return B200ATTN_ERR_VARIANT;
  rc = b200attn_kv_quant_append_bulk(shape, 1, k_new, v_new, k_cache, v_cache, k_scale, v_scale, seq_pos, 0,
                                     status, stream);
  if (rc) return rc;
  rc = decode_impl(shape, peers, q, nullptr, k_cache, v_cache, k_scale, v_scale, seq_pos, 1, softmax_scale, v, num_splits,
                   workspace, workspace_bytes, out, status, stream);
  if (rc) return rc;
  if (advance_pos) {
    cudaError_t e = launch_advance_pos(g, 1, seq_pos, (cudaStream_t)stream);
    if (e != cudaSuccess) return cuda_fail(e);
  }
  if (barrier_flags) return b200attn_peer_barrier(barrier_flags, peers->rank, peers->n_peers, status, stream);
  return B200ATTN_OK;
}

int b200attn_append_decode(const B200AttnShape* shape, const void* q, const void* k_new, const void* v_new,
                           void* k_cache, void* v_cache, float* k_scale, float* v_scale, int* seq_pos,
                           int advance_pos, float softmax_scale, int variant, int num_splits,
                           void* workspace, size_t workspace_bytes, void* out, int* status, void* stream) {
  if (!out) return B200ATTN_ERR_NULL;
  return step_impl(shape, nullptr, q, k_new, v_new, k_cache, v_cache, k_scale, v_scale, seq_pos, advance_pos, softmax_scale,
                   variant, num_splits, workspace, workspace_bytes, out, status, stream);
}

int b200attn_append_decode_peers(const B200AttnShape* shape, const B200AttnPeerOut* peers, const void* q, const void* k_new,
                                 const void* v_new, void* k_cache, void* v_cache, float* k_scale, float* v_scale,
                                 int* seq_pos, int advance_pos, float softmax_scale, int variant, int num_splits,
                                 void* workspace, size_t workspace_bytes, void* const* barrier_flags, int* status,
                                 void* stream) {
  if (!peers) return B200ATTN_ERR_NULL;
  if (barrier_flags)
    for (int r = 0; r < peers->n_peers && r < 8; ++r)
      if (!barrier_flags[r]) return B200ATTN_ERR_NULL;
  return step_impl(shape, peers, q, k_new, v_new, k_cache, v_cache, k_scale, v_scale, seq_pos, advance_pos, softmax_scale,
                   variant, num_splits, workspace, workspace_bytes, nullptr, status, stream, barrier_flags);
}

int b200attn_qk_norm_rope_append(const B200AttnShape* shape, const void* q_raw, const void* k_raw, const void* v_new,
                                 const void* q_norm_weight, const void* k_norm_weight, float eps, const void* cos,
                                 const void* sin, int rotary_dim, void* q_out, void* k_out, void* k_cache, void* v_cache,
                                 float* k_scale, float* v_scale, int* seq_pos, int advance_pos, int* status, void* stream) {
  Geometry g;
  int rc = resolve(shape, &g);
  if (rc) return rc;
  if (!q_raw || !k_raw || !v_new || !q_norm_weight || !k_norm_weight || !cos || !sin || !q_out || !k_cache || !v_cache ||
      !k_scale || !v_scale || !seq_pos || !status)
    return B200ATTN_ERR_NULL;
  // the rotated half must be a whole number of lanes away: rotary_dim a multiple of 2 * head_dim / 32
  if (rotary_dim < 0 || rotary_dim > g.head_dim || rotary_dim % (2 * (g.head_dim / 32)) != 0) return B200ATTN_ERR_SHAPE;
  if (!(eps >= 0.f)) return B200ATTN_ERR_SHAPE;
  if (!aligned16(q_raw) || !aligned16(k_raw) || !aligned16(v_new) || !aligned16(q_out) || !aligned16(k_out) ||
      !aligned16(k_cache) || !aligned16(v_cache))
    return B200ATTN_ERR_ALIGN;
  cudaError_t e = launch_producer(g, rotary_dim, eps, q_raw, k_raw, v_new, q_norm_weight, k_norm_weight, cos, sin, q_out,
                                  k_out, k_cache, v_cache, k_scale, v_scale, seq_pos, advance_pos, status,
                                  (cudaStream_t)stream);
  return e == cudaSuccess ? B200ATTN_OK : cuda_fail(e);
}

int b200attn_dequant_prefix(const B200AttnShape* shape, int n_tokens, const void* cache, long long layer_stride,
                            const float* scale, void* out, void* stream) {
  Geometry g;
  int rc = resolve(shape, &g);
  if (rc) return rc;
  if (!cache || !scale || !out) return B200ATTN_ERR_NULL;
  if (n_tokens < 0 || n_tokens > g.capacity) return B200ATTN_ERR_CAPACITY;
  if (!aligned16(cache) || !aligned16(out) || (layer_stride & 15)) return B200ATTN_ERR_ALIGN;
  if (layer_stride == 0) layer_stride = (long long)g.batch * g.h_kv * g.capacity * g.head_dim;
  cudaError_t e = launch_dequant_prefix(g, n_tokens, cache, layer_stride, scale, out, (cudaStream_t)stream);
  return e == cudaSuccess ? B200ATTN_OK : cuda_fail(e);
}

int b200attn_calibrate_scales(const B200AttnShape* shape, int n_tokens, const void* x, float* scale, void* stream) {
  Geometry g;
  int rc = resolve(shape, &g);
  if (rc) return rc;
  if (!x || !scale) return B200ATTN_ERR_NULL;
  if (n_tokens < 1) return B200ATTN_ERR_CAPACITY;
  if (!aligned16(x)) return B200ATTN_ERR_ALIGN;
  cudaError_t e = launch_calibrate(g, n_tokens, x, scale, (cudaStream_t)stream);
  return e == cudaSuccess ? B200ATTN_OK : cuda_fail(e);
}

}  // extern "C"
