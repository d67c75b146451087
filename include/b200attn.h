/*
 * b200attn — C-ABI of the B200 (sm_100a) decode-attention library.
 *
 * One hot path of xzzqqq/qwen38-5080 is replaced: bs=1 / batched decode attention over an
 * FP8-e4m3 static KV cache — (A) quantize-and-append of the step's K/V, (B) split-K GQA
 * attention partials, (C) log-sum-exp combine.  Every entry point takes plain pointers and
 * sizes; device pointers belong to the caller (torch tensors on the Python side), `stream`
 * is a cudaStream_t passed as void*, and every call is asynchronous on that stream: no host
 * synchronisation, no host read of device state, no allocation.  That makes a call sequence
 * CUDA-graph capturable as the reference's graph runner requires
 * (runner/model/graph_runner.py:127-198: fixed addresses, device-side position).
 *
 * Return value: 0 = launched; <0 = host-side argument error, nothing launched (the
 * counterpart of the reference's "reject before submitting kernels" capacity guard,
 * runner/model/decode_runner.py:323-332).  Soft errors seen on the device (position at
 * capacity, sequence length beyond capacity, a bounded wait that ran out) are OR-ed into
 * the caller's `status` word as B200ATTN_STATUS_* bits; the kernel then skips the
 * offending access and returns normally.
 */
#ifndef B200ATTN_H
#define B200ATTN_H

#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

#define B200ATTN_VERSION 100

/* host-side error codes */
#define B200ATTN_OK                 0
#define B200ATTN_ERR_NULL          -1   /* a required pointer is NULL */
#define B200ATTN_ERR_SHAPE         -2   /* unsupported head shape / group size / head_dim */
#define B200ATTN_ERR_ALIGN         -3   /* pointer or stride not 16-byte aligned */
#define B200ATTN_ERR_WORKSPACE     -4   /* workspace too small for the requested split count */
#define B200ATTN_ERR_SPLITS        -5   /* split count out of range */
#define B200ATTN_ERR_CUDA          -6   /* a CUDA runtime / driver call failed (see b200attn_last_cuda_error) */
#define B200ATTN_ERR_CAPACITY      -7   /* host-known length exceeds capacity */
#define B200ATTN_ERR_VARIANT       -8   /* unknown kernel variant */
#define B200ATTN_ERR_TOO_LARGE     -9   /* request exceeds the fixed scratch of b200attn_decode_static */

/* device status bits (OR-ed into *status) */
#define B200ATTN_STATUS_POS_AT_CAPACITY  1  /* append skipped: seq_pos[b] >= capacity */
#define B200ATTN_STATUS_LEN_OVER_CAP     2  /* seq_len[b] > capacity: clamped to capacity */
#define B200ATTN_STATUS_WAIT_TIMEOUT     4  /* a bounded wait on a copy barrier ran out */
#define B200ATTN_STATUS_LEN_NEGATIVE     8  /* seq_len[b] < 0: treated as 0 */
#define B200ATTN_STATUS_BOUNDS          16  /* index-checking build only (-DB200ATTN_BOUNDS=1): a kernel computed an index
                                               outside its buffer (reported, never trapped) */

/* kernel variants for b200attn_decode */
#define B200ATTN_VARIANT_AUTO     0   /* the library's default (the fastest validated variant) */
#define B200ATTN_VARIANT_SIMT     1   /* CUDA-core split-K partial kernel + separate combine kernel */
#define B200ATTN_VARIANT_MMA      2   /* TMA/mbarrier staged, tensor-core (mma.sync f16) stream-K kernel with fused combine */
/* 3 is retired (an intermediate kernel with only the score product on tcgen05): B200ATTN_ERR_VARIANT */
#define B200ATTN_VARIANT_UMMA2    4   /* both products on tcgen05.mma: S = K q^T and O += V^T P^T read the staged FP8 tiles
                                         directly (V as an MN-major operand), scores and the output accumulator live in
                                         tensor memory; both scale layouts */

/* scale granularity of the FP8 cache */
#define B200ATTN_SCALE_PER_HEAD   0   /* fp32 scale per (layer, kv_head): [n_layers][h_kv] */
#define B200ATTN_SCALE_PER_TOKEN  1   /* fp32 scale per (layer, seq, token, kv_head): [n_layers][batch][capacity][h_kv]
                                         — the layout the reference froze,
                                         docs/journal/2026-10-23-phase2-r3-coordinator.md:46-48 */

/*
 * Geometry of one call.  The cache is the FP8 counterpart of the reference's static cache
 * (runner/model/static_cache.py:135-158: keys/values [B, H_kv, capacity, D], fixed address,
 * zero-initialised), stacked over layers:
 *     k_cache / v_cache : u8 [n_layers][batch][h_kv][capacity][head_dim]   (e4m3fn bytes)
 * `k_layer_stride` / `v_layer_stride` are the byte distances between consecutive layers
 * (0 means dense = batch*h_kv*capacity*head_dim), so that per-layer tensors allocated
 * separately can be driven with n_layers = 1 and offset base pointers.
 * Tensor-parallel sharding by KV head is expressed by passing the local h_kv / h_q.
 */
typedef struct B200AttnShape {
  int n_layers;      /* 64 (the benchmark), 16 (the reference model), or 1 for the per-layer drop-in */
  int batch;         /* sequences, >= 1 */
  int h_q;           /* query heads (40 | 24); must be a multiple of h_kv, group size <= 8 */
  int h_kv;          /* KV heads (8 | 4) */
  int head_dim;      /* 128 or 256 */
  int capacity;      /* token slots per sequence */
  int scale_mode;    /* B200ATTN_SCALE_* */
  int reserved;      /* must be 0 */
  long long k_layer_stride;
  long long v_layer_stride;
} B200AttnShape;

/*
 * Output placement for KV-head tensor parallelism (no counterpart in the reference, which is
 * single-GPU): rank `rank` of `n_peers` computes h_q of the h_q_total query heads, and the
 * all-gather of the per-head outputs into bf16 [n_layers][batch][h_q_total][head_dim] on every rank
 * is done by the attention kernel itself, over NVLink peer memory (symmetric / peer-mapped buffers;
 * plain stores and loads only).  Three ways, `mode`:
 *
 * B200ATTN_GATHER_PACKETS — the fast one.  Every result leaves as an 8-byte packet {two bf16 values,
 *   step number} stored into the receiving rank's staging buffer, and at its end every CTA of a launch
 *   copies a share of the packets that arrived for this rank into this rank's own gathered tensor
 *   out[rank], waiting for each packet's step number.  Value and number travel in one store, so there
 *   is no fence, no flag and no barrier: when the launch is complete the gathered tensor is, and a
 *   rank that is a step ahead only ever writes staging, never a tensor a consumer may still be
 *   reading.  staging[r] is rank r's staging buffer as addressable from this GPU
 *   (b200attn_peer_staging_bytes() bytes each, zero-initialised); `step` is one int32 of this rank's
 *   device memory, zero at the start, advanced by every launch (all ranks must make the same calls in
 *   the same order).  The waits are bounded (1 s, B200ATTN_STATUS_WAIT_TIMEOUT).
 * B200ATTN_GATHER_STORES — every result is stored directly into every rank's gathered tensor out[r]
 *   at head offset rank*h_q; b200attn_peer_barrier (or the barrier_flags of
 *   b200attn_append_decode_peers) then makes the stores visible.  A tensor must not be rewritten by a
 *   later step while a slower rank still reads it.
 * B200ATTN_GATHER_STORES_2BUF — the same with two gathered tensors per rank used in turn, so that a
 *   fast rank's next step cannot touch what a slow rank's consumer still reads.  Which one a launch
 *   writes is decided on the device from the step counter the cross-GPU barrier keeps (`step` = word
 *   [n_peers] of this rank's flag buffer, see b200attn_peer_barrier): the launch that finds e there
 *   writes out[] when e + 1 is even and out_alt[] when it is odd, and the barrier that follows makes
 *   the counter e + 1.  Every step must be followed by exactly one barrier.
 */
#define B200ATTN_GATHER_STORES       1   /* 0 means the same */
#define B200ATTN_GATHER_STORES_2BUF  2
#define B200ATTN_GATHER_PACKETS      3
typedef struct B200AttnPeerOut {
  int n_peers;       /* 1..8 */
  int rank;          /* this rank */
  int h_q_total;     /* = n_peers * shape->h_q */
  int mode;          /* B200ATTN_GATHER_* */
  void* out[8];      /* gathered tensors; PACKETS reads out[rank] only */
  void* out_alt[8];  /* STORES_2BUF: every rank's second gathered tensor */
  void* staging[8];  /* PACKETS: every rank's staging buffer */
  int* step;         /* STORES_2BUF, PACKETS: this rank's step counter (device memory) */
} B200AttnPeerOut;

/* Bytes of one rank's staging buffer for B200ATTN_GATHER_PACKETS (shape = the per-rank shape). */
size_t b200attn_peer_staging_bytes(const B200AttnShape* shape, int n_peers);

/* Library version (B200ATTN_VERSION of the build). */
int b200attn_version(void);

/* 1 if this is the index-checking build (-DB200ATTN_BOUNDS=1), else 0. */
int b200attn_bounds_checked(void);

/* Hash of the sources the library was compiled from ("" for a build that did not record one); a
 * loader compares it with the sources beside the library to refuse a stale binary. */
const char* b200attn_source_hash(void);

/* Text for a host-side error code. */
const char* b200attn_error_string(int code);

/* Last CUDA error code seen by a failing call on this thread (0 if none). */
int b200attn_last_cuda_error(void);

/*
 * Split count for the SIMT variant / CTA count for the stream-K variant at a given maximum
 * sequence length, chosen to fill `num_sms` SMs (148 on B200).  Pure host function.
 * Replaces the split heuristic of the reference's fused kernel ("one program = (kv_head,
 * split)", docs/journal/2026-10-23-phase2-r3-coordinator.md:140-141).
 */
int b200attn_pick_splits(const B200AttnShape* shape, int max_seq_len, int num_sms, int variant);

/*
 * The kernel variant a request resolves to for this shape: B200ATTN_VARIANT_AUTO becomes the
 * variant the library would run, an explicit variant comes back unchanged, and a variant the
 * shape cannot use is the same negative error b200attn_decode would return.  Pure host function;
 * no counterpart in the reference, whose kernel choice is made by its Python caller.
 */
int b200attn_resolve_variant(const B200AttnShape* shape, int variant);

/*
 * Bytes of workspace b200attn_decode needs for `num_splits` (as returned by
 * b200attn_pick_splits, or larger).  The workspace holds the split-K partials (m, l, acc[G][D] in
 * fp32; the stream-K kernels keep each value in an 8-byte word with a tag that tells the CTA finishing the
 * pair that it has arrived) and the CTA counter of the one-launch step.
 */
int b200attn_workspace_bytes(const B200AttnShape* shape, int num_splits, int variant, size_t* bytes);

/*
 * Zero the workspace (the partial words and the counter must start at zero; a launch that ends without a
 * status error leaves them at zero again).  Call once after allocation, after any call that reported a
 * status error, and before a workspace that served one kernel variant is handed to another.
 */
int b200attn_workspace_init(void* workspace, size_t workspace_bytes, void* stream);

/*
 * A. Quantize-and-append one token per sequence for n_layers layers at once.
 * Replaces StaticCapFullAttentionLayer.update -> StaticLayer.update -> index_copy_
 * (runner/model/static_cache.py:69-77) with the FP8 format frozen in
 * docs/journal/2026-10-23-phase2-r3-coordinator.md:43-49:
 *     byte = e4m3fn_rne( clamp( float(x) / s, -448, 448 ) )
 * written at token slot seq_pos[b].  In B200ATTN_SCALE_PER_HEAD mode `k_scale`/`v_scale`
 * are inputs; in B200ATTN_SCALE_PER_TOKEN mode they are outputs (s = amax|x|/448 over the
 * head's head_dim values, written at [layer][b][seq_pos[b]][head]).
 *   k_new, v_new : bf16 [n_layers][batch][h_kv][head_dim]
 *   seq_pos      : int32 [batch], tokens already cached (device memory)
 *   advance_pos  : 1 -> seq_pos[b] += 1 after all layers were written (the reference's
 *                  cumulative_length.add_, static_cache.py:14-15)
 */
int b200attn_kv_quant_append(const B200AttnShape* shape,
                             const void* k_new_bf16, const void* v_new_bf16,
                             void* k_cache_u8, void* v_cache_u8,
                             float* k_scale, float* v_scale,
                             int* seq_pos, int advance_pos,
                             int* status, void* stream);

/*
 * Prefill-side bulk quantize-append: `n_tokens` consecutive tokens per sequence, written at
 * slots [seq_pos[b], seq_pos[b]+n_tokens).  Counterpart of the reference's q_len>1 update
 * (runner/model/static_cache.py:76-77; prefill chunk 128, runner/model/decode_runner.py:229-235).
 *   k_new, v_new : bf16 [n_layers][batch][h_kv][n_tokens][head_dim]
 */
int b200attn_kv_quant_append_bulk(const B200AttnShape* shape, int n_tokens,
                                  const void* k_new_bf16, const void* v_new_bf16,
                                  void* k_cache_u8, void* v_cache_u8,
                                  float* k_scale, float* v_scale,
                                  int* seq_pos, int advance_pos,
                                  int* status, void* stream);

/*
 * B+C. Decode attention for one query token per sequence: attends token slots
 * [0, seq_len[b] + seq_len_offset) of sequence b.  Replaces repeat_kv + eager attention
 * (bench/micro/attn_length_effect.py:41-66, the reference's replica of transformers'
 * eager_attention_forward) together with the capacity-length mask of
 * StaticCapFullAttentionLayer.get_mask_sizes (runner/model/static_cache.py:79-82): slots
 * at or beyond the valid length never influence the result, whatever bytes they hold.
 *   q            : bf16 [n_layers][batch][h_q][head_dim]
 *   k_scale,v_scale : fp32, layout by shape->scale_mode
 *   seq_len      : int32 [batch] on the device
 *   seq_len_offset : added to every seq_len[b] (pass seq_pos with offset 1 to attend the
 *                  token appended in the same step without bumping seq_pos first)
 *   softmax_scale: head_dim^-0.5
 *   num_splits   : from b200attn_pick_splits (0 = pick for capacity and 148 SMs)
 *   out          : bf16 [n_layers][batch][h_q][head_dim]  (the reference's
 *                  out.transpose(1,2).contiguous() layout, attn_length_effect.py:66)
 * The tensor-core kernels are launched with programmatic stream serialization: their thread blocks
 * may become resident while the previous kernel of the stream is finishing and wait for its
 * completion on the device before they read anything.  Nothing changes for the caller: stream order
 * holds, and the launch is captured into CUDA graphs like any other.
 */
int b200attn_decode(const B200AttnShape* shape,
                    const void* q_bf16,
                    const void* k_cache_u8, const void* v_cache_u8,
                    const float* k_scale, const float* v_scale,
                    const int* seq_len, int seq_len_offset,
                    float softmax_scale,
                    int variant, int num_splits,
                    void* workspace, size_t workspace_bytes,
                    void* out_bf16,
                    int* status, void* stream);

/*
 * b200attn_decode with the consumer-side fusion of the reference's attention block:
 *     out = bf16( bf16(attention) * bf16(sigmoid(gate)) )
 * i.e. `attn_output * sigmoid(gate)` with its two separate bf16 roundings
 * (docs/journal/2026-10-23-phase2-r3-coordinator.md:147-150).  Tensor-core variants only.
 *   gate : bf16 [n_layers][batch][h_q][head_dim]
 */
int b200attn_decode_gated(const B200AttnShape* shape,
                          const void* q_bf16, const void* gate_bf16,
                          const void* k_cache_u8, const void* v_cache_u8,
                          const float* k_scale, const float* v_scale,
                          const int* seq_len, int seq_len_offset,
                          float softmax_scale,
                          int variant, int num_splits,
                          void* workspace, size_t workspace_bytes,
                          void* out_bf16,
                          int* status, void* stream);

/*
 * b200attn_decode whose output all-gather is fused into the kernel (see B200AttnPeerOut).
 * Tensor-core variants only.  In packet mode the gathered tensor is complete when the call is; in
 * the stores modes follow it, on the same stream, with b200attn_peer_barrier before anything reads
 * the gathered tensor.
 */
int b200attn_decode_peers(const B200AttnShape* shape, const B200AttnPeerOut* peers,
                          const void* q_bf16,
                          const void* k_cache_u8, const void* v_cache_u8,
                          const float* k_scale, const float* v_scale,
                          const int* seq_len, int seq_len_offset,
                          float softmax_scale,
                          int variant, int num_splits,
                          void* workspace, size_t workspace_bytes,
                          int* status, void* stream);

/*
 * The decode step of b200attn_append_decode with the gathered output of b200attn_decode_peers:
 * append this rank's new K/V rows, attend seq_pos[b]+1 tokens, store the results into every
 * rank's gathered buffer, advance seq_pos if advance_pos.  One launch with the stream-K
 * kernels, three otherwise.  Packet mode: barrier_flags must be NULL, the launch itself waits for
 * the other ranks' packets.  Stores modes: with barrier_flags == NULL, follow it with
 * b200attn_peer_barrier as for b200attn_decode_peers; with barrier_flags (the flag buffers
 * b200attn_peer_barrier takes) the cross-GPU arrive-and-wait is part of the call: done by the
 * last CTA of the attention launch with the stream-K kernels, by the barrier kernel launched
 * behind the attention otherwise; same bounded wait and status bit.
 * (The reference has no multi-GPU path: no counterpart there.)
 */
int b200attn_append_decode_peers(const B200AttnShape* shape, const B200AttnPeerOut* peers,
                                 const void* q_bf16, const void* k_new_bf16, const void* v_new_bf16,
                                 void* k_cache_u8, void* v_cache_u8,
                                 float* k_scale, float* v_scale,
                                 int* seq_pos, int advance_pos,
                                 float softmax_scale,
                                 int variant, int num_splits,
                                 void* workspace, size_t workspace_bytes,
                                 void* const* barrier_flags,
                                 int* status, void* stream);

/*
 * Cross-GPU arrive-and-wait.  flags[r] = rank r's flag buffer (int32[24], zero-initialised,
 * symmetric / peer-mapped memory) as addressable from this GPU: words [0, world) are the arrival
 * epochs the ranks write, word [world] is the owner's epoch (= step) counter, words [16..19] hold two
 * 64-bit %globaltimer stamps of the owner's latest arrive-and-wait (arrival, end of the wait), there
 * for whoever wants to know how long a rank waited for the others.  Every rank launches it once per
 * step; it returns when all ranks have arrived.  The wait is bounded (1 s): on expiry
 * B200ATTN_STATUS_WAIT_TIMEOUT is OR-ed into *status and the kernel returns.  Graph-replayable:
 * the epoch counter lives in the flag buffer.
 */
int b200attn_peer_barrier(void* const* flags, int rank, int world, int* status, void* stream);

/*
 * b200attn_decode without a caller workspace (no counterpart in the reference: its fused kernel
 * takes its scratch from torch's allocator).  For hosts that may not allocate device memory where
 * they call the library — memory owned and budgeted by a framework pool, or a step that cannot
 * afford cudaMalloc's device synchronisation.  The split-K partials of the tensor-core
 * stream-K kernel (B200ATTN_VARIANT_MMA) live in a fixed 8 MiB array inside the library image
 * (b200attn_static_scratch_bytes()), held by every GPU that loads the library until exit.
 *   - a request whose workspace would not fit returns B200ATTN_ERR_TOO_LARGE, nothing launched
 *     (fits: 64 layers x bs 1 with the default CTA count; check b200attn_workspace_bytes);
 *   - all calls on a GPU share the array: calls that overlap on the device race — serialise them;
 *   - the first call on each device looks up the array's device address; make that first call
 *     before any stream capture;
 *   - nothing is allocated or freed, here or in any routine it calls.
 * Arguments as b200attn_decode, minus variant / workspace.
 */
int b200attn_decode_static(const B200AttnShape* shape,
                           const void* q_bf16,
                           const void* k_cache_u8, const void* v_cache_u8,
                           const float* k_scale, const float* v_scale,
                           const int* seq_len, int seq_len_offset,
                           float softmax_scale, int num_splits,
                           void* out_bf16,
                           int* status, void* stream);

/* Size in bytes of the fixed scratch array behind b200attn_decode_static. */
size_t b200attn_static_scratch_bytes(void);

/*
 * Producer side of the attention block fused with A: head-dim RMS norm of the query and key
 * heads (weight 1 + w, fp32 inside, one bf16 rounding), rotary embedding on the first
 * rotary_dim dims in bf16 arithmetic (two rounded products, one rounded sum), then the rotated
 * key and the value are quantised and appended at seq_pos exactly as b200attn_kv_quant_append
 * does; the rotated query is written for the attention call.  These are the steps between the
 * projections and the cache update / attention call of the attention block the reference runs
 * (transformers' Qwen3.5 model: q_norm, k_norm, apply_rotary_pos_emb; loaded by
 * runner/loader/nvfp4_model.py:82-88, rotary module rebuilt at :145) and the producer half of
 * the elementwise work the reference lists around its fused attention
 * (docs/journal/2026-10-23-phase2-r3-coordinator.md:147-150).  One launch for all layers.
 *   q_raw  : bf16 [n_layers][batch][h_q][head_dim]   (query half of the q projection)
 *   k_raw, v_new : bf16 [n_layers][batch][h_kv][head_dim]
 *   q_norm_weight, k_norm_weight : bf16 [n_layers][head_dim]
 *   cos, sin : bf16 [batch][rotary_dim] for each sequence's position (shared by all layers)
 *   rotary_dim : 0 .. head_dim, a multiple of head_dim / 16
 *   q_out  : bf16 [n_layers][batch][h_q][head_dim] (may be q_raw)
 *   k_out  : optional bf16 [n_layers][batch][h_kv][head_dim] copy of the rotated key, or NULL
 */
int b200attn_qk_norm_rope_append(const B200AttnShape* shape,
                                 const void* q_raw_bf16, const void* k_raw_bf16, const void* v_new_bf16,
                                 const void* q_norm_weight_bf16, const void* k_norm_weight_bf16, float eps,
                                 const void* cos_bf16, const void* sin_bf16, int rotary_dim,
                                 void* q_out_bf16, void* k_out_bf16,
                                 void* k_cache_u8, void* v_cache_u8,
                                 float* k_scale, float* v_scale,
                                 int* seq_pos, int advance_pos,
                                 int* status, void* stream);

/*
 * Fused convenience for one decode step: A (append at seq_pos) then B+C attending
 * seq_pos[b]+1 tokens, then seq_pos[b] += 1 if advance_pos.  Same stream, no host sync.
 * With the stream-K kernels (B200ATTN_VARIANT_UMMA2 for both scale layouts, B200ATTN_VARIANT_MMA
 * for per-head scales, i.e. whatever AUTO resolves to where a tensor-core kernel applies) the step
 * is ONE launch: the CTA that owns the tile holding a pair's new token quantises that row first
 * (per-token layout: after computing and storing its scale), and the last CTA to have read the
 * positions advances them; the CUDA-core variant launches append, attention and the position kernel one
 * after the other.  Cache bytes, scales, positions and status bits are the same either way.
 */
int b200attn_append_decode(const B200AttnShape* shape,
                           const void* q_bf16,
                           const void* k_new_bf16, const void* v_new_bf16,
                           void* k_cache_u8, void* v_cache_u8,
                           float* k_scale, float* v_scale,
                           int* seq_pos, int advance_pos,
                           float softmax_scale,
                           int variant, int num_splits,
                           void* workspace, size_t workspace_bytes,
                           void* out_bf16,
                           int* status, void* stream);

/*
 * On-demand dequantised view of a cache prefix for reference / prefill use
 * (the reference keeps dequant_kv for exactly these, never on the decode path:
 * docs/journal/2026-10-23-phase2-r3-coordinator.md:162-163):
 *     out_bf16[l][b][h][t][:] = bf16( float(byte) * s )   for t < n_tokens
 *   out : bf16 [n_layers][batch][h_kv][n_tokens][head_dim]
 */
int b200attn_dequant_prefix(const B200AttnShape* shape, int n_tokens,
                            const void* cache_u8, long long layer_stride,
                            const float* scale,
                            void* out_bf16, void* stream);

/*
 * Per-(layer, kv_head) scale calibration over a bf16 prefix on the device:
 *     scale[l][h] = max_{b,t<n_tokens,d} |x| / 448
 *   x : bf16 [n_layers][batch][h_kv][n_tokens][head_dim]
 * (the benchmark's cache is "quantised to FP8-e4m3 with a per-(layer, kv-head) fp32 absmax/448 scale").
 */
int b200attn_calibrate_scales(const B200AttnShape* shape, int n_tokens,
                              const void* x_bf16, float* scale, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* B200ATTN_H */
