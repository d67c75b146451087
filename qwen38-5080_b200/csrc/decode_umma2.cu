// All-tcgen05 variant of the stream-K decode attention: BOTH products run on the 5th-generation
// tensor cores straight from the TMA-staged FP8 tiles; no K or V byte passes through a register.
//
// One persistent CTA per SM, 128-token tiles, twenty warps:
//   1. producer warp: one lane streams K and V tiles with TMA into two shared-memory rings (and the
//      query rows of each pair);
//   2. S issuer warp: S[128 tokens x 16] = K q^T with tcgen05.mma kind::f8f6f4 — the K tile's TMA
//      128-byte-swizzle layout is the K-major canonical operand layout; the query is the B operand
//      as two e4m3 rows per head (leading part + remainder = the bf16 value exactly); scores land
//      in tensor memory (one buffer per softmax group);
//   3. sixteen softmax warps in four groups of four; group = tile index mod 4, each with its own
//      score buffer, probability operand, running state and output accumulators, so four tiles are
//      in flight and tiles are consumed strictly in ring order.  One thread per token: tcgen05.ld of
//      the token's scores, one group-wide reference maximum per head (redux.sync per warp + a
//      shared-memory exchange), p = 2^(s - m_ref).  The reference only moves when a tile's maximum
//      exceeds it by more than kTau (lazy rescale: p stays <= 2^kTau), so the accumulators in
//      tensor memory are rescaled (tcgen05.ld -> multiply -> tcgen05.st) only in the first tiles
//      of a pair;
//   4. the probabilities become the B operand of the second product: p * 2^13 is written as three
//      e5m2 terms (leading 3 significant bits, then the remainder twice: 9 significant bits, the
//      precision class of the reference's bf16 P, with e5m2's range down to 2^-29 of the
//      reference) into a 128-token shared-memory operand (rows 3h..3h+2 for head h);
//   5. P V issuer warp: O[128 dims x rows] += V^T P^T with tcgen05.mma, A = the V tile read
//      MN-major (its swizzled [token][dim] layout is the MN-major canonical layout), accumulating
//      in the group's tensor-memory accumulators over the whole segment; rows beyond the valid
//      length are zeroed in shared memory first (their bytes may be NaN patterns);
//   6. at the end of a segment each group reads its O once (one thread per dim), adds the terms
//      per head, and hands its state (m, l, acc) to the epilogue warp, which merges the four
//      states and writes the output or a split-K partial (tagged words); the CTA that holds a split pair's
//      last piece collects the pair's partials with all its warps when its own range is done.
// The same launch can be the whole decode step: the new token's K/V rows are quantised into the
// cache by the CTA that is going to load the tile that holds them, and the last CTA to have read the
// positions advances them (stores mode, tensor-parallel: the last CTA to finish, which also does the
// cross-GPU arrive-and-wait).
// Query groups of up to 5 heads use 16 probability-operand rows (3 G <= 16), groups of 6 to 8 an instance
// with 32 rows.
//
// All waits are bounded as in the other kernels; tensor memory is allocated by the S issuer warp at
// kernel start and always freed by it after the final barrier.
#include "tcgen05.cuh"

namespace b200attn {

namespace {

constexpr int kTile2 = 128;
constexpr int kGroups2 = 4;                          // softmax groups of four warps; group = tile index mod kGroups2
                                                     // (measured at depth 8192: 2 CTAs x 2 groups 175 us, 1 x 4 169 us)
constexpr int kMaxRingTiles2 = 12;                   // K + V tiles staged per CTA, at most (4 K + 8 V; 3 + 9 and 6 + 6 the same)
constexpr int kSoftmaxWarps2 = 4 * kGroups2;
constexpr int kProducer2 = kSoftmaxWarps2;           // TMA issue
constexpr int kEpilogue2 = kSoftmaxWarps2 + 1;       // merge, output, fused combine
constexpr int kIssuerS2 = kSoftmaxWarps2 + 2;        // query operand, S = K q^T issue, tensor memory owner
constexpr int kIssuerPV2 = kSoftmaxWarps2 + 3;       // O += V^T P^T issue
constexpr int kThreads2 = (kSoftmaxWarps2 + 4) * 32;
constexpr int kQRing2 = 4;                           // query operands / score scales in flight (segments)
constexpr float kTau = 2.0f;                         // lazy-rescale threshold, log2 units
constexpr float kPScale = 8192.f;                    // 2^13: p * 2^13 <= 2^15 < 57344 (e5m2 max)

// D f32, A e4m3 MN-major (V^T), B e5m2 K-major (P^T), N = 16, M = 128
constexpr uint32_t kIdescPV = (1u << 4) | (1u << 10) | (1u << 15) | ((16u >> 3) << 17) | ((128u >> 4) << 24);

__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
        "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]) : "memory");
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}
// Leading part of x that an e5m2 value holds exactly (sign, exponent, top two mantissa bits).
__device__ __forceinline__ float e5m2_head(float x) { return __uint_as_float(__float_as_uint(x) & 0xFFE00000u); }
// Two floats -> two e5m2 bytes: `lo` in the low byte, `hi` in the high byte.
__device__ __forceinline__ uint32_t pack_e5m2x2(float lo, float hi) {
  uint16_t r;
  asm("cvt.rn.satfinite.e5m2x2.f32 %0, %1, %2;" : "=h"(r) : "f"(hi), "f"(lo));
  return (uint32_t)r;
}
__device__ __forceinline__ void sts8(uint32_t addr, uint32_t v) {
  asm volatile("st.shared.u8 [%0], %1;" ::"r"(addr), "r"(v) : "memory");
}
__device__ __forceinline__ void sts128z(uint32_t addr) {
  asm volatile("st.shared.v4.u32 [%0], {%1, %1, %1, %1};" ::"r"(addr), "r"(0u) : "memory");
}
// Named barrier of one softmax group (128 threads): ids 1..kGroups2.
__device__ __forceinline__ void bar_group(int grp) {
  switch (grp) {
    case 0: asm volatile("bar.sync 1, 128;" ::: "memory"); break;
    case 1: asm volatile("bar.sync 2, 128;" ::: "memory"); break;
    case 2: asm volatile("bar.sync 3, 128;" ::: "memory"); break;
    default: asm volatile("bar.sync 4, 128;" ::: "memory"); break;
  }
}


// Shared-memory plan, computed the same way on the host and in the kernel.
struct Plan2 {
  int kstages, vstages;
  size_t bytes;
};
__host__ __device__ inline size_t umma2_fixed_bytes(int group, int head_dim, int batch) {
  const int dh = head_dim / 128;
  size_t b = 1024;                                                   // alignment slack
  b += (size_t)kQRing2 * dh * 16 * 128;                              // query operands
  b += (size_t)kGroups2 * (group <= 5 ? 16 : 32) * 128;              // probability operands
  b += (size_t)2 * group * head_dim * 2;                             // raw query rows
  b += (size_t)(kQRing2 * 8 + kGroups2 * 64 + kGroups2 * 32) * 4;    // scales, per-warp maxima and sums
  b += (size_t)kGroups2 * group * (head_dim + 4) * 4;                // dumped states
  b += (size_t)kGroups2 * 16 * 4;                                    // their m, l
  b += (size_t)(4 + 2 * kQRing2 + 4 * kGroups2 + 3) * 8;             // fixed barriers
  b += 64;                                                           // destinations of the tensor-parallel output
  b += sizeof(DeferredCombine);                                      // the pair finished at the CTA's end
  b += 32;                                                           // flags
  b += (size_t)(3 * batch + 2) * 4;                                  // sLen, sCum, sPos, the step counter
  return b;
}

// Fused step: quantise the new token of every pair whose last tile the CTA owns (the tile that holds it),
// exactly as the append kernel does.  Called by the softmax warps: one warp per K or V row at a time, D / 32 values
// per lane.  Per-token scale layout: the row's scale amax / 448 is computed here (a warp reduction) and written to
// [layer][sequence][slot][kv head] before the bytes.  Kept out of line: it runs once per launch and must not
// disturb the tile loop.
template <int D, bool PT>
__device__ __noinline__ void append_new_rows(int batch, int h_kv, int capacity, long long k_layer_stride,
                                             long long v_layer_stride, const uint16_t* k_new, const uint16_t* v_new,
                                             uint8_t* k_cache, uint8_t* v_cache, float* k_scale, float* v_scale,
                                             const int* sPos, int tid, long long r0, long long r1,
                                             const int* sCum, const int* sLen, int* status) {
  (void)status;
  constexpr int VPL = D / 32;   // values per lane: 4 or 8
  const int wid = tid >> 5, lane = tid & 31;
  Cursor a = locate(r0, sCum, sLen, batch, h_kv);
  long long cur = r0;
  int n = 0;
  while (cur < r1) {
    const long long pair_end = cur - a.tile + a.tiles_b;
    if (pair_end <= r1) {
      const int pos = sPos[a.b];   // as the prologue read it
      if (pos >= 0 && pos < capacity) {
#pragma unroll 1
        for (int which = 0; which < 2; ++which, ++n) {
          if (n % kSoftmaxWarps2 != wid) continue;
          const long long rowi = ((long long)a.layer * batch + a.b) * h_kv + a.h;
          const uint16_t* src = (which ? v_new : k_new) + rowi * D + lane * VPL;
          float x[VPL];
#pragma unroll
          for (int i = 0; i < VPL / 4; ++i) {
            const uint2 raw = *reinterpret_cast<const uint2*>(src + 4 * i);
            x[4 * i] = bf16_bits_to_float(raw.x & 0xFFFFu); x[4 * i + 1] = bf16_bits_to_float(raw.x >> 16);
            x[4 * i + 2] = bf16_bits_to_float(raw.y & 0xFFFFu); x[4 * i + 3] = bf16_bits_to_float(raw.y >> 16);
          }
          float sc;
          if (PT) {
            float amax = 0.f;
#pragma unroll
            for (int i = 0; i < VPL; ++i) amax = fmaxf(amax, fabsf(x[i]));
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
            sc = __fdiv_rn(amax, kE4m3Max);
            if (lane == 0) (which ? v_scale : k_scale)[(((long long)a.layer * batch + a.b) * capacity + pos) * h_kv + a.h] = sc;
          } else {
            sc = (which ? v_scale : k_scale)[a.layer * h_kv + a.h];
          }
          uint8_t* dst = (which ? v_cache : k_cache) + (long long)a.layer * (which ? v_layer_stride : k_layer_stride) +
                         (((long long)a.b * h_kv + a.h) * capacity + pos) * D + lane * VPL;
          B200ATTN_CHECK(status, a.b >= 0 && a.b < batch && a.h >= 0 && a.h < h_kv && a.layer >= 0 && pos / kTile2 == a.tiles_b - 1);
#pragma unroll
          for (int i = 0; i < VPL / 4; ++i)
            *reinterpret_cast<uint32_t*>(dst + 4 * i) = (uint32_t)quantize_e4m3(x[4 * i], sc) | ((uint32_t)quantize_e4m3(x[4 * i + 1], sc) << 8) |
                                                        ((uint32_t)quantize_e4m3(x[4 * i + 2], sc) << 16) | ((uint32_t)quantize_e4m3(x[4 * i + 3], sc) << 24);
        }
      }
    }
    cur = pair_end < r1 ? pair_end : r1;
    if (cur < r1) next_pair(a, sCum, sLen, batch, h_kv);
  }
}

// PT: per-token scale layout; GM: largest query group the instance takes, 5 (16 probability-operand rows) or 8 (32 rows).
// Instances of their own: the tile loop of the benchmark configuration (GM 5, per-head scales) stays as it is.
template <int D, bool PT, int GM>
__global__ void __launch_bounds__(kThreads2, 1)
attn_streamk_umma2_kernel(const __grid_constant__ CUtensorMap kmap, const __grid_constant__ CUtensorMap vmap,
                          const MmaParams p) {
  constexpr int NG = kGroups2;
  constexpr int DH = D / 128;
  constexpr int TILE_BYTES = kTile2 * D;
  constexpr int DP = D + 4;
  constexpr int QOP_BYTES = DH * 16 * 128;   // query operand
  constexpr int PROWS = GM <= 5 ? 16 : 32;   // rows of the probability operand / columns of an output accumulator
  constexpr int POP_BYTES = PROWS * 128;     // probability operand: PROWS rows x 128 tokens
  // The four 32-token products of a tile go to separate accumulators (summed once per segment): products
  // into one accumulator execute back to back at full latency, independent ones overlap.
  constexpr int OSPLIT = DH == 1 ? (GM <= 5 ? 4 : 2) : 1;
  constexpr uint32_t O_COL0 = NG * 16;       // tensor memory: S of each group, then O of each group
  constexpr uint32_t O_COLS = PROWS * DH * OSPLIT;   // per group
  constexpr uint32_t kIdescPVg = GM <= 5 ? kIdescPV : ((kIdescPV & ~(0x3Fu << 17)) | ((32u >> 3) << 17));   // N = PROWS
  constexpr uint32_t TMEM_NEED = NG * (16 + O_COLS);
  constexpr uint32_t TMEM_COLS = TMEM_NEED <= 64 ? 64 : TMEM_NEED <= 128 ? 128 : TMEM_NEED <= 256 ? 256 : 512;
  const Geometry& g = p.g;
  const int G = g.group;
  const int kstages = p.kstages, vstages = p.stages;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const uint32_t q_bytes = (uint32_t)G * D * 2;
  constexpr bool per_token = PT;   // scales [n_layers][batch][capacity][h_kv]

  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  uint8_t* smem = smem_raw + (((raw_addr + 1023u) & ~1023u) - raw_addr);
  uint8_t* sK = smem;                                                   // [kstages][TILE_BYTES]
  uint8_t* sV = sK + (size_t)kstages * TILE_BYTES;                      // [vstages][TILE_BYTES]
  uint8_t* sQop = sV + (size_t)vstages * TILE_BYTES;                    // [kQRing2][QOP_BYTES]
  uint8_t* sPop = sQop + kQRing2 * QOP_BYTES;                           // [NG][POP_BYTES], 1024-aligned
  uint8_t* sQraw = sPop + NG * POP_BYTES;                               // [2][G*D] bf16
  float* sScale = reinterpret_cast<float*>(sQraw + 2 * q_bytes);        // [kQRing2][8]
  float* sWmax = sScale + kQRing2 * 8;                                  // [NG][2][4 warps][8] tile maxima
  float* sWl = sWmax + NG * 64;                                         // [NG][4 warps][8] sums
  float* sDump = sWl + NG * 32;                                         // [NG][G][DP]
  float* sML = sDump + NG * G * DP;                                     // [NG][16]
  uint64_t* bars = reinterpret_cast<uint64_t*>(sML + NG * 16);
  const uint32_t kfull0 = smem_u32(bars), kempty0 = kfull0 + 8u * kstages;
  const uint32_t vfull0 = kempty0 + 8u * kstages, vempty0 = vfull0 + 8u * vstages;
  const uint32_t qrfull0 = vempty0 + 8u * vstages, qrempty0 = qrfull0 + 16u;
  const uint32_t qinfo0 = qrempty0 + 16u, qfree0 = qinfo0 + 8u * kQRing2;
  const uint32_t sfull0 = qfree0 + 8u * kQRing2, sempty0 = sfull0 + 8u * NG;
  const uint32_t pfull0 = sempty0 + 8u * NG, pvdone0 = pfull0 + 8u * NG;
  const uint32_t dfull0 = pvdone0 + 8u * NG, dempty0 = dfull0 + 8u, appended0 = dempty0 + 8u;
  constexpr int kFixedBars = 4 + 2 * kQRing2 + 4 * NG + 3;
  unsigned long long* sPeer = reinterpret_cast<unsigned long long*>(bars + kFixedBars + 2 * kstages + 2 * vstages);   // [8], see fill_peer_table
  DeferredCombine* sComb = reinterpret_cast<DeferredCombine*>(sPeer + 8);   // the pair this CTA finishes at its end
  int* sFlags = reinterpret_cast<int*>(sComb + 1);   // [0] timed_out [1] tmem [2] flags [3..7] issued counts
  int* sLen = sFlags + 8;
  int* sCum = sLen + g.batch;
  int* sPos = sCum + g.batch + 1;   // [batch] the positions as read
  int* sStep = sPos + g.batch;      // the step counter as read
  volatile int* timed_out = sFlags;

  if (tid == 0) {
    for (int s = 0; s < kstages; ++s) { mbar_init(kfull0 + 8u * s, 1); mbar_init(kempty0 + 8u * s, 1); }
    for (int s = 0; s < vstages; ++s) { mbar_init(vfull0 + 8u * s, 1); mbar_init(vempty0 + 8u * s, 1); }
    for (int i = 0; i < 2; ++i) { mbar_init(qrfull0 + 8u * i, 1); mbar_init(qrempty0 + 8u * i, 1); }
    for (int i = 0; i < kQRing2; ++i) { mbar_init(qinfo0 + 8u * i, 1); mbar_init(qfree0 + 8u * i, kSoftmaxWarps2); }
    for (int i = 0; i < NG; ++i) {
      mbar_init(sfull0 + 8u * i, 1);
      mbar_init(sempty0 + 8u * i, 4);     // the four warps of softmax group i
      mbar_init(pfull0 + 8u * i, 4);
      mbar_init(pvdone0 + 8u * i, 1);
    }
    mbar_init(dfull0, kSoftmaxWarps2);
    mbar_init(dempty0, 1);
    mbar_init(appended0, kSoftmaxWarps2);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    sFlags[0] = 0; sFlags[3] = 0; sFlags[4] = 0; sFlags[5] = 0; sFlags[6] = 0; sFlags[7] = 0;
    sComb->valid = 0;
    pdl_wait();   // the kernel before this one has completed: positions, cache rows and workspace are as it left them
    int acc = 0, any_empty = 0, st = 0, uniform = 1;
    for (int b = 0; b < g.batch; ++b) {
      const int raw = p.seq_len[b];
      int len = raw + p.seq_len_offset;
      if (p.k_new && (len < 1 || len > g.capacity)) st |= B200ATTN_STATUS_POS_AT_CAPACITY;   // the new token has no slot
      if (len < 0) { len = 0; st |= B200ATTN_STATUS_LEN_NEGATIVE; }
      if (len > g.capacity) { len = g.capacity; st |= B200ATTN_STATUS_LEN_OVER_CAP; }
      sPos[b] = raw;
      sLen[b] = len;
      sCum[b] = acc;
      acc += (len + kTile2 - 1) / kTile2;
      any_empty |= len == 0;
      uniform &= b == 0 || acc - sCum[b] == sCum[1] - sCum[0];
    }
    sCum[g.batch] = acc;
    *sStep = peer_step(p);
    sFlags[2] = any_empty | (uniform ? 2 : 0);
    if (st && blockIdx.x == 0) atomicOr(p.status, st);
  }
  if (warp == kProducer2 && lane == 0) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(&kmap) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&vmap) : "memory");
  }
  if (warp == kIssuerS2) tmem_alloc(smem_u32(sFlags + 1), TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = (uint32_t)sFlags[1];
  if (tid == 0) pdl_launch_dependents();
  const int step = *sStep;

  if (sFlags[2] & 1) {
    if (p.n_out) {   // tensor parallel: the destinations are needed here already (the epilogue warp writes them again later)
      if (tid < 8) fill_peer_table(p, sPeer, tid, step);
      __syncthreads();
    }
    const long long rows = (long long)g.n_layers * g.batch;
    for (long long r = blockIdx.x; r < rows; r += gridDim.x) {
      if (sLen[r % g.batch] == 0)
        for (int i = 2 * tid; i < g.h_q * D; i += 2 * kThreads2)
          emit_bits(p, sPeer, step, r * g.h_q * D + i, (r * p.out_hq_total + p.out_head_base) * D + i, 0u);
    }
  }

  const long long per_layer = (long long)sCum[g.batch] * g.h_kv;
  const long long total = per_layer * g.n_layers;
  int n_eff;
  long long r0, r1;
  cta_range(total, (int)gridDim.x, (int)blockIdx.x, (sFlags[2] & 2) ? sCum[1] - sCum[0] : 0, n_eff, r0, r1);
  const bool has_work = r0 < r1;

  if (warp == kProducer2) {
    // ===================== producer warp: one elected lane issues the copies =====================
    // (this lane, like the two issuer lanes, is a serial instruction stream that must keep up with one
    // tile per ~1300 cycles: stage indices, ring rounds and rows are carried, not recomputed)
    if (lane == 0 && has_work) {
      Cursor c = locate(r0, sCum, sLen, g.batch, g.h_kv);
      const uint64_t kv_policy = l2_policy_evict_first();
      const int total_it = (int)(r1 - r0);
      int seg = 0, ks = 0, kround = 0, vs = 0, vround = 0, kissued = 0, vissued = 0, row = 0;
      bool seg_start = true, ok = true, need_append = p.k_new != nullptr;
      for (int it = 0; it < total_it && ok; ++it) {
        if (seg_start) {
          const int qb = seg & 1;
          if (seg >= 2 && !mbar_wait_lean(qrempty0 + 8u * qb, ((seg >> 1) - 1) & 1, timed_out, p.status)) break;
          mbar_arrive_expect_tx(qrfull0 + 8u * qb, q_bytes);
          const long long lb = (long long)c.layer * g.batch + c.b;
          bulk_load(smem_u32(sQraw + qb * q_bytes), p.q + (lb * g.h_q + c.h * G) * D, q_bytes, qrfull0 + 8u * qb);
          ++seg;
          seg_start = false;
          row = (c.b * g.h_kv + c.h) * g.capacity + c.tile * kTile2;
        }
        if (need_append && c.tile == c.tiles_b - 1) {   // the tile that holds the new token: its row must be in the cache
          if (!mbar_wait_lean(appended0, 0, timed_out, p.status)) break;
          asm volatile("fence.proxy.async.global;" ::: "memory");
          need_append = false;
        }
        if (kround && !mbar_wait_lean(kempty0 + 8u * ks, (kround - 1) & 1, timed_out, p.status)) break;
        B200ATTN_CHECK(p.status, c.layer >= 0 && c.layer < g.n_layers && row >= 0 && (long long)row < (long long)g.batch * g.h_kv * g.capacity &&
                                     row == (c.b * g.h_kv + c.h) * g.capacity + c.tile * kTile2 && c.tile * kTile2 < c.len_b && ks < kstages && vs < vstages);
        mbar_arrive_expect_tx(kfull0 + 8u * ks, TILE_BYTES);
#pragma unroll
        for (int hf = 0; hf < DH; ++hf) {
          // K/V lines are used once: evict-first keeps L2 for what is used again (queries, partials, and in the
          // per-token layout the scale sectors, wanted once per KV head: 212 -> 171 us; per-head layout: -2.5 us)
          tma_load_3d_hint(smem_u32(sK) + ks * TILE_BYTES + hf * kTile2 * 128, &kmap, hf * 128, row, c.layer, kfull0 + 8u * ks, kv_policy);
        }
        ++kissued;
        if (++ks == kstages) { ks = 0; ++kround; }
        if (vround && !mbar_wait_lean(vempty0 + 8u * vs, (vround - 1) & 1, timed_out, p.status)) break;
        mbar_arrive_expect_tx(vfull0 + 8u * vs, TILE_BYTES);
#pragma unroll
        for (int hf = 0; hf < DH; ++hf) {
          tma_load_3d_hint(smem_u32(sV) + vs * TILE_BYTES + hf * kTile2 * 128, &vmap, hf * 128, row, c.layer, vfull0 + 8u * vs, kv_policy);
        }
        ++vissued;
        if (++vs == vstages) { vs = 0; ++vround; }
        row += kTile2;
        if (++c.tile == c.tiles_b) {
          seg_start = true;
          if (it + 1 < total_it) next_pair(c, sCum, sLen, g.batch, g.h_kv);
        }
      }
      sFlags[3] = kissued; sFlags[4] = vissued; sFlags[5] = seg;   // read by the drain after a timed-out wait
     
    }
  } else if (warp == kEpilogue2) {
    if (arrives_early(p)) arrive_early(p.seq_pos, p.exit_count, p.pkt ? p.epoch : nullptr, step, g.batch, g.capacity, lane);
    if (has_work)
      epilogue_warp<D, 1, NG, true, PT>(p, lane, r0, r1, total, n_eff, sCum, sLen, sDump, sML, dfull0, dempty0, timed_out, sPeer, sComb, step);
  } else if (warp == kIssuerS2) {
    // ===================== S issuer warp: query operand, S = K q^T =====================
    if (has_work) {
      Cursor c = locate(r0, sCum, sLen, g.batch, g.h_kv);
      const int total_it = (int)(r1 - r0);
      int seg = 0, qb = 0, ks = 0, kround = 0, issued = 0;
      bool seg_start = true, alive = true;
      const uint64_t descK0 = smem_desc_k128(smem_u32(sK)), descQ0 = smem_desc_k128(smem_u32(sQop));
      for (int it = 0; it < total_it && alive; ++it) {
        const int sb = it % NG;
        if (it >= NG) alive = mbar_wait_lean(sempty0 + 8u * sb, ((it / NG) - 1) & 1, timed_out, p.status);
        if (alive && seg_start) {
          qb = seg % kQRing2;
          alive = mbar_wait_lean(qrfull0 + 8u * (seg & 1), (seg >> 1) & 1, timed_out, p.status);
          // every softmax warp has taken the scales of the segment that used this slot before; its
          // score products completed before the score buffer waits above could pass
          if (alive && seg >= kQRing2) alive = mbar_wait_lean(qfree0 + 8u * qb, ((seg / kQRing2) - 1) & 1, timed_out, p.status);
          if (alive) {
            // Each head h: row h = leading e4m3 part of q * 2^e, row 8+h = remainder; lane owns 4 dims
            // per 128-dim block.  2^e puts the head's largest |q| into [128, 256).
            const uint32_t qraw = smem_u32(sQraw + (seg & 1) * q_bytes), qop = smem_u32(sQop + qb * QOP_BYTES);
            for (int h = 0; h < G; ++h) {
              float x[DH][4];
              float amax = 0.f;
#pragma unroll
              for (int hf = 0; hf < DH; ++hf) {
                uint32_t w0 = lds32(qraw + (h * D + hf * 128 + 4 * lane) * 2);
                uint32_t w1 = lds32(qraw + (h * D + hf * 128 + 4 * lane) * 2 + 4);
                x[hf][0] = bf16_bits_to_float(w0 & 0xFFFFu); x[hf][1] = bf16_bits_to_float(w0 >> 16);
                x[hf][2] = bf16_bits_to_float(w1 & 0xFFFFu); x[hf][3] = bf16_bits_to_float(w1 >> 16);
#pragma unroll
                for (int i = 0; i < 4; ++i) amax = fmaxf(amax, fabsf(x[hf][i]));
              }
#pragma unroll
              for (int off = 16; off > 0; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
              int ex = (int)((__float_as_uint(amax) >> 23) & 0xFF);
              ex = ex < 1 ? 127 : (ex < 8 ? 8 : (ex > 253 ? 253 : ex));   // zero / denormal / inf / NaN: no rescale worth doing
              const float down = __uint_as_float((uint32_t)(261 - ex) << 23);   // 2^(134-ex)
              const float up = __uint_as_float((uint32_t)(ex - 7) << 23);       // 2^(ex-134)
#pragma unroll
              for (int hf = 0; hf < DH; ++hf) {
                const float x0 = x[hf][0] * down, x1 = x[hf][1] * down, x2 = x[hf][2] * down, x3 = x[hf][3] * down;
                const float h0 = e4m3_head(x0), h1 = e4m3_head(x1), h2 = e4m3_head(x2), h3 = e4m3_head(x3);
                const uint32_t whi = pack_e4m3x2(h0, h1) | (pack_e4m3x2(h2, h3) << 16);
                const uint32_t wlo = pack_e4m3x2(x0 - h0, x1 - h1) | (pack_e4m3x2(x2 - h2, x3 - h3) << 16);
                // 128-byte swizzle: 16-byte chunk index xor (row & 7); rows h and 8+h share (row & 7)
                const uint32_t off = (uint32_t)hf * 2048u + ((((uint32_t)lane >> 2) ^ (uint32_t)(h & 7)) << 4) + ((4u * lane) & 15u);
                sts32(qop + off + (uint32_t)h * 128u, whi);
                sts32(qop + off + (uint32_t)(8 + h) * 128u, wlo);
              }
              // per-token scales are applied by the softmax threads, one token each
              if (lane == 0) sScale[qb * 8 + h] = up * (per_token ? 1.f : p.k_scale[c.layer * g.h_kv + c.h]) * p.score_scale;
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // operand bytes -> visible to the tensor core
            __syncwarp();
            if (lane == 0) {
              mbar_arrive(qrempty0 + 8u * (seg & 1));   // raw query buffer may be refilled
              mbar_arrive(qinfo0 + 8u * qb);            // scales are in place for the softmax warps
            }
          }
          ++seg;
        }
        seg_start = false;
        if (alive) alive = mbar_wait_lean(kfull0 + 8u * ks, kround & 1, timed_out, p.status);
        if (alive) {
          tc_fence_after();
          if (lane == 0) {
            // descriptors address shared memory in 16-byte units: stepping the start address is an add
            const uint64_t a0 = descK0 + (uint64_t)(ks * (TILE_BYTES >> 4)), b0 = descQ0 + (uint64_t)(qb * (QOP_BYTES >> 4));
            const uint32_t d = tmem_base + (uint32_t)sb * 16u;
#pragma unroll
            for (int hf = 0; hf < DH; ++hf)
#pragma unroll
              for (int kb = 0; kb < 4; ++kb)
                umma_f8(d, a0 + (uint64_t)(hf * (kTile2 * 128 >> 4) + kb * 2), b0 + (uint64_t)(hf * 128 + kb * 2),
                        kIdescQK, (hf | kb) ? 1u : 0u);
            umma_commit(sfull0 + 8u * sb);     // scores of this tile are complete
            umma_commit(kempty0 + 8u * ks);    // and the K tile has been read
          }
          __syncwarp();
          ++issued;
          if (++ks == kstages) { ks = 0; ++kround; }
        }
        if (++c.tile == c.tiles_b) {
          seg_start = true;
          if (it + 1 < total_it) next_pair(c, sCum, sLen, g.batch, g.h_kv);
        }
      }
      if (lane == 0) { sFlags[6] = issued; }
    }
  } else if (warp == kIssuerPV2) {
    // ===================== P V issuer warp: O[group] += V^T P^T =====================
    if (has_work) {
      Cursor c = locate(r0, sCum, sLen, g.batch, g.h_kv);
      const int total_it = (int)(r1 - r0);
      int seg_pos = 0, vs = 0, vround = 0, issued = 0;
      bool alive = true;
      const uint64_t descV0 = smem_desc_k128(smem_u32(sV)), descP0 = smem_desc_k128(smem_u32(sPop));
      for (int j = 0; j < total_it && alive; ++j) {
        const int pb = j % NG;
        const bool fresh = seg_pos < NG;   // the group's first tile of this segment: its accumulator starts over
        alive = mbar_wait_lean(pfull0 + 8u * pb, (j / NG) & 1, timed_out, p.status);
        if (alive) alive = mbar_wait_lean(vfull0 + 8u * vs, vround & 1, timed_out, p.status);
        if (alive) {
          tc_fence_after();
          if (lane == 0) {
            const uint64_t a0 = descV0 + (uint64_t)(vs * (TILE_BYTES >> 4)), b0 = descP0 + (uint64_t)(pb * (POP_BYTES >> 4));
            const uint32_t d0 = tmem_base + O_COL0 + (uint32_t)pb * O_COLS;
#pragma unroll
            for (int hf = 0; hf < DH; ++hf)
#pragma unroll
              for (int kb = 0; kb < 4; ++kb)   // 32 tokens per instruction: 32 rows of 128 bytes further in V, 32 bytes further in P;
                                             // accumulator block kb mod OSPLIT, started over by its first product of a fresh tile
                umma_f8(d0 + (uint32_t)PROWS * (hf + (OSPLIT > 1 ? kb % OSPLIT : 0)), a0 + (uint64_t)(hf * (kTile2 * 128 >> 4) + kb * (4096 >> 4)),
                        b0 + (uint64_t)(kb * 2), kIdescPVg, (kb >= OSPLIT || !fresh) ? 1u : 0u);
            umma_commit(pvdone0 + 8u * pb);    // O holds tile j; the group's probability operand is free
            umma_commit(vempty0 + 8u * vs);    // V tile has been read
          }
          __syncwarp();
          ++issued;
          if (++vs == vstages) { vs = 0; ++vround; }
        }
        ++seg_pos;
        if (++c.tile == c.tiles_b) {
          seg_pos = 0;
          if (j + 1 < total_it) next_pair(c, sCum, sLen, g.batch, g.h_kv);
        }
      }
      if (lane == 0) { sFlags[7] = issued; }
    }
  } else if (has_work) {
    // ===== softmax warps: groups of four; group = tile index mod NG; one thread = one token / one output dim =====
    if (p.k_new) {
      append_new_rows<D, PT>(g.batch, g.h_kv, g.capacity, g.k_layer_stride, g.v_layer_stride, p.k_new, p.v_new,
                             p.k_cache_w, p.v_cache_w, const_cast<float*>(p.k_scale), const_cast<float*>(p.v_scale), sPos, tid,
                             r0, r1, sCum, sLen, p.status);
      asm volatile("fence.proxy.async.global;" ::: "memory");   // the rows -> visible to the TMA loads of this CTA
      __syncwarp();
      if (lane == 0) mbar_arrive(appended0);
      // per-token layout: the new token's scales, written by one softmax warp, are read by another (its token's owner)
      if (PT) asm volatile("bar.sync 5, %0;" ::"n"(kSoftmaxWarps2 * 32) : "memory");
    }
    Cursor c = locate(r0, sCum, sLen, g.batch, g.h_kv);
    long long cur = r0;
    int it0 = 0, seg = 0;
    const int grp = warp >> 2, wq = warp & 3;
    const int tok_in_tile = wq * 32 + lane;
    const uint32_t tmem_lane = tmem_base + ((uint32_t)(wq * 32) << 16);
    const uint32_t tmem_s = tmem_lane + (uint32_t)grp * 16u;
    const uint32_t tmem_o = tmem_lane + O_COL0 + (uint32_t)grp * O_COLS;
    const uint32_t sfull = sfull0 + 8u * grp, sempty = sempty0 + 8u * grp, pfull = pfull0 + 8u * grp, pvdone = pvdone0 + 8u * grp;
    const uint32_t pop = smem_u32(sPop + grp * POP_BYTES);
    const uint32_t pcol = ((uint32_t)(tok_in_tile >> 4) << 4), pwithin = (uint32_t)tok_in_tile & 15u;
    const uint32_t sV_addr = smem_u32(sV);
    float* wmax = sWmax + grp * 64;
    float* wl = sWl + grp * 32;
    float* dump = sDump + grp * G * DP;
    if (GM > 5) {   // rows 24..31 of the probability operand are never written again: make them finite once
#pragma unroll
      for (int n = 24; n < 32; ++n) sts8(pop + n * 128 + (pcol ^ ((uint32_t)(n & 7) << 4)) + pwithin, 0u);
    }

    while (cur < r1) {
      const long long pair_start = cur - c.tile, pair_end = pair_start + c.tiles_b;
      const long long seg_end = pair_end < r1 ? pair_end : r1;
      const int ntiles = (int)(seg_end - cur);
      const int qb = seg % kQRing2;
      float sc[GM];
      {
        const bool ok = mbar_wait_lean(qinfo0 + 8u * qb, (seg / kQRing2) & 1, timed_out, p.status);
#pragma unroll
        for (int h = 0; h < GM; ++h) sc[h] = (ok && h < G) ? sScale[qb * 8 + h] : 0.f;
        __syncwarp();
        if (lane == 0) mbar_arrive(qfree0 + 8u * qb);
      }
      float mref[GM], l[GM];
#pragma unroll
      for (int h = 0; h < GM; ++h) { mref[h] = -INFINITY; l[h] = 0.f; }

      // this group's tiles: CTA-wide tile index j with j mod NG == grp
      const int jfirst = it0 + (((grp - it0) % NG) + NG) % NG;
      int jlast = -1;
      float kst_next = 1.f, vst_next = 1.f;
      if (per_token && jfirst < it0 + ntiles && (c.tile + (jfirst - it0)) * kTile2 + tok_in_tile < c.len_b) {
        const long long si = (((long long)c.layer * g.batch + c.b) * g.capacity + (c.tile + (jfirst - it0)) * kTile2 + tok_in_tile) * g.h_kv + c.h;
        kst_next = __ldcg(p.k_scale + si);
        vst_next = __ldcg(p.v_scale + si);
      }
      for (int j = jfirst; j < it0 + ntiles; j += NG) {
        jlast = j;
        const int ph = (j / NG) & 1;
        const int tile_tok0 = (c.tile + (j - it0)) * kTile2;
        // this token's K scale and V scale (the latter folded into the probability scaling): loaded one tile
        // of the group ahead, so the loads have a whole tile period to land
        const float kst = kst_next, vst = vst_next * kPScale;
        if (per_token && j + NG < it0 + ntiles && tile_tok0 + NG * kTile2 + tok_in_tile < c.len_b) {
          const long long si = (((long long)c.layer * g.batch + c.b) * g.capacity + tile_tok0 + NG * kTile2 + tok_in_tile) * g.h_kv + c.h;
          kst_next = __ldcg(p.k_scale + si);
          vst_next = __ldcg(p.v_scale + si);
        }
        const bool sok = mbar_wait_lean(sfull, ph, timed_out, p.status);
        uint32_t r[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) r[i] = 0;
        if (sok) {
          tc_fence_after();
          tmem_ld16(tmem_s, r);
          tc_fence_before();
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(sempty);
        const bool valid = sok && tile_tok0 + tok_in_tile < c.len_b;
        // scores and the tile maximum per head (over the group's 128 tokens)
        float s[GM];
        float* wm_w = wmax + ph * 32;
#pragma unroll
        for (int h = 0; h < GM; ++h) {
          s[h] = -INFINITY;
          if (h < G) {
            if (valid) s[h] = (__uint_as_float(r[h]) + __uint_as_float(r[8 + h])) * (sc[h] * kst);
            const float wm = warp_max(s[h]);
            if (lane == 0) wm_w[wq * 8 + h] = wm;
          }
        }
        bar_group(grp);
        bool rescale = false;
        float alpha[GM];
#pragma unroll
        for (int h = 0; h < GM; ++h) {
          alpha[h] = 1.f;
          if (h < G) {
            const float tmax = fmaxf(fmaxf(wm_w[h], wm_w[8 + h]), fmaxf(wm_w[16 + h], wm_w[24 + h]));
            if (tmax > mref[h] + kTau || mref[h] == -INFINITY) {   // the reference moves (always on the group's first tile)
              alpha[h] = mref[h] == -INFINITY ? 0.f : ex2(mref[h] - tmax);
              rescale |= mref[h] != -INFINITY;
              mref[h] = tmax;
              l[h] *= alpha[h];
            }
          }
        }
        // The P V of this group's previous tile has completed: the probability operand is free and the
        // accumulator holds everything up to that tile.
        bool pok = true;
        if (j >= NG) pok = mbar_wait_lean(pvdone, ph ^ 1, timed_out, p.status);
        if (rescale && pok) {   // O *= alpha per head, in tensor memory: thread = dim row
          tc_fence_after();
#pragma unroll
          for (int blk = 0; blk < DH * OSPLIT * (PROWS / 16); ++blk) {   // 16 columns at a time; column c belongs to head c / 3
            uint32_t o[16];
            tmem_ld16(tmem_o + 16u * blk, o);
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              const int col = (blk % (PROWS / 16)) * 16 + i;
              if (col < 3 * GM) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha[col / 3]);
            }
            tmem_st16(tmem_o + 16u * blk, o);
          }
          tc_fence_before();
        }
        // probabilities: p <= 2^kTau; p * 2^13 as three e5m2 terms, rows 3h..3h+2 of the operand
        if (pok) {
#pragma unroll
          for (int h = 0; h < GM; ++h) {
            float pr = 0.f;
            if (h < G && valid) pr = ex2(s[h] - mref[h]);
            l[h] += pr;
            const float q = pr * vst;
            const float t1 = e5m2_head(q), r1f = q - t1, t2 = e5m2_head(r1f), t3 = r1f - t2;
            const uint32_t b12 = pack_e5m2x2(t1, t2), b3 = pack_e5m2x2(t3, 0.f);
            sts8(pop + (3 * h) * 128 + (pcol ^ ((uint32_t)((3 * h) & 7) << 4)) + pwithin, b12);
            sts8(pop + (3 * h + 1) * 128 + (pcol ^ ((uint32_t)((3 * h + 1) & 7) << 4)) + pwithin, b12 >> 8);
            sts8(pop + (3 * h + 2) * 128 + (pcol ^ ((uint32_t)((3 * h + 2) & 7) << 4)) + pwithin, b3);
          }
          if (GM <= 5) sts8(pop + 15 * 128 + (pcol ^ (7u << 4)) + pwithin, 0u);   // unused 16th row: keep it finite (rows 24..31: zeroed once)
        }
        if (tile_tok0 + kTile2 > c.len_b) {
          // A token slot at or beyond the valid length: its V row may hold anything (NaN patterns
          // included) and 0 * NaN would poison O: zero the row in shared memory before the product.
          const int vs = j % vstages;
          const bool vok = mbar_wait_lean(vfull0 + 8u * vs, (j / vstages) & 1, timed_out, p.status);
          if (vok && !valid) {
#pragma unroll
            for (int hf = 0; hf < DH; ++hf)
#pragma unroll
              for (int ch = 0; ch < 8; ++ch)
                sts128z(sV_addr + vs * TILE_BYTES + hf * kTile2 * 128 + tok_in_tile * 128 + ch * 16);
          }
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // operand bytes -> visible to the tensor core
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(pfull);
      }

      // ---------------- end of segment: read O once, hand the group's state to the epilogue warp ----------------
      const bool ook = jlast < 0 || mbar_wait_lean(pvdone, (jlast / NG) & 1, timed_out, p.status);
#pragma unroll
      for (int h = 0; h < GM; ++h) {
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) l[h] += __shfl_xor_sync(0xffffffffu, l[h], off);
        if (lane == 0) wl[wq * 8 + h] = l[h];
      }
      const bool dok = seg < 1 || mbar_wait_lean(dempty0, (seg - 1) & 1, timed_out, p.status);
      bar_group(grp);
      if (ook && dok) {
        if (jlast >= 0) {
          tc_fence_after();
#pragma unroll
          for (int hf = 0; hf < DH; ++hf) {
            float acc[GM];
#pragma unroll
            for (int h = 0; h < GM; ++h) acc[h] = 0.f;
#pragma unroll
            for (int sp = 0; sp < OSPLIT; ++sp) {
              uint32_t o[PROWS];
#pragma unroll
              for (int cb = 0; cb < PROWS / 16; ++cb)
                tmem_ld16(tmem_o + (uint32_t)PROWS * (hf + sp) + 16u * cb, *reinterpret_cast<uint32_t(*)[16]>(o + 16 * cb));   // OSPLIT > 1 only with DH == 1
#pragma unroll
              for (int h = 0; h < GM; ++h)
                acc[h] += __uint_as_float(o[3 * h]) + __uint_as_float(o[3 * h + 1]) + __uint_as_float(o[3 * h + 2]);
            }
#pragma unroll
            for (int h = 0; h < GM; ++h)
              if (h < G) dump[h * DP + hf * 128 + tok_in_tile] = acc[h] * (1.f / kPScale);
          }
          tc_fence_before();
        } else {   // the segment had no tile for this group: an empty state (m = -inf) with finite contents
          for (int h = 0; h < G; ++h)
#pragma unroll
            for (int hf = 0; hf < DH; ++hf) dump[h * DP + hf * 128 + tok_in_tile] = 0.f;
        }
        if (wq == 0 && lane < GM) {
          float m = mref[0];
#pragma unroll
          for (int h = 1; h < GM; ++h) m = lane == h ? mref[h] : m;
          sML[grp * 16 + lane] = m;
          sML[grp * 16 + 8 + lane] = wl[lane] + wl[8 + lane] + wl[16 + lane] + wl[24 + lane];
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(dfull0);
      bar_group(grp);   // the sums are reused by the next segment
      ++seg;
      it0 += ntiles;
      cur = seg_end;
      if (cur < r1) next_pair(c, sCum, sLen, g.batch, g.h_kv);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == kIssuerS2) {
    if (sFlags[0] && lane == 0) {
      // A wait gave up: wait (bounded) for everything already issued into this CTA's shared / tensor memory.
      auto drain = [&](uint32_t bar0, int ring, int issued) {
        for (int s = 0; s < ring && s < issued; ++s) {
          const int lastu = ((issued - 1 - s) / ring) * ring + s;
          const unsigned long long t0 = global_timer_ns();
          while (!mbar_try_wait(bar0 + 8u * s, (lastu / ring) & 1) && global_timer_ns() - t0 < kWaitBudgetNs) {}
        }
      };
      drain(kfull0, kstages, sFlags[3]);
      drain(vfull0, vstages, sFlags[4]);
      drain(qrfull0, 2, sFlags[5]);
      drain(sfull0, NG, sFlags[6]);
      drain(pvdone0, NG, sFlags[7]);
    }
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
  // the pair whose last piece this CTA holds: all warps collect the other pieces (they end when this CTA's range does)
  if (sComb->valid && !sFlags[0]) combine_deferred<D>(combine_args_of(p, sPeer, step), *sComb, warp, kThreads2 / 32, lane);
  if (p.bar_world) __syncthreads();   // stores mode: every warp's peer stores are fenced before the CTA counts as finished
  end_of_launch(p, tid, kThreads2, step);
}

// Ring depths: all of the shared memory that the fixed part leaves, at most 4 K and 8 V tiles.
Plan2 plan2_for(const Geometry& g) {
  const size_t tile = (size_t)kTile2 * g.head_dim;
  const size_t fixed = umma2_fixed_bytes(g.group, g.head_dim, g.batch);
  const size_t budget = 227 * 1024 - 1024;
  Plan2 pl{2, 2, 0};
  for (int total = kMaxRingTiles2; total >= 4; --total) {
    const int ks = total >= 9 ? 4 : total >= 6 ? 3 : 2, vs = total - ks;
    const size_t b = fixed + (size_t)total * tile + (size_t)2 * total * 8;
    if (b <= budget && vs <= 8) { pl.kstages = ks; pl.vstages = vs; pl.bytes = (b + 15) & ~(size_t)15; return pl; }
  }
  pl.bytes = (fixed + 4 * tile + 64 + 15) & ~(size_t)15;
  return pl;
}

}  // namespace

bool umma2_supported(const Geometry& g) { return g.group <= 8; }

int umma2_pick_ctas(const Geometry& g, int max_seq_len, int num_sms) {
  (void)max_seq_len;
  const Plan2 pl = plan2_for(g);
  int per_sm = (int)((227 * 1024) / (pl.bytes + 1024));
  const int dh = g.head_dim / 128, need = kGroups2 * (16 + 16 * dh * (dh == 1 ? 4 : 1));
  const int tmem_cols = need <= 64 ? 64 : need <= 128 ? 128 : need <= 256 ? 256 : 512;
  if (per_sm > 512 / tmem_cols) per_sm = 512 / tmem_cols;
  if (per_sm > 2048 / kThreads2) per_sm = 2048 / kThreads2;
  if (per_sm < 1) per_sm = 1;
  return num_sms * per_sm;
}

cudaError_t launch_decode_umma2(const Geometry& g, const DecodeArgs& a, cudaStream_t stream) {
  if (g.batch > kMaxBatchMma || !umma2_supported(g)) return cudaErrorNotSupported;
  CUtensorMap kmap, vmap;
  if (!encode_cache_map(&kmap, a.k_cache, g, g.k_layer_stride, kTile2) ||
      !encode_cache_map(&vmap, a.v_cache, g, g.v_layer_stride, kTile2))
    return cudaErrorInvalidValue;
  MmaParams p{};
  p.g = g;
  p.q = (const uint16_t*)a.q;
  p.k_scale = a.k_scale;
  p.v_scale = a.v_scale;
  p.seq_len = a.seq_len;
  p.seq_len_offset = a.seq_len_offset;
  p.score_scale = a.softmax_scale * kLog2e;
  const int n = a.num_splits;
  p.ws_pkt = (unsigned long long*)a.workspace;
  p.out = (uint16_t*)a.out;
  p.gate = (const uint16_t*)a.gate;
  p.n_out = a.n_out;
  p.out_hq_total = a.n_out ? a.out_hq_total : g.h_q;
  p.out_head_base = a.n_out ? a.out_head_base : 0;
  for (int r = 0; r < 8; ++r) p.out_peer[r] = r < a.n_out ? (uint16_t*)a.out_peer[r] : nullptr;
  for (int r = 0; r < 8; ++r) p.out_peer[8 + r] = r < a.n_out ? (uint16_t*)a.out_peer_alt[r] : nullptr;
  p.epoch = a.n_out ? a.epoch : nullptr;
  p.pkt = a.n_out && a.pkt_src ? 1 : 0;
  p.pkt_src = (const unsigned long long*)a.pkt_src;
  p.pkt_slot_words = (long long)g.n_layers * g.batch * g.h_q * g.head_dim / 2;
  p.status = a.status;
  p.k_new = (const uint16_t*)a.k_new;
  p.v_new = (const uint16_t*)a.v_new;
  p.k_cache_w = (uint8_t*)a.k_cache;
  p.v_cache_w = (uint8_t*)a.v_cache;
  p.seq_pos = a.seq_pos;
  p.exit_count = (int*)(p.ws_pkt + (size_t)n * 2 * partial_slot_words(g.group, g.head_dim));
  for (int r = 0; r < 8; ++r) p.bar_flags[r] = r < a.bar_world ? a.bar_flags[r] : nullptr;
  p.bar_rank = a.bar_rank;
  p.bar_world = a.bar_world;
  const Plan2 pl = plan2_for(g);
  p.stages = pl.vstages;
  p.kstages = pl.kstages;
  auto launch = [&](auto kernel) -> cudaError_t {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)pl.bytes);
    if (e != cudaSuccess) return e;
    if (p.pkt) {   // may every CTA wait for remote packets?  only if the whole grid is resident at once
      int per_sm = 0;
      e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, kThreads2, pl.bytes);
      if (e != cudaSuccess) return e;
      p.pkt_resident = (long long)per_sm * device_sms() >= n ? 1 : 0;
    }
    return launch_pdl(kernel, n, kThreads2, pl.bytes, stream, kmap, vmap, p);
  };
  const bool pt = g.scale_mode == B200ATTN_SCALE_PER_TOKEN, wide = g.group > 5;
  if (g.head_dim == 128) {
    if (wide) return pt ? launch(attn_streamk_umma2_kernel<128, true, 8>) : launch(attn_streamk_umma2_kernel<128, false, 8>);
    return pt ? launch(attn_streamk_umma2_kernel<128, true, 5>) : launch(attn_streamk_umma2_kernel<128, false, 5>);
  }
  if (wide) return pt ? launch(attn_streamk_umma2_kernel<256, true, 8>) : launch(attn_streamk_umma2_kernel<256, false, 8>);
  return pt ? launch(attn_streamk_umma2_kernel<256, true, 5>) : launch(attn_streamk_umma2_kernel<256, false, 5>);
}

}  // namespace b200attn

