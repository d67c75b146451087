// mma.sync stream-K variant of the FP8-KV decode attention (the library's choice for short caches, where its
// finer split over three CTAs per SM beats the all-tcgen05 kernel's fixed cost).
//
// One persistent launch covers every (layer, sequence, kv head) of a decode step:
//   * the KV cache is cut into tiles of TILE_T tokens; all tiles of the step form one linear
//     sequence which is divided evenly over the resident CTAs (stream-K), so ragged batches and
//     any depth fill all 148 SMs and each CTA touches at most two partially owned
//     (layer, sequence, kv head) "pairs";
//   * a producer warp streams K and V tiles with TMA (cp.async.bulk.tensor, 128-byte swizzle)
//     into a ring of shared-memory stages guarded by full/empty mbarriers; every KV byte is read
//     from HBM exactly once and serves all G query heads of the group;
//   * the producer also stages the G query rows of each pair (one cp.async.bulk per segment);
//   * four consumer warps each own 16 tokens of a tile.  FP8 bytes go from shared memory to
//     registers, are widened to f16 in registers (cvt.rn.f16x2.e4m3x2, exact) and feed
//     mma.sync.m16n8k16 with the query heads on the N side (G <= 8): S^T = K q^T, then
//     O^T += V^T P^T after a warp-level movmatrix transpose of the probabilities.  Accumulation
//     and the log2-domain online softmax are fp32.  The per-head scales never enter the loop:
//     k_scale*softmax_scale*log2e multiplies the scores, v_scale the final normalisation;
//   * at the end of a pair (or of the CTA's range) the consumer warps dump their (m, l, acc)
//     state into a double-buffered shared-memory area and go straight on to the next pair; an
//     epilogue warp merges the four states off the critical path.  A pair owned by one CTA is
//     normalised and written directly; otherwise each owner leaves its (m, l, acc) piece in the workspace as
//     tagged 8-byte words, and the owner of the pair's last piece collects them with all its warps when its own
//     range is done, in CTA order (deterministic, so replays are bitwise identical).  It only waits for CTAs of
//     lower index.  Every wait — for copies, for pieces — is bounded: on expiry the CTA flags
//     B200ATTN_STATUS_WAIT_TIMEOUT, stops waiting, drains its copies and returns.
//
// It replaces repeat_kv + eager attention + the capacity mask of the reference
// (bench/micro/attn_length_effect.py:41-66, runner/model/static_cache.py:79-82) and follows the
// split/combine structure of its fused kernel
// (docs/journal/2026-10-23-phase2-r3-coordinator.md:137-141).
#include "streamk.cuh"

namespace b200attn {

namespace {

constexpr int kTileT = 64;                 // tokens per tile (16 per consumer warp)
constexpr int kThreads = kConsumerThreads + 64;   // + producer warp + epilogue warp
constexpr int kCtasPerSm = 3;                      // D = 128: the kernel is latency bound, three CTAs per SM hide it best
                                                   // (measured at depth 8192: 2 CTAs x 5 stages 187 us, 3 x 3 176 us, 4 x 2 with
                                                   // spills 191 us).  Co-resident CTAs do not progress equally (the first resident
                                                   // one ends ~10 % early); skewing the tile split per residency slot, or fusing the
                                                   // three CTAs into one 576-thread CTA, was measured and did not help (182 us).
                                                   // The 96-register cap of 18 warps per SM costs ~100 B of spills in the consumer
                                                   // loop; dropping the producer warp (lane 0 of consumer warp 0 issuing the copies,
                                                   // 15 warps, 127 registers, no spills) was slower still (198 us): the coupling of
                                                   // copy issue to one consumer's progress costs more than the spills.
constexpr int kDumpBufs = 2;                       // dump buffers per CTA

// Fused step: quantise the new token of every pair whose last tile (the tile that holds it) lies in the CTA's
// range [r0, r1), exactly as the append kernel does; called by all 32 lanes of the
// epilogue warp, which then releases the producer lane's wait in front of the first such tile.  Out of line: it runs
// once per launch and must not cost the tile loop registers or instruction-cache room.
template <int D>
__device__ __noinline__ void append_rows_by_warp(int batch, int h_kv, int capacity, long long k_layer_stride,
                                                 long long v_layer_stride, const uint16_t* k_new, const uint16_t* v_new,
                                                 uint8_t* k_cache, uint8_t* v_cache, const float* k_scale, const float* v_scale,
                                                 const int* sPos, int lane, long long r0, long long r1,
                                                 const int* sCum, const int* sLen, int* status) {
  (void)status;
  Cursor a = locate(r0, sCum, sLen, batch, h_kv);
  long long cur = r0;
  while (cur < r1) {
    const long long pair_end = cur - a.tile + a.tiles_b;
    if (pair_end <= r1) {
      const int pos = sPos[a.b];   // as the prologue read it
      if (pos >= 0 && pos < capacity) {
        const long long rowi = ((long long)a.layer * batch + a.b) * h_kv + a.h;
        B200ATTN_CHECK(status, a.b >= 0 && a.b < batch && a.h >= 0 && a.h < h_kv && a.layer >= 0 && pos / kTileT == a.tiles_b - 1);
        for (int e = lane; e < D / 2; e += 32) {   // 4 values of the K row (e < D/4) or of the V row
          const int which = e >= D / 4 ? 1 : 0, el = (e % (D / 4)) * 4;
          const uint2 raw = *reinterpret_cast<const uint2*>((which ? v_new : k_new) + rowi * D + el);
          const float sc = (which ? v_scale : k_scale)[a.layer * h_kv + a.h];
          const uint32_t bytes = (uint32_t)quantize_e4m3(bf16_bits_to_float(raw.x & 0xFFFFu), sc) |
                                 ((uint32_t)quantize_e4m3(bf16_bits_to_float(raw.x >> 16), sc) << 8) |
                                 ((uint32_t)quantize_e4m3(bf16_bits_to_float(raw.y & 0xFFFFu), sc) << 16) |
                                 ((uint32_t)quantize_e4m3(bf16_bits_to_float(raw.y >> 16), sc) << 24);
          uint8_t* dst = (which ? v_cache : k_cache) + (long long)a.layer * (which ? v_layer_stride : k_layer_stride) +
                         (((long long)a.b * h_kv + a.h) * capacity + pos) * D + el;
          *reinterpret_cast<uint32_t*>(dst) = bytes;
        }
      }
    }
    cur = pair_end < r1 ? pair_end : r1;
    if (cur < r1) next_pair(a, sCum, sLen, batch, h_kv);
  }
  asm volatile("fence.proxy.async.global;" ::: "memory");   // the rows -> visible to the CTA's TMA loads
  __syncwarp();
}

// MINB: CTAs per SM the instance is compiled for.  Three (96 registers, ~100 B of spills in the consumer loop) is
// the long-cache configuration; the instance for two has 168 registers to work with and serves the small grids of
// short caches, where nothing is gained from a third CTA per SM and the consumer chain's latency is what counts.
template <int D, int MINB>
__global__ void __launch_bounds__(kThreads, MINB)
attn_streamk_mma_kernel(const __grid_constant__ CUtensorMap kmap, const __grid_constant__ CUtensorMap vmap,
                        const MmaParams p) {
  constexpr int DH = D / 128;              // 128-byte column blocks per row
  constexpr int KSTEPS = D / 16;           // mma k-steps for QK^T == mma tiles for PV
  constexpr int TILE_BYTES = kTileT * D;   // one K (or V) tile
  constexpr int DP = D + 4;                // padded head row of a dumped state, in floats
  const Geometry& g = p.g;
  const int G = g.group;
  const int stages = p.stages;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int gq = lane >> 2, tq = lane & 3;  // mma fragment coordinates ("groupID", "threadID_in_group")
  const uint32_t q_bytes = (uint32_t)G * D * 2;
  const int dump_warp_floats = G * DP;

  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  uint8_t* smem = smem_raw + (((raw_addr + 1023u) & ~1023u) - raw_addr);
  uint8_t* sK = smem;
  uint8_t* sV = sK + (size_t)stages * TILE_BYTES;
  uint8_t* sQ = sV + (size_t)stages * TILE_BYTES;                                     // [2][G*D] bf16
  float* sDump = reinterpret_cast<float*>(sQ + 2 * q_bytes);                          // [2][4][G][DP]
  float* sML = sDump + kDumpBufs * kConsumerWarps * dump_warp_floats;                         // [2][4][16]: m[8], l[8]
  uint64_t* bars = reinterpret_cast<uint64_t*>(sML + kDumpBufs * kConsumerWarps * 16);
  unsigned long long* sPeer = reinterpret_cast<unsigned long long*>(bars + 2 * stages + 9);   // [8], see fill_peer_table
  DeferredCombine* sComb = reinterpret_cast<DeferredCombine*>(sPeer + 8);             // the pair this CTA finishes at its end
  int* sFlags = reinterpret_cast<int*>(sComb + 1);                                    // [0] timed_out [2] any_empty [3] copies
  int* sLen = sFlags + 4;                                                             // [batch]
  int* sCum = sLen + g.batch;                                                         // [batch+1]
  int* sPos = sCum + g.batch + 1;                                                     // [batch] the positions as read
  int* sStep = sPos + g.batch;                                                        // the step counter as read
  volatile int* timed_out = sFlags;
  const uint32_t full0 = smem_u32(bars), empty0 = full0 + 8u * stages;
  const uint32_t qfull0 = empty0 + 8u * stages, qempty0 = qfull0 + 16u;
  const uint32_t dfull0 = qempty0 + 16u, dempty0 = dfull0 + 16u, appended0 = dempty0 + 16u;

  if (tid == 0) {
    for (int s = 0; s < stages; ++s) {
      mbar_init(full0 + 8u * s, 1);
      mbar_init(empty0 + 8u * s, kConsumerWarps);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(qfull0 + 8u * i, 1);
      mbar_init(qempty0 + 8u * i, kConsumerWarps);
      mbar_init(dfull0 + 8u * i, kConsumerWarps);
      mbar_init(dempty0 + 8u * i, 1);
    }
    mbar_init(appended0, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    sFlags[0] = 0; sFlags[1] = 0; sFlags[3] = 0;
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
      acc += (len + kTileT - 1) / kTileT;
      any_empty |= len == 0;
      uniform &= b == 0 || acc - sCum[b] == sCum[1] - sCum[0];
    }
    sCum[g.batch] = acc;
    *sStep = peer_step(p);
    sFlags[2] = any_empty | (uniform ? 2 : 0);
    if (st && blockIdx.x == 0) atomicOr(p.status, st);
  }
  if (warp == kProducerWarp && lane == 0) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(&kmap) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&vmap) : "memory");
  }
  __syncthreads();
  if (tid == 0) pdl_launch_dependents();
  const int step = *sStep;

  // sequences of length 0 have no tiles: their outputs are zero, written by whoever gets there
  if (sFlags[2] & 1) {
    if (p.n_out) {   // tensor parallel: the destinations are needed here already (the epilogue warp writes them again later)
      if (tid < 8) fill_peer_table(p, sPeer, tid, step);
      __syncthreads();
    }
    const long long rows = (long long)g.n_layers * g.batch;
    for (long long r = blockIdx.x; r < rows; r += gridDim.x) {
      if (sLen[r % g.batch] == 0)
        for (int i = 2 * tid; i < g.h_q * D; i += 2 * kThreads)
          emit_bits(p, sPeer, step, r * g.h_q * D + i, (r * p.out_hq_total + p.out_head_base) * D + i, 0u);
    }
  }

  const long long per_layer = (long long)sCum[g.batch] * g.h_kv;
  const long long total = per_layer * g.n_layers;
  int n_eff;
  long long r0, r1;
  cta_range(total, (int)gridDim.x, (int)blockIdx.x, (sFlags[2] & 2) ? sCum[1] - sCum[0] : 0, n_eff, r0, r1);
  const bool has_work = r0 < r1;

  if (warp == kProducerWarp) {
    // ===================== producer warp: one elected lane issues the copies =====================
    if (lane == 0 && has_work) {
      bool need_append = p.k_new != nullptr;   // fused step: the epilogue warp appends the new rows meanwhile
      Cursor c = locate(r0, sCum, sLen, g.batch, g.h_kv);
      int it = 0, seg = 0;
      bool seg_start = true;
      for (long long idx = r0; idx < r1; ++idx, ++it) {
        if (seg_start) {   // the G query rows of this pair, once per segment
          const int qb = seg & 1;
          if (seg >= 2 && !mbar_wait(qempty0 + 8u * qb, ((seg >> 1) - 1) & 1, timed_out, p.status)) break;
          mbar_arrive_expect_tx(qfull0 + 8u * qb, q_bytes);
          const long long lb = (long long)c.layer * g.batch + c.b;
          bulk_load(smem_u32(sQ + qb * q_bytes), p.q + (lb * g.h_q + c.h * G) * D, q_bytes, qfull0 + 8u * qb);
          ++seg;
          seg_start = false;
        }
        const int s = it % stages;
        if (need_append && c.tile == c.tiles_b - 1) {   // the tile that holds the new token: its row must be in the cache
          if (!mbar_wait(appended0, 0, timed_out, p.status)) break;
          asm volatile("fence.proxy.async.global;" ::: "memory");
          need_append = false;
        }
        if (it >= stages && !mbar_wait(empty0 + 8u * s, ((it / stages) - 1) & 1, timed_out, p.status)) break;
        const uint32_t fb = full0 + 8u * s;
        mbar_arrive_expect_tx(fb, 2u * TILE_BYTES);
        const int row = (c.b * g.h_kv + c.h) * g.capacity + c.tile * kTileT;
        B200ATTN_CHECK(p.status, c.layer >= 0 && c.layer < g.n_layers && c.b >= 0 && c.b < g.batch && c.h >= 0 && c.h < g.h_kv &&
                                     c.tile >= 0 && c.tile * kTileT < c.len_b && (long long)row < (long long)g.batch * g.h_kv * g.capacity);
#pragma unroll
        for (int hf = 0; hf < DH; ++hf) {
          // K/V lines are used once: an L2 evict-first policy on the copies keeps L2 for what is used again
          // (queries, partials, outputs): 175.5 -> 169 us at depth 8192
          tma_load_3d_hint(smem_u32(sK + (size_t)s * TILE_BYTES + hf * kTileT * 128), &kmap, hf * 128, row, c.layer, fb, l2_policy_evict_first());
          tma_load_3d_hint(smem_u32(sV + (size_t)s * TILE_BYTES + hf * kTileT * 128), &vmap, hf * 128, row, c.layer, fb, l2_policy_evict_first());
        }
        if (++c.tile == c.tiles_b) {
          seg_start = true;
          if (idx + 1 < r1) next_pair(c, sCum, sLen, g.batch, g.h_kv);
        }
      }
      sFlags[3] = it;   // tile copies issued, for the drain at the end
      sFlags[1] = seg;  // query copies issued
    }
  } else if (warp == kEpilogueWarp) {
    if (p.k_new && has_work) {
      // fused step: this warp is idle until the first segment ends; it appends the new rows of the pairs
      // whose last tile this CTA loads while the producer is already streaming the tiles before them
      append_rows_by_warp<D>(g.batch, g.h_kv, g.capacity, g.k_layer_stride, g.v_layer_stride, p.k_new, p.v_new, p.k_cache_w,
                             p.v_cache_w, p.k_scale, p.v_scale, sPos, lane, r0, r1, sCum, sLen, p.status);
      if (lane == 0) mbar_arrive(appended0);
    }
    if (arrives_early(p)) arrive_early(p.seq_pos, p.exit_count, p.pkt ? p.epoch : nullptr, step, g.batch, g.capacity, lane);
    if (has_work)
      epilogue_warp<D, kDumpBufs>(p, lane, r0, r1, total, n_eff, sCum, sLen, sDump, sML, dfull0, dempty0, timed_out, sPeer, sComb, step);
  } else if (has_work) {
    // ================================ consumer warps ================================
    Cursor c = locate(r0, sCum, sLen, g.batch, g.h_kv);
    long long cur = r0;
    int it = 0, seg = 0;
    const uint32_t sK_addr = smem_u32(sK), sV_addr = smem_u32(sV);
    const int row_lo = warp * 16 + gq;   // K row of this thread inside a tile (and row_lo + 8)

    while (cur < r1) {
      const long long pair_start = cur - c.tile, pair_end = pair_start + c.tiles_b;
      const long long seg_end = pair_end < r1 ? pair_end : r1;
      const int ntiles = (int)(seg_end - cur);
      const int qb = seg & 1;

      // ---- query fragments (B operand of S^T = K q^T): head gq, dims hf*128 + 32*tq + 4*ks' ----
      // Each head is rescaled by a power of two so that its largest |q| lies in [1, 2): exact,
      // keeps every product inside f16 range whatever the magnitude of q.
      uint32_t qf[KSTEPS][2];
      float sc0, sc1;   // score multipliers of heads 2*tq and 2*tq+1 (this thread's S columns)
      {
        const bool qok = mbar_wait(qfull0 + 8u * qb, (seg >> 1) & 1, timed_out, p.status);
        float qv[DH][32];
        float amax = 0.f;
        if (gq < G && qok) {
          const uint32_t qaddr = smem_u32(sQ + qb * q_bytes) + (gq * D + 32 * tq) * 2;
#pragma unroll
          for (int hf = 0; hf < DH; ++hf) {
#pragma unroll
            for (int v4 = 0; v4 < 4; ++v4) {
              const uint4 raw = lds128(qaddr + hf * 256 + v4 * 16);
              const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                qv[hf][v4 * 8 + 2 * i] = bf16_bits_to_float(w[i] & 0xFFFFu);
                qv[hf][v4 * 8 + 2 * i + 1] = bf16_bits_to_float(w[i] >> 16);
              }
            }
          }
#pragma unroll
          for (int hf = 0; hf < DH; ++hf)
#pragma unroll
            for (int i = 0; i < 32; ++i) amax = fmaxf(amax, fabsf(qv[hf][i]));
        } else {
#pragma unroll
          for (int hf = 0; hf < DH; ++hf)
#pragma unroll
            for (int i = 0; i < 32; ++i) qv[hf][i] = 0.f;
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(qempty0 + 8u * qb);   // the query buffer may be refilled
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
        int ex = (int)((__float_as_uint(amax) >> 23) & 0xFF);
        // zero / denormal / inf / NaN heads: no rescale worth doing
        ex = ex < 1 ? 127 : (ex > 253 ? 253 : ex);
        const float down = __uint_as_float((uint32_t)(254 - ex) << 23);   // 2^(127-ex)
        const float up = __uint_as_float((uint32_t)ex << 23);             // 2^(ex-127)
#pragma unroll
        for (int hf = 0; hf < DH; ++hf)
#pragma unroll
          for (int w = 0; w < 8; ++w) {
            const float x0 = qv[hf][4 * w] * down, x1 = qv[hf][4 * w + 1] * down;
            const float x2 = qv[hf][4 * w + 2] * down, x3 = qv[hf][4 * w + 3] * down;
            __half2 b0 = __floats2half2_rn(x0, x1);
            __half2 b1 = __floats2half2_rn(x2, x3);
            qf[hf * 8 + w][0] = *reinterpret_cast<uint32_t*>(&b0);
            qf[hf * 8 + w][1] = *reinterpret_cast<uint32_t*>(&b1);
          }
        const float ks = p.k_scale[c.layer * g.h_kv + c.h] * p.score_scale;
        const float mult = up * ks;                       // held by the lanes of head gq
        sc0 = __shfl_sync(0xffffffffu, mult, 8 * tq);     // head 2*tq   lives in lanes 8*tq .. 8*tq+3
        sc1 = __shfl_sync(0xffffffffu, mult, 8 * tq + 4); // head 2*tq+1 lives in lanes 8*tq+4 ..
      }

      float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
      float o[KSTEPS][4];
#pragma unroll
      for (int j = 0; j < KSTEPS; ++j) { o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f; }

      for (int ti = 0; ti < ntiles; ++ti, ++it) {
        const int s = it % stages;
        const bool ok = mbar_wait(full0 + 8u * s, (it / stages) & 1, timed_out, p.status);
        const int tok0 = (c.tile + ti) * kTileT + warp * 16;   // first token of this warp's 16
        if (ok && tok0 < c.len_b) {
          // ---------------- S^T[16 tokens x 8 heads] = K q^T ----------------
          float sacc[4] = {0.f, 0.f, 0.f, 0.f}, sacc2[4] = {0.f, 0.f, 0.f, 0.f};   // two chains
          const uint32_t kt = sK_addr + s * TILE_BYTES;
#pragma unroll
          for (int hf = 0; hf < DH; ++hf) {
#pragma unroll
            for (int ch = 0; ch < 2; ++ch) {
              const uint32_t off = hf * kTileT * 128 + (((2 * tq + ch) ^ gq) << 4);
              const uint4 klo = lds128(kt + off + row_lo * 128);
              const uint4 khi = lds128(kt + off + (row_lo + 8) * 128);
              const uint32_t wl[4] = {klo.x, klo.y, klo.z, klo.w};
              const uint32_t wh[4] = {khi.x, khi.y, khi.z, khi.w};
#pragma unroll
              for (int wi = 0; wi < 4; ++wi) {
                const int ks = hf * 8 + ch * 4 + wi;
                if (wi & 1)
                  mma_f16(sacc2, cvt_lo(wl[wi]), cvt_lo(wh[wi]), cvt_hi(wl[wi]), cvt_hi(wh[wi]), qf[ks][0], qf[ks][1]);
                else
                  mma_f16(sacc, cvt_lo(wl[wi]), cvt_lo(wh[wi]), cvt_hi(wl[wi]), cvt_hi(wh[wi]), qf[ks][0], qf[ks][1]);
              }
            }
          }
          // ---------------- online softmax (log2 domain) ----------------
          float s0 = (sacc[0] + sacc2[0]) * sc0, s1 = (sacc[1] + sacc2[1]) * sc1;
          float s2 = (sacc[2] + sacc2[2]) * sc0, s3 = (sacc[3] + sacc2[3]) * sc1;
          if (tok0 + gq >= c.len_b) { s0 = -INFINITY; s1 = -INFINITY; }
          if (tok0 + gq + 8 >= c.len_b) { s2 = -INFINITY; s3 = -INFINITY; }
          float mx0 = fmaxf(s0, s2), mx1 = fmaxf(s1, s3);
#pragma unroll
          for (int off = 4; off < 32; off <<= 1) {
            mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, off));
            mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, off));
          }
          const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
          const float ms0 = mn0 == -INFINITY ? 0.f : mn0, ms1 = mn1 == -INFINITY ? 0.f : mn1;
          const float al0 = ex2(m0 - ms0), al1 = ex2(m1 - ms1);
          const float p0 = ex2(s0 - ms0), p1 = ex2(s1 - ms1), p2 = ex2(s2 - ms0), p3 = ex2(s3 - ms1);
          m0 = mn0; m1 = mn1;
          l0 = l0 * al0 + (p0 + p2);
          l1 = l1 * al1 + (p1 + p3);
          if (__any_sync(0xffffffffu, al0 != 1.f || al1 != 1.f)) {
#pragma unroll
            for (int j = 0; j < KSTEPS; ++j) { o[j][0] *= al0; o[j][1] *= al1; o[j][2] *= al0; o[j][3] *= al1; }
          }
          // P^T fragments (B operand of O^T += V^T P^T): transpose [token x head] -> [head x token]
          __half2 pa = __floats2half2_rn(p0, p1), pb = __floats2half2_rn(p2, p3);
          const uint32_t pb0 = movmatrix_trans(*reinterpret_cast<uint32_t*>(&pa));
          const uint32_t pb1 = movmatrix_trans(*reinterpret_cast<uint32_t*>(&pb));

          // ---------------- O^T[D dims x 8 heads] += V^T P^T ----------------
          const uint32_t vt = sV_addr + s * TILE_BYTES;
          const int vr = warp * 16 + 2 * tq;   // V rows vr, vr+1, vr+8, vr+9
          const bool tail = tok0 + 16 > c.len_b;
#pragma unroll
          for (int hf = 0; hf < DH; ++hf) {
            const uint32_t vb = vt + hf * kTileT * 128;
            uint4 va = lds128(vb + vr * 128 + ((gq ^ (2 * tq)) << 4));
            uint4 vbb = lds128(vb + (vr + 1) * 128 + ((gq ^ (2 * tq + 1)) << 4));
            uint4 vc = lds128(vb + (vr + 8) * 128 + ((gq ^ (2 * tq)) << 4));
            uint4 vd = lds128(vb + (vr + 9) * 128 + ((gq ^ (2 * tq + 1)) << 4));
            if (tail) {   // slots at or beyond the valid length may hold anything, NaN patterns included
              const int tv = tok0 + 2 * tq;
              const uint4 z = make_uint4(0, 0, 0, 0);
              if (tv >= c.len_b) va = z;
              if (tv + 1 >= c.len_b) vbb = z;
              if (tv + 8 >= c.len_b) vc = z;
              if (tv + 9 >= c.len_b) vd = z;
            }
            const uint32_t wa[4] = {va.x, va.y, va.z, va.w}, wb[4] = {vbb.x, vbb.y, vbb.z, vbb.w};
            const uint32_t wc[4] = {vc.x, vc.y, vc.z, vc.w}, wd[4] = {vd.x, vd.y, vd.z, vd.w};
#pragma unroll
            for (int wi = 0; wi < 4; ++wi) {
              const uint32_t x01 = prmt(wa[wi], wb[wi], 0x5140), x23 = prmt(wa[wi], wb[wi], 0x7362);
              const uint32_t y01 = prmt(wc[wi], wd[wi], 0x5140), y23 = prmt(wc[wi], wd[wi], 0x7362);
              mma_f16(o[hf * 8 + 2 * wi], cvt_lo(x01), cvt_hi(x01), cvt_lo(y01), cvt_hi(y01), pb0, pb1);
              mma_f16(o[hf * 8 + 2 * wi + 1], cvt_lo(x23), cvt_hi(x23), cvt_lo(y23), cvt_hi(y23), pb0, pb1);
            }
          }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(empty0 + 8u * s);
      }

      // ---------------- end of segment: hand the warp's state to the epilogue warp ----------------
#pragma unroll
      for (int off = 4; off < 32; off <<= 1) {
        l0 += __shfl_xor_sync(0xffffffffu, l0, off);
        l1 += __shfl_xor_sync(0xffffffffu, l1, off);
      }
      const int db = seg % kDumpBufs;
      if (seg < kDumpBufs || mbar_wait(dempty0 + 8u * db, ((seg / kDumpBufs) - 1) & 1, timed_out, p.status)) {
        float* ml = sML + (db * kConsumerWarps + warp) * 16;
        if (gq == 0) {
          ml[2 * tq] = m0; ml[2 * tq + 1] = m1;
          ml[8 + 2 * tq] = l0; ml[8 + 2 * tq + 1] = l1;
        }
        // o[j]: regs 0,1 -> dim (j>>3)*128 + 16*gq + 2*(j&7) of heads 2*tq, 2*tq+1; regs 2,3 -> that dim + 1
        const uint32_t dbase = smem_u32(sDump + (db * kConsumerWarps + warp) * dump_warp_floats);
        const int h0 = 2 * tq, h1 = 2 * tq + 1;
#pragma unroll
        for (int j = 0; j < KSTEPS; ++j) {
          const int u = (j >> 3) * 64 + 8 * gq + (j & 7);
          const uint32_t pos8 = 8u * (uint32_t)((u & ~7) | ((j & 7) ^ gq));
          if (h0 < G) sts64(dbase + h0 * DP * 4 + pos8, o[j][0], o[j][2]);
          if (h1 < G) sts64(dbase + h1 * DP * 4 + pos8, o[j][1], o[j][3]);
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(dfull0 + 8u * db);
      ++seg;
      cur = seg_end;
      if (cur < r1) next_pair(c, sCum, sLen, g.batch, g.h_kv);
    }
  }
  __syncthreads();
  if (sFlags[0] && tid == kConsumerThreads) {
    // A wait gave up.  Copies already issued still land in this CTA's shared memory: wait for
    // them (bounded) so the CTA does not retire underneath them.
    const int it = sFlags[3], segs = sFlags[1];
    for (int s = 0; s < stages && s < it; ++s) {
      const int last_it = ((it - 1 - s) / stages) * stages + s;   // last iteration that used stage s
      const uint32_t par = (last_it / stages) & 1;
      const unsigned long long t0 = global_timer_ns();
      while (!mbar_try_wait(full0 + 8u * s, par) && global_timer_ns() - t0 < kWaitBudgetNs) {}
    }
    for (int qb = 0; qb < 2 && qb < segs; ++qb) {
      const int last_seg = ((segs - 1 - qb) / 2) * 2 + qb;
      const unsigned long long t0 = global_timer_ns();
      while (!mbar_try_wait(qfull0 + 8u * qb, (last_seg >> 1) & 1) && global_timer_ns() - t0 < kWaitBudgetNs) {}
    }
  }
  // the pair whose last piece this CTA holds: all warps collect the other pieces (they end when this CTA's range does)
  if (sComb->valid && !sFlags[0]) combine_deferred<D>(combine_args_of(p, sPeer, step), *sComb, warp, kThreads / 32, lane);
  if (p.bar_world) __syncthreads();   // stores mode: every warp's peer stores are fenced before the CTA counts as finished
  end_of_launch(p, tid, kThreads, step);
}

constexpr int kStages = 3;   // ring depth.  A deeper ring where a small grid leaves shared memory unused (short caches, up to
                             // 12 stages at one CTA per SM) changed nothing: there the consumer chain is the limit, not the copies

size_t smem_bytes_for(const Geometry& g, int stages) {
  size_t b = 1024;                                            // alignment slack
  b += (size_t)2 * stages * kTileT * g.head_dim;              // K and V rings
  b += (size_t)2 * g.group * g.head_dim * 2;                  // query rows, double buffered
  b += (size_t)kDumpBufs * kConsumerWarps * g.group * (g.head_dim + 4) * 4;   // dumped warp states
  b += (size_t)kDumpBufs * kConsumerWarps * 16 * 4;                   // their m, l
  b += (size_t)(2 * stages + 9) * 8;                          // barriers
  b += 64;                                                    // destinations of the tensor-parallel output
  b += sizeof(DeferredCombine);                               // the pair finished at the CTA's end
  b += 16;                                                    // flags
  b += (size_t)(3 * g.batch + 2) * 4;                         // sLen, sCum, sPos, the step counter
  return (b + 15) & ~(size_t)15;
}

}  // namespace

size_t mma_workspace_bytes(const Geometry& g, int num_ctas) {
  size_t b = (size_t)num_ctas * 2 * partial_slot_words(g.group, g.head_dim) * 8;   // two tagged partials per CTA
  b += 16;                                                                            // exit counter of the fused step
  return (b + 255) & ~(size_t)255;
}

// The persistent grid: every CTA slot of the device.  Exception, short caches (at most kAlignMaxTiles tiles per
// pair at the given length): the kernel gives every CTA whole pairs (cta_range), and CTAs beyond the ones that
// get work only cost launch time (depth 512, 512 pairs: 444 CTAs 21.6 us, 256 CTAs 20.0 us; splitting the pairs
// of a small shard over more CTAs is slower than one pair per CTA: 128 pairs on 128 / 256 / 384 CTAs 11.8 / 15.4 /
// 17.0 us): the grid is the smallest one that gives every CTA the same number of pairs.
int mma_pick_ctas(const Geometry& g, int max_seq_len, int num_sms) {
  const size_t smem = smem_bytes_for(g, kStages);
  int per_sm = (int)((227 * 1024) / (smem + 1024));   // + per-CTA reservation
  if (per_sm < 1) per_sm = 1;
  if (per_sm > kCtasPerSm) per_sm = kCtasPerSm;
  const int full = num_sms * per_sm;
  const long long pairs = (long long)g.n_layers * g.batch * g.h_kv;
  const int tiles = (max_seq_len + kTileT - 1) / kTileT;
  if (tiles >= 1 && tiles <= kAlignMaxTiles) {
    const long long k = (pairs + full - 1) / full;
    return (int)((pairs + k - 1) / k);
  }
  // long caches: three CTAs per SM keep HBM busiest; a small amount of work (a KV-head shard: fewer than 256 tiles
  // per SM) runs better on two per SM, which is also the instance without the register cap (64 layers x 1 KV head
  // at depth 8192: 444 CTAs 34.4 us, 296 CTAs 32.3 us; 2 KV heads: 53.5 / 51.8 us)
  if (per_sm > 2 && pairs * tiles < 256LL * num_sms) return 2 * num_sms;
  return full;
}

cudaError_t launch_decode_mma(const Geometry& g, const DecodeArgs& a, cudaStream_t stream) {
  if (g.scale_mode != B200ATTN_SCALE_PER_HEAD || g.batch > kMaxBatchMma) return cudaErrorNotSupported;
  CUtensorMap kmap, vmap;
  if (!encode_cache_map(&kmap, a.k_cache, g, g.k_layer_stride, kTileT) || !encode_cache_map(&vmap, a.v_cache, g, g.v_layer_stride, kTileT))
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
  p.stages = kStages;
  p.k_new = (const uint16_t*)a.k_new;
  p.v_new = (const uint16_t*)a.v_new;
  p.k_cache_w = (uint8_t*)a.k_cache;
  p.v_cache_w = (uint8_t*)a.v_cache;
  p.seq_pos = a.seq_pos;
  p.exit_count = (int*)(p.ws_pkt + (size_t)n * 2 * partial_slot_words(g.group, g.head_dim));
  for (int r = 0; r < 8; ++r) p.bar_flags[r] = r < a.bar_world ? a.bar_flags[r] : nullptr;
  p.bar_rank = a.bar_rank;
  p.bar_world = a.bar_world;
  const size_t smem = smem_bytes_for(g, p.stages);
  auto launch = [&](auto kernel) -> cudaError_t {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    if (p.pkt) {   // may every CTA wait for remote packets?  only if the whole grid is resident at once
      int per_sm = 0;
      e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, kThreads, smem);
      if (e != cudaSuccess) return e;
      p.pkt_resident = (long long)per_sm * device_sms() >= n ? 1 : 0;
    }
    return launch_pdl(kernel, n, kThreads, smem, stream, kmap, vmap, p);
  };
  if (g.head_dim != 128) return launch(attn_streamk_mma_kernel<256, 1>);
  return n <= 2 * device_sms() ? launch(attn_streamk_mma_kernel<128, 2>) : launch(attn_streamk_mma_kernel<128, kCtasPerSm>);
}

}  // namespace b200attn


