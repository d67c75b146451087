// tcgen05 variant of the stream-K decode attention: the score GEMM runs on the 5th-generation
// tensor cores straight from the TMA-staged FP8 bytes.
//
// Same persistent stream-K structure, producer warp, epilogue warp, dump layout and fused combine
// as decode_mma.cu; what changes is who computes S = K q^T:
//   * tiles are 128 tokens; the K tile lands in shared memory in the TMA 128-byte-swizzle layout,
//     which is exactly the K-major canonical operand layout of tcgen05.mma, so an MMA-issuer warp
//     feeds it UNCONVERTED to `tcgen05.mma.cta_group::1.kind::f8f6f4` (M = 128 tokens, N = 16,
//     K = 32 dims per instruction).  No K byte ever passes through a register or a convert;
//   * the query is the B operand: per (layer, sequence, kv head) the issuer warp writes, for each
//     of the G heads, two e4m3 rows — the leading part of q (sign, exponent, 3 mantissa bits) in
//     N-row h and the remainder in N-row 8+h; a bf16 value has 8 significant bits, so the two
//     terms carry it exactly (up to a 2^-10 floor relative to the head's largest element);
//   * scores accumulate in fp32 in tensor memory (two 16-column buffers, so the tensor core works
//     on tile i+1 while tile i is in softmax); consumer warp w reads its 32 token rows with
//     `tcgen05.ld.32x32b.x16`: one thread = one token, s[h] = (col h + col 8+h) * scale;
//   * the online softmax keeps one running maximum per warp and head (`redux.sync.max`), the
//     probabilities go through a 512-byte per-warp shared-memory exchange into mma.sync B
//     fragments, and O^T += V^T P^T stays on mma.sync.m16n8k16.f16 with in-register widening of V
//     exactly as in decode_mma.cu (probabilities in f16, accumulation in fp32).
// This halves the FP8->f16 convert work (the limiter of decode_mma.cu: the XU pipe) and removes
// the K fragment loads and the score MMAs from the consumer warps.
//
// Every wait (TMA barriers, tcgen05.commit barriers, buffer hand-offs) is bounded as in
// decode_mma.cu; tensor memory is allocated by the issuer warp at kernel start and always freed
// by it at the end, after all warps have passed the final barrier.
#include "tcgen05.cuh"

namespace b200attn {

namespace {

constexpr int kTileU = 128;                          // tokens per tile = M of the score MMA
constexpr int kIssuerWarp = kConsumerWarps + 2;      // warp 6: tcgen05.mma issue, query operand, TMEM alloc
constexpr int kThreadsU = kConsumerThreads + 96;
constexpr int kKStages = 2;                          // K ring (freed as soon as the score MMA completes)
constexpr int kTmemCols = 32;                        // two score buffers of 16 fp32 columns

template <int D>
__global__ void __launch_bounds__(kThreadsU)
attn_streamk_umma_kernel(const __grid_constant__ CUtensorMap kmap, const __grid_constant__ CUtensorMap vmap,
                         const MmaParams p) {
  constexpr int DH = D / 128;              // 128-byte column blocks per row
  constexpr int KSTEPS = D / 16;           // mma.sync tiles for PV
  constexpr int TILE_BYTES = kTileU * D;   // one K (or V) tile
  constexpr int DP = D + 4;                // padded head row of a dumped state, in floats
  constexpr int QOP_BYTES = DH * 16 * 128; // query operand: 16 N-rows x 128 bytes per 128-dim block
  const Geometry& g = p.g;
  const int G = g.group;
  const int vstages = p.stages;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int gq = lane >> 2, tq = lane & 3;
  const uint32_t q_bytes = (uint32_t)G * D * 2;
  const int dump_warp_floats = G * DP;

  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  uint8_t* smem = smem_raw + (((raw_addr + 1023u) & ~1023u) - raw_addr);
  uint8_t* sK = smem;                                                                 // [kKStages][TILE_BYTES]
  uint8_t* sV = sK + (size_t)kKStages * TILE_BYTES;                                   // [vstages][TILE_BYTES]
  uint8_t* sQop = sV + (size_t)vstages * TILE_BYTES;                                  // [2][QOP_BYTES], 1024-aligned
  uint8_t* sQraw = sQop + 2 * QOP_BYTES;                                              // [2][G*D] bf16
  uint8_t* sP = sQraw + 2 * q_bytes;                                                  // [4 warps][8 heads][32 tokens] f16
  float* sScale = reinterpret_cast<float*>(sP + kConsumerWarps * 512);                // [2][8]
  float* sDump = sScale + 16;                                                         // [1][4][G][DP]
  float* sML = sDump + kConsumerWarps * dump_warp_floats;                             // [1][4][16]
  uint64_t* bars = reinterpret_cast<uint64_t*>(sML + kConsumerWarps * 16);
  // barrier map (8 bytes each)
  const uint32_t kfull0 = smem_u32(bars), kempty0 = kfull0 + 8u * kKStages;
  const uint32_t vfull0 = kempty0 + 8u * kKStages, vempty0 = vfull0 + 8u * vstages;
  const uint32_t qrfull0 = vempty0 + 8u * vstages, qrempty0 = qrfull0 + 16u;
  const uint32_t qinfo0 = qrempty0 + 16u, sfull0 = qinfo0 + 16u, sempty0 = sfull0 + 16u;
  const uint32_t dfull0 = sempty0 + 16u, dempty0 = dfull0 + 8u;
  constexpr int kFixedBars = 2 * kKStages + 12;
  int* sFlags = reinterpret_cast<int*>(bars + kFixedBars + 2 * vstages);   // [0] timed_out [1] tmem base [2] any_empty
  int* sLen = sFlags + 8;
  int* sCum = sLen + g.batch;
  volatile int* timed_out = sFlags;

  if (tid == 0) {
    for (int s = 0; s < kKStages; ++s) { mbar_init(kfull0 + 8u * s, 1); mbar_init(kempty0 + 8u * s, 1); }
    for (int s = 0; s < vstages; ++s) { mbar_init(vfull0 + 8u * s, 1); mbar_init(vempty0 + 8u * s, kConsumerWarps); }
    for (int i = 0; i < 2; ++i) {
      mbar_init(qrfull0 + 8u * i, 1);
      mbar_init(qrempty0 + 8u * i, 1);
      mbar_init(qinfo0 + 8u * i, 1);
      mbar_init(sfull0 + 8u * i, 1);
      mbar_init(sempty0 + 8u * i, kConsumerWarps);
    }
    mbar_init(dfull0, kConsumerWarps);
    mbar_init(dempty0, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    sFlags[0] = 0; sFlags[3] = 0; sFlags[4] = 0; sFlags[5] = 0; sFlags[6] = 0;
    int acc = 0, any_empty = 0, st = 0, uniform = 1;
    for (int b = 0; b < g.batch; ++b) {
      int len = p.seq_len[b] + p.seq_len_offset;
      if (len < 0) { len = 0; st |= B200ATTN_STATUS_LEN_NEGATIVE; }
      if (len > g.capacity) { len = g.capacity; st |= B200ATTN_STATUS_LEN_OVER_CAP; }
      sLen[b] = len;
      sCum[b] = acc;
      acc += (len + kTileU - 1) / kTileU;
      any_empty |= len == 0;
      uniform &= b == 0 || acc - sCum[b] == sCum[1] - sCum[0];
    }
    sCum[g.batch] = acc;
    sFlags[2] = any_empty | (uniform ? 2 : 0);
    if (st && blockIdx.x == 0) atomicOr(p.status, st);
  }
  if (warp == kProducerWarp && lane == 0) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(&kmap) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&vmap) : "memory");
  }
  if (warp == kIssuerWarp) tmem_alloc(smem_u32(sFlags + 1), kTmemCols);
  if (warp < kConsumerWarps) {   // the exchange area feeds unused N columns too: keep it finite
    for (int i = lane; i < 128; i += 32) reinterpret_cast<uint32_t*>(sP + warp * 512)[i] = 0;
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = (uint32_t)sFlags[1];

  if (sFlags[2] & 1) {   // sequences of length 0 have no tiles: their outputs are zero
    const long long rows = (long long)g.n_layers * g.batch;
    for (long long r = blockIdx.x; r < rows; r += gridDim.x) {
      if (sLen[r % g.batch] == 0)
        for (int i = tid; i < g.h_q * D; i += kThreadsU) {
          if (p.n_out == 0) p.out[r * g.h_q * D + i] = 0;
          else
            for (int pr = 0; pr < p.n_out; ++pr) p.out_peer[pr][(r * p.out_hq_total + p.out_head_base) * D + i] = 0;
        }
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
      Cursor c = locate(r0, sCum, sLen, g.batch, g.h_kv);
      int it = 0, seg = 0;
      bool seg_start = true;
      for (long long idx = r0; idx < r1; ++idx, ++it) {
        if (seg_start) {   // the G query rows of this pair, once per segment
          const int qb = seg & 1;
          if (seg >= 2 && !mbar_wait(qrempty0 + 8u * qb, ((seg >> 1) - 1) & 1, timed_out, p.status)) break;
          mbar_arrive_expect_tx(qrfull0 + 8u * qb, q_bytes);
          const long long lb = (long long)c.layer * g.batch + c.b;
          bulk_load(smem_u32(sQraw + qb * q_bytes), p.q + (lb * g.h_q + c.h * G) * D, q_bytes, qrfull0 + 8u * qb);
          ++seg;
          seg_start = false;
        }
        const int row = (c.b * g.h_kv + c.h) * g.capacity + c.tile * kTileU;
        const int ks = it % kKStages, vs = it % vstages;
        if (it >= kKStages && !mbar_wait(kempty0 + 8u * ks, ((it / kKStages) - 1) & 1, timed_out, p.status)) break;
        mbar_arrive_expect_tx(kfull0 + 8u * ks, TILE_BYTES);
#pragma unroll
        for (int hf = 0; hf < DH; ++hf)
          tma_load_3d(smem_u32(sK + (size_t)ks * TILE_BYTES + hf * kTileU * 128), &kmap, hf * 128, row, c.layer, kfull0 + 8u * ks);
        sFlags[3] = it + 1;   // K copies issued
        if (it >= vstages && !mbar_wait(vempty0 + 8u * vs, ((it / vstages) - 1) & 1, timed_out, p.status)) break;
        mbar_arrive_expect_tx(vfull0 + 8u * vs, TILE_BYTES);
#pragma unroll
        for (int hf = 0; hf < DH; ++hf)
          tma_load_3d(smem_u32(sV + (size_t)vs * TILE_BYTES + hf * kTileU * 128), &vmap, hf * 128, row, c.layer, vfull0 + 8u * vs);
        sFlags[4] = it + 1;   // V copies issued
        if (++c.tile == c.tiles_b) {
          seg_start = true;
          if (idx + 1 < r1) next_pair(c, sCum, sLen, g.batch, g.h_kv);
        }
      }
      sFlags[5] = seg;   // query copies issued
    }
  } else if (warp == kEpilogueWarp) {
    if (has_work)
      epilogue_warp<D, 1>(p, lane, r0, r1, total, n_eff, sCum, sLen, sDump, sML, dfull0, dempty0, timed_out);
  } else if (warp == kIssuerWarp) {
    // ===================== issuer warp: query operand + tcgen05.mma for S = K q^T =====================
    if (has_work) {
      Cursor c = locate(r0, sCum, sLen, g.batch, g.h_kv);
      int it = 0, seg = 0;
      bool seg_start = true;
      int qb = 0;
      bool alive = true;
      for (long long idx = r0; idx < r1 && alive; ++idx, ++it) {
        const int sb = it & 1;
        // the score buffer (and, two tiles back, the query operand of that segment) is free again
        if (it >= 2) alive = mbar_wait(sempty0 + 8u * sb, ((it >> 1) - 1) & 1, timed_out, p.status);
        if (alive && seg_start) {
          qb = seg & 1;
          alive = mbar_wait(qrfull0 + 8u * qb, (seg >> 1) & 1, timed_out, p.status);
          if (alive) {
            // Each head h: row h = leading e4m3 part of q * 2^e, row 8+h = remainder; lane owns 4 dims
            // per 128-dim block.  2^e puts the head's largest |q| into [128, 256).
            const uint32_t qraw = smem_u32(sQraw + qb * q_bytes), qop = smem_u32(sQop + qb * QOP_BYTES);
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
              if (lane == 0) sScale[qb * 8 + h] = up * p.k_scale[c.layer * g.h_kv + c.h] * p.score_scale;
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // operand bytes -> visible to the tensor core
            __syncwarp();
            if (lane == 0) {
              mbar_arrive(qrempty0 + 8u * qb);   // raw query buffer may be refilled
              mbar_arrive(qinfo0 + 8u * qb);     // scales are in place for the consumers
            }
          }
          ++seg;
          seg_start = false;
        }
        const int ks = it % kKStages;
        if (alive) alive = mbar_wait(kfull0 + 8u * ks, (it / kKStages) & 1, timed_out, p.status);
        if (alive) {
          tc_fence_after();
          if (lane == 0) {
            const uint32_t a0 = smem_u32(sK + (size_t)ks * TILE_BYTES), b0 = smem_u32(sQop + qb * QOP_BYTES);
            const uint32_t d = tmem_base + (uint32_t)sb * 16u;
#pragma unroll
            for (int hf = 0; hf < DH; ++hf)
#pragma unroll
              for (int kb = 0; kb < 4; ++kb)
                umma_f8(d, smem_desc_k128(a0 + hf * kTileU * 128 + kb * 32), smem_desc_k128(b0 + hf * 2048 + kb * 32),
                        kIdescQK, (hf | kb) ? 1u : 0u);
            umma_commit(sfull0 + 8u * sb);     // scores of this tile are complete
            umma_commit(kempty0 + 8u * ks);    // and the K tile has been read
          }
          __syncwarp();
        }
        if (++c.tile == c.tiles_b) {
          seg_start = true;
          if (idx + 1 < r1) next_pair(c, sCum, sLen, g.batch, g.h_kv);
        }
      }
      if (lane == 0) sFlags[6] = it;   // score MMAs issued
    }
  } else if (has_work) {
    // ================================ consumer warps ================================
    Cursor c = locate(r0, sCum, sLen, g.batch, g.h_kv);
    long long cur = r0;
    int it = 0, seg = 0;
    const uint32_t sV_addr = smem_u32(sV);
    const uint32_t sP_addr = smem_u32(sP + warp * 512);   // [8 heads][32 tokens] f16
    const uint32_t tmem_lane = tmem_base + ((uint32_t)(warp * 32) << 16);

    while (cur < r1) {
      const long long pair_start = cur - c.tile, pair_end = pair_start + c.tiles_b;
      const long long seg_end = pair_end < r1 ? pair_end : r1;
      const int ntiles = (int)(seg_end - cur);
      const int qb = seg & 1;

      float sc[kMaxGroup];   // score multipliers per head: 2^-e * k_scale * softmax_scale * log2(e)
      {
        const bool ok = mbar_wait(qinfo0 + 8u * qb, (seg >> 1) & 1, timed_out, p.status);
#pragma unroll
        for (int h = 0; h < kMaxGroup; ++h) sc[h] = (ok && h < G) ? sScale[qb * 8 + h] : 0.f;
      }
      float m[kMaxGroup], l[kMaxGroup];
#pragma unroll
      for (int h = 0; h < kMaxGroup; ++h) { m[h] = -INFINITY; l[h] = 0.f; }
      float o[KSTEPS][4];
#pragma unroll
      for (int j = 0; j < KSTEPS; ++j) { o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f; }

      for (int ti = 0; ti < ntiles; ++ti, ++it) {
        const int sb = it & 1, vs = it % vstages;
        const int tok0 = (c.tile + ti) * kTileU + warp * 32;   // first token of this warp's 32
        const bool sok = mbar_wait(sfull0 + 8u * sb, (it >> 1) & 1, timed_out, p.status);
        uint32_t r[16];
        const bool active = sok && tok0 < c.len_b;
        if (active) {
          tc_fence_after();
          tmem_ld16(tmem_lane + (uint32_t)sb * 16u, r);
          tc_fence_before();
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(sempty0 + 8u * sb);   // the score buffer may be overwritten
        if (active) {
          // ---------------- online softmax: one thread = one token ----------------
          const bool valid = tok0 + lane < c.len_b;
          float pr[kMaxGroup], al[kMaxGroup];
          bool changed = false;
#pragma unroll
          for (int h = 0; h < kMaxGroup; ++h) {
            if (h < G) {
              float s = (__uint_as_float(r[h]) + __uint_as_float(r[8 + h])) * sc[h];
              if (!valid) s = -INFINITY;
              const float mn = fmaxf(m[h], warp_max(s));
              const float ms = mn == -INFINITY ? 0.f : mn;
              al[h] = ex2(m[h] - ms);
              pr[h] = ex2(s - ms);
              changed |= al[h] != 1.f;
              m[h] = mn;
              l[h] = l[h] * al[h] + pr[h];
            } else {
              al[h] = 1.f;
              pr[h] = 0.f;
            }
          }
          if (changed) {   // m is warp-uniform, so is this branch
            const float a0 = tq == 0 ? al[0] : tq == 1 ? al[2] : tq == 2 ? al[4] : al[6];
            const float a1 = tq == 0 ? al[1] : tq == 1 ? al[3] : tq == 2 ? al[5] : al[7];
#pragma unroll
            for (int j = 0; j < KSTEPS; ++j) { o[j][0] *= a0; o[j][1] *= a1; o[j][2] *= a0; o[j][3] *= a1; }
          }
          // probabilities -> [head][token] f16 exchange -> mma.sync B fragments
          __syncwarp();
#pragma unroll
          for (int h = 0; h < kMaxGroup; ++h)
            if (h < G) sts16(sP_addr + (h * 32 + lane) * 2, __half_as_ushort(__float2half_rn(pr[h])));
          __syncwarp();

        }
        // Every warp waits for the V tile before releasing it, working on it or not: an arrival
        // must never run ahead into the stage's next use.
        const bool vok = mbar_wait(vfull0 + 8u * vs, (it / vstages) & 1, timed_out, p.status);
        if (active) {
          // ---------------- O^T[D dims x 8 heads] += V^T P^T, two 16-token blocks ----------------
          if (vok) {
            const uint32_t vt = sV_addr + vs * TILE_BYTES;
#pragma unroll
            for (int bk = 0; bk < 2; ++bk) {
              const int t0 = tok0 + 16 * bk;
              if (t0 < c.len_b) {
                const uint32_t pb0 = lds32(sP_addr + (gq * 32 + 16 * bk + 2 * tq) * 2);
                const uint32_t pb1 = lds32(sP_addr + (gq * 32 + 16 * bk + 2 * tq + 8) * 2);
                const int vr = warp * 32 + 16 * bk + 2 * tq;   // V rows vr, vr+1, vr+8, vr+9
                const bool tail = t0 + 16 > c.len_b;
#pragma unroll
                for (int hf = 0; hf < DH; ++hf) {
                  const uint32_t vb = vt + hf * kTileU * 128;
                  uint4 va = lds128(vb + vr * 128 + ((gq ^ (2 * tq)) << 4));
                  uint4 vbb = lds128(vb + (vr + 1) * 128 + ((gq ^ (2 * tq + 1)) << 4));
                  uint4 vc = lds128(vb + (vr + 8) * 128 + ((gq ^ (2 * tq)) << 4));
                  uint4 vd = lds128(vb + (vr + 9) * 128 + ((gq ^ (2 * tq + 1)) << 4));
                  if (tail) {   // slots at or beyond the valid length may hold anything, NaN patterns included
                    const int tv = t0 + 2 * tq;
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
            }
          }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(vempty0 + 8u * vs);
      }

      // ---------------- end of segment: hand the warp's state to the epilogue warp ----------------
#pragma unroll
      for (int h = 0; h < kMaxGroup; ++h) {
        if (h < G) {
#pragma unroll
          for (int off = 16; off > 0; off >>= 1) l[h] += __shfl_xor_sync(0xffffffffu, l[h], off);
        }
      }
      if (seg < 1 || mbar_wait(dempty0, (seg - 1) & 1, timed_out, p.status)) {
        float* ml = sML + warp * 16;
        if (lane == 0) {
#pragma unroll
          for (int h = 0; h < kMaxGroup; ++h) { ml[h] = m[h]; ml[8 + h] = l[h]; }
        }
        const uint32_t dbase = smem_u32(sDump + warp * dump_warp_floats);
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
      if (lane == 0) mbar_arrive(dfull0);
      ++seg;
      cur = seg_end;
      if (cur < r1) next_pair(c, sCum, sLen, g.batch, g.h_kv);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == kIssuerWarp) {
    if (sFlags[0] && lane == 0) {
      // A wait gave up.  Operations already issued still target this CTA's shared and tensor
      // memory: wait for them (bounded) before the CTA retires and the columns are freed.
      const int nk = sFlags[3], nv = sFlags[4], nq = sFlags[5], ns = sFlags[6];
      auto drain = [&](uint32_t bar0, int ring, int issued) {
        for (int s = 0; s < ring && s < issued; ++s) {
          const int last = ((issued - 1 - s) / ring) * ring + s;
          const unsigned long long t0 = global_timer_ns();
          while (!mbar_try_wait(bar0 + 8u * s, (last / ring) & 1) && global_timer_ns() - t0 < kWaitBudgetNs) {}
        }
      };
      drain(kfull0, kKStages, nk);
      drain(vfull0, vstages, nv);
      drain(qrfull0, 2, nq);
      drain(sfull0, 2, ns);
    }
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

int vstages_for(const Geometry& g) { return g.head_dim == 128 ? 3 : 2; }

size_t umma_smem_bytes(const Geometry& g, int vstages) {
  const int dh = g.head_dim / 128;
  size_t b = 1024;                                                   // alignment slack
  b += (size_t)(kKStages + vstages) * kTileU * g.head_dim;           // K and V rings
  b += (size_t)2 * dh * 16 * 128;                                    // query operand, double buffered
  b += (size_t)2 * g.group * g.head_dim * 2;                         // raw query rows, double buffered
  b += (size_t)kConsumerWarps * 512;                                 // probability exchange
  b += 16 * 4;                                                       // scales
  b += (size_t)kConsumerWarps * g.group * (g.head_dim + 4) * 4;      // dumped warp states
  b += (size_t)kConsumerWarps * 16 * 4;                              // their m, l
  b += (size_t)(2 * kKStages + 12 + 2 * vstages) * 8;                // barriers
  b += 32;                                                           // flags
  b += (size_t)(2 * g.batch + 1) * 4;                                // sLen, sCum
  return (b + 15) & ~(size_t)15;
}

}  // namespace

int umma_pick_ctas(const Geometry& g, int max_seq_len, int num_sms) {
  (void)max_seq_len;
  const size_t smem = umma_smem_bytes(g, vstages_for(g));
  int per_sm = (int)((227 * 1024) / (smem + 1024));
  if (per_sm < 1) per_sm = 1;
  if (per_sm > 2) per_sm = 2;
  return num_sms * per_sm;
}

cudaError_t launch_decode_umma(const Geometry& g, const DecodeArgs& a, cudaStream_t stream) {
  if (g.scale_mode != B200ATTN_SCALE_PER_HEAD || g.batch > kMaxBatchMma) return cudaErrorNotSupported;
  CUtensorMap kmap, vmap;
  if (!encode_cache_map(&kmap, a.k_cache, g, g.k_layer_stride, kTileU) ||
      !encode_cache_map(&vmap, a.v_cache, g, g.v_layer_stride, kTileU))
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
  p.ws_acc = (float*)a.workspace;
  p.ws_ml = p.ws_acc + (size_t)n * 2 * g.group * g.head_dim;
  p.tickets = (int*)(p.ws_ml + (size_t)n * 2 * 16);
  p.out = (uint16_t*)a.out;
  p.gate = (const uint16_t*)a.gate;
  p.n_out = a.n_out;
  p.out_hq_total = a.n_out ? a.out_hq_total : g.h_q;
  p.out_head_base = a.n_out ? a.out_head_base : 0;
  for (int r = 0; r < 8; ++r) p.out_peer[r] = r < a.n_out ? (uint16_t*)a.out_peer[r] : nullptr;
  p.status = a.status;
  p.stages = vstages_for(g);
  const size_t smem = umma_smem_bytes(g, p.stages);
  auto launch = [&](auto kernel) -> cudaError_t {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    kernel<<<n, kThreadsU, smem, stream>>>(kmap, vmap, p);
    return cudaGetLastError();
  };
  return g.head_dim == 128 ? launch(attn_streamk_umma_kernel<128>) : launch(attn_streamk_umma_kernel<256>);
}

}  // namespace b200attn
