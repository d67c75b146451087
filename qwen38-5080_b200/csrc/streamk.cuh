// Shared pieces of the stream-K decode-attention kernels: parameters, PTX wrappers, the linear
// tile walk, and the epilogue warp (merge of dumped warp states, output, fused combine).
#pragma once

#include <cuda.h>

#include <mutex>

#include "common.cuh"

namespace b200attn {
namespace {

constexpr int kConsumerWarps = 4;
constexpr int kConsumerThreads = kConsumerWarps * 32;
constexpr int kProducerWarp = kConsumerWarps;          // warp 4: TMA issue
constexpr int kEpilogueWarp = kConsumerWarps + 1;      // warp 5: merge, output, fused combine
constexpr int kMaxBatchMma = 2048;
constexpr unsigned long long kWaitBudgetNs = 2000000000ull;  // 2 s per wait

struct MmaParams {
  Geometry g;
  const uint16_t* q;
  const float* k_scale;
  const float* v_scale;
  const int* seq_len;
  int seq_len_offset;
  float score_scale;     // softmax_scale * log2(e)
  unsigned long long* ws_pkt;   // split-K partials as tagged words, [num_ctas][2 slots][G * D + 16]: see partial_slot_words
  uint16_t* out;         // local output [n_layers][batch][h_q][D] (peer mode: unused)
  // peer mode (tensor-parallel by KV head): every result is stored into the output buffer of all
  // n_out ranks, laid out [n_layers][batch][out_hq_total][D], at head offset out_head_base
  uint16_t* out_peer[16];      // [0..8): every rank's gathered tensor; [8..16): every rank's second one (double buffering)
  int* epoch;                  // this rank's step counter: the launch that finds e there is step e + 1 and uses table entries
                               // [0..8) when e + 1 is even, [8..16) when it is odd; null = [0..8) always.  (Stores mode: the
                               // barrier's own-epoch word, advanced by the barrier.  Packet mode: advanced by the launch.)
  int n_out;             // 0 = local output only
  int out_hq_total, out_head_base;
  // packet mode (pkt != 0): results travel to the other ranks as 8-byte packets {two bf16 values, step number} into
  // their staging buffers: out_peer[r] / out_peer[8 + r] are this rank's slots there for even / odd steps (null for
  // the own rank), `out` is this rank's own gathered tensor; at its end every CTA unpacks a share of what the other
  // ranks sent here (pkt_src: own staging, [2 parities][n_out slots][pkt_slot_words]), waiting for each packet's step
  // number — that wait is all the cross-GPU synchronisation there is: no fence, no flag, no barrier
  int pkt;
  int pkt_resident;            // the whole grid is resident at once: every CTA may wait for remote packets (see unpack_packets)
  const unsigned long long* pkt_src;
  long long pkt_slot_words;
  const uint16_t* gate;  // optional bf16 [n_layers][batch][h_q][D]: out *= sigmoid(gate), see store_out
  int* status;
  int stages;            // ring depth (the V ring where K and V have their own)
  int kstages;           // K ring depth, kernels with separate rings only
  // fused step (kernels that implement it): new-token rows to quantise into the cache first, positions
  // to advance at the end, and the exit counter that elects the last CTA
  const uint16_t* k_new;
  const uint16_t* v_new;
  uint8_t* k_cache_w;
  uint8_t* v_cache_w;
  int* seq_pos;
  int* exit_count;
  // cross-GPU arrive-and-wait by the last CTA to finish (protocol of peer_barrier.cu); bar_world 0 = none
  int* bar_flags[8];
  int bar_rank, bar_world;
};

// ---------------------------------------------------------------------------------------------
// PTX wrappers
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{ .reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }"
      : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
  return ok != 0;
}
__device__ __forceinline__ unsigned long long global_timer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
// Bounded wait.  Returns false (and raises the CTA's timeout flag) when the budget runs out or
// when another thread of the CTA already gave up.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* timed_out, int* status) {
  if (mbar_try_wait(bar, parity)) return true;
  if (*timed_out) return false;
#pragma unroll 1
  for (int i = 0; i < 64; ++i)
    if (mbar_try_wait(bar, parity)) return true;
  const unsigned long long t0 = global_timer_ns();
#pragma unroll 1
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 256; ++i)
      if (mbar_try_wait(bar, parity)) return true;
    if (*timed_out) return false;
    if (global_timer_ns() - t0 > kWaitBudgetNs) {
      *timed_out = 1;
      atomicOr(status, B200ATTN_STATUS_WAIT_TIMEOUT);
      return false;
    }
  }
}
// The same wait with only the first try inline, for kernels with many wait sites and registers to
// spare: the spin / time-out code at every site costs instruction-cache room that the tile loops need
// (the all-tcgen05 kernel's role loops are instruction-fetch sensitive; in the register-tight mma.sync
// kernel the call's spills cost more than the code size saves: 175 -> 180 us).
__device__ __noinline__ bool mbar_wait_slow(uint32_t bar, uint32_t parity, volatile int* timed_out, int* status) {
  return mbar_wait(bar, parity, timed_out, status);
}
__device__ __forceinline__ bool mbar_wait_lean(uint32_t bar, uint32_t parity, volatile int* timed_out, int* status) {
  if (mbar_try_wait(bar, parity)) return true;
  return mbar_wait_slow(bar, parity, timed_out, status);
}
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, int x, int y, int z, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
      ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(z), "r"(bar) : "memory");
}
// The same copy with an L2 eviction policy (createpolicy) for the fetched lines.
__device__ __forceinline__ void tma_load_3d_hint(uint32_t dst, const CUtensorMap* map, int x, int y, int z, uint32_t bar,
                                                 uint64_t policy) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%2, %3, %4}], [%5], %6;"
      ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(z), "r"(bar), "l"(policy) : "memory");
}
// Programmatic dependent launch: the stream-K kernels are launched with programmatic stream serialization, so their
// CTAs may become resident while the kernel before them in the stream is still finishing (the set-up of the CTA's
// barriers and tensor memory runs meanwhile); pdl_wait() returns once that kernel has completed and its memory is
// visible — it stands before the CTA's first read of global memory — and pdl_launch_dependents() lets the next
// kernel's CTAs in as soon as SMs have room.  A kernel launched without the attribute sees both as no-ops.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

__device__ __forceinline__ uint64_t l2_policy_evict_first() {
  uint64_t pol;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
  return pol;
}
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
  return v;
}
__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
__device__ __forceinline__ void sts64(uint32_t addr, float x, float y) {
  asm volatile("st.shared.v2.f32 [%0], {%1, %2};" ::"r"(addr), "f"(x), "f"(y) : "memory");
}

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ uint32_t cvt_lo(uint32_t w) { return e4m3x2_to_f16x2((uint16_t)(w & 0xFFFFu)); }
__device__ __forceinline__ uint32_t cvt_hi(uint32_t w) { return e4m3x2_to_f16x2((uint16_t)(w >> 16)); }
__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
  uint32_t d;
  asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(sel));
  return d;
}
__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t a) {
  uint32_t d;
  asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(d) : "r"(a));
  return d;
}
// D(16x8,f32) += A(16x16,f16,row) * B(16x8,f16,col)
__device__ __forceinline__ void mma_f16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                        uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
      "{%0, %1, %2, %3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}


// Two floats -> two e4m3 bytes in a 16-bit register: `lo` in the low byte, `hi` in the high byte.
__device__ __forceinline__ uint32_t pack_e4m3x2(float lo, float hi) {
  uint16_t r;
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(r) : "f"(hi), "f"(lo));
  return (uint32_t)r;
}
// Leading part of x that an e4m3 value holds exactly (sign, exponent, top three mantissa bits).
__device__ __forceinline__ float e4m3_head(float x) { return __uint_as_float(__float_as_uint(x) & 0xFFF00000u); }

// ---------------------------------------------------------------------------------------------
// the stream-K walk: linear tile index -> (layer, sequence, kv head, tile)
// ---------------------------------------------------------------------------------------------
struct Cursor {
  int layer, b, h, tile;   // position of the current tile
  int tiles_b;             // tiles of sequence b
  int len_b;               // valid tokens of sequence b
};

// cum[b] = tiles of sequences < b; len[] clamped lengths.  Both in shared memory.
__device__ __forceinline__ Cursor locate(long long idx, const int* cum, const int* len, int batch, int h_kv) {
  const long long per_layer = (long long)cum[batch] * h_kv;
  Cursor c;
  c.layer = (int)(idx / per_layer);
  const long long r = idx - (long long)c.layer * per_layer;
  int lo = 0, hi = batch - 1;   // largest b with cum[b]*h_kv <= r (and tiles_b > 0 follows from r < cum[b+1]*h_kv)
  while (lo < hi) {
    const int mid = (lo + hi + 1) >> 1;
    if ((long long)cum[mid] * h_kv <= r) lo = mid; else hi = mid - 1;
  }
  // sequences with zero tiles share cum[] with their successor: step forward to the one that owns r
  while (cum[lo + 1] == cum[lo]) ++lo;
  c.b = lo;
  c.tiles_b = cum[lo + 1] - cum[lo];
  c.len_b = len[lo];
  const long long rr = r - (long long)cum[lo] * h_kv;
  c.h = (int)(rr / c.tiles_b);
  c.tile = (int)(rr - (long long)c.h * c.tiles_b);
  return c;
}

// Move to the first tile of the next pair.
__device__ __forceinline__ void next_pair(Cursor& c, const int* cum, const int* len, int batch, int h_kv) {
  c.tile = 0;
  if (++c.h < h_kv) return;
  c.h = 0;
  for (;;) {
    if (++c.b == batch) { c.b = 0; ++c.layer; }
    if (cum[c.b + 1] != cum[c.b]) break;   // at least one sequence is non-empty when total > 0
  }
  c.tiles_b = cum[c.b + 1] - cum[c.b];
  c.len_b = len[c.b];
}

// CTA that owns linear tile x when `total` tiles are divided over n CTAs as [c*total/n, (c+1)*total/n).
__device__ __forceinline__ int owner_of(long long x, long long total, int n) {
  return (int)(((x + 1) * n - 1) / total);
}


// Tile range [r0, r1) of CTA `cta`.  Default: the even stream-K split of `total` tiles over n_eff
// CTAs.  Short sequences are the exception: when every pair has the same small number of tiles
// (`pair_tiles` <= kAlignMaxTiles, i.e. depth <= 1024 with 64-token tiles), a split pair costs its
// owners a partial and a combine at the end of the launch, more than the few tiles of imbalance it saves
// (depth 512, 512 pairs: whole pairs on 256 CTAs 18.5 us, the even split over 296 CTAs 19.6 us).  So
//   * with more than half as many pairs as CTAs, every CTA takes whole pairs, and only as many CTAs work as
//     it takes to give each the same number k = ceil(pairs / grid) of them (512 pairs on a grid of 444:
//     256 CTAs with two pairs each, 20.0 us, against 444 CTAs of which 68 have two, 21.6 us);
//   * with fewer pairs (few KV heads per GPU), every pair is cut into the same number of equal pieces, one
//     piece per CTA, as many as the grid has room for: n_eff = pairs * pieces, so the even split below puts
//     its boundaries on the pairs by itself.  The host chooses the grid for that (mma_pick_ctas).
constexpr int kAlignMaxTiles = 16;
__device__ __forceinline__ void cta_range(long long total, int grid, int cta, int pair_tiles,
                                          int& n_eff, long long& r0, long long& r1) {
  n_eff = (int)(total < (long long)grid ? total : (long long)grid);
  r0 = r1 = 0;
  if (pair_tiles > 0 && pair_tiles <= kAlignMaxTiles) {
    const long long pairs = total / pair_tiles;
    if (2 * pairs > (long long)grid) {
      const long long k = (pairs + grid - 1) / grid;
      n_eff = (int)((pairs + k - 1) / k);
      if (cta < n_eff) {
        r0 = ((long long)cta * pairs / n_eff) * pair_tiles;
        r1 = (((long long)cta + 1) * pairs / n_eff) * pair_tiles;
      }
      return;
    }
    long long pieces = (long long)grid / pairs;
    if (pieces > pair_tiles) pieces = pair_tiles;
    n_eff = (int)(pairs * pieces);
  }
  if (cta < n_eff) {
    r0 = (long long)cta * total / n_eff;
    r1 = ((long long)cta + 1) * total / n_eff;
  }
}

// Position (in float2 units) of dim pair u inside a dumped head row.  The xor spreads the
// consumer fragments (dims 16*gq + 2*j per lane) over all banks; it permutes within groups of 8.
__device__ __forceinline__ int dump_pos(int u) { return (u & ~7) | ((u & 7) ^ ((u >> 3) & 7)); }

// The number of the step this launch is (see MmaParams::epoch), and the half of out_peer it uses.
__device__ __forceinline__ int peer_step(const MmaParams& p) {
  return p.epoch != nullptr ? *reinterpret_cast<const volatile int*>(p.epoch) + 1 : 0;
}
__device__ __forceinline__ int peer_buffer_base(int step) { return (step & 1) ? 8 : 0; }

// Tensor-parallel output: where this launch's results go on the other GPUs.  The epilogue warp of a CTA writes the
// (up to 8) destinations of this step into shared memory once (fill_peer_table), and the results of a pair then go
// out together through one out-of-line function that reads them from there (send_pair).  All of it is about code
// size and latency: the kernels' tile loops are sensitive to the size of the code around them (destination loops
// inlined at the twenty places of the epilogue that produce output cost the long-cache kernel 3 % of its time),
// kernel parameters can only be read by the kernel function itself, a lookup in the parameter block per destination
// and value costs ~150 cycles, and so does an out-of-line call per value (both ~2 us per pair).
//   packet mode: entry r = this rank's slot in rank r's staging buffer for this step's parity (0 for the own rank)
//   stores mode: entry r = rank r's gathered tensor of this step's parity (0 beyond n_out)
__device__ __forceinline__ void fill_peer_table(const MmaParams& p, unsigned long long* tab, int r, int step) {   // entry r < 8
  unsigned long long v = 0;
  if (p.pkt) {
    if (p.out_peer[r]) v = (unsigned long long)p.out_peer[r] + (unsigned long long)(step & 1) * p.n_out * p.pkt_slot_words * 8ull;
  } else if (r < p.n_out) {
    v = (unsigned long long)p.out_peer[peer_buffer_base(step) + r];
  }
  tab[r] = v;
}
// Packet mode: one 8-byte store per rank, value and step number arrive together or not at all.  Stores mode: the
// output all-gather as plain stores into every rank's gathered tensor (own one included) over NVLink.
__device__ __noinline__ void emit_peer(const unsigned long long* tab, int pkt, int step, long long idx, long long peer_idx, uint32_t bits) {
  if (pkt) {
    const unsigned long long w = (unsigned long long)bits | ((unsigned long long)(uint32_t)step << 32);
    const unsigned long long off = (unsigned long long)(idx >> 1) * 8ull;
#pragma unroll
    for (int r = 0; r < 8; ++r) {
      const unsigned long long dst = tab[r];
      if (dst) asm volatile("st.relaxed.sys.global.b64 [%0], %1;" ::"l"(dst + off), "l"(w) : "memory");
    }
  } else {
#pragma unroll
    for (int r = 0; r < 8; ++r) {
      const unsigned long long dst = tab[r];
      if (dst) *reinterpret_cast<uint32_t*>(dst + (unsigned long long)peer_idx * 2ull) = bits;
    }
  }
}

// One pair of adjacent bf16 outputs on its way: `idx` is its element index in this rank's [n_layers][batch][h_q][D]
// layout, `peer_idx` in the gathered [n_layers][batch][out_hq_total][D] layout.
__device__ __forceinline__ void emit_bits(const MmaParams& p, const unsigned long long* peer_tab, int step, long long idx,
                                          long long peer_idx, uint32_t bits) {
  if (p.n_out == 0) {
    *reinterpret_cast<uint32_t*>(p.out + idx) = bits;
  } else {
    if (p.pkt) *reinterpret_cast<uint32_t*>(p.out + peer_idx) = bits;   // this rank's rows of its own gathered tensor
    emit_peer(peer_tab, p.pkt, step, idx, peer_idx, bits);
  }
}

// Two adjacent outputs -> bf16 bits.  With a gate, the consumer-side fusion of the reference's attention
// block, attn_output * sigmoid(gate), with its two separate bf16 roundings
// (docs/journal/2026-10-23-phase2-r3-coordinator.md:147-150): s = bf16(sigmoid(gate)), then
// bf16(bf16(attn) * s).  `idx`: element index in this rank's [n_layers][batch][h_q][D] layout.
__device__ __forceinline__ uint32_t out_bits(const MmaParams& p, long long idx, float x, float y) {
  const uint16_t* gate = p.gate;
  __nv_bfloat162 ob = __floats2bfloat162_rn(x, y);
  if (gate) {
    const uint32_t gw = *reinterpret_cast<const uint32_t*>(gate + idx);
    const float g0 = bf16_bits_to_float(gw & 0xFFFFu), g1 = bf16_bits_to_float(gw >> 16);
    const __nv_bfloat162 s = __floats2bfloat162_rn(__fdiv_rn(1.f, 1.f + expf(-g0)), __fdiv_rn(1.f, 1.f + expf(-g1)));
    ob = __floats2bfloat162_rn(__low2float(ob) * __low2float(s), __high2float(ob) * __high2float(s));
  }
  return *reinterpret_cast<uint32_t*>(&ob);
}

// The finished rows of one (layer, sequence, kv head) pair, G heads x D dims, on their way to the other GPUs: lane
// `lane` of the epilogue warp holds words[h * (D / 64) + r] = dims 2 * (lane + 32 r), + 1 of head h.  `orow`: the
// pair's first element in this rank's [n_layers][batch][h_q][D] layout, `prow` in the gathered layout.
template <int D>
__device__ __noinline__ void send_pair(const unsigned long long* tab, int pkt, int step, const uint32_t* words, int G,
                                       long long orow, long long prow, uint16_t* own, int lane) {
  constexpr int UR = D / 64;
  if (pkt) {   // this rank's rows of its own gathered tensor
    for (int h = 0; h < G; ++h)
#pragma unroll
      for (int r = 0; r < UR; ++r) *reinterpret_cast<uint32_t*>(own + prow + h * D + 2 * (lane + 32 * r)) = words[h * UR + r];
  }
  const unsigned long long tag = (unsigned long long)(uint32_t)step << 32;
#pragma unroll 1
  for (int d = 0; d < 8; ++d) {
    const unsigned long long dst = tab[d];
    if (!dst) continue;
    if (pkt) {   // one 8-byte store per value pair: value and step number arrive together or not at all
      const unsigned long long base = dst + (unsigned long long)((orow >> 1) + lane) * 8ull;
      for (int h = 0; h < G; ++h)
#pragma unroll
        for (int r = 0; r < UR; ++r)
          asm volatile("st.relaxed.sys.global.b64 [%0], %1;" ::"l"(base + (unsigned long long)(h * (D / 2) + 32 * r) * 8ull),
                       "l"((unsigned long long)words[h * UR + r] | tag) : "memory");
    } else {     // plain stores into rank d's gathered tensor
      const unsigned long long base = dst + (unsigned long long)(prow + 2 * lane) * 2ull;
      for (int h = 0; h < G; ++h)
#pragma unroll
        for (int r = 0; r < UR; ++r)
          *reinterpret_cast<uint32_t*>(base + (unsigned long long)(h * D + 64 * r) * 2ull) = words[h * UR + r];
    }
  }
}

// ---------------------------------------------------------------------------------------------
// Split-K hand-over.  A pair whose tiles are spread over the CTAs c_first .. c_last is finished by c_last, the
// owner of its final piece.  Every owner (c_last included) leaves its piece's merged state (m, l, acc) in its own
// workspace slot as 8-byte words {fp32 value, tag = pair + 1}: value and tag become visible together, so the
// words need no fence, no flag and no arrival counter, and the writer is done when its stores are issued.  c_last
// holds the pair's FINAL tiles, which are the first of its own range: it notes the pair (DeferredCombine) and
// goes on; when its whole range is done, all its warps collect the pair's pieces (combine_deferred) — each
// word is polled until its tag is the pair's (bounded), summed in CTA order (the result is the same from launch to
// launch) and set back to zero, which is the state every launch must find (the workspace starts zeroed and every
// launch that ends without a time-out leaves it so).  c_last only ever waits for CTAs of lower index, which the
// hardware dispatches first: this cannot deadlock on a grid that is not resident all at once.  The other
// owners reach the end of their pieces when they reach the end of their ranges, i.e. when c_last does: the
// hand-over costs the pair one trip through L2, where the ticket scheme it replaces cost five in a row under
// full memory load (partials, release, ticket, two dependent rounds of loads): 7-10 us at the end of a launch.
// ---------------------------------------------------------------------------------------------
__host__ __device__ __forceinline__ long long partial_slot_words(int G, int D) { return (long long)G * D + 16; }   // acc, m[8], l[8]

struct DeferredCombine {   // in shared memory; written by lane 0 of the epilogue warp, read after the CTA's last barrier
  long long orow, prow;    // the pair's first output element, local and gathered layout
  int pair, c_first, first_slot, valid;
  float vs;
  int pad;
};

__device__ __forceinline__ void st_tagged(unsigned long long* dst, float v, unsigned long long tag) {
  asm volatile("st.relaxed.gpu.global.b64 [%0], %1;" ::"l"(dst), "l"((unsigned long long)__float_as_uint(v) | tag) : "memory");
}
__device__ __forceinline__ unsigned long long ld_tagged(const unsigned long long* src) {
  unsigned long long v;
  asm volatile("ld.relaxed.gpu.global.b64 %0, [%1];" : "=l"(v) : "l"(src) : "memory");
  return v;
}

// What combine_deferred needs of the kernel's parameters, by value (handing the parameter block itself to an
// out-of-line function by reference would make the tile loops read their parameters through memory).
struct CombineArgs {
  unsigned long long* ws_pkt;
  uint16_t* out;
  const uint16_t* gate;
  const unsigned long long* peer_tab;
  int* status;
  int G, n_out, pkt, step;
};
__device__ __forceinline__ CombineArgs combine_args_of(const MmaParams& p, const unsigned long long* peer_tab, int step) {
  return CombineArgs{p.ws_pkt, p.out, p.gate, peer_tab, p.status, p.g.group, p.n_out, p.pkt, step};
}

// All warps of c_last, after the CTA's last barrier.  Warp w takes heads w, w + nwarps, ...; lane j polls owner j's
// (m, l) and every lane its UR dim pairs of every owner's accumulator, CH owners at a time, all loads of a round in
// flight together.
template <int D>
__device__ __noinline__ void combine_deferred(CombineArgs a, DeferredCombine dc, int warp, int nwarps, int lane) {
  constexpr int UR = D / 64;               // dim pairs per lane
  constexpr int CH = 8 / UR;               // owners per round: 16 words in flight per lane
  const long long SW = partial_slot_words(a.G, D);
  const int c_last = (int)blockIdx.x, n = c_last - dc.c_first + 1;
  const uint32_t tag32 = (uint32_t)(dc.pair + 1);
  const unsigned long long t0 = global_timer_ns();
  for (int h = warp; h < a.G; h += nwarps) {
    // the pieces in CTA order, CH at a time, against a running maximum (one round when the pair has at most CH pieces)
    float M = -INFINITY, ll = 0.f, ax[UR], ay[UR];
#pragma unroll
    for (int r = 0; r < UR; ++r) { ax[r] = 0.f; ay[r] = 0.f; }
    for (int c0 = 0; c0 < n; c0 += CH) {
      unsigned long long w[CH][2 * UR], wm[CH], wl[CH];
      uint32_t pending = 0;   // bit per word of the round: CH * (2 * UR + 2) <= 32
#pragma unroll
      for (int i = 0; i < CH; ++i)
        if (c0 + i < n) pending |= ((1u << (2 * UR + 2)) - 1u) << (i * (2 * UR + 2));
      for (int tries = 0; pending; ++tries) {
#pragma unroll
        for (int i = 0; i < CH; ++i) {
          const int cc = dc.c_first + c0 + i;
          const unsigned long long* slot = a.ws_pkt + ((long long)cc * 2 + (cc == dc.c_first ? dc.first_slot : 0)) * SW;
          const uint32_t bit0 = i * (2 * UR + 2);
#pragma unroll
          for (int r = 0; r < UR; ++r) {
            if (pending & (1u << (bit0 + 2 * r))) w[i][2 * r] = ld_tagged(slot + h * D + 2 * (lane + 32 * r));
            if (pending & (1u << (bit0 + 2 * r + 1))) w[i][2 * r + 1] = ld_tagged(slot + h * D + 2 * (lane + 32 * r) + 1);
          }
          if (pending & (1u << (bit0 + 2 * UR))) wm[i] = ld_tagged(slot + (long long)a.G * D + h);
          if (pending & (1u << (bit0 + 2 * UR + 1))) wl[i] = ld_tagged(slot + (long long)a.G * D + 8 + h);
        }
#pragma unroll
        for (int i = 0; i < CH; ++i) {
          const uint32_t bit0 = i * (2 * UR + 2);
#pragma unroll
          for (int k = 0; k < 2 * UR; ++k)
            if ((pending & (1u << (bit0 + k))) && (uint32_t)(w[i][k] >> 32) == tag32) pending &= ~(1u << (bit0 + k));
          if ((pending & (1u << (bit0 + 2 * UR))) && (uint32_t)(wm[i] >> 32) == tag32) pending &= ~(1u << (bit0 + 2 * UR));
          if ((pending & (1u << (bit0 + 2 * UR + 1))) && (uint32_t)(wl[i] >> 32) == tag32) pending &= ~(1u << (bit0 + 2 * UR + 1));
        }
        if (pending && (tries & 63) == 63 && global_timer_ns() - t0 > kWaitBudgetNs) {
          atomicOr(a.status, B200ATTN_STATUS_WAIT_TIMEOUT);
          return;
        }
      }
      float Mn = M;
#pragma unroll
      for (int i = 0; i < CH; ++i)
        if (c0 + i < n) Mn = fmaxf(Mn, __uint_as_float((uint32_t)wm[i]));
      const float keep = M == -INFINITY ? 0.f : ex2(M - Mn);   // what is summed so far, on the new maximum's scale
      M = Mn;
      ll *= keep;
#pragma unroll
      for (int r = 0; r < UR; ++r) { ax[r] *= keep; ay[r] *= keep; }
#pragma unroll
      for (int i = 0; i < CH; ++i) {
        if (c0 + i < n) {
          const int cc = dc.c_first + c0 + i;
          unsigned long long* slot = a.ws_pkt + ((long long)cc * 2 + (cc == dc.c_first ? dc.first_slot : 0)) * SW;
          B200ATTN_CHECK(a.status, cc >= 0 && cc <= c_last && cc < (int)gridDim.x);
          const float mc = __uint_as_float((uint32_t)wm[i]);
          const float f = mc == -INFINITY ? 0.f : ex2(mc - M);
          ll += __uint_as_float((uint32_t)wl[i]) * f;
#pragma unroll
          for (int r = 0; r < UR; ++r) {
            ax[r] += __uint_as_float((uint32_t)w[i][2 * r]) * f;
            ay[r] += __uint_as_float((uint32_t)w[i][2 * r + 1]) * f;
            // 16 bytes of zeros: the two words are consumed
            *reinterpret_cast<ulonglong2*>(slot + h * D + 2 * (lane + 32 * r)) = make_ulonglong2(0ull, 0ull);
          }
          if (lane == 0) { slot[(long long)a.G * D + h] = 0ull; slot[(long long)a.G * D + 8 + h] = 0ull; }
        }
      }
    }
    const float inv = ll > 0.f ? dc.vs / ll : 0.f;
    uint32_t words[UR];
#pragma unroll
    for (int r = 0; r < UR; ++r) {
      const long long idx = dc.orow + h * D + 2 * (lane + 32 * r);
      __nv_bfloat162 ob = __floats2bfloat162_rn(ax[r] * inv, ay[r] * inv);
      if (a.gate) {   // as out_bits
        const uint32_t gw = *reinterpret_cast<const uint32_t*>(a.gate + idx);
        const float g0 = bf16_bits_to_float(gw & 0xFFFFu), g1 = bf16_bits_to_float(gw >> 16);
        const __nv_bfloat162 sg = __floats2bfloat162_rn(__fdiv_rn(1.f, 1.f + expf(-g0)), __fdiv_rn(1.f, 1.f + expf(-g1)));
        ob = __floats2bfloat162_rn(__low2float(ob) * __low2float(sg), __high2float(ob) * __high2float(sg));
      }
      words[r] = *reinterpret_cast<uint32_t*>(&ob);
      if (a.n_out == 0) *reinterpret_cast<uint32_t*>(a.out + idx) = words[r];
    }
    if (a.n_out) {
      send_pair<D>(a.peer_tab, a.pkt, a.step, words, 1, dc.orow + h * D, dc.prow + h * D, a.out, lane);
      if (!a.pkt) __threadfence_system();   // stores mode: see the end of epilogue_warp
    }
  }
}

// ---------------------------------------------------------------------------------------------
// epilogue warp: walks the CTA's segments in the consumers' order.  For each it waits for the
// NW dumped states (m[8], l[8], acc[G][D]; head rows in the xor layout of dump_pos, or in plain
// dim order when PLAIN), merges them (UNIT_V: the V scales are already in the accumulators: per-token layout),
// and either writes the normalised bf16 output (pair fully owned by this CTA) or leaves the merged state in the
// CTA's workspace slot as tagged words; if the piece is the pair's last one, it notes the pair in `deferred` for
// combine_deferred.
// ---------------------------------------------------------------------------------------------
template <int D, int NDUMP, int NW = kConsumerWarps, bool PLAIN = false, bool UNIT_V = false>
__device__ __forceinline__ void epilogue_warp(const MmaParams& p, int lane, long long r0, long long r1,
                                              long long total, int n_eff, const int* sCum, const int* sLen,
                                              const float* sDump, const float* sML, uint32_t dfull0,
                                              uint32_t dempty0, volatile int* timed_out, const unsigned long long* peer_tab,
                                              DeferredCombine* deferred, int step) {
  constexpr int DP = D + 4;                // padded head row of a dumped state, in floats
  constexpr int UR = D / 64;               // dim pairs per epilogue lane
  const Geometry& g = p.g;
  const int G = g.group;
  const int dump_warp_floats = G * DP;
  uint32_t obuf[kMaxGroup * UR];   // peer mode: the bf16 rows of the pair being finished, sent together (send_pair)
  if (p.n_out) {
    if (lane < 8) fill_peer_table(p, const_cast<unsigned long long*>(peer_tab), lane, step);
    __syncwarp();
  }
{
  Cursor c = locate(r0, sCum, sLen, g.batch, g.h_kv);
  long long cur = r0;
  int seg = 0;
  while (cur < r1) {
    const long long pair_start = cur - c.tile, pair_end = pair_start + c.tiles_b;
    const long long seg_end = pair_end < r1 ? pair_end : r1;
    const long long lb = (long long)c.layer * g.batch + c.b;
    const long long pair = lb * g.h_kv + c.h;
    const bool complete = cur == pair_start && seg_end == pair_end;
    const float vs = UNIT_V ? 1.f : p.v_scale[c.layer * g.h_kv + c.h];
    const int db = seg % NDUMP;
    const bool ok = mbar_wait(dfull0 + 8u * db, (seg / NDUMP) & 1, timed_out, p.status);
    const float* dump = sDump + db * NW * dump_warp_floats;
    const float* ml = sML + db * NW * 16;
    const int slot = cur == r0 ? 0 : 1;
    unsigned long long* pslot = p.ws_pkt + ((long long)blockIdx.x * 2 + slot) * partial_slot_words(G, D);
    const unsigned long long tag = (unsigned long long)(uint32_t)(pair + 1) << 32;
    const long long orow = (lb * g.h_q + c.h * G) * D;
    const long long prow = (lb * p.out_hq_total + p.out_head_base + c.h * G) * D;   // row in the gathered layout
    B200ATTN_CHECK(p.status, c.layer >= 0 && c.layer < g.n_layers && c.b >= 0 && c.b < g.batch && c.h >= 0 && c.h < g.h_kv);
    B200ATTN_CHECK(p.status, orow >= 0 && orow + (long long)G * D <= (long long)g.n_layers * g.batch * g.h_q * D);
    B200ATTN_CHECK(p.status, seg_end > cur && seg_end <= r1 && c.tile >= 0 && c.tile < c.tiles_b);
    if (ok) {
      for (int h = 0; h < G; ++h) {
        float mw[NW], M = -INFINITY;
#pragma unroll
        for (int w = 0; w < NW; ++w) { mw[w] = ml[w * 16 + h]; M = fmaxf(M, mw[w]); }
        float ll = 0.f, ax[UR], ay[UR];
#pragma unroll
        for (int r = 0; r < UR; ++r) { ax[r] = 0.f; ay[r] = 0.f; }
#pragma unroll
        for (int w = 0; w < NW; ++w) {
          const float f = mw[w] == -INFINITY ? 0.f : ex2(mw[w] - M);
          ll += ml[w * 16 + 8 + h] * f;
#pragma unroll
          for (int r = 0; r < UR; ++r) {
            const float2 v = *reinterpret_cast<const float2*>(dump + w * dump_warp_floats + h * DP + 2 * (PLAIN ? lane + 32 * r : dump_pos(lane + 32 * r)));
            ax[r] += v.x * f;
            ay[r] += v.y * f;
          }
        }
        if (complete) {
          const float inv = ll > 0.f ? vs / ll : 0.f;
#pragma unroll
          for (int r = 0; r < UR; ++r) {
            const long long idx = orow + h * D + 2 * (lane + 32 * r);
            const uint32_t bits = out_bits(p, idx, ax[r] * inv, ay[r] * inv);
            if (p.n_out == 0) *reinterpret_cast<uint32_t*>(p.out + idx) = bits;
            else obuf[h * UR + r] = bits;
          }
        } else {
#pragma unroll
          for (int r = 0; r < UR; ++r) {
            st_tagged(pslot + h * D + 2 * (lane + 32 * r), ax[r], tag);
            st_tagged(pslot + h * D + 2 * (lane + 32 * r) + 1, ay[r], tag);
          }
          if (lane == 0) { st_tagged(pslot + G * D + h, M, tag); st_tagged(pslot + G * D + 8 + h, ll, tag); }
        }
      }
      if (complete && p.n_out) send_pair<D>(peer_tab, p.pkt, step, obuf, G, orow, prow, p.out, lane);
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(dempty0 + 8u * db);   // the dump buffer may be overwritten
    if (!complete && ok && seg_end == pair_end) {
      // the pair's last piece: this CTA finishes the pair when its own range is done
      const int c_first = owner_of(pair_start, total, n_eff);
      B200ATTN_CHECK(p.status, c_first >= 0 && c_first < (int)blockIdx.x && owner_of(pair_end - 1, total, n_eff) == (int)blockIdx.x && cur == r0);
      if (lane == 0) {
        deferred->orow = orow; deferred->prow = prow;
        deferred->pair = (int)pair; deferred->c_first = c_first;
        deferred->first_slot = (long long)c_first * total / n_eff < pair_start ? 1 : 0;
        deferred->vs = vs;
        deferred->valid = 1;
      }
    }
    ++seg;
    cur = seg_end;
    if (cur < r1) next_pair(c, sCum, sLen, g.batch, g.h_kv);
  }
  // Stores mode: every lane's stores into the other GPUs' tensors are made visible system-wide here, by the warp
  // that issued them, so that the fence of the CTA that finishes the launch finds nothing of them outstanding.
  if (p.n_out && !p.pkt) __threadfence_system();
}
}

// Layout of a barrier flag buffer (int32 words, peer-writable): [0, world) arrival epochs written by the ranks,
// [world] the owner's epoch counter, [16..19] two 64-bit %globaltimer stamps of the owner's latest
// arrive-and-wait (when it arrived, when the wait ended).
constexpr int kFlagStampWord = 16;
constexpr unsigned long long kBarrierBudgetNs = 1000000000ull;   // 1 s

// Cross-GPU arrive-and-wait by one warp: bump the own epoch, publish it into every rank's flag buffer, wait
// (bounded) until every rank's epoch has reached it.  Lane r talks to rank r, so the flag stores go out
// together and the polls run side by side.  The caller has made the launch's peer stores happen-before this
// warp (exit counter + warp shuffle); each publishing lane's system-scope fence orders them before its flag.
__device__ __forceinline__ void warp_peer_barrier(int* const* flags, int rank, int world, int lane, int* status) {
  int* mine = flags[rank];
  const int e = *reinterpret_cast<volatile int*>(mine + world) + 1;
  const unsigned long long t0 = global_timer_ns();
  if (lane < world) {
    __threadfence_system();
    asm volatile("st.relaxed.sys.global.s32 [%0], %1;" ::"l"(flags[lane] + rank), "r"(e) : "memory");
    for (;;) {
      int v;
      asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(mine + lane) : "memory");
      if (v - e >= 0) break;
      if (global_timer_ns() - t0 > kBarrierBudgetNs) { atomicOr(status, B200ATTN_STATUS_WAIT_TIMEOUT); break; }
    }
  }
  __syncwarp();
  if (lane == 0) {
    unsigned long long* stamp = reinterpret_cast<unsigned long long*>(mine + kFlagStampWord);
    stamp[0] = t0;
    stamp[1] = global_timer_ns();
    *reinterpret_cast<volatile int*>(mine + world) = e;
  }
}

// Last act of a launch whose end does need an election among the CTAs (stores mode: someone has to run the cross-GPU
// barrier after everybody's peer stores; packets on a grid that is not resident at once: someone has to unpack after
// everything is sent; see arrives_early for all other launches), called by warp 0 of every CTA after the CTA's final
// __syncthreads: the warp of the last CTA to arrive advances the positions and does the barrier or the unpacking.
// Out of line: it runs once per CTA and must not cost the tile loops registers.  Its arguments travel by value:
// handing the kernel's parameter block to an out-of-line function by reference takes that block's address, and
// the tile loops then read their parameters through memory instead of as constant operands (measured: +6 % on
// the long-cache kernel, +30 % at depth 512).
struct StepEnd {
  int* seq_pos;
  int* exit_count;
  int* status;
  int batch, capacity, bar_rank, bar_world;
  int* flags[8];
  int* step_counter;   // packet mode: the counter the last CTA advances (null otherwise)
  int step;
};
__device__ __forceinline__ StepEnd step_end_of(const MmaParams& p, int step) {
  return StepEnd{p.seq_pos, p.exit_count, p.status, p.g.batch, p.g.capacity, p.bar_rank, p.bar_world,
                 {p.bar_flags[0], p.bar_flags[1], p.bar_flags[2], p.bar_flags[3], p.bar_flags[4], p.bar_flags[5], p.bar_flags[6],
                  p.bar_flags[7]}, p.pkt ? p.epoch : nullptr, step};
}

// Packet mode, receiving side.  The other ranks' results arrive in this rank's staging buffer as 8-byte packets
// {two bf16 values, step number}, slot s = sender s, in the sender's own [n_layers][batch][h_q][D] order.  Share
// `part` of `parts` of the (n_out - 1) * slot_words packets is copied into this rank's gathered tensor, each packet
// as soon as its step number is this step's (bounded wait: after kBarrierBudgetNs the status bit is set and the rest
// is skipped).  Every CTA calls it after its own work (part = its index), so the copy is spread over the grid and
// runs while slower CTAs and slower ranks are still computing.  That needs the whole grid resident: a CTA waiting
// here for a rank whose progress depends, through that rank's own waiting CTAs, on CTAs of this grid that have not
// started yet would wait for ever; a grid larger than the device holds at once is unpacked by the last CTA instead.
struct Unpack {
  const unsigned long long* src;   // this rank's staging, already at this step's parity
  uint16_t* out;                   // this rank's gathered tensor
  int* status;
  long long slot_words;
  int row_words;                   // packets per (layer, sequence) row of one sender: h_q * D / 2
  long long out_row;               // elements per (layer, sequence) row of the gathered tensor: out_hq_total * D
  int n_out, rank, step;
};
__device__ __forceinline__ Unpack unpack_of(const MmaParams& p, int step) {
  return Unpack{p.pkt_src + (long long)(step & 1) * p.n_out * p.pkt_slot_words, p.out, p.status, p.pkt_slot_words,
                p.g.h_q * p.g.head_dim / 2, (long long)p.out_hq_total * p.g.head_dim, p.n_out, p.out_head_base / p.g.h_q, step};
}
__device__ __noinline__ void unpack_packets(Unpack u, int part, int parts, int tid, int nthreads) {
  // 32-bit index arithmetic: the host refuses staging buffers of 2^31 packets or more
  constexpr int U = 8;   // packets a thread has in flight: one L2 round trip per U packets, not per packet (a small
                         // shard of a short cache runs on few CTAs, and each of its threads has a dozen packets to wait for)
  const uint32_t slot = (uint32_t)u.slot_words, total = (uint32_t)(u.n_out - 1) * slot;
  const uint32_t t0 = (uint32_t)((unsigned long long)part * total / parts), t1 = (uint32_t)(((unsigned long long)part + 1) * total / parts);
  const unsigned long long start = global_timer_ns();
  for (uint32_t base = t0 + tid; base < t1; base += (uint32_t)nthreads * U) {
    uint32_t sender[U], word[U];
    unsigned long long v[U];
    uint32_t pending = 0;
#pragma unroll
    for (int i = 0; i < U; ++i) {
      const uint32_t t = base + (uint32_t)i * nthreads;
      if (t < t1) {
        const uint32_t si = t / slot;
        word[i] = t - si * slot;
        sender[i] = si < (uint32_t)u.rank ? si : si + 1;
        pending |= 1u << i;
      }
    }
    for (int tries = 0; pending; ++tries) {
#pragma unroll
      for (int i = 0; i < U; ++i)
        if (pending & (1u << i))
          asm volatile("ld.relaxed.sys.global.b64 %0, [%1];" : "=l"(v[i]) : "l"(u.src + (size_t)sender[i] * slot + word[i]) : "memory");
#pragma unroll
      for (int i = 0; i < U; ++i)
        if ((pending & (1u << i)) && (int)(v[i] >> 32) == u.step) {
          pending &= ~(1u << i);
          const uint32_t row = word[i] / (uint32_t)u.row_words, rem = word[i] - row * (uint32_t)u.row_words;
          B200ATTN_CHECK(u.status, sender[i] < (uint32_t)u.n_out && sender[i] != (uint32_t)u.rank && row < slot / (uint32_t)u.row_words);
          *reinterpret_cast<uint32_t*>(u.out + (long long)row * u.out_row + (size_t)sender[i] * u.row_words * 2 + rem * 2) = (uint32_t)v[i];
        }
      if (pending && (tries & 63) == 63 && global_timer_ns() - start > kBarrierBudgetNs) {
        atomicOr(u.status, B200ATTN_STATUS_WAIT_TIMEOUT);
        return;
      }
    }
  }
}

__device__ __noinline__ void finish_step(StepEnd s, Unpack u, int unpack_all, int lane) {
  // the positions of the first 32 sequences are fetched while the counter's round trip is under way: whoever turns
  // out to be last has them at hand (nobody writes them before that)
  int pos0 = 0;
  if (s.seq_pos && lane < s.batch) pos0 = s.seq_pos[lane];
  int last = 0;
  if (lane == 0) {
    int arrived;
    if (s.bar_world)   // stores mode: the counter also carries this CTA's peer stores to the CTA that publishes the flags
      asm volatile("atom.add.acq_rel.gpu.global.s32 %0, [%1], 1;" : "=r"(arrived) : "l"(s.exit_count) : "memory");
    else               // otherwise it only counts: the CTA's reads of the positions are long complete
      asm volatile("atom.add.relaxed.gpu.global.s32 %0, [%1], 1;" : "=r"(arrived) : "l"(s.exit_count) : "memory");
    last = arrived == (int)gridDim.x - 1;
  }
  last = __shfl_sync(0xffffffffu, last, 0);
  if (!last) return;
  if (unpack_all) {   // a grid that is not resident all at once: everything this rank sent is out, one warp waits for the rest
    unpack_packets(u, 0, 1, lane, 32);
    __syncwarp();
  }
  if (s.seq_pos)
    for (int b = lane; b < s.batch; b += 32) {
      const int pos = b < 32 ? pos0 : s.seq_pos[b];
      if (pos >= 0 && pos + 1 <= s.capacity) s.seq_pos[b] = pos + 1;
    }
  if (lane == 0) {
    *s.exit_count = 0;   // ready for the next launch
    if (s.step_counter) *s.step_counter = s.step;
  }
  if (s.bar_world) warp_peer_barrier(s.flags, s.bar_rank, s.bar_world, lane, s.status);
}

// A launch whose end needs no election among the CTAs — a whole step on one GPU, or with the packet exchange on a grid
// that is resident at once — advances the positions and the step counter as soon as every CTA has READ them, which
// each does once, in its prologue (later uses take them from shared memory): an idle warp takes the arrival counter
// right after the prologue, and the counter's round trip and the last arrival's updates run under the tile loop
// instead of after the unpacking.
__device__ __forceinline__ bool arrives_early(const MmaParams& p) {
  return (p.seq_pos || p.pkt) && !p.bar_world && !(p.pkt && p.n_out > 1 && !p.pkt_resident);
}
__device__ __noinline__ void arrive_early(int* seq_pos, int* exit_count, int* step_counter, int step, int batch, int capacity, int lane) {
  int last = 0;
  if (lane == 0) {
    int arrived;   // after this CTA's reads of positions and step counter (ordered by its __syncthreads), before the last arrival's writes
    asm volatile("atom.add.acq_rel.gpu.global.s32 %0, [%1], 1;" : "=r"(arrived) : "l"(exit_count) : "memory");
    last = arrived == (int)gridDim.x - 1;
  }
  if (!__shfl_sync(0xffffffffu, last, 0)) return;
  if (seq_pos)
    for (int b = lane; b < batch; b += 32) {
      const int pos = seq_pos[b];
      if (pos >= 0 && pos + 1 <= capacity) seq_pos[b] = pos + 1;
    }
  if (lane == 0) {
    *exit_count = 0;   // ready for the next launch
    if (step_counter) *step_counter = step;
  }
}

// What every CTA does after its final __syncthreads when the launch is a whole step and / or sends packets.
// `step`: the step counter as the CTA's prologue read it.
__device__ __forceinline__ void end_of_launch(const MmaParams& p, int tid, int nthreads, int step) {
  if (!(p.seq_pos || p.bar_world || p.pkt)) return;
  const bool receive = p.pkt && p.n_out > 1;
  const bool early = arrives_early(p);
  if (receive && p.pkt_resident) {
    unpack_packets(unpack_of(p, step), (int)blockIdx.x, (int)gridDim.x, tid, nthreads);
    if (!early) __syncthreads();   // this CTA's copies are done before it counts as finished
  }
  if (early) return;
  if (tid < 32) finish_step(step_end_of(p, step), unpack_of(p, step), receive && !p.pkt_resident, tid);
}

// ---------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// <<<grid, threads, smem, stream>>> with programmatic stream serialization (see pdl_wait).
template <typename Kernel, typename... Args>
inline cudaError_t launch_pdl(Kernel kernel, int grid, int threads, size_t smem, cudaStream_t stream, Args... args) {
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3((unsigned)grid);
  cfg.blockDim = dim3((unsigned)threads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, args...);
}

inline EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
  });
  return fn;
}

// u8 view [n_layers][rows = batch*h_kv*capacity][D], box = 128 bytes x box_rows rows, 128-byte swizzle.
inline bool encode_cache_map(CUtensorMap* map, const void* base, const Geometry& g, long long layer_stride, int box_rows) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return false;
  const cuuint64_t dims[3] = {(cuuint64_t)g.head_dim, (cuuint64_t)g.batch * g.h_kv * g.capacity, (cuuint64_t)g.n_layers};
  const cuuint64_t strides[2] = {(cuuint64_t)g.head_dim, (cuuint64_t)layer_stride};
  const cuuint32_t box[3] = {128, (cuuint32_t)box_rows, 1};
  const cuuint32_t estr[3] = {1, 1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<void*>(base), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace
}  // namespace b200attn
