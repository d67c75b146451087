/*
 * Plain-C restatement of the reference's FP8-KV decode-attention path.
 * TEST INFRASTRUCTURE, NOT PRODUCT: only tests, the smoke check and the CPU-baseline legs of
 * the bench may load this library; the CUDA library never links or calls it.
 *
 * What it follows (paths inside the reference project):
 *   - FP8 format: docs/journal/2026-10-23-phase2-r3-coordinator.md:43-49
 *       s = amax|x|/448, q = clamp(x/s, -448, 448).to(float8_e4m3fn), x^ = q.float()*s
 *   - attention arithmetic: bench/micro/attn_length_effect.py:49-66 (eager_attention):
 *       bf16 matmul (fp32 accumulate, bf16 result) -> * scaling (bf16) -> + mask (bf16)
 *       -> softmax in fp32 -> bf16 -> bf16 matmul -> [H_q, D] output
 *   - valid-length mask over a capacity-long cache: bench/micro/attn_length_effect.py:106-111,
 *       runner/model/static_cache.py:79-82.  A masked slot gets finfo(bf16).min added, which
 *       underflows to exactly 0 after the fp32 softmax, so this file simply skips slots >= L.
 *
 * Pinning: bit-exactness of the byte conversion against torch's float8_e4m3fn cast, and
 * agreement of the attention with the torch restatement / the reference's golden outputs, are
 * checked by tests/test_oracle.py.  Summation order differs from torch's matmul, so the
 * attention agrees to bf16 rounding, not bitwise.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

static inline float bf16_to_f32(uint16_t h) {
  uint32_t u = (uint32_t)h << 16;
  float f;
  memcpy(&f, &u, 4);
  return f;
}

static inline uint16_t f32_to_bf16(float f) { /* round to nearest even, NaN kept quiet */
  uint32_t u;
  memcpy(&u, &f, 4);
  if ((u & 0x7FFFFFFFu) > 0x7F800000u) return (uint16_t)((u >> 16) | 0x40);
  u += 0x7FFFu + ((u >> 16) & 1u);
  return (uint16_t)(u >> 16);
}

static inline float round_bf16(float f) { return bf16_to_f32(f32_to_bf16(f)); }

/* float32 -> e4m3fn byte: round to nearest even; |y| >= 480, inf, NaN -> 0x7F | sign. */
uint8_t oracle_f32_to_e4m3(float y) {
  uint32_t u;
  memcpy(&u, &y, 4);
  uint8_t sign = (uint8_t)((u >> 31) << 7);
  uint32_t mag = u & 0x7FFFFFFFu;
  if (mag >= 0x43F00000u) return (uint8_t)(0x7F | sign);            /* >= 480, inf, NaN */
  if (mag >= 0x3C800000u) {                                         /* normal: |y| >= 2^-6 */
    uint32_t m = mag + 0x7FFFFu + ((mag >> 20) & 1u);
    return (uint8_t)(((m >> 20) - (120u << 3)) | sign);
  }
  float a = fabsf(y) * 512.0f;                                      /* subnormal: units of 2^-9 */
  return (uint8_t)((uint8_t)nearbyintf(a) | sign);                  /* default mode = half-even */
}

float oracle_e4m3_to_f32(uint8_t b) {
  int e = (b >> 3) & 0xF, m = b & 7;
  float v;
  if (e == 0xF && m == 7) v = NAN;
  else if (e == 0) v = ldexpf((float)m, -9);
  else v = ldexpf(1.0f + (float)m / 8.0f, e - 7);
  return (b & 0x80) ? -v : v;
}

/* q = clamp(float(x)/s, -448, 448) -> e4m3; NaN stays NaN (torch.clamp propagates NaN); a zero
 * scale (an all-zero row or head) gives zero bytes. */
void oracle_quantize(const uint16_t* x_bf16, float scale, uint8_t* out, long n) {
  for (long i = 0; i < n; ++i) {
    if (scale == 0.0f) { out[i] = 0; continue; }
    float y = bf16_to_f32(x_bf16[i]) / scale;
    if (y == y) y = y < -448.0f ? -448.0f : (y > 448.0f ? 448.0f : y);
    out[i] = oracle_f32_to_e4m3(y);
  }
}

/*
 * One (layer, sequence): q bf16 [h_q][d]; k, v bytes [h_kv][capacity][d]; scales per head
 * (token_stride == 0) or per token (scale[t*token_stride + h]); out bf16 [h_q][d].
 */
static void attend_one(const uint16_t* q, const uint8_t* k, const uint8_t* v, const float* ks,
                       const float* vs, int token_stride, int h_q, int h_kv, int d, int capacity,
                       int len, float scaling, uint16_t* out, float* w /* [len] scratch */) {
  int g = h_q / h_kv;
  for (int hq = 0; hq < h_q; ++hq) {
    int h = hq / g;
    const uint8_t* kh = k + (size_t)h * capacity * d;
    const uint8_t* vh = v + (size_t)h * capacity * d;
    float mx = -INFINITY;
    for (int t = 0; t < len; ++t) {
      float s_k = token_stride ? ks[(size_t)t * token_stride + h] : ks[h];
      float acc = 0.f;
      for (int i = 0; i < d; ++i)
        acc += bf16_to_f32(q[hq * d + i]) * round_bf16(oracle_e4m3_to_f32(kh[(size_t)t * d + i]) * s_k);
      float sc = round_bf16(round_bf16(acc) * scaling); /* matmul -> bf16, * scaling -> bf16 */
      w[t] = sc;
      if (sc > mx) mx = sc;
    }
    float sum = 0.f;
    for (int t = 0; t < len; ++t) { w[t] = expf(w[t] - mx); sum += w[t]; }
    for (int t = 0; t < len; ++t) w[t] = round_bf16(w[t] / sum); /* softmax fp32 -> bf16 */
    for (int i = 0; i < d; ++i) {
      float acc = 0.f;
      for (int t = 0; t < len; ++t) {
        float s_v = token_stride ? vs[(size_t)t * token_stride + h] : vs[h];
        acc += w[t] * round_bf16(oracle_e4m3_to_f32(vh[(size_t)t * d + i]) * s_v);
      }
      out[hq * d + i] = f32_to_bf16(acc);
    }
  }
}

/*
 * Multi-layer batched decode attention over the FP8 cache.
 *   q, out : bf16 [n_layers][batch][h_q][d];  caches u8 [n_layers][batch][h_kv][capacity][d]
 *   scale_mode 0: scales [n_layers][h_kv]; 1: [n_layers][batch][capacity][h_kv]
 * Returns 0, or -1 on bad arguments.  Parallel over (layer, sequence) when built with OpenMP.
 */
int oracle_decode_attention(int n_layers, int batch, int h_q, int h_kv, int d, int capacity,
                            int scale_mode, const uint16_t* q, const uint8_t* k_cache,
                            const uint8_t* v_cache, const float* k_scale, const float* v_scale,
                            const int* seq_len, float scaling, uint16_t* out) {
  if (!q || !k_cache || !v_cache || !k_scale || !v_scale || !seq_len || !out) return -1;
  if (h_kv <= 0 || h_q % h_kv) return -1;
  long n = (long)n_layers * batch;
#pragma omp parallel for schedule(dynamic, 1)
  for (long idx = 0; idx < n; ++idx) {
    int layer = (int)(idx / batch), b = (int)(idx % batch);
    int len = seq_len[b] < 0 ? 0 : (seq_len[b] > capacity ? capacity : seq_len[b]);
    uint16_t* o = out + (size_t)idx * h_q * d;
    if (len == 0) { memset(o, 0, (size_t)h_q * d * 2); continue; }
    float* w = (float*)malloc((size_t)len * sizeof(float));
    const float *ks, *vs;
    int ts = 0;
    if (scale_mode == 0) { ks = k_scale + (size_t)layer * h_kv; vs = v_scale + (size_t)layer * h_kv; }
    else { ks = k_scale + (size_t)idx * capacity * h_kv; vs = v_scale + (size_t)idx * capacity * h_kv; ts = h_kv; }
    attend_one(q + (size_t)idx * h_q * d, k_cache + (size_t)idx * h_kv * capacity * d,
               v_cache + (size_t)idx * h_kv * capacity * d, ks, vs, ts, h_q, h_kv, d, capacity, len,
               scaling, o, w);
    free(w);
  }
  return 0;
}
