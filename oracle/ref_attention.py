"""CPU oracle for the FP8-KV decode-attention path.  TEST INFRASTRUCTURE, NOT PRODUCT.

Only tests, the smoke check and the CPU-baseline legs of the bench may import this module;
the product path (the CUDA library) never does and has no CPU fallback.

It restates, in plain torch on the CPU, the reference's algorithm for this path:

* ``repeat_kv`` / ``eager_attention`` / ``fp64_reference`` follow
  bench/micro/attn_length_effect.py:41-46, :49-66, :69-75 of the reference (its replica of
  transformers' ``eager_attention_forward``): bf16 matmul, scores scaled and kept in bf16,
  additive mask, fp32 softmax cast back to bf16, bf16 matmul, transpose(1, 2).
* the zero padding to capacity and the ``finfo(bf16).min`` mask follow
  bench/micro/attn_length_effect.py:106-111 and runner/model/padded_reference.py:35-44.
* the FP8 format follows the scheme frozen in
  docs/journal/2026-10-23-phase2-r3-coordinator.md:43-49:
  ``s = amax|x|/448``, ``q = clamp(x/s, -448, 448).to(float8_e4m3fn)``, ``x^ = q.float()*s``.
  Scale granularity per (layer, kv head) is the benchmark's; per (layer, kv head, token) is
  the reference's own.
* seeded inputs follow bench/micro/attn_length_effect.py:99-102 (one CPU generator; q, then
  k, then v; fp32 normal cast to bf16).

Pinning: tests/golden/ holds outputs of the reference's own functions (imported from the
reference checkout by tests/golden/make_golden.py); tests/test_oracle.py checks this
restatement against them.  The FP8 pieces have no source in the reference checkout, so their
byte-level behaviour is pinned to torch's float8_e4m3fn cast (the operation the frozen
formula names) by an exhaustive known-answer test, and restated bit by bit in
``e4m3_bytes_from_f32`` (numpy) and oracle/ref_attention.c.
"""

from __future__ import annotations

import math

import numpy as np
import torch

E4M3_MAX = 448.0
LOG2E = 1.4426950408889634


# --------------------------------------------------------------------------------------
# attention (bench/micro/attn_length_effect.py)
# --------------------------------------------------------------------------------------
def repeat_kv(hidden_states: torch.Tensor, n_rep: int) -> torch.Tensor:
    """Expand KV heads to query heads (attn_length_effect.py:41-46)."""
    b, h_kv, s, d = hidden_states.shape
    if n_rep == 1:
        return hidden_states
    x = hidden_states[:, :, None, :, :].expand(b, h_kv, n_rep, s, d)
    return x.reshape(b, h_kv * n_rep, s, d)


def eager_attention(q, k, v, mask=None, *, scaling: float | None = None) -> torch.Tensor:
    """bf16 eager GQA attention (attn_length_effect.py:49-66).

    q [B,H_q,1,D], k/v [B,H_kv,S,D] -> [B,1,H_q,D].  Head counts come from the shapes and
    ``scaling`` defaults to D**-0.5 (module globals H_Q/H_KV/SCALING in the reference).
    """
    h_q, h_kv, d = q.shape[1], k.shape[1], q.shape[-1]
    scaling = d ** -0.5 if scaling is None else scaling
    ks = repeat_kv(k, h_q // h_kv)
    vs = repeat_kv(v, h_q // h_kv)
    w = torch.matmul(q, ks.transpose(2, 3)) * scaling
    if mask is not None:
        w = w + mask
    w = torch.nn.functional.softmax(w, dim=-1, dtype=torch.float32).to(q.dtype)
    out = torch.matmul(w, vs)
    return out.transpose(1, 2).contiguous()


def fp64_reference(q, k, v, *, scaling: float | None = None) -> torch.Tensor:
    """float64 attention over the valid keys only (attn_length_effect.py:69-75)."""
    h_q, h_kv, d = q.shape[1], k.shape[1], q.shape[-1]
    scaling = d ** -0.5 if scaling is None else scaling
    q64 = q.double()
    k64 = repeat_kv(k.double(), h_q // h_kv)
    v64 = repeat_kv(v.double(), h_q // h_kv)
    w = torch.softmax(torch.matmul(q64, k64.transpose(2, 3)) * scaling, dim=-1)
    return torch.matmul(w, v64).transpose(1, 2).contiguous()


def pad_and_mask(k, v, capacity: int, fill: float = 0.0):
    """Pad K/V [B,H_kv,L,D] to capacity and build the additive mask
    (attn_length_effect.py:106-111; fill value as in padded_reference.py:41-43)."""
    b, h_kv, length, d = k.shape
    pad = capacity - length
    if pad < 0:
        raise ValueError(f"length {length} exceeds capacity {capacity}")
    k_pad = torch.cat([k, torch.full((b, h_kv, pad, d), fill, dtype=k.dtype)], dim=-2)
    v_pad = torch.cat([v, torch.full((b, h_kv, pad, d), fill, dtype=v.dtype)], dim=-2)
    mask = torch.full((1, 1, 1, capacity), torch.finfo(torch.bfloat16).min, dtype=torch.bfloat16)
    mask[..., :length] = 0
    return k_pad, v_pad, mask


# --------------------------------------------------------------------------------------
# FP8 e4m3 (docs/journal/2026-10-23-phase2-r3-coordinator.md:43-49)
# --------------------------------------------------------------------------------------
def head_scales(x: torch.Tensor) -> torch.Tensor:
    """Per-(kv head) scale of x [B,H_kv,L,D] bf16: amax|x| / 448 in fp32 -> [H_kv].  A head that is
    zero everywhere gets scale 1 (the formula's 0 would turn every later x/s into NaN or +-448)."""
    s = x.float().abs().amax(dim=(0, 2, 3)) / E4M3_MAX
    return torch.where(s == 0, torch.ones_like(s), s)


def token_scales(x: torch.Tensor) -> torch.Tensor:
    """Per-(token, kv head) scale of x [B,H_kv,L,D]: amax over D / 448 -> [B,L,H_kv]
    (the reference's `[capacity, kv_heads]` layout per layer)."""
    return (x.float().abs().amax(dim=3) / E4M3_MAX).permute(0, 2, 1).contiguous()


def quantize_e4m3(x: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    """clamp(x/s, -448, 448).to(e4m3fn) -> uint8 bytes.  `scale` broadcasts against x.  A zero scale
    (an all-zero row or head; the formula's 0/0 has no frozen meaning) gives zero bytes."""
    scale = torch.as_tensor(scale, dtype=torch.float32)
    zero = scale == 0
    y = (x.float() / torch.where(zero, torch.ones_like(scale), scale)).clamp(-E4M3_MAX, E4M3_MAX)
    q = y.to(torch.float8_e4m3fn).view(torch.uint8)
    return torch.where(zero.expand_as(q), torch.zeros_like(q), q)


def quantize_per_head(x: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    """x [B,H_kv,L,D] bf16, scale [H_kv] -> uint8 [B,H_kv,L,D]."""
    return quantize_e4m3(x, scale.view(1, -1, 1, 1))


def quantize_per_token(x: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    """x [B,H_kv,L,D] bf16, scale [B,L,H_kv] -> uint8 [B,H_kv,L,D].  An all-zero head row
    has scale 0; its bytes are defined as 0 (the formula's 0/0 has no frozen meaning)."""
    return quantize_e4m3(x, scale.permute(0, 2, 1).unsqueeze(-1))


def dequantize(bytes_u8: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    """q.float()*s rounded to bf16 (what the padded torch attention consumes)."""
    return (bytes_u8.view(torch.float8_e4m3fn).float() * scale).to(torch.bfloat16)


def e4m3_bytes_from_f32(y: np.ndarray) -> np.ndarray:
    """Bit-level restatement of the float32 -> float8_e4m3fn cast (round to nearest even,
    subnormals down to 2^-9, |y| > 464 and NaN -> 0x7F with the sign bit kept).  numpy only."""
    y = np.ascontiguousarray(y, dtype=np.float32)
    bits = y.view(np.uint32).astype(np.uint64)
    sign = ((bits >> 31) & 1).astype(np.uint8) << 7
    mag = (bits & 0x7FFFFFFF).astype(np.int64)
    out = np.zeros(y.shape, dtype=np.uint8)
    # NaN / inf / beyond the largest value that still rounds to 448 (i.e. >= 480): NaN byte
    nan_like = mag >= 0x43F00000  # 480.0f
    # normal e4m3 range: |y| >= 2^-6
    normal = (~nan_like) & (mag >= 0x3C800000)
    m = mag[normal]
    # drop 20 mantissa bits with round-to-nearest-even, rebias exponent 127 -> 7
    lsb = (m >> 20) & 1
    m = m + 0x7FFFF + lsb
    m = (m >> 20) - ((127 - 7) << 3)
    out[normal] = m.astype(np.uint8)
    # subnormal e4m3: multiples of 2^-9; RNE via float arithmetic on exact values
    sub = (~nan_like) & (~normal)
    a = np.abs(y[sub]).astype(np.float64) * 512.0  # exact
    r = np.rint(a)  # numpy rint is round-half-even
    out[sub] = r.astype(np.uint8)  # 8 -> 0x08 = smallest normal, consistent
    out[nan_like] = 0x7F
    return out | sign


# --------------------------------------------------------------------------------------
# seeded inputs and the full padded-reference pipeline
# --------------------------------------------------------------------------------------
def make_inputs(seed: int, h_q: int, h_kv: int, d: int, length: int, batch: int = 1):
    """q [B,H_q,1,D], k, v [B,H_kv,L,D] bf16 from one CPU generator, in that order
    (attn_length_effect.py:99-102)."""
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(batch, h_q, 1, d, generator=g, dtype=torch.float32).to(torch.bfloat16)
    k = torch.randn(batch, h_kv, length, d, generator=g, dtype=torch.float32).to(torch.bfloat16)
    v = torch.randn(batch, h_kv, length, d, generator=g, dtype=torch.float32).to(torch.bfloat16)
    return q, k, v


def padded_fp8_reference(q, k_bytes, v_bytes, k_scale, v_scale, capacity: int,
                         *, scaling: float | None = None, fill: float = 0.0) -> torch.Tensor:
    """The parity target: the reference's padded torch attention over the dequantised cache.

    q [B,H_q,1,D] bf16; k_bytes/v_bytes uint8 [B,H_kv,L,D] (valid prefix only);
    k_scale/v_scale [H_kv] (per head) or [B,L,H_kv] (per token).  Returns [B,1,H_q,D] bf16.
    """
    def bc(s):
        return s.view(1, -1, 1, 1) if s.dim() == 1 else s.permute(0, 2, 1).unsqueeze(-1)
    kd = dequantize(k_bytes, bc(k_scale))
    vd = dequantize(v_bytes, bc(v_scale))
    k_pad, v_pad, mask = pad_and_mask(kd, vd, capacity, fill)
    return eager_attention(q, k_pad, v_pad, mask=mask, scaling=scaling)


def fp64_fp8_reference(q, k_bytes, v_bytes, k_scale, v_scale, *, scaling=None) -> torch.Tensor:
    """float64 attention over the same quantised KV, exact dequant (no bf16 rounding)."""
    def bc(s):
        return s.view(1, -1, 1, 1) if s.dim() == 1 else s.permute(0, 2, 1).unsqueeze(-1)
    kd = k_bytes.view(torch.float8_e4m3fn).double() * bc(k_scale).double()
    vd = v_bytes.view(torch.float8_e4m3fn).double() * bc(v_scale).double()
    h_q, h_kv, d = q.shape[1], kd.shape[1], q.shape[-1]
    scaling = d ** -0.5 if scaling is None else scaling
    w = torch.softmax(torch.matmul(q.double(), repeat_kv(kd, h_q // h_kv).transpose(2, 3)) * scaling, dim=-1)
    return torch.matmul(w, repeat_kv(vd, h_q // h_kv)).transpose(1, 2).contiguous()


def error_metrics(out: torch.Tensor, ref: torch.Tensor) -> dict:
    """max abs error, cosine, nrmse (metric definitions of runner/ops/nvfp4/reference.py:179-195)."""
    a = out.double().flatten()
    b = ref.double().flatten()
    diff = a - b
    denom = float(b.norm()) or 1.0
    cos = float(torch.dot(a, b) / (a.norm() * b.norm())) if float(a.norm()) > 0 and float(b.norm()) > 0 else (
        1.0 if float(diff.abs().max()) == 0 else 0.0)
    return {
        "max_abs": float(diff.abs().max()) if diff.numel() else 0.0,
        "cosine": cos,
        "nrmse": float(diff.norm()) / denom,
    }


def decode_step_reference(q, k_cache_bytes, v_cache_bytes, k_scale, v_scale, seq_len, capacity,
                          *, scaling=None):
    """Multi-layer, batched wrapper used by the parity tests.

    q [N,B,H_q,D] bf16; caches uint8 [N,B,H_kv,capacity,D]; scales [N,H_kv] or
    [N,B,capacity,H_kv]; seq_len list[int] of B valid lengths.  Returns bf16 [N,B,H_q,D]:
    each (layer, sequence) goes through ``padded_fp8_reference`` separately, as the
    reference runs bs=1.
    """
    n, b, h_q, d = q.shape
    out = torch.zeros(n, b, h_q, d, dtype=torch.bfloat16)
    for layer in range(n):
        for s in range(b):
            length = int(seq_len[s])
            if length == 0:
                continue
            kb = k_cache_bytes[layer, s:s + 1, :, :length]
            vb = v_cache_bytes[layer, s:s + 1, :, :length]
            if k_scale.dim() == 2:
                ks, vs = k_scale[layer], v_scale[layer]
            else:
                ks, vs = k_scale[layer, s:s + 1, :length], v_scale[layer, s:s + 1, :length]
            o = padded_fp8_reference(q[layer, s].view(1, h_q, 1, d), kb, vb, ks, vs, capacity,
                                     scaling=scaling)
            out[layer, s] = o.view(h_q, d)
    return out


def cpu_attention_seconds(h_q: int, h_kv: int, d: int, depth: int, capacity: int, layers: int,
                          repeats: int, threads: int, seed: int = 0) -> dict:
    """Time the padded torch attention (dequant + pad + attention) on the host cores.

    Returns seconds per layer (median) for the full pipeline and for attention alone.
    """
    import time
    torch.set_num_threads(threads)
    q, k, v = make_inputs(seed, h_q, h_kv, d, depth)
    sk, sv = head_scales(k), head_scales(v)
    kb, vb = quantize_per_head(k, sk), quantize_per_head(v, sv)
    full, attn_only = [], []
    for i in range(repeats + 1):
        for _ in range(layers):
            t0 = time.perf_counter()
            kd = dequantize(kb, sk.view(1, -1, 1, 1))
            vd = dequantize(vb, sv.view(1, -1, 1, 1))
            k_pad, v_pad, mask = pad_and_mask(kd, vd, capacity)
            t1 = time.perf_counter()
            eager_attention(q, k_pad, v_pad, mask=mask)
            t2 = time.perf_counter()
            if i > 0:
                full.append(t2 - t0)
                attn_only.append(t2 - t1)
    full.sort()
    attn_only.sort()
    return {"full_s_per_layer": full[len(full) // 2], "attn_s_per_layer": attn_only[len(attn_only) // 2],
            "threads": threads, "samples": len(full)}



# ------------------------------------------------------------------------------------------
# producer side of the attention block: q_norm / k_norm + rotary embedding
# ------------------------------------------------------------------------------------------
def qk_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """The head-dim RMS norm the reference's model applies to query and key heads before the
    rotary embedding (Qwen3_5Attention.q_norm / k_norm of transformers 5.5.0, the model class the
    reference loads: runner/loader/nvfp4_model.py:82-88,145).  Zero-centred weight: computed in
    fp32 as x * rsqrt(mean(x^2) + eps) * (1 + w), then rounded to x's dtype."""
    xf = x.float()
    return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * (1.0 + weight.float())).to(x.dtype)


def partial_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """Rotary embedding on the first cos.shape[-1] dims of every head, the rest passes through
    (apply_rotary_pos_emb of the same model file).  x [B, H, T, D]; cos, sin [B, T, R] in x's
    dtype.  Evaluated in x's dtype as the model does: two rounded products and a rounded sum."""
    r = cos.shape[-1]
    c, s = cos.unsqueeze(1), sin.unsqueeze(1)
    xr, xp = x[..., :r], x[..., r:]
    rot = torch.cat([-xr[..., r // 2:], xr[..., : r // 2]], dim=-1)
    return torch.cat([(xr * c) + (rot * s), xp], dim=-1)


def producer_reference(q_raw, k_raw, wq, wk, eps, cos, sin):
    """q_raw [B, H_q, 1, D], k_raw [B, H_kv, 1, D] (projection outputs of one decode step, bf16)
    -> (q, k) as the attention function and the cache update receive them."""
    return partial_rope(qk_norm(q_raw, wq, eps), cos, sin), partial_rope(qk_norm(k_raw, wk, eps), cos, sin)


def softmax_scale(d: int) -> float:
    return 1.0 / math.sqrt(d)
