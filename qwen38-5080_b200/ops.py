"""Attention-op level API: torch tensors in, C-ABI calls out.

Signature follows the op the reference runs inside its decode step (q, KV-cache handles,
per-head scales, sequence lengths, cache capacity): the FP8 counterpart of
``StaticCapFullAttentionLayer.update`` + eager attention
(runner/model/static_cache.py:69-82, bench/micro/attn_length_effect.py:49-66 in the reference).
torch only owns memory and streams here; all arithmetic runs in libb200attn.so.

Layouts (n_layers may be dropped for a single layer):
    q, out           bf16  [n_layers, batch, h_q, head_dim]
    k_cache, v_cache uint8 / float8_e4m3fn [n_layers, batch, h_kv, capacity, head_dim]
    k_new, v_new     bf16  [n_layers, batch, h_kv, head_dim]  (bulk: [..., h_kv, n_tokens, head_dim])
    k_scale, v_scale fp32  [n_layers, h_kv]  or  [n_layers, batch, capacity, h_kv] (per token)
    seq_len, seq_pos int32 [batch] on the device
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass

import torch

from . import _lib
from ._lib import B200AttnShape, B200AttnError, VARIANTS, check


def _ptr(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _need_cuda(*tensors: torch.Tensor) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise ValueError("b200attn ops need CUDA tensors: there is no CPU path")
        if t is not None and not t.is_contiguous():
            raise ValueError("b200attn ops need contiguous tensors")


def _as5(cache: torch.Tensor) -> torch.Tensor:
    return cache if cache.dim() == 5 else cache.unsqueeze(0)


@dataclass
class Geometry:
    shape: B200AttnShape

    @property
    def pairs(self) -> int:
        s = self.shape
        return s.n_layers * s.batch * s.h_kv


def make_shape(h_q: int, k_cache: torch.Tensor, v_cache: torch.Tensor, k_scale: torch.Tensor) -> B200AttnShape:
    """Geometry from the cache handles.  A 5-d cache may be strided over layers (dim 0) only."""
    kc, vc = _as5(k_cache), _as5(v_cache)
    if kc.shape != vc.shape:
        raise ValueError("k_cache and v_cache must have the same shape")
    n, b, h_kv, cap, d = kc.shape
    for c in (kc, vc):
        if c.element_size() != 1:
            raise ValueError("KV cache must be uint8 / float8_e4m3fn")
        if c.stride()[1:] != (h_kv * cap * d, cap * d, d, 1):
            raise ValueError("KV cache must be dense within a layer")
    scale_mode = _lib.SCALE_PER_HEAD if k_scale.numel() == n * h_kv else _lib.SCALE_PER_TOKEN
    if scale_mode == _lib.SCALE_PER_TOKEN and k_scale.numel() != n * b * cap * h_kv:
        raise ValueError("scales must be [n_layers, h_kv] or [n_layers, batch, capacity, h_kv]")
    return B200AttnShape(n, b, h_q, h_kv, d, cap, scale_mode, 0,
                         kc.stride(0) if n > 1 else 0, vc.stride(0) if n > 1 else 0)


def pick_splits(shape: B200AttnShape, max_seq_len: int | None = None, num_sms: int | None = None,
                variant: str = "auto") -> int:
    if num_sms is None:
        num_sms = torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count \
            if torch.cuda.is_available() else 148
    n = _lib.lib().b200attn_pick_splits(ctypes.byref(shape), shape.capacity if max_seq_len is None else max_seq_len,
                                        num_sms, VARIANTS[variant])
    return check(n, "b200attn_pick_splits")


def workspace_bytes(shape: B200AttnShape, num_splits: int, variant: str = "auto") -> int:
    out = ctypes.c_size_t(0)
    check(_lib.lib().b200attn_workspace_bytes(ctypes.byref(shape), num_splits, VARIANTS[variant], ctypes.byref(out)),
          "b200attn_workspace_bytes")
    return out.value


class Workspace:
    """Split-K partials (tagged words) + the step's CTA counter, allocated once (before any graph capture)."""

    def __init__(self, shape: B200AttnShape, device, variant: str = "auto", num_splits: int = 0,
                 max_seq_len: int | None = None):
        self.variant = variant
        code = check(_lib.lib().b200attn_resolve_variant(ctypes.byref(shape), VARIANTS[variant]), "b200attn_resolve_variant")
        self.resolved = next(name for name, c in VARIANTS.items() if c == code)   # the kernel "auto" stands for
        self.num_splits = num_splits or pick_splits(shape, max_seq_len, variant=variant)
        self.nbytes = max(256, workspace_bytes(shape, self.num_splits, variant))
        self.buf = torch.empty(self.nbytes, dtype=torch.uint8, device=device)
        self.status = torch.zeros(1, dtype=torch.int32, device=device)
        self.init()

    def init(self) -> None:
        check(_lib.lib().b200attn_workspace_init(self.buf.data_ptr(), self.nbytes, _stream()), "b200attn_workspace_init")

    def read_status(self) -> int:
        """Device status bits (synchronises; not for use inside a captured step)."""
        return int(self.status.item())


def kv_quant_append(k_new, v_new, k_cache, v_cache, k_scale, v_scale, seq_pos, *, h_q: int | None = None,
                    advance: bool = True, status: torch.Tensor, n_tokens: int | None = None) -> None:
    """FP8 quantize-and-append of one token (or `n_tokens` tokens) per sequence, all layers at once."""
    _need_cuda(k_new, v_new, k_scale, v_scale, seq_pos, status)
    kc = _as5(k_cache)
    shape = make_shape(h_q or kc.shape[2], k_cache, v_cache, k_scale)
    n, b, h_kv, cap, d = kc.shape
    want = n * b * h_kv * d * (n_tokens or 1)
    if k_new.numel() != want or v_new.numel() != want or k_new.dtype != torch.bfloat16 or v_new.dtype != torch.bfloat16:
        raise ValueError(f"k_new/v_new must be bf16 with {want} elements")
    if seq_pos.dtype != torch.int32 or seq_pos.numel() != b:
        raise ValueError("seq_pos must be int32 [batch]")
    L = _lib.lib()
    if n_tokens is None:
        rc = L.b200attn_kv_quant_append(ctypes.byref(shape), _ptr(k_new), _ptr(v_new), _ptr(k_cache), _ptr(v_cache),
                                        _ptr(k_scale), _ptr(v_scale), _ptr(seq_pos), int(advance), _ptr(status), _stream())
    else:
        rc = L.b200attn_kv_quant_append_bulk(ctypes.byref(shape), n_tokens, _ptr(k_new), _ptr(v_new), _ptr(k_cache),
                                             _ptr(v_cache), _ptr(k_scale), _ptr(v_scale), _ptr(seq_pos), int(advance),
                                             _ptr(status), _stream())
    check(rc, "b200attn_kv_quant_append")


def decode_attention(q, k_cache, v_cache, k_scale, v_scale, seq_len, *, workspace: Workspace,
                     softmax_scale: float | None = None, seq_len_offset: int = 0, out: torch.Tensor | None = None,
                     variant: str | None = None, gate: torch.Tensor | None = None, peer_out=None) -> torch.Tensor:
    """Split-K GQA decode attention over the FP8 cache; returns bf16 with q's shape.
    With `gate` (bf16, q's shape) the result is bf16(bf16(attention) * bf16(sigmoid(gate))).
    With `peer_out` (tensor parallel) the results go into every rank's gathered buffer and nothing is returned:
    after the barrier, `peer_out.current()` is the gathered tensor."""
    _need_cuda(q, k_scale, v_scale, seq_len)
    if q.dtype != torch.bfloat16:
        raise ValueError("q must be bf16")
    h_q, d = q.shape[-2], q.shape[-1]
    shape = make_shape(h_q, k_cache, v_cache, k_scale)
    if q.numel() != shape.n_layers * shape.batch * h_q * d or d != shape.head_dim:
        raise ValueError("q must be [n_layers, batch, h_q, head_dim]")
    if seq_len.dtype != torch.int32 or seq_len.numel() != shape.batch:
        raise ValueError("seq_len must be int32 [batch]")
    scale = d ** -0.5 if softmax_scale is None else softmax_scale
    if peer_out is not None:   # tensor parallel: results go straight into every rank's gathered buffer
        rc = _lib.lib().b200attn_decode_peers(
            ctypes.byref(shape), ctypes.byref(peer_out.c_peers), _ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(k_scale),
            _ptr(v_scale), _ptr(seq_len), seq_len_offset, scale, VARIANTS[variant or workspace.variant],
            workspace.num_splits, _ptr(workspace.buf), workspace.nbytes, _ptr(workspace.status), _stream())
        check(rc, "b200attn_decode_peers")
        return None     # after the barrier: peer_out.current()
    if out is None:
        out = torch.empty_like(q)
    if gate is not None:
        _need_cuda(gate)
        if gate.dtype != torch.bfloat16 or gate.numel() != q.numel():
            raise ValueError("gate must be bf16 with q's shape")
        rc = _lib.lib().b200attn_decode_gated(
            ctypes.byref(shape), _ptr(q), _ptr(gate), _ptr(k_cache), _ptr(v_cache), _ptr(k_scale), _ptr(v_scale),
            _ptr(seq_len), seq_len_offset, scale, VARIANTS[variant or workspace.variant], workspace.num_splits,
            _ptr(workspace.buf), workspace.nbytes, _ptr(out), _ptr(workspace.status), _stream())
    else:
        rc = _lib.lib().b200attn_decode(
            ctypes.byref(shape), _ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(k_scale), _ptr(v_scale), _ptr(seq_len),
            seq_len_offset, scale, VARIANTS[variant or workspace.variant], workspace.num_splits, _ptr(workspace.buf),
            workspace.nbytes, _ptr(out), _ptr(workspace.status), _stream())
    check(rc, "b200attn_decode")
    return out


def peer_barrier(peer_out, status: torch.Tensor) -> None:
    """Cross-GPU arrive-and-wait after `decode_attention(..., peer_out=...)` (same stream); nothing to do in packet mode."""
    if not peer_out.needs_barrier:
        return
    check(_lib.lib().b200attn_peer_barrier(peer_out.c_flags, peer_out.rank, peer_out.world, _ptr(status), _stream()),
          "b200attn_peer_barrier")


def append_decode(q, k_new, v_new, k_cache, v_cache, k_scale, v_scale, seq_pos, *, workspace: Workspace,
                  softmax_scale: float | None = None, advance: bool = True, out: torch.Tensor | None = None,
                  variant: str | None = None, peer_out=None, barrier: bool = False) -> torch.Tensor:
    """One decode step: append this token's K/V at seq_pos, attend seq_pos+1 tokens, bump seq_pos.
    With `peer_out` (tensor parallel) the results go into every rank's gathered tensor (`peer_out.current()`); in its
    stores mode either pass `barrier=True` (the cross-GPU arrive-and-wait becomes part of the step) or follow with
    `peer_barrier`; in packet mode the step is complete by itself."""
    _need_cuda(q, k_new, v_new, k_scale, v_scale, seq_pos)
    h_q, d = q.shape[-2], q.shape[-1]
    shape = make_shape(h_q, k_cache, v_cache, k_scale)
    if peer_out is not None:
        rc = _lib.lib().b200attn_append_decode_peers(
            ctypes.byref(shape), ctypes.byref(peer_out.c_peers), _ptr(q), _ptr(k_new), _ptr(v_new), _ptr(k_cache),
            _ptr(v_cache), _ptr(k_scale), _ptr(v_scale), _ptr(seq_pos), int(advance),
            d ** -0.5 if softmax_scale is None else softmax_scale, VARIANTS[variant or workspace.variant],
            workspace.num_splits, _ptr(workspace.buf), workspace.nbytes, peer_out.c_flags if barrier and peer_out.needs_barrier else None,
            _ptr(workspace.status), _stream())
        check(rc, "b200attn_append_decode_peers")
        return None     # after the barrier: peer_out.current()
    if out is None:
        out = torch.empty_like(q)
    scale = d ** -0.5 if softmax_scale is None else softmax_scale
    rc = _lib.lib().b200attn_append_decode(
        ctypes.byref(shape), _ptr(q), _ptr(k_new), _ptr(v_new), _ptr(k_cache), _ptr(v_cache), _ptr(k_scale),
        _ptr(v_scale), _ptr(seq_pos), int(advance), scale, VARIANTS[variant or workspace.variant],
        workspace.num_splits, _ptr(workspace.buf), workspace.nbytes, _ptr(out), _ptr(workspace.status), _stream())
    check(rc, "b200attn_append_decode")
    return out


def qk_norm_rope_append(q_raw, k_raw, v_new, q_norm_weight, k_norm_weight, cos, sin, k_cache, v_cache, k_scale, v_scale,
                        seq_pos, *, eps: float = 1e-6, advance: bool = False, status: torch.Tensor,
                        q_out: torch.Tensor | None = None, k_out: torch.Tensor | None = None) -> torch.Tensor:
    """Producer side of the attention block for one decode step of all layers: q_norm / k_norm, rotary
    embedding, FP8 quantize-and-append of the rotated key and the value.  Returns the rotated query
    (bf16, q_raw's shape) for `decode_attention`.  cos, sin: bf16 [batch, rotary_dim]."""
    _need_cuda(q_raw, k_raw, v_new, q_norm_weight, k_norm_weight, cos, sin, k_scale, v_scale, seq_pos, status)
    h_q, d = q_raw.shape[-2], q_raw.shape[-1]
    shape = make_shape(h_q, k_cache, v_cache, k_scale)
    for t in (q_raw, k_raw, v_new, q_norm_weight, k_norm_weight, cos, sin):
        if t.dtype != torch.bfloat16 or not t.is_contiguous():
            raise ValueError("q_raw, k_raw, v_new, norm weights, cos and sin must be contiguous bf16")
    if q_raw.numel() != shape.n_layers * shape.batch * h_q * d or k_raw.numel() != shape.n_layers * shape.batch * shape.h_kv * d \
            or v_new.numel() != k_raw.numel():
        raise ValueError("q_raw / k_raw / v_new must be [n_layers, batch, heads, head_dim]")
    if q_norm_weight.numel() != shape.n_layers * d or k_norm_weight.numel() != shape.n_layers * d:
        raise ValueError("norm weights must be [n_layers, head_dim]")
    rotary_dim = cos.shape[-1]
    if cos.numel() != shape.batch * rotary_dim or sin.shape != cos.shape:
        raise ValueError("cos and sin must be [batch, rotary_dim]")
    if q_out is None:
        q_out = torch.empty_like(q_raw)
    rc = _lib.lib().b200attn_qk_norm_rope_append(
        ctypes.byref(shape), _ptr(q_raw), _ptr(k_raw), _ptr(v_new), _ptr(q_norm_weight), _ptr(k_norm_weight), eps, _ptr(cos),
        _ptr(sin), rotary_dim, _ptr(q_out), _ptr(k_out) if k_out is not None else None, _ptr(k_cache), _ptr(v_cache),
        _ptr(k_scale), _ptr(v_scale), _ptr(seq_pos), int(advance), _ptr(status), _stream())
    check(rc, "b200attn_qk_norm_rope_append")
    return q_out


def dequant_prefix(cache, scale, n_tokens: int, *, h_q: int | None = None) -> torch.Tensor:
    """bf16 [n_layers, batch, h_kv, n_tokens, head_dim] view of the first n_tokens slots."""
    c5 = _as5(cache)
    shape = make_shape(h_q or c5.shape[2], cache, cache, scale)
    n, b, h_kv, cap, d = c5.shape
    out = torch.empty(n, b, h_kv, n_tokens, d, dtype=torch.bfloat16, device=cache.device)
    if n_tokens:
        check(_lib.lib().b200attn_dequant_prefix(ctypes.byref(shape), n_tokens, _ptr(cache), c5.stride(0) if n > 1 else 0,
                                                 _ptr(scale), _ptr(out), _stream()), "b200attn_dequant_prefix")
    return out


def calibrate_scales(x: torch.Tensor, capacity: int) -> torch.Tensor:
    """scale[layer, head] = amax|x| / 448 over x bf16 [n_layers, batch, h_kv, n_tokens, head_dim]."""
    _need_cuda(x)
    n, b, h_kv, t, d = x.shape
    shape = B200AttnShape(n, b, h_kv, h_kv, d, max(capacity, 1), _lib.SCALE_PER_HEAD, 0, 0, 0)
    scale = torch.empty(n, h_kv, dtype=torch.float32, device=x.device)
    check(_lib.lib().b200attn_calibrate_scales(ctypes.byref(shape), t, _ptr(x), _ptr(scale), _stream()),
          "b200attn_calibrate_scales")
    return scale


__all__ = ["B200AttnError", "B200AttnShape", "Workspace", "make_shape", "pick_splits", "workspace_bytes",
           "kv_quant_append", "decode_attention", "peer_barrier", "append_decode", "dequant_prefix", "calibrate_scales",
           "qk_norm_rope_append"]
