"""Drop-in shim for the two plug points the reference's decode step uses.

(i)  cache-layer protocol — the object the model calls as ``past_key_values.update(k, v, layer_idx)``.
     The reference's layers (runner/model/static_cache.py:44-82) expose
     ``update(key_states[B,H_kv,q_len,D], value_states, ...) -> (K, V)``, ``get_mask_sizes``,
     ``get_seq_length``, ``reset``, and attributes ``keys``, ``values``, ``cumulative_length``,
     ``max_cache_len``, ``is_initialized``.  ``FP8StaticAttentionLayer`` keeps that surface over
     e4m3 bytes + fp32 scales: decode (q_len == 1) quantize-appends in place and returns the FP8
     cache handles; prefill (q_len > 1) bulk-appends and returns a dequantised bf16 prefix, the
     one use the reference keeps ``dequant_kv`` for
     (docs/journal/2026-10-23-phase2-r3-coordinator.md:162-163).
(ii) attention interface — a callable ``fn(module, query[B,H_q,q_len,D], key, value,
     attention_mask, scaling=..., dropout=..., **kw) -> (attn_output[B,q_len,H_q,D], None)``
     selected by ``config._attn_implementation`` (runner/loader/nvfp4_model.py:82,88 selects
     "eager").  ``fp8_decode_attention`` consumes the handles ``update`` returned.

Wiring is counted, as the reference's integration did (fused-call counters, zero fallbacks
asserted: docs/journal/2026-10-23-phase2-r3-coordinator.md:198): ``COUNTERS``.
"""
from __future__ import annotations

import torch

from . import ops

ATTENTION_NAME = "b200_fp8_decode"
COUNTERS = {"fused_decode_calls": 0, "prefill_calls": 0, "appends": 0, "bulk_appends": 0}
_LAYERS: dict[int, "FP8StaticAttentionLayer"] = {}      # id(k handle storage) -> layer


class FP8StaticAttentionLayer:
    """One decoder layer's FP8 static KV cache (fixed address, device-side length)."""

    is_sliding = False
    supports_early_init = True

    def __init__(self, max_cache_len: int, h_q: int | None = None, k_scale=None, v_scale=None):
        self.max_cache_len = int(max_cache_len)
        self.h_q = h_q
        self.is_initialized = False
        self._init_scales = (k_scale, v_scale)
        self.host_len = 0

    # -- allocation (StaticLayer.lazy/early initialisation in the reference) --------------------
    def early_initialization(self, batch_size, num_heads, head_dim, dtype=None, device="cuda"):
        dev = torch.device(device)
        shape = (batch_size, num_heads, self.max_cache_len, head_dim)
        self.keys = torch.zeros(shape, dtype=torch.uint8, device=dev)
        self.values = torch.zeros(shape, dtype=torch.uint8, device=dev)
        ks, vs = self._init_scales
        self.k_scale = torch.ones(1, num_heads, device=dev) if ks is None else ks.to(dev).view(1, num_heads).float()
        self.v_scale = torch.ones(1, num_heads, device=dev) if vs is None else vs.to(dev).view(1, num_heads).float()
        self.cumulative_length = torch.zeros(batch_size, dtype=torch.int32, device=dev)
        self.h_kv, self.head_dim, self.batch = num_heads, head_dim, batch_size
        self.h_q = self.h_q or num_heads
        shp = ops.make_shape(self.h_q, self.keys, self.values, self.k_scale)
        self.workspace = ops.Workspace(shp, dev)
        self.is_initialized = True
        _LAYERS[self.keys.data_ptr()] = self

    def set_scales(self, k_scale: torch.Tensor, v_scale: torch.Tensor) -> None:
        self.k_scale.copy_(k_scale.view(1, -1))
        self.v_scale.copy_(v_scale.view(1, -1))

    # -- cache protocol ------------------------------------------------------------------------
    def update(self, key_states: torch.Tensor, value_states: torch.Tensor, *args, **kwargs):
        if not self.is_initialized:
            b, h, _, d = key_states.shape
            self.early_initialization(b, h, d, device=key_states.device)
        q_len = key_states.shape[2]
        if q_len == 1:
            # [B,H_kv,1,D] -> [1,B,H_kv,D]: same memory order, no copy
            k_new = key_states.reshape(1, self.batch, self.h_kv, self.head_dim)
            v_new = value_states.reshape(1, self.batch, self.h_kv, self.head_dim)
            ops.kv_quant_append(k_new, v_new, self.keys, self.values, self.k_scale, self.v_scale,
                                self.cumulative_length, h_q=self.h_q, advance=True, status=self.workspace.status)
            COUNTERS["appends"] += 1
            self.host_len += 1
            return self.keys, self.values           # FP8 handles, full capacity (the "cap" decode shape)
        if self.host_len + q_len > self.max_cache_len:
            raise ValueError(f"capacity {self.max_cache_len} exceeded: {self.host_len} cached + {q_len}")
        k_new = key_states.reshape(1, self.batch, self.h_kv, q_len, self.head_dim).contiguous()
        v_new = value_states.reshape(1, self.batch, self.h_kv, q_len, self.head_dim).contiguous()
        ops.kv_quant_append(k_new, v_new, self.keys, self.values, self.k_scale, self.v_scale,
                            self.cumulative_length, h_q=self.h_q, advance=True, status=self.workspace.status,
                            n_tokens=q_len)
        COUNTERS["bulk_appends"] += 1
        self.host_len += q_len
        kd = ops.dequant_prefix(self.keys, self.k_scale, self.host_len, h_q=self.h_q)[0]
        vd = ops.dequant_prefix(self.values, self.v_scale, self.host_len, h_q=self.h_q)[0]
        COUNTERS["prefill_calls"] += 1
        return kd, vd                               # bf16 valid prefix for the stock prefill attention

    def get_mask_sizes(self, query_length: int) -> tuple[int, int]:
        if query_length == 1:
            return self.max_cache_len, 0
        return self.host_len + query_length, 0

    def get_seq_length(self) -> int:
        return self.host_len

    def get_max_cache_shape(self) -> int:
        return self.max_cache_len

    def reset(self) -> None:
        """In place: positions to zero, buffers and addresses kept (static_cache.py:161-164)."""
        if self.is_initialized:
            self.cumulative_length.zero_()
            self.keys.zero_()
            self.values.zero_()
            self.workspace.status.zero_()
            self.workspace.init()
        self.host_len = 0


def fp8_decode_attention(module, query, key, value, attention_mask=None, scaling=None, dropout=0.0, **kwargs):
    """Attention-interface function.  `key`/`value` are the FP8 handles a decode ``update`` returned;
    the mask is not read: the kernel bounds the scan by the layer's device-side length."""
    layer = _LAYERS.get(key.data_ptr()) if key.dtype == torch.uint8 else None
    if layer is None or query.shape[2] != 1:
        raise ValueError("fp8_decode_attention serves q_len == 1 over handles returned by "
                         "FP8StaticAttentionLayer.update; prefill goes through the stock attention")
    b, h_q, _, d = query.shape
    q = query.reshape(1, b, h_q, d)
    out = ops.decode_attention(q, layer.keys, layer.values, layer.k_scale, layer.v_scale, layer.cumulative_length,
                               workspace=layer.workspace, softmax_scale=scaling)
    COUNTERS["fused_decode_calls"] += 1
    return out.view(b, 1, h_q, d), None


def register() -> str:
    """Register under transformers' attention-function table; returns the implementation name."""
    from transformers.modeling_utils import ALL_ATTENTION_FUNCTIONS
    ALL_ATTENTION_FUNCTIONS[ATTENTION_NAME] = fp8_decode_attention
    return ATTENTION_NAME


def cache_layout_gate(layers, kv_format: str = "fp8-e4m3") -> bool:
    """Format-declared layout check, the counterpart of the reference's `cache_gate`, which
    hard-codes bf16 (scripts/m3_check.py:228-250) and was to become format-declared
    (docs/journal/2026-10-23-phase2-r3-coordinator.md:53-55)."""
    want = torch.uint8 if kv_format == "fp8-e4m3" else torch.bfloat16
    return all(getattr(l, "is_initialized", False) and l.keys.dtype == want and l.values.dtype == want
               and l.keys.shape[2] == l.max_cache_len for l in layers)


__all__ = ["FP8StaticAttentionLayer", "fp8_decode_attention", "register", "cache_layout_gate", "COUNTERS",
           "ATTENTION_NAME"]
