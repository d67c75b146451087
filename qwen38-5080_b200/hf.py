"""Drop-in shim for the two plug points the reference's decode step uses.

(i)  cache protocol — the container the model calls as ``past_key_values.update(k, v, layer_idx)``
     and its per-layer objects.  The reference builds a ``Cache`` whose full-attention layers are
     static layers (runner/model/static_cache.py:44-82, container and pre-allocation at :89-158)
     exposing ``update(key_states[B,H_kv,q_len,D], value_states, ...) -> (K, V)``,
     ``get_mask_sizes``, ``get_seq_length``, ``reset`` and the attributes ``keys``, ``values``,
     ``cumulative_length`` (a 0-dim device tensor), ``max_cache_len``, ``is_initialized``.
     ``FP8StaticAttentionLayer`` keeps that surface over e4m3 bytes + fp32 scales: decode
     (q_len == 1) quantize-appends in place and returns the FP8 cache handles; prefill
     (q_len > 1) bulk-appends and returns a dequantised bf16 prefix, the one use the reference
     keeps ``dequant_kv`` for (docs/journal/2026-10-23-phase2-r3-coordinator.md:162-163).
     ``build_fp8_static_cache`` / ``preallocate_kv`` mirror the reference's ``build_static_cache`` /
     ``preallocate_kv`` for a config's ``layer_types``.
(ii) attention interface — a callable ``fn(module, query[B,H_q,q_len,D], key, value,
     attention_mask, scaling=..., dropout=..., **kw) -> (attn_output[B,q_len,H_q,D], None)``
     selected by ``config._attn_implementation`` (runner/loader/nvfp4_model.py:82,88 selects
     "eager").  ``fp8_decode_attention`` consumes the handles ``update`` returned; for anything else
     (prefill, a cache that is not FP8) it runs the stock eager attention and counts that.

Wiring is counted, as the reference's integration did (fused-call counters, zero fallbacks
asserted: docs/journal/2026-10-23-phase2-r3-coordinator.md:198; fall back and count rather than
raise: ...-r4-coordinator.md:58-60): ``COUNTERS``.
"""
from __future__ import annotations

import torch
from transformers.cache_utils import Cache, CacheLayerMixin, LinearAttentionLayer

from . import ops

ATTENTION_NAME = "b200_fp8_decode"
COUNTERS = {"fused_decode_calls": 0, "fused_step_calls": 0, "prefill_attention_calls": 0, "decode_fallbacks": 0,
            "appends": 0, "bulk_appends": 0}
_LAYERS: dict[int, "FP8StaticAttentionLayer"] = {}      # data_ptr of the K handle -> layer


class FP8StaticAttentionLayer(CacheLayerMixin):
    """One decoder layer's FP8 static KV cache (fixed address, device-side length).

    ``fuse_append``: the decode ``update`` only notes the new rows; ``fp8_decode_attention`` then runs
    append + attention + position advance as the library's one-launch step.  Use it only when that
    function is the model's attention implementation (a decode ``update`` without the attention call
    that follows would lose its token)."""

    is_compileable = False
    is_sliding = False
    supports_early_init = True

    def __init__(self, max_cache_len: int, h_q: int | None = None, k_scale=None, v_scale=None, fuse_append: bool = False):
        super().__init__()
        self.max_cache_len = int(max_cache_len)
        self.h_q = h_q
        self.fuse_append = fuse_append
        self._init_scales = (k_scale, v_scale)
        self._pending = None
        self.host_len = 0

    # -- allocation (StaticLayer's lazy / early initialisation in the reference) ------------------
    def lazy_initialization(self, key_states: torch.Tensor, value_states: torch.Tensor) -> None:
        b, h, _, d = key_states.shape
        self.early_initialization(b, h, d, device=key_states.device)

    def early_initialization(self, batch_size, num_heads, head_dim, dtype=None, device="cuda"):
        dev = torch.device(device)
        self.device = dev
        shape = (batch_size, num_heads, self.max_cache_len, head_dim)
        self.keys = torch.zeros(shape, dtype=torch.uint8, device=dev)
        self.values = torch.zeros(shape, dtype=torch.uint8, device=dev)
        ks, vs = self._init_scales
        self.k_scale = torch.ones(1, num_heads, device=dev) if ks is None else ks.to(dev).view(1, num_heads).float()
        self.v_scale = torch.ones(1, num_heads, device=dev) if vs is None else vs.to(dev).view(1, num_heads).float()
        # the reference's counter is a 0-dim device tensor (static_cache.py:14-15); a batch needs one per sequence
        self.cumulative_length = torch.zeros((), dtype=torch.int32, device=dev) if batch_size == 1 \
            else torch.zeros(batch_size, dtype=torch.int32, device=dev)
        self.h_kv, self.head_dim, self.batch = num_heads, head_dim, batch_size
        self.h_q = self.h_q or num_heads
        shp = ops.make_shape(self.h_q, self.keys, self.values, self.k_scale)
        self.workspace = ops.Workspace(shp, dev)
        self.is_initialized = True
        _LAYERS[self.keys.data_ptr()] = self

    def set_scales(self, k_scale: torch.Tensor, v_scale: torch.Tensor) -> None:
        self.k_scale.copy_(k_scale.view(1, -1))
        self.v_scale.copy_(v_scale.view(1, -1))

    def _positions(self) -> torch.Tensor:
        return self.cumulative_length.view(-1)     # [batch] view of the same memory

    # -- cache protocol ------------------------------------------------------------------------
    def update(self, key_states: torch.Tensor, value_states: torch.Tensor, *args, **kwargs):
        if not self.is_initialized:
            self.lazy_initialization(key_states, value_states)
        q_len = key_states.shape[2]
        # reject on the host before any launch (runner/model/decode_runner.py:323-332)
        if self.host_len + q_len > self.max_cache_len:
            raise ValueError(f"capacity {self.max_cache_len} exceeded: {self.host_len} cached + {q_len}")
        if q_len == 1:
            # [B,H_kv,1,D] -> [1,B,H_kv,D]: same memory order, no copy when the projection output is dense
            k_new = key_states.reshape(1, self.batch, self.h_kv, self.head_dim).contiguous()
            v_new = value_states.reshape(1, self.batch, self.h_kv, self.head_dim).contiguous()
            if self.fuse_append:
                self._pending = (k_new, v_new)       # appended by the attention call that follows
            else:
                ops.kv_quant_append(k_new, v_new, self.keys, self.values, self.k_scale, self.v_scale,
                                    self._positions(), h_q=self.h_q, advance=True, status=self.workspace.status)
                COUNTERS["appends"] += 1
            self.host_len += 1
            return self.keys, self.values           # FP8 handles, full capacity (the "cap" decode shape)
        k_new = key_states.reshape(1, self.batch, self.h_kv, q_len, self.head_dim).contiguous()
        v_new = value_states.reshape(1, self.batch, self.h_kv, q_len, self.head_dim).contiguous()
        ops.kv_quant_append(k_new, v_new, self.keys, self.values, self.k_scale, self.v_scale,
                            self._positions(), h_q=self.h_q, advance=True, status=self.workspace.status,
                            n_tokens=q_len)
        COUNTERS["bulk_appends"] += 1
        self.host_len += q_len
        kd = ops.dequant_prefix(self.keys, self.k_scale, self.host_len, h_q=self.h_q)[0]
        vd = ops.dequant_prefix(self.values, self.v_scale, self.host_len, h_q=self.h_q)[0]
        return kd, vd                               # bf16 valid prefix for the stock prefill attention

    def get_mask_sizes(self, query_length: int) -> tuple[int, int]:
        if query_length == 1:
            return self.max_cache_len, 0
        return self.host_len + query_length, 0

    def get_seq_length(self) -> int:
        return self.host_len

    def get_max_cache_shape(self) -> int:
        return self.max_cache_len

    def check_status(self) -> int:
        """Device status bits of this layer's launches (synchronises: call it outside a captured step)."""
        return self.workspace.read_status()

    def reset(self) -> None:
        """In place: positions to zero, buffers and addresses kept (static_cache.py:161-164)."""
        if self.is_initialized:
            self.cumulative_length.zero_()
            self.keys.zero_()
            self.values.zero_()
            self.workspace.status.zero_()
            self.workspace.init()
        self._pending = None
        self.host_len = 0


class FP8StaticAdapterCache(Cache):
    """The container the model holds as ``past_key_values``: one layer object per decoder layer,
    assembled from ``config.layer_types`` (the reference's StaticAdapterCache, static_cache.py:89-108)."""

    def __init__(self, layers: list, capacity: int):
        super().__init__(layers=layers)
        self.capacity = int(capacity)
        self.kv_format = "fp8-e4m3"

    def __repr__(self) -> str:
        return f"FP8StaticAdapterCache(capacity={self.capacity})"

    def kv_layers(self) -> list[FP8StaticAttentionLayer]:
        return [l for l in self.layers if isinstance(l, FP8StaticAttentionLayer)]

    def check_status(self) -> int:
        st = 0
        for layer in self.kv_layers():
            if layer.is_initialized:
                st |= layer.check_status()
        return st


def build_fp8_static_cache(config, capacity: int, *, k_scales=None, v_scales=None, fuse_append: bool = False) -> FP8StaticAdapterCache:
    """FP8 static cache for a model config: an FP8 layer per ``full_attention`` entry of
    ``config.layer_types``, the stock linear-attention state layer per ``linear_attention`` entry
    (the reference's build_static_cache, static_cache.py:111-132).  ``k_scales`` / ``v_scales``:
    optional per full-attention layer [h_kv] scale tensors, in layer order."""
    layers: list = []
    n_full = 0
    h_q = config.num_attention_heads
    for idx, kind in enumerate(config.layer_types):
        if kind == "linear_attention":
            layers.append(LinearAttentionLayer())
        elif kind == "full_attention":
            ks = None if k_scales is None else k_scales[n_full]
            vs = None if v_scales is None else v_scales[n_full]
            layers.append(FP8StaticAttentionLayer(capacity, h_q=h_q, k_scale=ks, v_scale=vs, fuse_append=fuse_append))
            n_full += 1
        else:
            raise ValueError(f"unsupported layer_type {kind!r} at {idx}")
    return FP8StaticAdapterCache(layers, capacity)


def preallocate_kv(cache: FP8StaticAdapterCache, config, *, batch_size: int = 1, device="cuda") -> int:
    """Allocate every FP8 layer at capacity before the first forward; returns the KV bytes
    (the reference's preallocate_kv, static_cache.py:135-158)."""
    for layer in cache.kv_layers():
        layer.early_initialization(batch_size, config.num_key_value_heads, config.head_dim, device=torch.device(device))
    return sum(2 * layer.keys.numel() for layer in cache.kv_layers())


def fp8_decode_attention(module, query, key, value, attention_mask=None, scaling=None, dropout=0.0, **kwargs):
    """Attention-interface function.  With the FP8 handles a decode ``update`` returned, the mask is
    not read: the kernel bounds the scan by the layer's device-side length.  Prefill (q_len > 1, bf16
    prefix from ``update``) and a decode over anything but those handles run the stock eager attention."""
    layer = _LAYERS.get(key.data_ptr()) if key.dtype == torch.uint8 else None
    if layer is None or query.shape[2] != 1:
        if key.dtype == torch.uint8:
            raise ValueError("FP8 cache handles reach the attention function only from a q_len == 1 update")
        from transformers.models.qwen3_5.modeling_qwen3_5 import eager_attention_forward
        COUNTERS["prefill_attention_calls" if query.shape[2] != 1 else "decode_fallbacks"] += 1
        return eager_attention_forward(module, query, key, value, attention_mask, scaling=scaling, dropout=dropout, **kwargs)
    b, h_q, _, d = query.shape
    q = query.reshape(1, b, h_q, d).contiguous()
    if layer._pending is not None:
        k_new, v_new = layer._pending
        layer._pending = None
        out = ops.append_decode(q, k_new, v_new, layer.keys, layer.values, layer.k_scale, layer.v_scale, layer._positions(),
                                workspace=layer.workspace, softmax_scale=scaling, advance=True)
        COUNTERS["fused_step_calls"] += 1
    else:
        out = ops.decode_attention(q, layer.keys, layer.values, layer.k_scale, layer.v_scale, layer._positions(),
                                   workspace=layer.workspace, softmax_scale=scaling)
    COUNTERS["fused_decode_calls"] += 1
    return out.view(b, 1, h_q, d), None


def register() -> str:
    """Register the attention function (and the mask builder the stock prefill path needs under that
    name) in transformers' tables; returns the name to put into ``config._attn_implementation``."""
    from transformers.masking_utils import ALL_MASK_ATTENTION_FUNCTIONS, eager_mask
    from transformers.modeling_utils import ALL_ATTENTION_FUNCTIONS
    ALL_ATTENTION_FUNCTIONS.register(ATTENTION_NAME, fp8_decode_attention)
    ALL_MASK_ATTENTION_FUNCTIONS.register(ATTENTION_NAME, eager_mask)
    return ATTENTION_NAME


def cache_layout_gate(layers, kv_format: str = "fp8-e4m3") -> bool:
    """Format-declared layout check, the counterpart of the reference's `cache_gate`, which
    hard-codes bf16 (scripts/m3_check.py:228-250) and was to become format-declared
    (docs/journal/2026-10-23-phase2-r3-coordinator.md:53-55)."""
    want = torch.uint8 if kv_format == "fp8-e4m3" else torch.bfloat16
    layers = [l for l in layers if isinstance(l, CacheLayerMixin)]
    return bool(layers) and all(getattr(l, "is_initialized", False) and l.keys.dtype == want and l.values.dtype == want
                                and l.keys.shape[2] == l.max_cache_len for l in layers)


__all__ = ["FP8StaticAttentionLayer", "FP8StaticAdapterCache", "build_fp8_static_cache", "preallocate_kv",
           "fp8_decode_attention", "register", "cache_layout_gate", "COUNTERS", "ATTENTION_NAME"]
