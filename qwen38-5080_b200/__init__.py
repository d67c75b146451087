"""B200-native FP8-KV decode attention (drop-in for the reference's decode attention path)."""
from . import _lib, dist, ops
from ._lib import B200AttnError, B200AttnShape
from .cache import FP8StaticCache
from .ops import (Workspace, append_decode, peer_barrier, calibrate_scales, decode_attention, dequant_prefix, kv_quant_append,
                  make_shape, pick_splits, qk_norm_rope_append, workspace_bytes)

__all__ = ["B200AttnError", "B200AttnShape", "FP8StaticCache", "Workspace", "append_decode", "calibrate_scales",
           "decode_attention", "dequant_prefix", "kv_quant_append", "make_shape", "peer_barrier", "pick_splits", "qk_norm_rope_append",
           "workspace_bytes",
           "ops", "dist", "_lib"]
