"""FP8 static KV cache: the storage the reference's static cache adapter provides
(runner/model/static_cache.py in the reference: pre-allocated, fixed-address, zero-initialised
K/V per layer, a device-side length that advances inside the captured graph, in-place reset),
restated for e4m3 bytes + fp32 scales and for all layers in one allocation so that one launch
covers a whole decode step.
"""
from __future__ import annotations

import torch

from . import _lib, ops


class FP8StaticCache:
    """K/V bytes [n_layers, batch, h_kv, capacity, head_dim], scales, device-side positions.

    ``seq_pos[b]`` counts the tokens cached for sequence b (the reference's
    ``cumulative_length``, static_cache.py:14-15); it lives on the device and is advanced by the
    append kernel, so a captured step never needs the host.  ``host_len`` mirrors it on the host
    for the capacity guard only.
    """

    def __init__(self, n_layers: int, batch: int, h_q: int, h_kv: int, head_dim: int, capacity: int,
                 device="cuda", scale_mode: str = "per_head", variant: str = "auto", num_splits: int = 0):
        self.n_layers, self.batch, self.h_q, self.h_kv = n_layers, batch, h_q, h_kv
        self.head_dim, self.capacity = head_dim, capacity
        self.device = torch.device(device)
        self.per_token = scale_mode == "per_token"
        shape5 = (n_layers, batch, h_kv, capacity, head_dim)
        self.k_cache = torch.zeros(shape5, dtype=torch.uint8, device=self.device)
        self.v_cache = torch.zeros(shape5, dtype=torch.uint8, device=self.device)
        sshape = (n_layers, batch, capacity, h_kv) if self.per_token else (n_layers, h_kv)
        self.k_scale = torch.zeros(sshape, dtype=torch.float32, device=self.device) if self.per_token \
            else torch.ones(sshape, dtype=torch.float32, device=self.device)
        self.v_scale = self.k_scale.clone()
        self.seq_pos = torch.zeros(batch, dtype=torch.int32, device=self.device)
        self.host_len = [0] * batch
        self.shape = ops.make_shape(h_q, self.k_cache, self.v_cache, self.k_scale)
        self.workspace = ops.Workspace(self.shape, self.device, variant=variant, num_splits=num_splits)

    # ---- bookkeeping -----------------------------------------------------------------------
    @property
    def status(self) -> torch.Tensor:
        return self.workspace.status

    def nbytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in (self.k_cache, self.v_cache, self.k_scale, self.v_scale))

    def require_capacity(self, steps: int) -> None:
        """Reject on the host, before any launch, a run that would overflow the cache
        (DecodeRunner.require_capacity, runner/model/decode_runner.py:323-332)."""
        used = max(self.host_len)
        if used + steps > self.capacity:
            raise ValueError(f"capacity {self.capacity} exceeded: {used} cached + {steps} steps")

    def reset(self, zero_fill: bool = False) -> None:
        """In-place reset: positions to zero, addresses unchanged (static_cache.py:161-164)."""
        self.seq_pos.zero_()
        self.host_len = [0] * self.batch
        if zero_fill:
            self.k_cache.zero_()
            self.v_cache.zero_()
        self.workspace.status.zero_()
        self.workspace.init()

    def set_scales(self, k_scale: torch.Tensor, v_scale: torch.Tensor) -> None:
        self.k_scale.copy_(k_scale.to(self.device))
        self.v_scale.copy_(v_scale.to(self.device))

    # ---- the three operations ----------------------------------------------------------------
    def prefill(self, k: torch.Tensor, v: torch.Tensor, calibrate: bool = False) -> None:
        """Bulk quantize-append of k, v bf16 [n_layers, batch, h_kv, n_tokens, head_dim]."""
        n_tokens = k.shape[3]
        self.require_capacity(n_tokens)
        if calibrate and not self.per_token:
            self.k_scale.copy_(ops.calibrate_scales(k, self.capacity))
            self.v_scale.copy_(ops.calibrate_scales(v, self.capacity))
        ops.kv_quant_append(k.contiguous(), v.contiguous(), self.k_cache, self.v_cache, self.k_scale, self.v_scale,
                            self.seq_pos, h_q=self.h_q, advance=True, status=self.status, n_tokens=n_tokens)
        self.host_len = [x + n_tokens for x in self.host_len]

    def append(self, k_new: torch.Tensor, v_new: torch.Tensor, advance: bool = True) -> None:
        ops.kv_quant_append(k_new, v_new, self.k_cache, self.v_cache, self.k_scale, self.v_scale, self.seq_pos,
                            h_q=self.h_q, advance=advance, status=self.status)
        if advance:
            self.host_len = [x + 1 for x in self.host_len]

    def attend(self, q: torch.Tensor, out: torch.Tensor | None = None, seq_len_offset: int = 0) -> torch.Tensor:
        return ops.decode_attention(q, self.k_cache, self.v_cache, self.k_scale, self.v_scale, self.seq_pos,
                                    workspace=self.workspace, seq_len_offset=seq_len_offset, out=out)

    def step(self, q, k_new, v_new, out: torch.Tensor | None = None, count: bool = True) -> torch.Tensor:
        """Append + attend + advance: one decode step for every layer (graph capturable)."""
        out = ops.append_decode(q, k_new, v_new, self.k_cache, self.v_cache, self.k_scale, self.v_scale,
                                self.seq_pos, workspace=self.workspace, out=out)
        if count:
            self.host_len = [x + 1 for x in self.host_len]
        return out


__all__ = ["FP8StaticCache"]
