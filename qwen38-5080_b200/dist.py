"""Multi-GPU partitioning of the decode-attention path (one process per GPU, torch.distributed).

The reference is single-GPU; these shardings follow the benchmark's configurations:

* KV-head tensor parallel for one long sequence: rank r owns KV heads
  [r*h_kv/P, (r+1)*h_kv/P) and the query heads of those groups, for every layer.  Attention per
  KV head is independent (softmax is per query head), so ranks never exchange partials; the one
  exchange per step is an all-gather of the bf16 output.
* sequence sharding for batched decode: whole sequences per rank, balanced on total depth; no
  collective on the data path.
"""
from __future__ import annotations

import torch


def head_shard(h_q: int, h_kv: int, world: int, rank: int) -> tuple[slice, slice]:
    """(kv-head slice, query-head slice) owned by `rank`."""
    if h_kv % world or h_q % h_kv:
        raise ValueError(f"cannot shard {h_kv} KV heads over {world} ranks")
    per = h_kv // world
    group = h_q // h_kv
    return slice(rank * per, (rank + 1) * per), slice(rank * per * group, (rank + 1) * per * group)


def assign_sequences(depths: list[int], world: int) -> list[list[int]]:
    """Assignment of sequence indices to ranks that balances total depth: greedy longest-first, then moves and swaps
    between pairs of ranks for as long as one lowers the larger load of its pair (with two sequences per rank the
    greedy plan alone leaves the busiest rank 18 % above the mean on the benchmark's ragged batch).  Deterministic
    (ties broken by index), so every rank computes the same plan.  A rank may end up with no sequence only when
    there are fewer sequences than ranks."""
    load = [0] * world
    plan: list[list[int]] = [[] for _ in range(world)]
    for idx in sorted(range(len(depths)), key=lambda i: (-depths[i], i)):
        r = min(range(world), key=lambda j: (load[j], len(plan[j]), j))
        plan[r].append(idx)
        load[r] += depths[idx]
    # pairwise balancing: the move or swap between any two ranks that lowers the larger of their two loads the most;
    # every accepted step lowers the sum of squared loads, so this ends by itself (the bound is a safety belt)
    for _ in range(64 * max(1, len(depths)) * world):
        best = None                                     # (gain, kind, a, b, i, j)
        for a in range(world):
            for b in range(world):
                if b == a or load[a] <= load[b]:
                    continue
                for i in plan[a]:
                    if len(plan[a]) > 1:                # move i from a to b
                        gain = load[a] - max(load[a] - depths[i], load[b] + depths[i])
                        if gain > 0 and (best is None or (-gain, 0, a, b, i, -1) < best):
                            best = (-gain, 0, a, b, i, -1)
                    for j in plan[b]:                   # swap i and j
                        gain = load[a] - max(load[a] - depths[i] + depths[j], load[b] - depths[j] + depths[i])
                        if gain > 0 and (best is None or (-gain, 1, a, b, i, j) < best):
                            best = (-gain, 1, a, b, i, j)
        if best is None:
            break
        _, kind, a, b, i, j = best
        plan[a].remove(i); plan[b].append(i)
        load[a] -= depths[i]; load[b] += depths[i]
        if kind == 1:
            plan[b].remove(j); plan[a].append(j)
            load[b] -= depths[j]; load[a] += depths[j]
    for p in plan:
        p.sort()
    return plan


class HeadGather:
    """All-gather of per-rank outputs [n_layers, batch, h_q/P, D] into [n_layers, batch, h_q, D].

    Buffers are allocated once; `gather()` issues one collective on the current stream plus one
    strided copy that puts every rank's heads in place (query head order = rank order).
    """

    def __init__(self, local_like: torch.Tensor, world: int, group=None):
        import torch.distributed as dist
        self.dist, self.world, self.group = dist, world, group
        n, b, hq, d = local_like.shape
        self.staging = torch.empty(world, n, b, hq, d, dtype=local_like.dtype, device=local_like.device)
        self.full = torch.empty(n, b, world * hq, d, dtype=local_like.dtype, device=local_like.device)

    def gather(self, local: torch.Tensor) -> torch.Tensor:
        n, b, hq, d = local.shape
        self.dist.all_gather_into_tensor(self.staging.view(self.world * n, b, hq, d), local.contiguous(), group=self.group)
        self.full.view(n, b, self.world, hq, d).copy_(self.staging.permute(1, 2, 0, 3, 4))
        return self.full


class PeerOutput:
    """The gathered output [n_layers, batch, h_q_total, D] of a tensor-parallel step and what the fused
    all-gather needs around it.  The attention kernel of every rank sends its heads to all ranks over
    NVLink peer memory (symmetric memory); the all-gather is part of the kernel.

    mode "packets" (default): results travel as 8-byte packets {two bf16 values, step number} into the
    receivers' staging buffers and every launch copies what arrived for it into its own gathered tensor;
    no fence, no flag, no barrier, one gathered tensor per rank (``current()``), complete when the launch is.
    mode "stores": results are stored directly into every rank's gathered tensors — two per rank, used in
    turn, because a fast rank may start its next step while a slow rank's consumer still reads this one's —
    and a cross-GPU arrive-and-wait follows (``ops.peer_barrier`` or ``barrier=True`` on the step); which
    tensor a step writes follows, on the device, from the parity of the step counter the barrier keeps.

    Allocate once, before any graph capture; all ranks make the same calls in the same order."""

    def __init__(self, local_like: torch.Tensor, world: int, rank: int, group=None, mode: str = "packets"):
        import ctypes
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm_mem
        from . import _lib
        group = group if group is not None else dist.group.WORLD
        n, b, hq, d = local_like.shape
        dev = local_like.device
        self.world, self.rank, self.mode = world, rank, mode
        zeros8 = (ctypes.c_void_p * 8)()
        if mode == "packets":
            shape = _lib.B200AttnShape(n, b, hq, hq, d, 1, 0, 0, 0, 0)     # only layers, batch, query heads and head_dim count
            nbytes = _lib.lib().b200attn_peer_staging_bytes(ctypes.byref(shape), world)
            if nbytes == 0:
                raise ValueError("unsupported shape for the packet staging buffer")
            self.full = torch.zeros(n, b, world * hq, d, dtype=local_like.dtype, device=dev)
            self.staging = symm_mem.empty((nbytes // 8,), dtype=torch.int64, device=dev)
            self.staging.zero_()
            self._stage_hdl = symm_mem.rendezvous(self.staging, group)
            self.step = torch.zeros(1, dtype=torch.int32, device=dev)
            torch.cuda.synchronize()
            dist.barrier(group)
            out = (ctypes.c_void_p * 8)()
            out[rank] = self.full.data_ptr()
            self.c_peers = _lib.B200AttnPeerOut(world, rank, world * hq, _lib.GATHER_PACKETS, out, zeros8,
                                                (ctypes.c_void_p * 8)(*[int(p) for p in self._stage_hdl.buffer_ptrs]),
                                                self.step.data_ptr())
            self.c_flags = None
            return
        if mode != "stores":
            raise ValueError("mode must be 'packets' or 'stores'")
        self.buffers = symm_mem.empty((2, n, b, world * hq, d), dtype=local_like.dtype, device=dev)
        self.buffers.zero_()
        self._out_hdl = symm_mem.rendezvous(self.buffers, group)
        self.flags = symm_mem.empty((64,), dtype=torch.int32, device=dev)
        self.flags.zero_()
        self._flag_hdl = symm_mem.rendezvous(self.flags, group)
        torch.cuda.synchronize()
        dist.barrier(group)
        half = self.buffers[0].numel() * self.buffers.element_size()
        bases = [int(p) for p in self._out_hdl.buffer_ptrs]
        flag_ptrs = [int(p) for p in self._flag_hdl.buffer_ptrs]
        self.c_peers = _lib.B200AttnPeerOut(world, rank, world * hq, _lib.GATHER_STORES_2BUF, (ctypes.c_void_p * 8)(*bases),
                                            (ctypes.c_void_p * 8)(*[p + half for p in bases]), zeros8, flag_ptrs[rank] + 4 * world)
        self.c_flags = (ctypes.c_void_p * 8)(*flag_ptrs)

    @property
    def needs_barrier(self) -> bool:
        return self.mode == "stores"

    def steps_done(self) -> int:
        """The step counter (synchronises: not for use inside a captured step)."""
        return int(self.step.item()) if self.mode == "packets" else int(self.flags[self.world].item())

    def current(self) -> torch.Tensor:
        """The gathered tensor of the latest completed step (stores mode: synchronises)."""
        return self.full if self.mode == "packets" else self.buffers[self.steps_done() & 1]

    def poison_next(self) -> None:
        """Fill the tensor the next step is going to write with NaN (for tests: a step must overwrite all of it)."""
        (self.full if self.mode == "packets" else self.buffers[(self.steps_done() + 1) & 1]).fill_(float("nan"))

    def last_wait_us(self) -> float | None:
        """Stores mode: how long this rank's latest arrive-and-wait took, from the two device time stamps the barrier leaves."""
        if self.mode == "packets":
            return None
        t = self.flags[16:20].view(torch.int64).cpu().tolist()
        return (t[1] - t[0]) / 1e3


def gather_sequences(local: torch.Tensor, plan: list[list[int]], batch: int, group=None) -> torch.Tensor:
    """Off-clock gather for parity checks of the sequence-sharded path: every rank contributes
    [n_layers, len(plan[rank]), h_q, D]; returns [n_layers, batch, h_q, D] in original order."""
    import torch.distributed as dist
    world = dist.get_world_size(group)
    n, _, hq, d = local.shape
    width = max(len(p) for p in plan)
    padded = torch.zeros(n, width, hq, d, dtype=local.dtype, device=local.device)
    padded[:, : local.shape[1]] = local
    parts = [torch.empty_like(padded) for _ in range(world)]
    dist.all_gather(parts, padded, group=group)
    out = torch.empty(n, batch, hq, d, dtype=local.dtype, device=local.device)
    for r, idxs in enumerate(plan):
        for j, b in enumerate(idxs):
            out[:, b] = parts[r][:, j]
    return out


__all__ = ["head_shard", "assign_sequences", "HeadGather", "PeerOutput", "gather_sequences"]
