"""Host-side logic of the multi-GPU shardings, run as two gloo ranks on the CPU."""
import importlib
import os
import sys
from pathlib import Path

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parents[1]


def _load_dist():
    if str(ROOT) not in sys.path:
        sys.path.insert(0, str(ROOT))
    return importlib.import_module("qwen38-5080_b200.dist")


def test_head_shard_and_sequence_plan():
    d = _load_dist()
    kv, q = d.head_shard(40, 8, 4, 2)
    assert (kv.start, kv.stop, q.start, q.stop) == (4, 6, 20, 30)
    with pytest.raises(ValueError):
        d.head_shard(40, 8, 3, 0)
    g = torch.Generator().manual_seed(0)
    depths = torch.randint(1024, 16385, (16,), generator=g).tolist()
    for world in (1, 2, 4, 8):
        plan = d.assign_sequences(depths, world)
        assert sorted(i for p in plan for i in p) == list(range(16))
        loads = [sum(depths[i] for i in p) for p in plan]
        assert max(loads) - min(loads) <= max(depths)          # greedy bound
        assert max(loads) <= 1.08 * sum(depths) / world          # greedy alone: 1.18 on 8 ranks (two sequences per rank)


def _worker(rank, world, port, ret):
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        d = _load_dist()
        n, b, h_q, h_kv, dim = 3, 2, 40, 8, 16
        full = torch.arange(n * b * h_q * dim, dtype=torch.float32).view(n, b, h_q, dim).to(torch.bfloat16)
        _, qs = d.head_shard(h_q, h_kv, world, rank)
        local = full[:, :, qs].contiguous()
        hg = d.HeadGather(local, world)
        got = hg.gather(local)
        ok1 = torch.equal(got, full)
        # sequence sharding: ragged plan, gather back in original order
        depths = [900, 100, 500, 300, 50]
        plan = d.assign_sequences(depths, world)
        seq_full = torch.arange(n * 5 * 4 * dim, dtype=torch.float32).view(n, 5, 4, dim)
        mine = seq_full[:, plan[rank]].contiguous()
        back = d.gather_sequences(mine, plan, 5)
        ok2 = torch.equal(back, seq_full)
        ret[rank] = (ok1, ok2)
    finally:
        dist.destroy_process_group()


def test_two_rank_gather_paths_on_gloo():
    world = 2
    port = 29500 + os.getpid() % 2000
    with mp.Manager() as mgr:
        ret = mgr.dict()
        mp.spawn(_worker, args=(world, port, ret), nprocs=world, join=True)
        assert dict(ret) == {0: (True, True), 1: (True, True)}
