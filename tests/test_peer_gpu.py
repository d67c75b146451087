"""Fused output all-gather over peer memory: two ranks, one GPU each (skipped with fewer than 2 GPUs).
Sharded result == single-GPU result, bit for bit (heads are independent)."""
import importlib
import os
import sys
from pathlib import Path

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parents[1]


def _worker(rank, world, port, ret):
    import torch.distributed as dist
    sys.path.insert(0, str(ROOT)); sys.path.insert(0, str(ROOT / "tests"))
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    pkg = importlib.import_module("qwen38-5080_b200")
    from oracle import ref_attention as oracle
    from helpers import build_case
    n_layers, batch, h_q, h_kv, d, cap, lens = 3, 2, 40, 8, 128, 512, [300, 77]
    case = build_case(oracle, n_layers, batch, h_q, h_kv, d, lens, cap, seed=17)
    kv, qs = pkg.dist.head_shard(h_q, h_kv, world, rank)
    loc = {"q": case["q"][:, :, qs].contiguous().to(dev), "k": case["k_cache"][:, :, kv].contiguous().to(dev),
           "v": case["v_cache"][:, :, kv].contiguous().to(dev), "ks": case["k_scale"][:, kv].contiguous().to(dev),
           "vs": case["v_scale"][:, kv].contiguous().to(dev)}
    shape = pkg.make_shape(h_q // world, loc["k"], loc["v"], loc["ks"])
    seq = torch.tensor(lens, dtype=torch.int32, device=dev)
    peer = pkg.dist.PeerOutput(loc["q"], world, rank)
    ref_case = {k: (v.to(dev) if isinstance(v, torch.Tensor) else v) for k, v in case.items()}
    shape1 = pkg.make_shape(h_q, ref_case["k_cache"], ref_case["v_cache"], ref_case["k_scale"])
    g = torch.Generator().manual_seed(5)
    k_new = torch.randn(n_layers, batch, h_kv, d, generator=g).to(torch.bfloat16)
    v_new = torch.randn(n_layers, batch, h_kv, d, generator=g).to(torch.bfloat16)
    ok = True
    for variant in ("mma", "umma2"):
        ws = pkg.Workspace(shape, dev, variant=variant)
        ws1 = pkg.Workspace(shape1, dev, variant=variant)
        for step in range(3):      # repeated steps: the barrier's epoch advances on the device
            peer.full.fill_(float("nan"))
            torch.cuda.synchronize(); dist.barrier()
            full = pkg.decode_attention(loc["q"], loc["k"], loc["v"], loc["ks"], loc["vs"], seq, workspace=ws, peer_out=peer)
            pkg.peer_barrier(peer, ws.status)
            torch.cuda.synchronize()
            # single-GPU answer on this rank for comparison
            want = pkg.decode_attention(ref_case["q"], ref_case["k_cache"], ref_case["v_cache"], ref_case["k_scale"],
                                        ref_case["v_scale"], seq, workspace=ws1)
            torch.cuda.synchronize()
            ok = ok and torch.equal(full.view(torch.int16), want.view(torch.int16)) and ws.read_status() == 0
            dist.barrier()
        # the whole decode step (append + attend + advance) with the gathered output, against one GPU
        kc, vc = loc["k"].clone(), loc["v"].clone()
        kc1, vc1 = ref_case["k_cache"].clone(), ref_case["v_cache"].clone()
        pos, pos1 = seq.clone(), seq.clone()
        for step in range(2):
            peer.full.fill_(float("nan"))
            torch.cuda.synchronize(); dist.barrier()
            full = pkg.append_decode(loc["q"], k_new[:, :, kv].contiguous().to(dev), v_new[:, :, kv].contiguous().to(dev), kc, vc,
                                     loc["ks"], loc["vs"], pos, workspace=ws, peer_out=peer, barrier=step == 1)
            if step == 0:          # the barrier as a call of its own, then as part of the step
                pkg.peer_barrier(peer, ws.status)
            want = pkg.append_decode(ref_case["q"], k_new.to(dev), v_new.to(dev), kc1, vc1, ref_case["k_scale"],
                                     ref_case["v_scale"], pos1, workspace=ws1)
            torch.cuda.synchronize()
            ok = ok and torch.equal(full.view(torch.int16), want.view(torch.int16)) and ws.read_status() == 0
            ok = ok and torch.equal(kc, kc1[:, :, kv]) and torch.equal(vc, vc1[:, :, kv]) and torch.equal(pos, pos1)
            ok = ok and pos.cpu().tolist() == [x + step + 1 for x in lens]
            dist.barrier()
    ret[rank] = bool(ok)
    torch.cuda.synchronize(); dist.barrier()
    os._exit(0)


def test_fused_all_gather_matches_single_gpu():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    import torch.multiprocessing as mp
    world, port = 2, 29600 + os.getpid() % 300
    with mp.Manager() as mgr:
        ret = mgr.dict()
        procs = [mp.get_context("spawn").Process(target=_worker, args=(r, world, port, ret)) for r in range(world)]
        for p in procs:
            p.start()
        for p in procs:
            p.join(timeout=180)
        alive = [p for p in procs if p.is_alive()]
        for p in alive:
            p.kill()
        assert not alive, "a rank did not finish"
        assert dict(ret) == {0: True, 1: True}
