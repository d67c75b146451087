"""The two multi-GPU shardings on real GPUs, one process per GPU (skipped with fewer than 2 GPUs; runs
on min(GPUs, 8) ranks, a divisor of the 8 KV heads).

* KV-head tensor parallel with the output all-gather fused into the attention kernel (value+step packets
  into the other ranks' staging, or plain stores into every rank's gathered tensors followed by a
  barrier): a small ragged case against the single-GPU result (bit for bit where the split points coincide), and a case big
  enough that the default kernel choice is the all-tcgen05 kernel with (layer, sequence, head) pairs
  split over several CTAs, checked against the single-GPU result and the CPU oracle.
* sequence sharding of a ragged batch: every rank steps its own sequences; the gathered result is the
  single-GPU batch's.
"""
import importlib
import os
import sys
from pathlib import Path

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parents[1]


def _setup(rank, world, port):
    import torch.distributed as dist
    sys.path.insert(0, str(ROOT)); sys.path.insert(0, str(ROOT / "tests"))
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    return dist, dev, importlib.import_module("qwen38-5080_b200")


class _Checks:
    """Collects the labels of failed checks, so that a failing rank says what failed."""

    def __init__(self):
        self.failed = []

    def __call__(self, label, cond):
        if not cond:
            self.failed.append(label)


def _finish(dist, ret, rank, chk):
    ret[rank] = chk.failed if isinstance(chk, _Checks) else ([] if chk else ["failed"])
    torch.cuda.synchronize(); dist.barrier()
    os._exit(0)


def _small_worker(rank, world, port, ret):
    dist, dev, pkg = _setup(rank, world, port)
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
    peers = {mode: pkg.dist.PeerOutput(loc["q"], world, rank, mode=mode) for mode in ("packets", "stores")}
    ref_case = {k: (v.to(dev) if isinstance(v, torch.Tensor) else v) for k, v in case.items()}
    shape1 = pkg.make_shape(h_q, ref_case["k_cache"], ref_case["v_cache"], ref_case["k_scale"])
    g = torch.Generator().manual_seed(5)
    k_new = torch.randn(n_layers, batch, h_kv, d, generator=g).to(torch.bfloat16)
    v_new = torch.randn(n_layers, batch, h_kv, d, generator=g).to(torch.bfloat16)
    chk = _Checks()
    done = {"packets": 0, "stores": 0}

    def same(got, want, variant):
        # The all-tcgen05 kernel cuts this small case into one tile per CTA on one GPU and on a shard alike, so the
        # partials and their merge order are the same: bit-identical.  The mma.sync kernel sizes its grid by the number
        # of pairs, the shard's split points fall elsewhere inside the pairs of this ragged batch: last-bit differences.
        if variant == "umma2":
            return torch.equal(got.view(torch.int16), want.view(torch.int16))
        m = oracle.error_metrics(got.cpu(), want.cpu())
        return m["max_abs"] <= 2.0 ** -7 and m["cosine"] >= 0.99999
    for variant, mode in (("mma", "packets"), ("umma2", "packets"), ("mma", "stores"), ("umma2", "stores")):
        peer = peers[mode]
        ws = pkg.Workspace(shape, dev, variant=variant)
        ws1 = pkg.Workspace(shape1, dev, variant=variant)
        for step in range(3):      # repeated steps: the step counter advances on the device
            peer.poison_next()
            torch.cuda.synchronize(); dist.barrier()
            pkg.decode_attention(loc["q"], loc["k"], loc["v"], loc["ks"], loc["vs"], seq, workspace=ws, peer_out=peer)
            pkg.peer_barrier(peer, ws.status)
            torch.cuda.synchronize()
            # single-GPU answer on this rank for comparison
            want = pkg.decode_attention(ref_case["q"], ref_case["k_cache"], ref_case["v_cache"], ref_case["k_scale"],
                                        ref_case["v_scale"], seq, workspace=ws1)
            torch.cuda.synchronize()
            done[mode] += 1
            chk(f"{variant} {mode} attention {step}: result", same(peer.current(), want, variant))
            chk(f"{variant} {mode} attention {step}: status", ws.read_status() == 0)
            chk(f"{variant} {mode} attention {step}: counter {peer.steps_done()} != {done[mode]}", peer.steps_done() == done[mode])
            dist.barrier()
        # the whole decode step (append + attend + advance) with the gathered output, against one GPU
        kc, vc = loc["k"].clone(), loc["v"].clone()
        kc1, vc1 = ref_case["k_cache"].clone(), ref_case["v_cache"].clone()
        pos, pos1 = seq.clone(), seq.clone()
        for step in range(2):
            peer.poison_next()
            torch.cuda.synchronize(); dist.barrier()
            pkg.append_decode(loc["q"], k_new[:, :, kv].contiguous().to(dev), v_new[:, :, kv].contiguous().to(dev), kc, vc,
                              loc["ks"], loc["vs"], pos, workspace=ws, peer_out=peer, barrier=step == 1)
            if step == 0:          # the barrier as a call of its own, then as part of the step
                pkg.peer_barrier(peer, ws.status)
            want = pkg.append_decode(ref_case["q"], k_new.to(dev), v_new.to(dev), kc1, vc1, ref_case["k_scale"],
                                     ref_case["v_scale"], pos1, workspace=ws1)
            torch.cuda.synchronize()
            done[mode] += 1
            chk(f"{variant} {mode} step {step}: result", same(peer.current(), want, variant))
            chk(f"{variant} {mode} step {step}: status", ws.read_status() == 0)
            chk(f"{variant} {mode} step {step}: cache", torch.equal(kc, kc1[:, :, kv]) and torch.equal(vc, vc1[:, :, kv]) and torch.equal(pos, pos1))
            chk(f"{variant} {mode} step {step}: positions", pos.cpu().tolist() == [x + step + 1 for x in lens])
            chk(f"{variant} {mode} step {step}: counter {peer.steps_done()} != {done[mode]}", peer.steps_done() == done[mode])
            dist.barrier()
    _finish(dist, ret, rank, chk)


def _random_bytes(shape, gen, dev):
    x = torch.randn(shape, generator=gen, device=dev, dtype=torch.bfloat16)
    return (x.float() / (4.5 / 448)).clamp(-448, 448).to(torch.float8_e4m3fn).view(torch.uint8)


def _big_worker(rank, world, port, ret):
    """64 layers x 2 sequences in capacity 4096: the persistent grids of both stream-K kernels split the (layer,
    sequence, head) pairs of a rank's shard, so the pieces go through the split-K hand-over.  Graph-replayed steps;
    the idle gathered buffer is poisoned before every step (a step must never read or leave stale data)."""
    dist, dev, pkg = _setup(rank, world, port)
    from oracle import ref_attention as oracle
    n_layers, batch, h_q, h_kv, d, cap, lens, steps = 64, 2, 40, 8, 128, 4096, [4000, 2500], 4
    g = torch.Generator(device=dev).manual_seed(99)          # the same data on every rank
    kc = torch.full((n_layers, batch, h_kv, cap, d), 0xFF, dtype=torch.uint8, device=dev)
    vc = torch.full_like(kc, 0xFF)
    for b, L in enumerate(lens):
        kc[:, b, :, :L] = _random_bytes((n_layers, h_kv, L, d), g, dev)
        vc[:, b, :, :L] = _random_bytes((n_layers, h_kv, L, d), g, dev)
    ks = torch.full((n_layers, h_kv), 4.5 / 448, device=dev)
    vs = ks.clone()
    q = torch.randn(n_layers, batch, h_q, d, generator=g, device=dev, dtype=torch.bfloat16)
    kn = torch.randn(steps, n_layers, batch, h_kv, d, generator=g, device=dev, dtype=torch.bfloat16)
    vn = torch.randn(steps, n_layers, batch, h_kv, d, generator=g, device=dev, dtype=torch.bfloat16)
    kv, qs = pkg.dist.head_shard(h_q, h_kv, world, rank)
    # single GPU, all heads, eager steps
    one = pkg.FP8StaticCache(n_layers, batch, h_q, h_kv, d, cap, device=dev)
    one.k_cache.copy_(kc); one.v_cache.copy_(vc); one.set_scales(ks, vs)
    one.seq_pos.copy_(torch.tensor(lens, dtype=torch.int32))
    want = [one.step(q, kn[i], vn[i]).clone() for i in range(steps)]
    # this rank's heads, one graph-replayed launch per step with the gather inside; both stream-K kernels (the default
    # choice depends on the shard's size: the all-tcgen05 kernel on two GPUs, the mma.sync kernel on small shards)
    chk = _Checks()
    chk("single GPU resolves to umma2", one.workspace.resolved == "umma2")
    start = torch.tensor(lens, dtype=torch.int32, device=dev)
    q_loc = q[:, :, qs].contiguous()
    worst = 0.0
    for variant in ("umma2", "mma"):
        mine = pkg.FP8StaticCache(n_layers, batch, h_q // world, h_kv // world, d, cap, device=dev, variant=variant)
        chk(f"{variant}: resolved", mine.workspace.resolved == variant)
        mine.k_cache.copy_(kc[:, :, kv]); mine.v_cache.copy_(vc[:, :, kv]); mine.set_scales(ks[:, kv], vs[:, kv])
        k_buf, v_buf = kn[0][:, :, kv].contiguous(), vn[0][:, :, kv].contiguous()
        peer = pkg.dist.PeerOutput(q_loc, world, rank)

        def launch():
            pkg.append_decode(q_loc, k_buf, v_buf, mine.k_cache, mine.v_cache, mine.k_scale, mine.v_scale, mine.seq_pos,
                              workspace=mine.workspace, peer_out=peer, barrier=True)
        mine.seq_pos.copy_(start)
        side = torch.cuda.Stream(); side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            launch(); launch()                      # warm-up: an even number of steps keeps the buffer parity
        torch.cuda.current_stream().wait_stream(side); torch.cuda.synchronize(); dist.barrier()
        mine.k_cache.copy_(kc[:, :, kv]); mine.v_cache.copy_(vc[:, :, kv]); mine.seq_pos.copy_(start)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            launch()
        torch.cuda.synchronize(); dist.barrier()
        for i in range(steps):
            k_buf.copy_(kn[i][:, :, kv]); v_buf.copy_(vn[i][:, :, kv])
            peer.poison_next()                      # the buffer this step writes holds NaN everywhere beforehand
            torch.cuda.synchronize(); dist.barrier()
            graph.replay()
            torch.cuda.synchronize()
            got = peer.current()
            chk(f"{variant} step {i}: no NaN left", not bool(torch.isnan(got.float()).any()))
            m = oracle.error_metrics(got.cpu(), want[i].cpu())
            worst = max(worst, m["max_abs"])
            chk(f"{variant} step {i}: {m}", m["max_abs"] <= 2.0 ** -7 and m["cosine"] >= 0.99999)
            dist.barrier()
        chk(f"{variant}: status and positions", mine.workspace.read_status() == 0 and mine.seq_pos.cpu().tolist() == [x + steps for x in lens])
        chk(f"{variant}: cache bytes", torch.equal(mine.k_cache, one.k_cache[:, :, kv]) and torch.equal(mine.v_cache, one.v_cache[:, :, kv]))
    if rank == 0:      # the last step's gathered tensor against the CPU oracle, first and last layer
        got = peer.current().cpu()
        final = [x + steps for x in lens]
        for layer in (0, n_layers - 1):
            kb, vb = one.k_cache[layer:layer + 1].cpu(), one.v_cache[layer:layer + 1].cpu()
            for b, L in enumerate(final):
                kb[:, b, :, L:] = 0
                vb[:, b, :, L:] = 0
            ref = oracle.decode_step_reference(q[layer:layer + 1].cpu(), kb, vb, ks[layer:layer + 1].cpu(), vs[layer:layer + 1].cpu(), final, cap)
            m = oracle.error_metrics(got[layer:layer + 1], ref)
            chk(f"oracle layer {layer}: {m}", m["max_abs"] <= 2e-2 and m["cosine"] >= 0.9999)
    _finish(dist, ret, rank, chk)


def _sequence_worker(rank, world, port, ret):
    """Ragged batch of 8 sequences sharded by sequence (greedy longest-first plan): each rank runs the fused
    step on its own sequences, no collective on the data path; gathered off the clock and compared with the
    single-GPU batch; the local cache bytes are the single-GPU cache's rows."""
    dist, dev, pkg = _setup(rank, world, port)
    from oracle import ref_attention as oracle
    n_layers, batch, h_q, h_kv, d, cap = 8, 8, 40, 8, 128, 3200
    depths = torch.randint(200, 3001, (batch,), generator=torch.Generator().manual_seed(1)).tolist()
    g = torch.Generator(device=dev).manual_seed(7)
    kc = torch.full((n_layers, batch, h_kv, cap, d), 0xFF, dtype=torch.uint8, device=dev)
    vc = torch.full_like(kc, 0xFF)
    for b, L in enumerate(depths):
        kc[:, b, :, :L] = _random_bytes((n_layers, h_kv, L, d), g, dev)
        vc[:, b, :, :L] = _random_bytes((n_layers, h_kv, L, d), g, dev)
    ks = torch.full((n_layers, h_kv), 4.5 / 448, device=dev)
    q = torch.randn(n_layers, batch, h_q, d, generator=g, device=dev, dtype=torch.bfloat16)
    kn = torch.randn(n_layers, batch, h_kv, d, generator=g, device=dev, dtype=torch.bfloat16)
    vn = torch.randn(n_layers, batch, h_kv, d, generator=g, device=dev, dtype=torch.bfloat16)
    one = pkg.FP8StaticCache(n_layers, batch, h_q, h_kv, d, cap, device=dev)
    one.k_cache.copy_(kc); one.v_cache.copy_(vc); one.set_scales(ks, ks)
    one.seq_pos.copy_(torch.tensor(depths, dtype=torch.int32))
    want = one.step(q, kn, vn)
    plan = pkg.dist.assign_sequences(depths, world)
    idx = plan[rank]
    mine = pkg.FP8StaticCache(n_layers, len(idx), h_q, h_kv, d, cap, device=dev)
    mine.k_cache.copy_(kc[:, idx]); mine.v_cache.copy_(vc[:, idx]); mine.set_scales(ks, ks)
    mine.seq_pos.copy_(torch.tensor([depths[i] for i in idx], dtype=torch.int32))
    out = mine.step(q[:, idx].contiguous(), kn[:, idx].contiguous(), vn[:, idx].contiguous())
    torch.cuda.synchronize()
    got = pkg.dist.gather_sequences(out, plan, batch)
    m = oracle.error_metrics(got.cpu(), want.cpu())
    ok = m["max_abs"] <= 2.0 ** -7 and m["cosine"] >= 0.99999
    ok = ok and torch.equal(mine.k_cache, one.k_cache[:, idx]) and torch.equal(mine.v_cache, one.v_cache[:, idx])
    ok = ok and mine.seq_pos.cpu().tolist() == [depths[i] + 1 for i in idx] and mine.workspace.read_status() == 0
    if rank == 0:
        layer, final = n_layers - 1, [x + 1 for x in depths]
        kb, vb = one.k_cache[layer:layer + 1].cpu(), one.v_cache[layer:layer + 1].cpu()
        for b, L in enumerate(final):
            kb[:, b, :, L:] = 0
            vb[:, b, :, L:] = 0
        ref = oracle.decode_step_reference(q[layer:layer + 1].cpu(), kb, vb, ks[layer:layer + 1].cpu(), ks[layer:layer + 1].cpu(), final, cap)
        mo = oracle.error_metrics(got[layer:layer + 1].cpu(), ref)
        ok = ok and mo["max_abs"] <= 2e-2 and mo["cosine"] >= 0.9999
    _finish(dist, ret, rank, bool(ok))


def _world():
    n = torch.cuda.device_count()
    return 8 if n >= 8 else 4 if n >= 4 else 2 if n >= 2 else 0


def _run(worker, port_base, timeout=300):
    world = _world()
    if world < 2:
        pytest.skip("needs at least 2 GPUs")
    import torch.multiprocessing as mp
    port = port_base + os.getpid() % 300
    with mp.Manager() as mgr:
        ret = mgr.dict()
        procs = [mp.get_context("spawn").Process(target=worker, args=(r, world, port, ret)) for r in range(world)]
        for p in procs:
            p.start()
        for p in procs:
            p.join(timeout=timeout)
        alive = [p for p in procs if p.is_alive()]
        for p in alive:
            p.kill()
        assert not alive, "a rank did not finish"
        assert dict(ret) == {r: [] for r in range(world)}


def test_fused_all_gather_matches_single_gpu():
    _run(_small_worker, 29600)


def test_tensor_parallel_steps_with_split_pairs_and_double_buffer():
    _run(_big_worker, 30000)


def test_sequence_sharded_batched_step_matches_single_gpu():
    _run(_sequence_worker, 30400)
