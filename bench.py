#!/usr/bin/env python3
"""Benchmark of the FP8-KV decode-attention step (64 layers) on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload cfg2] [--impl ours|reference]

A "step" is one decode step of the attention path for all 64 layers: quantize-and-append of the
new token's K/V plus split-K GQA attention over the FP8 cache, replayed as one CUDA graph.
Headline workload (cfg2): depth 8192, capacity 8192, bs=1, H_q=40, H_kv=8, D=128; the cache is
full, so every step re-quantises the newest token into the last slot and attends 8192 tokens.
Other depths of the metric (512, 32768) are measured in the same run and reported under
"per_depth".  With N > 1 ranks the KV heads are sharded (tensor parallel, strong scaling) and
every step ends with an all-gather of the per-head outputs over NVLink.

Synthetic data: seeded N(0,1) bf16 K/V quantised to e4m3 with per-(layer, kv head) absmax/448
scales by the library's own calibration + bulk-append kernels (the reference's fixed-depth
prompts are token ids for a checkpoint that is not available).

`--impl reference` times the CPU restatement of the reference's padded torch attention
(oracle/ref_attention.py) on the host cores instead; it is the baseline arm, not the product.
"""
from __future__ import annotations

import argparse
import importlib
import json
import os
import statistics
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

N_LAYERS, H_Q, H_KV, D = 64, 40, 8, 128
METRIC = "decode-attn us/step (64 layers)"
WORKLOADS = {
    # name: (depth, capacity, advance)
    "cfg1": (512, 1024, True),
    "cfg2": (8192, 8192, False),
    "cfg3": (32768, 32768 + 256, True),
}
PEAK_FALLBACK_GBS = 6650.0
REF_SAMPLE_LAYERS = 4


def kv_bytes_per_step(depth: int, h_kv: int | None = None) -> int:
    """Algorithmic bytes of one step: K and V e4m3 bytes of every attended token, all layers."""
    return N_LAYERS * (H_KV if h_kv is None else h_kv) * depth * D * 2


def load_peak() -> tuple[float, str]:
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            return float(json.loads(p.read_text())["hbm_gbs"]), "measured"
        except Exception:  # noqa: BLE001
            pass
    return PEAK_FALLBACK_GBS, "fallback"


DTYPES = {"umma2": "fp8-e4m3 KV fed to tcgen05 as stored; query as two e4m3 terms (exact), probabilities as three e5m2 terms; "
                    "fp32 accumulate/softmax, bf16 in/out",
          "mma": "fp8-e4m3 KV, f16 tensor-core products, fp32 accumulate/softmax, bf16 in/out",
          "simt": "fp8-e4m3 KV, fp32 CUDA-core products, fp32 accumulate/softmax, bf16 in/out"}


def kernel_name(variant: str, per_token: bool = False) -> str:
    """Name of the dominant kernel as a profiler lists it, for the head shape of this run."""
    group = H_Q // H_KV
    return {"simt": f"attn_splitk_simt_kernel<{D},{group}>", "mma": f"attn_streamk_mma_kernel<{D}>",
            "umma2": f"attn_streamk_umma2_kernel<{D}, {'true' if per_token else 'false'}, {5 if group <= 5 else 8}>"}[variant]


def load_traffic(workload: str, variant: str):
    """DRAM bytes per launch of the dominant kernel from the committed ncu summary, if any
    (keyed by workload, then by kernel variant)."""
    p = ROOT / "profiles" / "dram_traffic.json"
    if p.exists():
        try:
            entry = json.loads(p.read_text()).get(workload)
            return entry.get(variant) if isinstance(entry, dict) else entry
        except Exception:  # noqa: BLE001
            return None
    return None


class ClockSampler:
    """SM clock and throttle reasons read through NVML (read-only) every few ms by a thread
    while the timed region runs."""

    REASONS = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap",
               0x80: "hw_power_brake_slowdown"}

    def __init__(self, torch, index: int, period_s: float = 0.004):
        self.samples, self.bits, self.max_mhz, self.period = [], 0, None, period_s
        self.stop_flag = threading.Event()
        self.handle = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            uuid = str(torch.cuda.get_device_properties(index).uuid)
            self.handle = pynvml.nvmlDeviceGetHandleByUUID(("GPU-" + uuid).encode() if not uuid.startswith("GPU-") else uuid.encode())
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(self.handle, pynvml.NVML_CLOCK_SM))
        except Exception:  # noqa: BLE001 - NVML missing: clocks are reported as unknown
            self.handle = None

    def _loop(self):
        nv = self.nv
        while not self.stop_flag.is_set():
            try:
                self.samples.append(float(nv.nvmlDeviceGetClockInfo(self.handle, nv.NVML_CLOCK_SM)))
                self.bits |= int(nv.nvmlDeviceGetCurrentClocksEventReasons(self.handle))
            except Exception:  # noqa: BLE001
                pass
            time.sleep(self.period)

    def __enter__(self):
        if self.handle is not None:
            self.thread = threading.Thread(target=self._loop, daemon=True)
            self.thread.start()
        return self

    def __exit__(self, *exc):
        self.stop_flag.set()
        if self.handle is not None:
            self.thread.join(timeout=1)

    def summary(self) -> dict:
        reasons = sorted(name for bit, name in self.REASONS.items() if self.bits & bit)
        return {"sm_mhz": statistics.median(self.samples) if self.samples else None, "sm_max_mhz": self.max_mhz,
                "reasons": reasons, "samples": len(self.samples)}


# ------------------------------------------------------------------------------------------
# reference arm: the oracle port on the host cores
# ------------------------------------------------------------------------------------------
def run_reference(args) -> int:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    import torch
    from oracle import ref_attention as oracle
    depth, cap, _ = WORKLOADS[args.workload]
    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    q, k, v = oracle.make_inputs(0, H_Q, H_KV, D, depth)
    sk, sv = oracle.head_scales(k), oracle.head_scales(v)
    kb, vb = oracle.quantize_per_head(k, sk), oracle.quantize_per_head(v, sv)
    cap = max(cap, depth)

    def sample_step():
        for _ in range(REF_SAMPLE_LAYERS):
            oracle.padded_fp8_reference(q, kb, vb, sk, sv, cap)

    for _ in range(args.warmup):
        sample_step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        sample_step()
    dt = (time.perf_counter() - t0) / args.steps
    us_per_step = dt * 1e6 * (N_LAYERS / REF_SAMPLE_LAYERS)
    sample = (f"each timed step = {REF_SAMPLE_LAYERS} of {N_LAYERS} layers of dequant+pad+padded torch attention "
              f"at depth {depth}, scaled x{N_LAYERS // REF_SAMPLE_LAYERS}")
    line = {
        "impl": "reference", "metric": METRIC, "value": us_per_step, "unit": "us/step", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": us_per_step / 1e3, "higher_is_better": False,
        "scaling": "strong", "vs_baseline": None, "dtype": "bf16 (torch CPU, fp32 softmax)", "data": "synthetic",
        "config": {"workload": workload_name(args.workload, depth, cap), "timing": "host wall clock"},
        "cpu_baseline": {"value": us_per_step, "unit": "us/step", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": us_per_step, "unit": "us/step", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)
    return 0


SCALES_TEXT = "per-(layer,kv-head)"


def workload_name(key: str, depth: int, cap: int) -> str:
    return (f"{key}: {N_LAYERS}-layer bs=1 decode attention, depth {depth}, capacity {cap}, H_q={H_Q} H_kv={H_KV} "
            f"D={D}, FP8-e4m3 KV with {SCALES_TEXT} scales, append+attend per step")


# ------------------------------------------------------------------------------------------
# our arm
# ------------------------------------------------------------------------------------------
class StepRunner:
    """One workload resident on one GPU: cache, static step buffers, captured graph."""

    def __init__(self, pkg, torch, device, depth, cap, advance, h_q, h_kv, seed, dist=None, world=1, variant="auto",
                 num_splits=0, gather="peer", scale_mode="per_head"):
        self.pkg, self.torch, self.device, self.depth, self.advance = pkg, torch, device, depth, advance
        self.h_q, self.h_kv, self.dist, self.world = h_q, h_kv, dist, world
        g = torch.Generator(device=device).manual_seed(seed)
        self.cache = pkg.FP8StaticCache(N_LAYERS, 1, h_q, h_kv, D, cap, device=device, variant=variant,
                                        num_splits=num_splits, scale_mode=scale_mode)
        prefix = depth if advance else depth - 1      # cfg2: slot depth-1 is rewritten by every step
        chunk = 8192
        scales_done = False
        for t0 in range(0, prefix, chunk):
            n = min(chunk, prefix - t0)
            k = torch.randn(N_LAYERS, 1, h_kv, n, D, generator=g, device=device, dtype=torch.bfloat16)
            v = torch.randn(N_LAYERS, 1, h_kv, n, D, generator=g, device=device, dtype=torch.bfloat16)
            self.cache.prefill(k, v, calibrate=not scales_done and scale_mode == "per_head")
            scales_done = True
        self.start_pos = prefix
        self.q = torch.randn(N_LAYERS, 1, h_q, D, generator=g, device=device, dtype=torch.bfloat16)
        self.k_new = torch.randn(N_LAYERS, 1, h_kv, D, generator=g, device=device, dtype=torch.bfloat16)
        self.v_new = torch.randn(N_LAYERS, 1, h_kv, D, generator=g, device=device, dtype=torch.bfloat16)
        self.out = torch.empty_like(self.q)
        distmod = importlib.import_module("qwen38-5080_b200.dist")
        self.peer = None
        self.gatherer = None
        if world > 1 and gather == "peer":
            self.peer = distmod.PeerOutput(self.out, world, dist.get_rank())
            self.full_out = self.peer.full
        elif world > 1:
            self.gatherer = distmod.HeadGather(self.out, world)
            self.full_out = self.gatherer.full
        else:
            self.full_out = None
        self.graph = None

    def launch_step(self):
        c = self.cache
        if self.peer is not None:
            # append + attention storing into every rank's gathered buffer (+ position bump), then the cross-GPU barrier
            self.pkg.append_decode(self.q, self.k_new, self.v_new, c.k_cache, c.v_cache, c.k_scale, c.v_scale, c.seq_pos,
                                   workspace=c.workspace, advance=self.advance, peer_out=self.peer, barrier=True)
            return
        self.pkg.append_decode(self.q, self.k_new, self.v_new, c.k_cache, c.v_cache, c.k_scale, c.v_scale, c.seq_pos,
                               workspace=c.workspace, advance=self.advance, out=self.out)

    def gather(self):
        if self.gatherer is not None:
            self.gatherer.gather(self.out)     # NCCL all-gather + one strided copy into [n, b, h_q, D]

    def capture(self):
        torch = self.torch
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(3):
                self.launch_step()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        self.reset_pos()
        self.gather_in_graph = False
        if self.gatherer is not None:          # the all-gather belongs to the step: capture it with the kernels
            with torch.cuda.stream(side):
                self.gather()
            torch.cuda.current_stream().wait_stream(side)
            torch.cuda.synchronize()
            try:
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph):
                    self.launch_step()
                    self.gather()
                self.graph, self.gather_in_graph = graph, True
            except Exception as exc:  # noqa: BLE001 - NCCL capture unsupported here: gather after the replay instead
                print(f"[bench] all-gather not captured ({type(exc).__name__}); issuing it after the replay", file=sys.stderr)
                torch.cuda.synchronize()
                self.reset_pos()
        if self.graph is None:
            self.graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(self.graph):
                self.launch_step()
        torch.cuda.synchronize()
        self.reset_pos()

    def reset_pos(self):
        self.cache.seq_pos.fill_(self.start_pos)

    def step(self):
        self.graph.replay()
        if not self.gather_in_graph:
            self.gather()

    def kernels_per_step(self) -> int:
        fused = self.cache.workspace.resolved in ("umma2", "mma") and not self.cache.per_token
        if self.peer is not None:                # (append, bump,) attention with fused gather, barrier
            return (1 if self.cache.workspace.resolved == "umma2" else 2) if fused else (3 if self.advance else 2) + 1
        if fused:
            return 1                         # the fused step: append, attention, combine and position bump in one launch
        n = 3 if self.advance else 2         # append, attention (+ fused combine), position bump
        return n + (1 if self.cache.workspace.variant == "simt" and self.cache.workspace.num_splits > 1 else 0)


def barrier(dist, world):
    if world > 1:
        dist.barrier()


def timed_steps(torch, dist, world, runner, steps, warmup, sampler=None) -> float:
    """Seconds per step on the device: W warm-up steps, then K steps between CUDA events,
    barrier + synchronize on both sides, max over ranks."""
    runner.reset_pos()
    for _ in range(warmup):
        runner.step()
    torch.cuda.synchronize()
    barrier(dist, world)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        runner.step()
    e1.record()
    torch.cuda.synchronize()
    barrier(dist, world)
    sec = e0.elapsed_time(e1) / 1e3 / steps
    if world > 1:
        t = torch.tensor([sec], device=runner.device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        sec = float(t.item())
    return sec


def timed_kernel(torch, runner, steps, warmup) -> float:
    """Average duration of the attention kernel alone: the launch is captured in its own CUDA graph
    (so the host cannot be the limit) and replayed back to back between CUDA events."""
    c = runner.cache
    off = 0 if runner.advance else 1

    def launch():
        runner.pkg.decode_attention(runner.q, c.k_cache, c.v_cache, c.k_scale, c.v_scale, c.seq_pos,
                                    workspace=c.workspace, seq_len_offset=off, out=runner.out)
    runner.reset_pos()
    if runner.advance:
        c.seq_pos.fill_(runner.depth)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        launch()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    per_graph = 4                     # launches per replay: keeps graph-launch gaps out of the per-kernel figure
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for _ in range(per_graph):
            launch()
    for _ in range(max(1, warmup // per_graph)):
        graph.replay()
    torch.cuda.synchronize()
    replays = max(1, (steps + per_graph - 1) // per_graph)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(replays):
        graph.replay()
    e1.record()
    torch.cuda.synchronize()
    runner.reset_pos()
    return e0.elapsed_time(e1) / 1e3 / (replays * per_graph)


def timed_e2e(torch, dist, world, runner, steps, warmup) -> tuple[float, int, int]:
    """Through the public API with HOST buffers: per step, pinned-host q/k/v -> device, the decode
    step, device -> pinned-host output, and a synchronize (the caller needs the result).  The
    copies and the step are captured into one CUDA graph (memcpy nodes + the library's launches),
    as a host that replays its decode step would do; if that capture is refused the same sequence
    is issued call by call."""
    hq, hk, hv = (t.cpu().pin_memory() for t in (runner.q, runner.k_new, runner.v_new))
    src = runner.full_out if world > 1 else runner.out
    hout = torch.empty(src.shape, dtype=src.dtype).pin_memory()
    h2d = sum(t.numel() * t.element_size() for t in (hq, hk, hv))
    d2h = hout.numel() * hout.element_size()

    def sequence():
        runner.q.copy_(hq, non_blocking=True)
        runner.k_new.copy_(hk, non_blocking=True)
        runner.v_new.copy_(hv, non_blocking=True)
        runner.launch_step()
        if runner.gatherer is not None:
            runner.gather()
        hout.copy_(src, non_blocking=True)

    graph = None
    try:
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            sequence()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            sequence()
    except Exception as exc:  # noqa: BLE001 - e.g. NCCL capture unsupported: issue the calls one by one
        print(f"[bench] e2e sequence not captured ({type(exc).__name__}); issuing it call by call", file=sys.stderr)
        graph = None
        torch.cuda.synchronize()

    def one():
        if graph is not None:
            graph.replay()
        else:
            sequence()
        torch.cuda.synchronize()

    runner.reset_pos()
    for _ in range(warmup):
        one()
    barrier(dist, world)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        one()
    e1.record()
    torch.cuda.synchronize()
    wall = (time.perf_counter() - t0) / steps
    barrier(dist, world)
    runner.reset_pos()
    sec = max(e0.elapsed_time(e1) / 1e3 / steps, wall)
    if world > 1:
        t = torch.tensor([sec], device=runner.device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        sec = float(t.item())
    return sec, h2d, d2h


def cpu_baseline(depth: int, cap: int) -> dict:
    from oracle import ref_attention as oracle
    threads = os.cpu_count() or 1
    layers, repeats = 4, 2
    r = oracle.cpu_attention_seconds(H_Q, H_KV, D, depth, max(cap, depth), layers, repeats, threads)
    return {"value": r["full_s_per_layer"] * N_LAYERS * 1e6, "unit": "us/step", "cores": threads, "kind": "port",
            "attn_only_us_per_step": r["attn_s_per_layer"] * N_LAYERS * 1e6,
            "sample": f"median of {r['samples']} single-layer runs (dequant + pad + padded torch attention) at depth "
                      f"{depth}, capacity {max(cap, depth)}, scaled x{N_LAYERS} layers"}


def run_ours(args) -> int:
    import torch
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit(f"--gpus {args.gpus} needs torchrun with {args.gpus} ranks")
    dist = None
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product has no CPU path")
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if world > 1:
        import torch.distributed as dist
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=device)
    pkg = importlib.import_module("qwen38-5080_b200")
    if H_KV % world:
        raise SystemExit("KV-head sharding needs a GPU count that divides 8")
    h_kv, h_q = H_KV // world, H_Q // world

    per_depth, runners = {}, {}
    order = [args.workload] + [w for w in WORKLOADS if w != args.workload and not args.only]
    headline = None
    for key in order:
        depth, cap, advance = WORKLOADS[key]
        room = cap - depth - args.warmup - 4 if advance else 1 << 30   # the cache must not overflow
        steps = max(1, min(args.steps, room))
        runner = StepRunner(pkg, torch, device, depth, cap, advance, h_q, h_kv, seed=rank, dist=dist, world=world,
                            variant=args.variant, num_splits=args.ctas, gather=args.gather, scale_mode=args.scales)
        runner.capture()
        if world > 1:   # every rank in step before the first timed (or barrier-carrying) launch
            torch.cuda.synchronize()
            dist.barrier()
        with ClockSampler(torch, local) as sampler:
            sec = timed_steps(torch, dist, world, runner, steps, args.warmup)
            ksec = timed_kernel(torch, runner, steps, args.warmup)
        status = runner.cache.workspace.read_status()
        if status:
            raise SystemExit(f"device status {status} after {key}")
        total_bytes = kv_bytes_per_step(depth)                 # whole job (all ranks)
        entry = {"us_per_step": sec * 1e6, "us_per_layer": sec * 1e6 / N_LAYERS,
                 "hbm_gbs_whole_job": total_bytes / sec / 1e9, "hbm_gbs_per_gpu": total_bytes / world / sec / 1e9,
                 "frac_of_8TBs_per_gpu": total_bytes / world / sec / 8e12,
                 "attn_kernel_us": ksec * 1e6, "attn_kernel_gbs_per_gpu": total_bytes / world / ksec / 1e9,
                 "steps": steps}
        per_depth[str(depth)] = entry
        if key == args.workload:
            headline = (key, runner, sec, ksec, sampler.summary(), steps)
            e2e_sec, h2d, d2h = timed_e2e(torch, dist, world, runner, steps, args.warmup)
        else:
            del runner
            torch.cuda.empty_cache()

    key, runner, sec, ksec, clocks, steps = headline
    depth, cap, advance = WORKLOADS[key]
    peak, peak_kind = load_peak()
    bytes_per_launch = kv_bytes_per_step(depth, h_kv)           # one GPU's launch
    achieved = bytes_per_launch / ksec / 1e9
    line = {
        "metric": METRIC, "value": sec * 1e6, "unit": "us/step", "n_gpus": world, "steps": steps,
        "warmup": args.warmup, "ms_per_step": sec * 1e3, "higher_is_better": False, "scaling": "strong",
        "vs_baseline": None, "dtype": DTYPES[runner.cache.workspace.resolved],
        "data": "synthetic",
        "config": {"workload": workload_name(key, depth, cap), "sharding": f"kv-head tensor parallel x{world}",
                   "l2": f"inputs larger than L2 ({kv_bytes_per_step(depth, h_kv) / 1e6:.0f} MB KV per GPU per step)"
                         if bytes_per_launch > 200e6 else "KV working set smaller than L2: L2-warm figure",
                   "execution": "CUDA graph replay of " + ("the fused append + attention launch" if runner.kernels_per_step() == 1 else "append + attention")
                                + ((" with the output all-gather fused into the attention kernel (peer stores over NVLink into "
                                     "every rank's gathered buffer) + a cross-GPU barrier kernel, all in the graph"
                                     if runner.peer is not None else
                                     " + NCCL all-gather + head reorder copy, captured in the graph" if runner.gather_in_graph
                                     else " then NCCL all-gather + head reorder copy after the replay") if world > 1 else "")},
        "hbm_gbs": kv_bytes_per_step(depth) / sec / 1e9,
        "frac_of_8TBs": kv_bytes_per_step(depth) / world / sec / 8e12,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "traffic": load_traffic(key, runner.cache.workspace.resolved), "kernel": kernel_name(runner.cache.workspace.resolved, runner.cache.per_token), "peak_kind": peak_kind,
                     "algorithmic_bytes_per_launch": bytes_per_launch, "launch_us": ksec * 1e6},
        "e2e": {"value": e2e_sec * 1e6, "unit": "us/step", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
        "gpu_launches": runner.kernels_per_step() * steps,
        "clocks": clocks,
        "per_depth": per_depth,
    }
    if world == 1 and rank == 0 and not args.no_cpu:
        line["cpu_baseline"] = cpu_baseline(depth, cap)
    if rank == 0:
        print(json.dumps(line), flush=True)
    finish(torch, dist, world)
    return 0


def finish(torch, dist, world) -> None:
    """Leave a multi-rank run: all ranks idle and in step, then exit without tearing the NCCL
    communicator down (graphs that captured its collectives are still alive; destroying the
    process group under them has been seen to block forever)."""
    if world > 1:
        torch.cuda.synchronize()
        dist.barrier()
        torch.cuda.synchronize()
        sys.stdout.flush()
        sys.stderr.flush()
        os._exit(0)


def run_cfg4(args) -> int:
    """Batched decode (BASELINE config 4): bs=16 ragged depths U[1024, 16384] (seed 0), sharded by
    sequence over the ranks with no data-path collective; a step = fused one-token K/V
    quantize-append per sequence + attention, replayed as a CUDA graph."""
    import torch
    world = int(os.environ.get("WORLD_SIZE", "1")); rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    dist = None
    if world > 1:
        import torch.distributed as dist
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=device)
    pkg = importlib.import_module("qwen38-5080_b200")
    g0 = torch.Generator().manual_seed(0)
    depths_all = torch.randint(1024, 16384 + 1, (16,), generator=g0).tolist()
    plan = pkg.dist.assign_sequences(depths_all, world)
    depths = [depths_all[i] for i in plan[rank]]
    batch, cap = len(depths), 16384 + 256
    room = 256 - args.warmup - 8
    steps = max(1, min(args.steps, room))
    g = torch.Generator(device=device).manual_seed(rank)
    cache = pkg.FP8StaticCache(N_LAYERS, batch, H_Q, H_KV, D, cap, device=device, variant=args.variant,
                               num_splits=args.ctas)
    done = False
    for t0 in range(0, max(depths), 2048):      # fill every slot up to the longest depth, then set the ragged lengths
        n = min(2048, max(depths) - t0)
        k = torch.randn(N_LAYERS, batch, H_KV, n, D, generator=g, device=device, dtype=torch.bfloat16)
        v = torch.randn(N_LAYERS, batch, H_KV, n, D, generator=g, device=device, dtype=torch.bfloat16)
        cache.prefill(k, v, calibrate=not done)
        done = True
    start = torch.tensor(depths, dtype=torch.int32, device=device)
    q = torch.randn(N_LAYERS, batch, H_Q, D, generator=g, device=device, dtype=torch.bfloat16)
    kn = torch.randn(N_LAYERS, batch, H_KV, D, generator=g, device=device, dtype=torch.bfloat16)
    vn = torch.randn(N_LAYERS, batch, H_KV, D, generator=g, device=device, dtype=torch.bfloat16)
    out = torch.empty_like(q)

    def launch():
        pkg.append_decode(q, kn, vn, cache.k_cache, cache.v_cache, cache.k_scale, cache.v_scale, cache.seq_pos,
                          workspace=cache.workspace, advance=True, out=out)
    cache.seq_pos.copy_(start)
    side = torch.cuda.Stream(); side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(3):
            launch()
    torch.cuda.current_stream().wait_stream(side); torch.cuda.synchronize()
    cache.seq_pos.copy_(start)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        launch()
    torch.cuda.synchronize()
    cache.seq_pos.copy_(start)
    for _ in range(args.warmup):
        graph.replay()
    torch.cuda.synchronize(); barrier(dist, world); torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(torch, local) as sampler:
        e0.record()
        for _ in range(steps):
            graph.replay()
        e1.record()
        torch.cuda.synchronize()
    barrier(dist, world)
    sec = e0.elapsed_time(e1) / 1e3 / steps
    if world > 1:
        t = torch.tensor([sec], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        sec = float(t.item())
    status = cache.workspace.read_status()
    if status:
        raise SystemExit(f"device status {status}")
    mean_len = [d + args.warmup + (steps + 1) / 2 for d in depths_all]      # lengths grow by one per step
    total_bytes = N_LAYERS * H_KV * D * 2 * sum(mean_len)
    line = {"metric": METRIC, "value": sec * 1e6, "unit": "us/step", "n_gpus": world, "steps": steps, "warmup": args.warmup,
            "ms_per_step": sec * 1e3, "higher_is_better": False, "scaling": "strong", "vs_baseline": None,
            "dtype": DTYPES[cache.workspace.resolved], "data": "synthetic",
            "config": {"workload": f"cfg4: {N_LAYERS}-layer batched decode, bs=16, ragged depths U[1024,16384] seed 0 "
                                   f"(sum {sum(depths_all)}), capacity {cap}, fused one-token append per sequence per step",
                       "sharding": f"by sequence x{world} (greedy longest-first on depth), no collective",
                       "execution": "CUDA graph replay of " + ("one fused launch: append + attention + position bump" if cache.workspace.resolved in ("umma2", "mma") else "append + attention + position bump")},
            "hbm_gbs": total_bytes / sec / 1e9, "frac_of_8TBs": total_bytes / world / sec / 8e12,
            "tokens_per_s": 16 / sec, "gpu_launches": (1 if cache.workspace.resolved in ("umma2", "mma") else 3) * steps, "clocks": sampler.summary()}
    if rank == 0:
        print(json.dumps(line), flush=True)
    finish(torch, dist, world)
    return 0


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--workload", choices=sorted(WORKLOADS) + ["cfg4"], default="cfg2")
    ap.add_argument("--only", action="store_true", help="measure only the headline workload")
    ap.add_argument("--variant", choices=["auto", "mma", "umma2", "simt"], default="auto", help="attention kernel variant")
    ap.add_argument("--gather", choices=["peer", "nccl"], default="peer",
                    help="N > 1: fused peer-store all-gather (default) or NCCL all-gather + reorder copy")
    ap.add_argument("--scales", choices=["per_head", "per_token"], default="per_head",
                    help="scale granularity of the FP8 cache (per_token = the reference's frozen [capacity, kv_heads] layout)")
    ap.add_argument("--heads", default="", help="H_q,H_kv,head_dim instead of the metric's 40,8,128 (e.g. 24,4,256: the "
                    "reference model's own attention shape; not the metric)")
    ap.add_argument("--ctas", type=int, default=0, help="override the split / CTA count (0 = library default)")
    ap.add_argument("--layers", type=int, default=64, help="layers per step (64 = the metric; fewer only for profiling)")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    global N_LAYERS, SCALES_TEXT, H_Q, H_KV, D
    N_LAYERS = args.layers
    if args.heads:
        H_Q, H_KV, D = (int(x) for x in args.heads.split(","))
    if args.scales == "per_token":
        SCALES_TEXT = "per-(token,kv-head)"
    if args.workload == "cfg4":
        if args.impl == "reference":
            raise SystemExit("--impl reference times the bs=1 workloads (cfg1..cfg3)")
        return run_cfg4(args)
    if args.impl == "reference":
        return run_reference(args)
    return run_ours(args)


if __name__ == "__main__":
    raise SystemExit(main())
