#!/usr/bin/env python3
"""Benchmark of the FP8-KV decode-attention step (64 layers) on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload cfg2] [--impl ours|reference]

A "step" is one decode step of the attention path for all 64 layers: quantize-and-append of the
new token's K/V plus split-K GQA attention over the FP8 cache: one kernel launch, replayed from CUDA
graphs (five steps to a graph in the timed passes, so that the host's replay rate cannot be the limit
of a 20 us step; single steps where every step is timed by itself).
Headline workload (cfg2): depth 8192, capacity 8192, bs=1, H_q=40, H_kv=8, D=128; the cache is
full, so every step re-quantises the newest token into the last slot and attends 8192 tokens.
The other depths of the metric (512, 32768) are measured in the same run under "per_depth", the
batched ragged workload (bs=16, sharded by sequence) under "per_workload".  With N > 1 ranks the KV
heads of the single-sequence workloads are sharded (tensor parallel, strong scaling) and every
step ends with the all-gather of the per-head outputs over NVLink, fused into the kernel.

Protocol (the reference's: within-run step distribution apart from between-run spread,
runner/report.py:228-258): 10 ms or more of the workload's own steps so that the clocks are up (a pass of the
short-cache workload lasts one millisecond), then W warm-up steps, then K steps between two CUDA events —
that pass is
`value` — then four more such passes (median / min / max over the five) and one pass with an event
pair around every step (p50 / p95).  After the clock has stopped, two layers of the step's result
are compared with the CPU oracle and reported as "parity".

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
STEPS_PER_GRAPH = 5
WORKLOADS = {
    # name: (depth, capacity, advance)
    "cfg1": (512, 1024, True),
    "cfg2": (8192, 8192, False),
    "cfg3": (32768, 32768 + 256, True),
}
CFG4_BATCH, CFG4_LO, CFG4_HI, CFG4_CAP = 16, 1024, 16384, 16384 + 256
PEAK_FALLBACK_GBS = 6650.0
REF_SAMPLE_LAYERS = 4
PASSES = 5
L2_FREE_COPIES = 6
PARITY_TOL = {"max_abs": 2e-2, "cosine": 0.9999}


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


def kernel_name(variant: str, per_token: bool = False, ctas: int = 0, sms: int = 148) -> str:
    """Name of the dominant kernel as a profiler lists it, for the head shape of this run (the mma.sync kernel has an
    instance for grids of up to two CTAs per SM and one for three)."""
    group = H_Q // H_KV
    inst = "*" if D != 128 or ctas <= 0 else ("2" if ctas <= 2 * sms else "3")
    return {"simt": f"attn_splitk_simt_kernel<{D},{group}>", "mma": f"attn_streamk_mma_kernel<{D}, {inst}>",
            "umma2": f"attn_streamk_umma2_kernel<{D}, {'true' if per_token else 'false'}, {5 if group <= 5 else 8}>"}[variant]


def load_traffic(workload: str, variant: str):
    """DRAM bytes per launch of the dominant kernel on ONE GPU holding all KV heads, from the committed
    ncu summary, if any (keyed by workload, then by kernel variant)."""
    p = ROOT / "profiles" / "dram_traffic.json"
    if p.exists():
        try:
            entry = json.loads(p.read_text()).get(workload)
            return entry.get(variant) if isinstance(entry, dict) else entry
        except Exception:  # noqa: BLE001
            return None
    return None


SCALES_TEXT = "per-(layer,kv-head)"


def workload_name(key: str) -> str:
    if key == "cfg4":
        return (f"cfg4: {N_LAYERS}-layer batched decode, bs={CFG4_BATCH}, ragged depths U[{CFG4_LO},{CFG4_HI}] seed 0, "
                f"capacity {CFG4_CAP}, H_q={H_Q} H_kv={H_KV} D={D}, FP8-e4m3 KV with {SCALES_TEXT} scales, fused one-token "
                f"append per sequence per step")
    depth, cap, _ = WORKLOADS[key]
    return (f"{key}: {N_LAYERS}-layer bs=1 decode attention, depth {depth}, capacity {cap}, H_q={H_Q} H_kv={H_KV} "
            f"D={D}, FP8-e4m3 KV with {SCALES_TEXT} scales, append+attend per step")


def make_config(key: str, world: int) -> dict:
    """The `config` object of the JSON line: the same for this arm and for the reference arm."""
    if key == "cfg4":
        sharding = f"by sequence x{world} (greedy longest-first on depth), no collective"
        per_gpu = N_LAYERS * H_KV * D * 2 * CFG4_BATCH * (CFG4_LO + CFG4_HI) // 2 // world
    else:
        sharding = f"kv-head tensor parallel x{world}"
        per_gpu = kv_bytes_per_step(WORKLOADS[key][0]) // world
    l2 = (f"inputs larger than L2 (about {per_gpu / 1e6:.0f} MB of KV per GPU per step)" if per_gpu > 200e6 else
          f"KV working set ({per_gpu / 1e6:.0f} MB per GPU) smaller than L2: L2-warm figure; an L2-free figure that rotates "
          f"{L2_FREE_COPIES} cache copies is reported beside it where measured")
    return {"workload": workload_name(key), "sharding": sharding, "l2": l2,
            "execution": f"CUDA-graph replays of {STEPS_PER_GRAPH} steps, one launch per step: quantize-append + split-K attention + combine"
                         + (" + output all-gather over NVLink, in the same launch" if world > 1 and key != "cfg4" else "")}


class ClockSampler:
    """SM clock and throttle reasons read through NVML (read-only) every few ms by a thread
    while the timed region runs."""

    REASONS = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap",
               0x80: "hw_power_brake_slowdown"}

    def __init__(self, torch, index: int, period_s: float = 0.002):
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
            t0 = time.time()     # NVML's first queries are slow: they are over before anything is timed
            while len(self.samples) < 2 and time.time() - t0 < 1.0:
                time.sleep(0.005)
        return self

    def __exit__(self, *exc):
        self.stop_flag.set()
        if self.handle is not None:
            self.thread.join(timeout=1)

    def summary(self) -> dict:
        reasons = sorted(name for bit, name in self.REASONS.items() if self.bits & bit)
        return {"sm_mhz": statistics.median(self.samples) if self.samples else None, "sm_max_mhz": self.max_mhz,
                "reasons": reasons, "samples": len(self.samples)}


def percentile(values, q: float) -> float:
    s = sorted(values)
    if not s:
        return float("nan")
    k = (len(s) - 1) * q
    lo, hi = int(k), min(int(k) + 1, len(s) - 1)
    return s[lo] + (s[hi] - s[lo]) * (k - lo)


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
    cap = max(cap, depth)
    layers = []
    for layer in range(REF_SAMPLE_LAYERS):             # every sampled layer has its own q / K / V
        q, k, v = oracle.make_inputs(layer, H_Q, H_KV, D, depth)
        sk, sv = oracle.head_scales(k), oracle.head_scales(v)
        layers.append((q, oracle.quantize_per_head(k, sk), oracle.quantize_per_head(v, sv), sk, sv))

    def sample_step():
        for q, kb, vb, sk, sv in layers:
            oracle.padded_fp8_reference(q, kb, vb, sk, sv, cap)

    for _ in range(args.warmup):
        sample_step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        sample_step()
    dt = (time.perf_counter() - t0) / args.steps
    us_per_step = dt * 1e6 * (N_LAYERS / REF_SAMPLE_LAYERS)
    sample = (f"each timed step = {REF_SAMPLE_LAYERS} of {N_LAYERS} layers (own K/V each) of dequant+pad+padded torch attention "
              f"at depth {depth}, scaled x{N_LAYERS // REF_SAMPLE_LAYERS}; host wall clock")
    line = {
        "impl": "reference", "metric": METRIC, "value": us_per_step, "unit": "us/step", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": us_per_step / 1e3, "higher_is_better": False,
        "scaling": "strong", "vs_baseline": None, "dtype": "bf16 (torch CPU, fp32 softmax)", "data": "synthetic",
        "config": make_config(args.workload, args.gpus),
        "cpu_baseline": {"value": us_per_step, "unit": "us/step", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": us_per_step, "unit": "us/step", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)
    return 0


# ------------------------------------------------------------------------------------------
# our arm
# ------------------------------------------------------------------------------------------
class StepRunner:
    """One workload resident on one GPU: cache, static step buffers, captured graph.

    Single-sequence workloads: `depths` is one depth, the KV heads are this rank's share and, with more
    than one rank, the results go into every rank's gathered buffers.  Batched workload: `depths` are this
    rank's sequences, all heads, no exchange."""

    def __init__(self, pkg, torch, device, depths, cap, advance, h_q, h_kv, seed, dist=None, world=1, variant="auto",
                 num_splits=0, gather="packets", scale_mode="per_head", tensor_parallel=True):
        self.pkg, self.torch, self.device, self.depths, self.advance = pkg, torch, device, list(depths), advance
        self.h_q, self.h_kv, self.dist, self.world, self.cap = h_q, h_kv, dist, world, cap
        batch = len(self.depths)
        g = torch.Generator(device=device).manual_seed(seed)
        self.cache = pkg.FP8StaticCache(N_LAYERS, batch, h_q, h_kv, D, cap, device=device, variant=variant,
                                        num_splits=num_splits, scale_mode=scale_mode)
        longest = max(self.depths)
        prefix = longest if advance else longest - 1      # cfg2: slot depth-1 is rewritten by every step
        chunk = 8192 if batch == 1 else 2048
        scales_done = False
        for t0 in range(0, prefix, chunk):                # every slot up to the longest depth; ragged lengths are set below
            n = min(chunk, prefix - t0)
            k = torch.randn(N_LAYERS, batch, h_kv, n, D, generator=g, device=device, dtype=torch.bfloat16)
            v = torch.randn(N_LAYERS, batch, h_kv, n, D, generator=g, device=device, dtype=torch.bfloat16)
            self.cache.prefill(k, v, calibrate=not scales_done and scale_mode == "per_head")
            scales_done = True
        self.start_pos = torch.tensor([d if advance else d - 1 for d in self.depths], dtype=torch.int32, device=device)
        # the step's inputs share one device buffer, so that a host that owns them can send them with one copy
        nq, nk = N_LAYERS * batch * h_q * D, N_LAYERS * batch * h_kv * D
        self.inputs = torch.randn(nq + 2 * nk, generator=g, device=device, dtype=torch.bfloat16)
        self.q = self.inputs[:nq].view(N_LAYERS, batch, h_q, D)
        self.k_new = self.inputs[nq:nq + nk].view(N_LAYERS, batch, h_kv, D)
        self.v_new = self.inputs[nq + nk:].view(N_LAYERS, batch, h_kv, D)
        self.out = torch.empty_like(self.q)
        distmod = importlib.import_module("qwen38-5080_b200.dist")
        self.peer = None
        self.gatherer = None
        if world > 1 and tensor_parallel and gather in ("packets", "stores"):
            self.peer = distmod.PeerOutput(self.out, world, dist.get_rank(), mode=gather)
        elif world > 1 and tensor_parallel:
            self.gatherer = distmod.HeadGather(self.out, world)
        self.graph = None
        self.graph_multi = None
        self.gather_in_graph = False

    def launch_step(self):
        c = self.cache
        if self.peer is not None:
            # one launch: append + attention sending its results to every rank's gathered tensor + position bump
            # (+ cross-GPU barrier in the stores mode; the packet mode needs none)
            self.pkg.append_decode(self.q, self.k_new, self.v_new, c.k_cache, c.v_cache, c.k_scale, c.v_scale, c.seq_pos,
                                   workspace=c.workspace, advance=self.advance, peer_out=self.peer, barrier=True)
            return
        self.pkg.append_decode(self.q, self.k_new, self.v_new, c.k_cache, c.v_cache, c.k_scale, c.v_scale, c.seq_pos,
                               workspace=c.workspace, advance=self.advance, out=self.out)

    def gather(self):
        if self.gatherer is not None:
            self.gatherer.gather(self.out)     # NCCL all-gather + one strided copy into [n, b, h_q, D]

    def result(self):
        """The step's result as a consumer on this rank sees it (all heads)."""
        if self.peer is not None:
            return self.peer.current()
        return self.gatherer.full if self.gatherer is not None else self.out

    def capture(self):
        torch = self.torch
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(4):
                self.launch_step()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        self.reset_pos()
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
        # The same step STEPS_PER_GRAPH times in one graph, for the timed passes: a 20 us step replayed one by one
        # from Python is at the edge of what the host can issue (the pass then times the host, 22.5 us a step on the
        # slower hosts of the pool), and a caller with steps that short would not replay them one by one either.
        if self.gatherer is None or self.gather_in_graph:
            self.graph_multi = torch.cuda.CUDAGraph()
            with torch.cuda.graph(self.graph_multi):
                for _ in range(STEPS_PER_GRAPH):
                    self.launch_step()
                    if self.gatherer is not None:
                        self.gather()
            torch.cuda.synchronize()
            self.reset_pos()

    def run(self, n: int):
        """n steps: graphs of STEPS_PER_GRAPH steps, the remainder one by one."""
        if self.graph_multi is not None:
            while n >= STEPS_PER_GRAPH:
                self.graph_multi.replay()
                n -= STEPS_PER_GRAPH
        for _ in range(n):
            self.step()

    def reset_pos(self):
        self.cache.seq_pos.copy_(self.start_pos)

    def step(self):
        self.graph.replay()
        if self.gatherer is not None and not self.gather_in_graph:
            self.gather()

    def kernels_per_step(self) -> int:
        fused = self.cache.workspace.resolved == "umma2" or (self.cache.workspace.resolved == "mma" and not self.cache.per_token)
        if fused:
            return 1                         # the fused step: append, attention, combine, position bump (and barrier) in one launch
        n = 3 if self.advance else 2         # append, attention (+ fused combine), position bump
        n += 1 if self.cache.workspace.resolved == "simt" and self.cache.workspace.num_splits > 1 else 0
        return n + (1 if self.peer is not None and self.peer.needs_barrier else 0)


def barrier(dist, world):
    if world > 1:
        dist.barrier()


def max_over_ranks(torch, dist, world, device, value: float) -> float:
    if world == 1:
        return value
    t = torch.tensor([value], device=device, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def timed_pass(torch, dist, world, runner, steps, warmup, per_step=False):
    """One pass: W warm-up steps, then K steps between CUDA events (barrier + synchronize on both sides).
    Returns seconds per step (max over ranks); with per_step=True an event pair brackets every step
    instead and the list of this rank's step times (seconds) is returned too."""
    runner.reset_pos()
    runner.run(warmup)
    torch.cuda.synchronize()
    barrier(dist, world)
    torch.cuda.synchronize()
    if per_step:
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(steps + 1)]
        ev[0].record()
        for i in range(steps):
            runner.step()
            ev[i + 1].record()
        torch.cuda.synchronize()
        barrier(dist, world)
        each = [ev[i].elapsed_time(ev[i + 1]) / 1e3 for i in range(steps)]
        return max_over_ranks(torch, dist, world, runner.device, sum(each) / steps), each
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    runner.run(steps)
    e1.record()
    torch.cuda.synchronize()
    barrier(dist, world)
    return max_over_ranks(torch, dist, world, runner.device, e0.elapsed_time(e1) / 1e3 / steps), None


def prewarm(torch, dist, world, runner, steps, seconds=0.01) -> None:
    """Keep the GPU busy with the workload's own steps for ten milliseconds or more before anything is timed: a
    workload whose timed pass lasts a millisecond would otherwise be measured while the clocks still come up from
    the idle period of its set-up.  A few steps at a time (positions reset each time), so that a workload whose step
    takes milliseconds is not run hot before its first pass either."""
    t0 = time.time()
    chunk = min(steps, STEPS_PER_GRAPH)
    while True:
        runner.reset_pos()
        runner.run(chunk)
        torch.cuda.synchronize()
        done = torch.tensor([1.0 if time.time() - t0 >= seconds else 0.0], device=runner.device)
        if world > 1:   # every rank leaves the loop in the same round (tensor-parallel steps wait for each other)
            dist.all_reduce(done, op=dist.ReduceOp.MIN)
        if done.item() > 0:
            break


def measure(torch, dist, world, runner, steps, warmup) -> dict:
    """The protocol of the module docstring for one workload; seconds."""
    prewarm(torch, dist, world, runner, steps)
    passes = [timed_pass(torch, dist, world, runner, steps, warmup)[0] for _ in range(PASSES)]
    _, each = timed_pass(torch, dist, world, runner, steps, warmup, per_step=True)
    return {"first": passes[0], "passes": passes, "each": each}


def stats_entry(m: dict) -> dict:
    us = [x * 1e6 for x in m["passes"]]
    each = [x * 1e6 for x in m["each"]]
    return {"passes_us": {"n": len(us), "median": statistics.median(us), "min": min(us), "max": max(us)},
            "step_us": {"n": len(each), "p50": percentile(each, 0.5), "p95": percentile(each, 0.95),
                        "note": "one event pair per step (this rank); the events add to the gap between replays"}}


def timed_kernel(torch, runner, steps, warmup) -> float:
    """Average duration of the attention kernel alone: the launch is captured in its own CUDA graph
    (so the host cannot be the limit) and replayed back to back between CUDA events."""
    c = runner.cache
    off = 0 if runner.advance else 1

    def launch():
        runner.pkg.decode_attention(runner.q, c.k_cache, c.v_cache, c.k_scale, c.v_scale, c.seq_pos,
                                    workspace=c.workspace, seq_len_offset=off, out=runner.out)
    runner.reset_pos()
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
    step, device -> pinned-host result, and a synchronize (the caller needs the result).  With one
    rank the result is the whole output; tensor-parallel, every rank reads back the heads it computed
    from its gathered buffer (together the ranks read the whole result once; the gathered tensor itself
    stays on the device, where its consumer is).  The copies and the step are captured into one CUDA
    graph (memcpy nodes + the library's launch), as a host that replays its decode step would do; two
    steps per graph, because the stores mode of the tensor-parallel step alternates between two gathered buffers."""
    hin = runner.inputs.cpu().pin_memory()   # q, k_new, v_new of the step: one pinned buffer, one copy
    if runner.peer is not None:
        rank, hq_loc, peer = runner.peer.rank, runner.h_q, runner.peer
        tensors = [peer.full, peer.full] if peer.mode == "packets" else [peer.buffers[(peer.steps_done() + 1 + i) & 1] for i in range(2)]
        sources = [t[:, :, rank * hq_loc:(rank + 1) * hq_loc] for t in tensors]
    else:
        sources = [runner.result()] * 2
    hout = torch.empty(sources[0].shape, dtype=sources[0].dtype).pin_memory()
    h2d = hin.numel() * hin.element_size()
    d2h = hout.numel() * hout.element_size()

    def sequence():
        for src in sources:
            runner.inputs.copy_(hin, non_blocking=True)
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

    def two_steps():
        if graph is not None:
            graph.replay()
        else:
            sequence()
        torch.cuda.synchronize()

    reps = max(1, (steps + 1) // 2)
    runner.reset_pos()
    for _ in range(max(1, warmup // 2)):
        two_steps()
    runner.reset_pos()
    barrier(dist, world)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        two_steps()
    e1.record()
    torch.cuda.synchronize()
    wall = (time.perf_counter() - t0) / (2 * reps)
    barrier(dist, world)
    runner.reset_pos()
    sec = max(e0.elapsed_time(e1) / 1e3 / (2 * reps), wall)
    return max_over_ranks(torch, dist, world, runner.device, sec), h2d, d2h * (world if runner.peer is not None else 1)


def timed_l2_free(pkg, torch, device, depth, cap, advance, h_q, h_kv, variant, steps, warmup) -> float:
    """Seconds per step when the cache cannot stay in L2: the step rotates through several copies of the cache
    (each with its own data), one graph replay = one step on every copy.  This rank's heads, no exchange.
    0.0 if a device status bit was set (the caller withholds the figure; every rank still takes part in the
    reduction that follows)."""
    runners = [StepRunner(pkg, torch, device, [depth], cap, advance, h_q, h_kv, seed=100 + i, variant=variant)
               for i in range(L2_FREE_COPIES)]
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for r in runners:
            r.launch_step()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for r in runners:
            r.launch_step()
    reps = max(1, steps // L2_FREE_COPIES)
    for r in runners:
        r.reset_pos()
    for _ in range(max(1, warmup // L2_FREE_COPIES)):
        graph.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        graph.replay()
    e1.record()
    torch.cuda.synchronize()
    for r in runners:
        if r.cache.workspace.read_status():
            print(f"[bench] device status {r.cache.workspace.read_status()} in the L2-free run", file=sys.stderr)
            return 0.0
    return e0.elapsed_time(e1) / 1e3 / (reps * L2_FREE_COPIES)


def parity_check(torch, dist, world, runner, seq_plan=None, layers=None) -> dict | None:
    """Off the clock: one more step from the start positions, then two layers of its result (as rank 0 sees it:
    the gathered tensor when tensor-parallel) against the CPU oracle — the reference's padded torch attention over
    the dequantised cache.  The other ranks' K/V bytes, scales and queries of those layers are gathered for it.
    Sequence-sharded: every rank checks its own sequences; the worst figures over the ranks are reported."""
    from oracle import ref_attention as oracle
    layers = [0, N_LAYERS - 1] if layers is None else layers
    c = runner.cache
    runner.reset_pos()
    runner.step()
    torch.cuda.synchronize()
    barrier(dist, world)
    lens = [int(x) + 1 for x in runner.start_pos.cpu().tolist()]
    longest = max(lens)
    idx = torch.tensor(layers, device=runner.device)
    mine = {"k": c.k_cache.index_select(0, idx)[:, :, :, :longest].contiguous(), "v": c.v_cache.index_select(0, idx)[:, :, :, :longest].contiguous(),
            "ks": c.k_scale.index_select(0, idx).contiguous(), "vs": c.v_scale.index_select(0, idx).contiguous(),
            "q": runner.q.index_select(0, idx).contiguous()}
    result = runner.result().index_select(0, idx).contiguous()
    rank = dist.get_rank() if world > 1 else 0
    if world > 1 and seq_plan is None:         # tensor parallel: heads of all ranks, in rank order
        full = {}
        for name, t in mine.items():
            parts = [torch.empty_like(t) for _ in range(world)]
            dist.all_gather(parts, t)
            full[name] = torch.cat(parts, dim=t.dim() - 1 if name in ("ks", "vs") else 2)   # the KV-head axis
        mine = full
    worst = {"max_abs": 0.0, "cosine": 1.0}
    if rank == 0 or seq_plan is not None:
        ref = oracle.decode_step_reference(mine["q"].cpu(), mine["k"].cpu(), mine["v"].cpu(), mine["ks"].cpu(), mine["vs"].cpu(),
                                           lens, longest)
        got = result.cpu()
        for b in range(len(lens)):
            m = oracle.error_metrics(got[:, b], ref[:, b])
            worst = {"max_abs": max(worst["max_abs"], m["max_abs"]), "cosine": min(worst["cosine"], m["cosine"])}
    if world > 1:
        t = torch.tensor([worst["max_abs"], -worst["cosine"]], device=runner.device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        worst = {"max_abs": float(t[0].item()), "cosine": -float(t[1].item())}
    runner.reset_pos()
    worst.update({"layers": layers, "against": "CPU oracle (the reference's padded torch attention on the dequantised cache)",
                  "ok": worst["max_abs"] <= PARITY_TOL["max_abs"] and worst["cosine"] >= PARITY_TOL["cosine"]})
    return worst


def cpu_baseline(depth: int, cap: int) -> dict:
    from oracle import ref_attention as oracle
    threads = os.cpu_count() or 1
    layers, repeats = 4, 2
    r = oracle.cpu_attention_seconds(H_Q, H_KV, D, depth, max(cap, depth), layers, repeats, threads)
    return {"value": r["full_s_per_layer"] * N_LAYERS * 1e6, "unit": "us/step", "cores": threads, "kind": "port",
            "attn_only_us_per_step": r["attn_s_per_layer"] * N_LAYERS * 1e6,
            "sample": f"median of {r['samples']} single-layer runs (dequant + pad + padded torch attention) at depth "
                      f"{depth}, capacity {max(cap, depth)}, scaled x{N_LAYERS} layers"}


def cfg4_depths(torch) -> list[int]:
    return torch.randint(CFG4_LO, CFG4_HI + 1, (CFG4_BATCH,), generator=torch.Generator().manual_seed(0)).tolist()


def build_runner(pkg, torch, device, dist, world, rank, key, args):
    """(runner, steps, extra) for a workload key on this rank."""
    if key == "cfg4":
        depths_all = cfg4_depths(torch)
        plan = pkg.dist.assign_sequences(depths_all, world)
        depths = [depths_all[i] for i in plan[rank]]
        steps = max(1, min(args.steps, 256 - args.warmup - 8))
        runner = StepRunner(pkg, torch, device, depths, CFG4_CAP, True, H_Q, H_KV, seed=rank, dist=dist, world=world,
                            variant=args.variant, num_splits=args.ctas, tensor_parallel=False)
        loads = [sum(depths_all[i] for i in p) for p in plan]
        return runner, steps, {"plan": plan, "depths": depths_all, "loads": loads}
    depth, cap, advance = WORKLOADS[key]
    room = cap - depth - args.warmup - 8 if advance else 1 << 30   # the cache must not overflow
    steps = max(1, min(args.steps, room))
    runner = StepRunner(pkg, torch, device, [depth], cap, advance, H_Q // world, H_KV // world, seed=rank, dist=dist, world=world,
                        variant=args.variant, num_splits=args.ctas, gather=args.gather, scale_mode=args.scales)
    return runner, steps, {}


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
    if H_KV % world or CFG4_BATCH % world:
        raise SystemExit("KV-head sharding needs a GPU count that divides 8")

    others = [] if args.only else [w for w in list(WORKLOADS) + ["cfg4"] if w != args.workload]
    if args.scales != "per_head":
        others = [w for w in others if w != "cfg4"]
    per_depth, per_workload = {}, {}
    headline = None
    for key in [args.workload] + others:
        runner, steps, extra = build_runner(pkg, torch, device, dist, world, rank, key, args)
        runner.capture()
        if world > 1:   # every rank in step before the first timed (or barrier-carrying) launch
            torch.cuda.synchronize()
            dist.barrier()
        is_headline = key == args.workload
        warm = args.warmup
        with ClockSampler(torch, local) as sampler:
            m = measure(torch, dist, world, runner, steps, warm)
            ksec = timed_kernel(torch, runner, steps, warm)
        sec = m["first"]
        if runner.cache.workspace.read_status():
            raise SystemExit(f"device status {runner.cache.workspace.read_status()} after {key}")
        waits = None
        if runner.peer is not None and runner.peer.mode == "stores":     # how long each rank's last arrive-and-wait took (device time stamps)
            w = torch.tensor([runner.peer.last_wait_us()], device=device, dtype=torch.float64)
            allw = [torch.empty_like(w) for _ in range(world)]
            dist.all_gather(allw, w)
            waits = [float(x.item()) for x in allw]
        parity = None if args.no_parity else parity_check(torch, dist, world, runner, seq_plan=extra.get("plan"))
        if key == "cfg4":
            mean_len = [d + warm + (steps + 1) / 2 for d in extra["depths"]]      # lengths grow by one per step
            total_bytes = N_LAYERS * H_KV * D * 2 * sum(mean_len)
            share = max(extra["loads"]) / sum(extra["loads"])
            entry = {"us_per_step": sec * 1e6, "hbm_gbs_whole_job": total_bytes / sec / 1e9,
                     "hbm_gbs_busiest_gpu": total_bytes * share / sec / 1e9, "frac_of_8TBs_busiest_gpu": total_bytes * share / sec / 8e12,
                     "tokens_per_s": CFG4_BATCH / sec, "sum_depth_per_rank": extra["loads"],
                     "busiest_rank_share": share, "load_imbalance": max(extra["loads"]) * world / sum(extra["loads"]),
                     "kernel": runner.cache.workspace.resolved, "gpu_launches_per_step": runner.kernels_per_step(), "steps": steps}
            bytes_per_launch = total_bytes * share
        else:
            depth = WORKLOADS[key][0]
            total_bytes = kv_bytes_per_step(depth)                 # whole job (all ranks)
            entry = {"us_per_step": sec * 1e6, "us_per_layer": sec * 1e6 / N_LAYERS,
                     "hbm_gbs_whole_job": total_bytes / sec / 1e9, "hbm_gbs_per_gpu": total_bytes / world / sec / 1e9,
                     "frac_of_8TBs_per_gpu": total_bytes / world / sec / 8e12,
                     "attn_kernel_us": ksec * 1e6, "attn_kernel_gbs_per_gpu": total_bytes / world / ksec / 1e9,
                     "kernel": runner.cache.workspace.resolved, "steps": steps}
            bytes_per_launch = kv_bytes_per_step(depth, H_KV // world)
            # the workload whose whole KV working set fits L2 (the short cache) also gets an L2-free figure
            if total_bytes < 200e6 and not args.no_l2_free:
                l2f = timed_l2_free(pkg, torch, device, depth, WORKLOADS[key][1], WORKLOADS[key][2], H_Q // world, H_KV // world,
                                    args.variant, steps, args.warmup)
                bad = max_over_ranks(torch, dist, world, device, 1.0 if l2f <= 0 else 0.0)
                l2f = max_over_ranks(torch, dist, world, device, l2f)
                if bad == 0:
                    entry["l2_free"] = {"us_per_step": l2f * 1e6, "hbm_gbs_per_gpu": total_bytes / world / l2f / 1e9,
                                        "copies": L2_FREE_COPIES, "note": "this rank's heads, no exchange; the step rotates through "
                                        f"{L2_FREE_COPIES} caches so that none of them stays in L2"}
                else:
                    entry["l2_free"] = {"error": "a rank's device status was set in the L2-free run; figure withheld"}
        entry.update(stats_entry(m))
        entry["clocks"] = sampler.summary()     # this workload's own timed passes
        if waits is not None:
            entry["exchange_wait_us"] = {"min": min(waits), "max": max(waits),
                                         "note": "last step: from a rank's arrival at the in-launch barrier to its release"}
        if parity is not None:
            entry["parity"] = parity
        (per_workload if key == "cfg4" else per_depth)[key if key == "cfg4" else str(WORKLOADS[key][0])] = entry
        if is_headline:
            e2e_sec, h2d, d2h = timed_e2e(torch, dist, world, runner, steps, args.warmup)
            headline = {"key": key, "sec": sec, "ksec": ksec, "clocks": sampler.summary(), "steps": steps, "m": m,
                        "ctas": runner.cache.workspace.num_splits, "sms": torch.cuda.get_device_properties(device).multi_processor_count,
                        "resolved": runner.cache.workspace.resolved, "per_token": runner.cache.per_token,
                        "launches": runner.kernels_per_step(), "bytes_per_launch": bytes_per_launch, "total_bytes": total_bytes,
                        "e2e": (e2e_sec, h2d, d2h), "parity": parity, "entry": entry}
        del runner
        torch.cuda.empty_cache()

    h = headline
    key = h["key"]
    peak, peak_kind = load_peak()
    achieved = h["bytes_per_launch"] / h["ksec"] / 1e9
    traffic = load_traffic(key, h["resolved"])
    one_gpu_bytes = kv_bytes_per_step(WORKLOADS[key][0]) if key in WORKLOADS else None
    line = {
        "metric": METRIC if args.layers == 64 else METRIC.replace("64 layers", f"{args.layers} layers: profiling only"),
        "value": h["sec"] * 1e6, "unit": "us/step", "n_gpus": world, "steps": h["steps"],
        "warmup": args.warmup, "ms_per_step": h["sec"] * 1e3, "higher_is_better": False, "scaling": "strong",
        "vs_baseline": None, "dtype": DTYPES[h["resolved"]], "data": "synthetic",
        "config": make_config(key, world),
        "hbm_gbs": h["total_bytes"] / h["sec"] / 1e9,
        "frac_of_8TBs": h["bytes_per_launch"] / h["sec"] / 8e12,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "traffic": None if traffic is None or not one_gpu_bytes else traffic * h["bytes_per_launch"] / one_gpu_bytes,
                     "traffic_note": "ncu DRAM bytes of a 16-layer launch on one GPU, scaled by the KV bytes this launch reads",
                     "kernel": kernel_name(h["resolved"], h["per_token"], h["ctas"], h["sms"]), "peak_kind": peak_kind,
                     "algorithmic_bytes_per_launch": h["bytes_per_launch"], "launch_us": h["ksec"] * 1e6},
        "e2e": {"value": h["e2e"][0] * 1e6, "unit": "us/step", "h2d_bytes_per_step": h["e2e"][1], "d2h_bytes_per_step": h["e2e"][2]},
        "gpu_launches": h["launches"] * h["steps"],
        "clocks": h["clocks"],
    }
    line.update(stats_entry(h["m"]))
    if h["parity"] is not None:
        line["parity"] = h["parity"]
    if "exchange_wait_us" in h["entry"]:
        line["exchange_wait_us"] = h["entry"]["exchange_wait_us"]
    line["per_depth"] = per_depth
    if per_workload:
        line["per_workload"] = per_workload
    if world == 1 and rank == 0 and not args.no_cpu and key in WORKLOADS:
        line["cpu_baseline"] = cpu_baseline(*WORKLOADS[key][:2])
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


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--workload", choices=sorted(WORKLOADS) + ["cfg4"], default="cfg2")
    ap.add_argument("--only", action="store_true", help="measure only the headline workload")
    ap.add_argument("--variant", choices=["auto", "mma", "umma2", "simt"], default="auto", help="attention kernel variant")
    ap.add_argument("--gather", choices=["packets", "stores", "nccl"], default="packets",
                    help="N > 1: all-gather fused into the kernel as 8-byte value+step packets (default), as plain peer stores "
                         "followed by a cross-GPU barrier, or NCCL all-gather + reorder copy after the kernel")
    ap.add_argument("--scales", choices=["per_head", "per_token"], default="per_head",
                    help="scale granularity of the FP8 cache (per_token = the reference's frozen [capacity, kv_heads] layout)")
    ap.add_argument("--heads", default="", help="H_q,H_kv,head_dim instead of the metric's 40,8,128 (e.g. 24,4,256: the "
                    "reference model's own attention shape; not the metric)")
    ap.add_argument("--ctas", type=int, default=0, help="override the split / CTA count (0 = library default)")
    ap.add_argument("--layers", type=int, default=64, help="layers per step (64 = the metric; fewer only for profiling)")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-parity", action="store_true", help="skip the off-clock comparison with the CPU oracle")
    ap.add_argument("--no-l2-free", action="store_true", help="skip the L2-free variant of the short-cache workload")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    global N_LAYERS, SCALES_TEXT, H_Q, H_KV, D
    N_LAYERS = args.layers
    if args.heads:
        H_Q, H_KV, D = (int(x) for x in args.heads.split(","))
    if args.scales == "per_token":
        SCALES_TEXT = "per-(token,kv-head)"
    if args.impl == "reference":
        if args.workload == "cfg4":
            raise SystemExit("--impl reference times the bs=1 workloads (cfg1..cfg3)")
        return run_reference(args)
    return run_ours(args)


if __name__ == "__main__":
    raise SystemExit(main())
