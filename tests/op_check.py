#!/usr/bin/env python3
"""Op check of the FP8-KV decode attention in the shape of the reference's op-check scripts
(scripts/phase2_attn_check.py / phase2_fp8kv_check.py are registered in runner/experiment/schema.py:81-94;
their artifact contract is runner/experiment/op_artifact.py): runs a few cases on cuda:0 against the CPU
oracle and writes ``op.json`` (schema phase2-op/1) with gates, diagnostics and metrics per case.

    python tests/op_check.py --out <dir> [--steps K]
"""
from __future__ import annotations

import argparse
import importlib
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parents[1]
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests"))

CASES = {   # name: (layers, h_q, h_kv, head_dim, depth, capacity)
    "bench-shape-depth512": (4, 40, 8, 128, 512, 1024),
    "bench-shape-depth4096": (4, 40, 8, 128, 4096, 4096 + 64),
    "model-shape-depth1024": (4, 24, 4, 256, 1024, 2048),
}


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", required=True)
    ap.add_argument("--steps", type=int, default=8)
    args = ap.parse_args()
    import torch
    from oracle import ref_attention as oracle
    pkg = importlib.import_module("qwen38-5080_b200")
    art = importlib.import_module("qwen38-5080_b200.op_artifact")
    dev = torch.device("cuda:0")
    report = art.OpReport(args.out, "b200attn-fp8kv-decode", "fp8-kv", candidate_extra={"backend": "cuda-sm100a"},
                          steps=args.steps, environment={"torch": torch.__version__, "gpu": torch.cuda.get_device_name(0)})
    for name, (n, h_q, h_kv, d, depth, cap) in CASES.items():
        case = report.case(name, layers=n, h_q=h_q, h_kv=h_kv, head_dim=d, depth=depth, capacity=cap, steps=args.steps,
                           kv_format="fp8-e4m3", scales="per-(layer,kv-head)")
        g = torch.Generator().manual_seed(0)
        k0 = torch.randn(n, 1, h_kv, depth, d, generator=g).to(torch.bfloat16)
        v0 = torch.randn(n, 1, h_kv, depth, d, generator=g).to(torch.bfloat16)
        qs = torch.randn(args.steps, n, 1, h_q, d, generator=g).to(torch.bfloat16)
        kn = torch.randn(args.steps, n, 1, h_kv, d, generator=g).to(torch.bfloat16)
        vn = torch.randn(args.steps, n, 1, h_kv, d, generator=g).to(torch.bfloat16)
        cache = pkg.FP8StaticCache(n, 1, h_q, h_kv, d, cap, device=dev)
        cache.prefill(k0.to(dev), v0.to(dev), calibrate=True)
        ks, vs = cache.k_scale.cpu(), cache.v_scale.cpu()
        want_k = oracle.quantize_e4m3(k0, ks.view(n, 1, h_kv, 1, 1))
        bytes_ok = torch.equal(cache.k_cache[:, :, :, :depth].cpu(), want_k)
        worst_abs, worst_cos, append_ok = 0.0, 1.0, True
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        outs = []
        e0.record()
        for i in range(args.steps):
            outs.append(cache.step(qs[i].to(dev), kn[i].to(dev), vn[i].to(dev)).clone())
        e1.record()
        torch.cuda.synchronize()
        for i in (0, args.steps - 1):
            length = depth + i + 1
            kc, vc = cache.k_cache.cpu().clone(), cache.v_cache.cpu().clone()
            kc[:, :, :, length:] = 0
            vc[:, :, :, length:] = 0
            ref = oracle.decode_step_reference(qs[i], kc, vc, ks, vs, [length], cap)
            m = oracle.error_metrics(outs[i].cpu(), ref)
            worst_abs, worst_cos = max(worst_abs, m["max_abs"]), min(worst_cos, m["cosine"])
            append_ok = append_ok and torch.equal(cache.k_cache[:, :, :, length - 1].cpu(),
                                                  oracle.quantize_e4m3(kn[i], ks.view(n, 1, h_kv, 1)))
        case.gate("coverage: prefill bytes, appended bytes, first and last step vs the padded reference", True,
                  {"steps_checked": [0, args.steps - 1]})
        case.gate("prefill bytes bit-exact", bytes_ok)
        case.gate("appended bytes bit-exact", append_ok)
        case.gate("max_abs <= 2e-2", worst_abs <= 2e-2, worst_abs)
        case.gate("cosine >= 0.9999", worst_cos >= 0.9999, worst_cos)
        case.gate("device status clean", cache.workspace.read_status() == 0)
        case.diag("kernel", True, cache.workspace.resolved)
        us = e0.elapsed_time(e1) * 1e3 / args.steps
        case.metric("us_per_step_eager", us)
        case.metric("max_abs", worst_abs)
        case.metric("cosine", worst_cos)
    payload = report.finish()
    print(f"op.json: ok={payload['summary']['ok']} -> {Path(args.out) / 'op.json'}")
    return 0 if payload["summary"]["ok"] else 1


if __name__ == "__main__":
    raise SystemExit(main())
