#!/usr/bin/env python3
"""Generate tests/golden/attn_golden.npz from the reference's OWN functions.

Run where the reference checkout is available (pass its root with --reference); the fixtures
are committed because the checkout does not travel to the GPU box.

For every case the inputs are seeded exactly as bench/micro/attn_length_effect.py:99-102 does
(one CPU generator: q, k, v), K/V are quantised to e4m3 with per-(kv head) absmax/448 scales
and dequantised to bf16 (docs/journal/2026-10-23-phase2-r3-coordinator.md:43-49), padded with
zeros to capacity and masked (attn_length_effect.py:106-111), and then the reference module's
``eager_attention`` and ``fp64_reference`` are called with its globals H_Q/H_KV/HEAD_DIM/SCALING
set to the case's head shape.  Stored per case: the bf16 output bits, the fp64 output (as
float32), the scales, and sha256 digests of q and of the quantised K/V bytes so a test can
prove it rebuilt the same inputs.

    python tests/golden/make_golden.py --reference <reference checkout>
"""
from __future__ import annotations

import argparse
import hashlib
import importlib.util
import json
import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parents[1]))
from oracle import ref_attention as oracle  # noqa: E402  (input generation + quantisation only)

# (name, h_q, h_kv, d, length, capacity, seed)
CASES = [
    ("b40x8x128_L1_c1024_s0", 40, 8, 128, 1, 1024, 0),
    ("b40x8x128_L127_c1024_s0", 40, 8, 128, 127, 1024, 0),
    ("b40x8x128_L128_c1024_s0", 40, 8, 128, 128, 1024, 0),
    ("b40x8x128_L129_c1024_s0", 40, 8, 128, 129, 1024, 0),
    ("b40x8x128_L300_c1024_s0", 40, 8, 128, 300, 1024, 0),
    ("b40x8x128_L513_c1024_s0", 40, 8, 128, 513, 1024, 0),
    ("b40x8x128_L513_c1024_s1", 40, 8, 128, 513, 1024, 1),
    ("b40x8x128_L1024_c1024_s0", 40, 8, 128, 1024, 1024, 0),
    ("b40x8x128_L8192_c8192_s0", 40, 8, 128, 8192, 8192, 0),
    ("r24x4x256_L513_c1024_s0", 24, 4, 256, 513, 1024, 0),
    ("r24x4x256_L300_c1024_s3", 24, 4, 256, 300, 1024, 3),
]


def load_reference_module(root: Path):
    path = root / "bench" / "micro" / "attn_length_effect.py"
    spec = importlib.util.spec_from_file_location("ref_attn_length_effect", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def sha(t: torch.Tensor) -> str:
    return hashlib.sha256(t.contiguous().view(torch.uint8).numpy().tobytes()).hexdigest()


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", type=Path, required=True, help="root of the reference checkout")
    args = ap.parse_args()
    ref = load_reference_module(args.reference)
    torch.set_num_threads(1)  # one thread: the stored bits do not depend on the thread count

    arrays, meta = {}, {}
    for name, h_q, h_kv, d, length, cap, seed in CASES:
        ref.H_Q, ref.H_KV, ref.HEAD_DIM, ref.SCALING = h_q, h_kv, d, d ** -0.5
        q, k, v = oracle.make_inputs(seed, h_q, h_kv, d, length)
        sk, sv = oracle.head_scales(k), oracle.head_scales(v)
        kb, vb = oracle.quantize_per_head(k, sk), oracle.quantize_per_head(v, sv)
        kd = oracle.dequantize(kb, sk.view(1, -1, 1, 1))
        vd = oracle.dequantize(vb, sv.view(1, -1, 1, 1))
        pad = cap - length
        k_pad = torch.cat([kd, torch.zeros(1, h_kv, pad, d, dtype=kd.dtype)], dim=-2)
        v_pad = torch.cat([vd, torch.zeros(1, h_kv, pad, d, dtype=vd.dtype)], dim=-2)
        mask = torch.full((1, 1, 1, cap), torch.finfo(torch.bfloat16).min, dtype=torch.bfloat16)
        mask[..., :length] = 0
        out = ref.eager_attention(q, k_pad, v_pad, mask=mask)          # the reference's function
        out64 = ref.fp64_reference(q, kd, vd)                          # the reference's function
        arrays[f"{name}/out_bf16_bits"] = out.view(torch.int16).numpy().view(np.uint16)
        arrays[f"{name}/out_fp64_as_f32"] = out64.float().numpy()
        arrays[f"{name}/k_scale"] = sk.numpy()
        arrays[f"{name}/v_scale"] = sv.numpy()
        meta[name] = {
            "h_q": h_q, "h_kv": h_kv, "d": d, "length": length, "capacity": cap, "seed": seed,
            "sha_q": sha(q), "sha_k_bytes": sha(kb), "sha_v_bytes": sha(vb),
        }
        print(name, "ok", flush=True)
    arrays["meta_json"] = np.frombuffer(json.dumps(meta).encode(), dtype=np.uint8)
    np.savez_compressed(HERE / "attn_golden.npz", **arrays)
    print("wrote", HERE / "attn_golden.npz")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
