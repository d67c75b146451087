#!/usr/bin/env python3
"""Generate tests/golden/producer_golden.npz from the model code the reference runs.

The reference loads transformers' Qwen3.5 text model (runner/loader/nvfp4_model.py:82-88,145) and
its attention block normalises and rotates q and k before the cache update.  That code lives in
the third-party package (transformers 5.5.0 in this image), so the fixtures are produced by
calling ITS ``Qwen3_5RMSNorm`` and ``apply_rotary_pos_emb`` on seeded inputs; the oracle's
restatement (oracle/ref_attention.py::producer_reference) is pinned against them bit for bit.

    python tests/golden/make_golden_producer.py
"""
from __future__ import annotations

import json
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent

# (name, batch, h_q, h_kv, head_dim, rotary_dim, eps, seed)
CASES = [
    ("b2_40x8x128_r32", 2, 40, 8, 128, 32, 1e-6, 0),
    ("b2_40x8x128_r64", 2, 40, 8, 128, 64, 1e-6, 1),
    ("b1_40x8x128_r128", 1, 40, 8, 128, 128, 1e-5, 2),
    ("b3_24x4x256_r64", 3, 24, 4, 256, 64, 1e-6, 3),      # the reference model's head shape (partial rotary 0.25)
]


def bits(t: torch.Tensor) -> np.ndarray:
    return t.contiguous().view(torch.int16).numpy().view(np.uint16)


def main() -> int:
    import transformers
    from transformers.models.qwen3_5 import modeling_qwen3_5 as m
    torch.set_num_threads(1)
    arrays, meta = {}, {"transformers": transformers.__version__}
    for name, b, h_q, h_kv, d, r, eps, seed in CASES:
        g = torch.Generator().manual_seed(seed)
        q_raw = (torch.randn(b, h_q, 1, d, generator=g) * 3).to(torch.bfloat16)
        k_raw = (torch.randn(b, h_kv, 1, d, generator=g) * 3).to(torch.bfloat16)
        wq = (torch.randn(d, generator=g) * 0.3).to(torch.bfloat16)
        wk = (torch.randn(d, generator=g) * 0.3).to(torch.bfloat16)
        ang = torch.rand(b, 1, r, generator=g) * 6.283
        cos, sin = torch.cos(ang).to(torch.bfloat16), torch.sin(ang).to(torch.bfloat16)
        norm_q, norm_k = m.Qwen3_5RMSNorm(d, eps=eps).to(torch.bfloat16), m.Qwen3_5RMSNorm(d, eps=eps).to(torch.bfloat16)
        with torch.no_grad():
            norm_q.weight.copy_(wq)
            norm_k.weight.copy_(wk)
            # the block's own order: norm on [B, T, H, D], transpose to [B, H, T, D], rotary
            qn = norm_q(q_raw.transpose(1, 2)).transpose(1, 2)
            kn = norm_k(k_raw.transpose(1, 2)).transpose(1, 2)
            q_out, k_out = m.apply_rotary_pos_emb(qn, kn, cos, sin)
        for key, t in (("q_raw", q_raw), ("k_raw", k_raw), ("wq", wq), ("wk", wk), ("cos", cos), ("sin", sin),
                       ("q_out", q_out), ("k_out", k_out)):
            arrays[f"{name}/{key}"] = bits(t)
        meta[name] = {"batch": b, "h_q": h_q, "h_kv": h_kv, "d": d, "rotary_dim": r, "eps": eps, "seed": seed}
        print(name, "ok", flush=True)
    arrays["meta_json"] = np.frombuffer(json.dumps(meta).encode(), dtype=np.uint8)
    np.savez_compressed(HERE / "producer_golden.npz", **arrays)
    print("wrote", HERE / "producer_golden.npz")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
