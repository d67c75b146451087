"""GPU parity of the producer-side fusion (q_norm / k_norm + rotary embedding + FP8 append) against
the oracle and against the fixtures made by the model code the reference runs."""
import json

import numpy as np
import pytest
import torch

from test_oracle import producer_case

pytestmark = pytest.mark.gpu


def ulp_distance(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """Distance in bf16 steps (sign-magnitude bits mapped to a monotone integer line)."""
    def line(t):
        i = t.contiguous().view(torch.int16).to(torch.int32)
        return torch.where(i < 0, -(i & 0x7FFF), i)
    return (line(a) - line(b)).abs()


def run_producer(pkg, dev, q_raw, k_raw, v_new, wq, wk, cos, sin, eps, cap, pos, scale_mode, k_scale=None, v_scale=None):
    """q_raw [n, b, h_q, d] etc. on the CPU -> (q_out, k_out, cache) through the C-ABI."""
    n, b, h_q, d = q_raw.shape
    h_kv = k_raw.shape[2]
    cache = pkg.FP8StaticCache(n, b, h_q, h_kv, d, cap, device=dev, variant="simt", scale_mode=scale_mode)
    if scale_mode == "per_head":
        cache.set_scales(k_scale.to(dev), v_scale.to(dev))
    cache.seq_pos.copy_(torch.tensor(pos, dtype=torch.int32))
    k_out = torch.empty_like(k_raw, device=dev)
    q_out = pkg.qk_norm_rope_append(q_raw.to(dev), k_raw.to(dev), v_new.to(dev), wq.to(dev), wk.to(dev), cos.to(dev),
                                    sin.to(dev), cache.k_cache, cache.v_cache, cache.k_scale, cache.v_scale,
                                    cache.seq_pos, eps=eps, advance=True, status=cache.status, k_out=k_out)
    torch.cuda.synchronize()
    return q_out.cpu(), k_out.cpu(), cache


def test_producer_golden_parity(pkg, oracle, producer_golden, cuda_device):
    """Every fixture of the model code: the kernel's q and rotated k are within one bf16 step of it
    (the fp32 sum of squares is a warp tree, not the CPU's order) and identical almost everywhere;
    the appended bytes are exactly the quantisation of the kernel's own rotated k, and V's of v."""
    data, meta = producer_golden
    for name in [n for n in meta if n != "transformers"]:
        m = meta[name]
        c = producer_case(data, name, m)
        b, h_q, h_kv, d = m["batch"], m["h_q"], m["h_kv"], m["d"]
        g = torch.Generator().manual_seed(m["seed"] + 100)
        v_new = torch.randn(1, b, h_kv, d, generator=g).to(torch.bfloat16)
        pos = [5 + 3 * i for i in range(b)]
        for scale_mode in ("per_head", "per_token"):
            ks = (torch.rand(1, h_kv, generator=g) * 0.05 + 0.01) if scale_mode == "per_head" else None
            vs = (torch.rand(1, h_kv, generator=g) * 0.05 + 0.01) if scale_mode == "per_head" else None
            q_out, k_out, cache = run_producer(
                pkg, cuda_device, c["q_raw"].transpose(1, 2).contiguous().view(1, b, h_q, d),
                c["k_raw"].transpose(1, 2).contiguous().view(1, b, h_kv, d), v_new, c["wq"].view(1, d), c["wk"].view(1, d),
                c["cos"].view(b, -1).contiguous(), c["sin"].view(b, -1).contiguous(), m["eps"], 64, pos, scale_mode, ks, vs)
            assert cache.workspace.read_status() == 0
            want_q = c["q_out"].transpose(1, 2).contiguous().view(1, b, h_q, d)
            want_k = c["k_out"].transpose(1, 2).contiguous().view(1, b, h_kv, d)
            for got, want, what in ((q_out, want_q, "q"), (k_out, want_k, "k")):
                dist = ulp_distance(got, want)
                assert int(dist.max()) <= 1, (name, scale_mode, what, int(dist.max()))
                assert float((dist == 0).float().mean()) >= 0.995, (name, what)
            assert cache.seq_pos.cpu().tolist() == [p + 1 for p in pos]
            kc, vc = cache.k_cache.cpu(), cache.v_cache.cpu()
            for i, p in enumerate(pos):
                krow, vrow = k_out[0, i].unsqueeze(0), v_new[0, i].unsqueeze(0)          # [1, h_kv, d]
                if scale_mode == "per_head":
                    wk_bytes = oracle.quantize_e4m3(krow, cache.k_scale.cpu().view(1, h_kv, 1))
                    wv_bytes = oracle.quantize_e4m3(vrow, cache.v_scale.cpu().view(1, h_kv, 1))
                else:
                    sk = krow.float().abs().amax(dim=-1) / 448.0
                    sv = vrow.float().abs().amax(dim=-1) / 448.0
                    assert torch.equal(cache.k_scale[0, i, p].cpu(), sk[0]) and torch.equal(cache.v_scale[0, i, p].cpu(), sv[0])
                    wk_bytes = oracle.quantize_e4m3(krow, sk.unsqueeze(-1))
                    wv_bytes = oracle.quantize_e4m3(vrow, sv.unsqueeze(-1))
                assert torch.equal(kc[0, i, :, p], wk_bytes[0]), (name, scale_mode, "K bytes")
                assert torch.equal(vc[0, i, :, p], wv_bytes[0]), (name, scale_mode, "V bytes")
                assert int(kc[0, i, :, p + 1].max()) == 0 and (p == 0 or int(kc[0, i, :, p - 1].max()) == 0)   # nothing else written


def test_producer_then_attention_all_layers(pkg, oracle, cuda_device):
    """64-layer shape of the benchmark, one step: producer launch, then decode attention over the
    cache it appended to; against the oracle chain (norm + rope on the CPU, quantise, attention)."""
    n, b, h_q, h_kv, d, cap, r, depth = 4, 2, 40, 8, 128, 256, 64, 130
    g = torch.Generator().manual_seed(9)
    k0 = torch.randn(n, b, h_kv, depth, d, generator=g).to(torch.bfloat16)
    v0 = torch.randn(n, b, h_kv, depth, d, generator=g).to(torch.bfloat16)
    q_raw = (torch.randn(n, b, h_q, d, generator=g) * 2).to(torch.bfloat16)
    k_raw = (torch.randn(n, b, h_kv, d, generator=g) * 2).to(torch.bfloat16)
    v_new = torch.randn(n, b, h_kv, d, generator=g).to(torch.bfloat16)
    wq = (torch.randn(n, d, generator=g) * 0.2).to(torch.bfloat16)
    wk = (torch.randn(n, d, generator=g) * 0.2).to(torch.bfloat16)
    ang = torch.rand(b, r, generator=g) * 6.283
    cos, sin = torch.cos(ang).to(torch.bfloat16), torch.sin(ang).to(torch.bfloat16)
    cache = pkg.FP8StaticCache(n, b, h_q, h_kv, d, cap, device=cuda_device, variant="mma")
    cache.prefill(k0.to(cuda_device), v0.to(cuda_device), calibrate=True)
    dev = cuda_device
    q = pkg.qk_norm_rope_append(q_raw.to(dev), k_raw.to(dev), v_new.to(dev), wq.to(dev), wk.to(dev), cos.to(dev), sin.to(dev),
                                cache.k_cache, cache.v_cache, cache.k_scale, cache.v_scale, cache.seq_pos, eps=1e-6,
                                advance=True, status=cache.status)
    out = cache.attend(q)
    torch.cuda.synchronize()
    assert cache.workspace.read_status() == 0 and cache.seq_pos.cpu().tolist() == [depth + 1] * b
    # oracle chain, layer by layer
    ks, vs = cache.k_scale.cpu(), cache.v_scale.cpu()
    kc, vc = cache.k_cache.cpu().clone(), cache.v_cache.cpu().clone()
    q_ref = torch.empty_like(q_raw)
    for layer in range(n):
        qr, kr = oracle.producer_reference(q_raw[layer].unsqueeze(2), k_raw[layer].unsqueeze(2), wq[layer], wk[layer], 1e-6,
                                           cos.unsqueeze(1), sin.unsqueeze(1))
        q_ref[layer] = qr.squeeze(2)
        kc[layer, :, :, depth] = oracle.quantize_e4m3(kr.squeeze(2), ks[layer].view(1, h_kv, 1))
        vc[layer, :, :, depth] = oracle.quantize_e4m3(v_new[layer], vs[layer].view(1, h_kv, 1))
    assert int(ulp_distance(q.cpu(), q_ref).max()) <= 1
    same = (cache.k_cache.cpu() == kc).float().mean().item()
    assert same >= 0.9999 and torch.equal(cache.v_cache.cpu(), vc)      # a k that differs by one bf16 step may round to the next code
    ref = oracle.decode_step_reference(q_ref, kc, vc, ks, vs, [depth + 1] * b, cap)
    m = oracle.error_metrics(out.cpu(), ref)
    assert m["max_abs"] <= 2e-2 and m["cosine"] >= 0.9999, m
