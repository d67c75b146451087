"""The cache-layer + attention-interface shim, driven the way the model's attention module drives it."""
import types

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_prefill_then_decode_through_the_plug_points(pkg, oracle, cuda_device):
    from importlib import import_module
    hf = import_module("qwen38-5080_b200.hf")
    h_q, h_kv, d, cap, prefix, steps = 24, 4, 256, 128, 37, 3
    g = torch.Generator().manual_seed(2)
    k0 = torch.randn(1, h_kv, prefix, d, generator=g).to(torch.bfloat16)
    v0 = torch.randn(1, h_kv, prefix, d, generator=g).to(torch.bfloat16)
    ks, vs = oracle.head_scales(k0) * 1.2, oracle.head_scales(v0) * 1.2
    layer = hf.FP8StaticAttentionLayer(cap, h_q=h_q, k_scale=ks, v_scale=vs)
    module = types.SimpleNamespace(layer_idx=0, num_key_value_groups=h_q // h_kv)
    before = dict(hf.COUNTERS)

    kd, vd = layer.update(k0.to(cuda_device), v0.to(cuda_device))             # prefill, q_len > 1
    assert kd.dtype == torch.bfloat16 and kd.shape == (1, h_kv, prefix, d)
    want_k = oracle.quantize_per_head(k0, ks)
    assert torch.equal(layer.keys[:, :, :prefix].cpu(), want_k)
    assert torch.equal(kd.cpu(), oracle.dequantize(want_k, ks.view(1, -1, 1, 1)))
    assert layer.get_mask_sizes(1) == (cap, 0) and layer.get_seq_length() == prefix
    assert hf.cache_layout_gate([layer])

    kb, vb = want_k, oracle.quantize_per_head(v0, vs)
    for _ in range(steps):
        q = torch.randn(1, h_q, 1, d, generator=g).to(torch.bfloat16)
        kn = torch.randn(1, h_kv, 1, d, generator=g).to(torch.bfloat16)
        vn = torch.randn(1, h_kv, 1, d, generator=g).to(torch.bfloat16)
        kh, vh = layer.update(kn.to(cuda_device), vn.to(cuda_device))         # decode, q_len == 1
        assert kh.dtype == torch.uint8 and kh.data_ptr() == layer.keys.data_ptr()
        out, weights = hf.fp8_decode_attention(module, q.to(cuda_device), kh, vh, None, scaling=d ** -0.5)
        assert weights is None and out.shape == (1, 1, h_q, d)
        kb = torch.cat([kb, oracle.quantize_per_head(kn, ks)], dim=2)
        vb = torch.cat([vb, oracle.quantize_per_head(vn, vs)], dim=2)
        ref = oracle.padded_fp8_reference(q, kb, vb, ks, vs, cap)
        m = oracle.error_metrics(out.cpu(), ref)
        assert m["max_abs"] <= 2e-2 and m["cosine"] >= 0.9999, m
    assert torch.equal(layer.keys[:, :, :prefix + steps].cpu(), kb)           # appended bytes bit-exact
    assert layer.cumulative_length.cpu().tolist() == [prefix + steps]
    assert hf.COUNTERS["fused_decode_calls"] - before["fused_decode_calls"] == steps
    assert hf.COUNTERS["appends"] - before["appends"] == steps
    ptr = layer.keys.data_ptr()
    layer.reset()
    assert layer.keys.data_ptr() == ptr and layer.get_seq_length() == 0 and int(layer.keys.max()) == 0
    with pytest.raises(ValueError):
        hf.fp8_decode_attention(module, torch.zeros(1, h_q, 2, d, dtype=torch.bfloat16, device=cuda_device),
                                layer.keys, layer.values)
