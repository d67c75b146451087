"""The cache-layer + attention-interface shim: first driven by hand the way the model's attention
module drives it, then by the real attention module of transformers' Qwen3.5 implementation (the
model code the reference runs: runner/loader/nvfp4_model.py:82-88) with the attention function
selected by name on the config and the FP8 layers behind a cache container."""
import types
from importlib import import_module

import pytest
import torch

from helpers import TOL_COSINE, TOL_MAX_ABS

pytestmark = pytest.mark.gpu


def test_prefill_then_decode_through_the_plug_points(pkg, oracle, cuda_device):
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
    assert layer.cumulative_length.dim() == 0                                  # the reference's 0-dim device counter
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
        assert m["max_abs"] <= TOL_MAX_ABS and m["cosine"] >= TOL_COSINE, m
    assert torch.equal(layer.keys[:, :, :prefix + steps].cpu(), kb)           # appended bytes bit-exact
    assert int(layer.cumulative_length) == prefix + steps
    assert hf.COUNTERS["fused_decode_calls"] - before["fused_decode_calls"] == steps
    assert hf.COUNTERS["appends"] - before["appends"] == steps
    assert hf.COUNTERS["decode_fallbacks"] == before["decode_fallbacks"]
    assert layer.check_status() == 0
    ptr = layer.keys.data_ptr()
    layer.reset()
    assert layer.keys.data_ptr() == ptr and layer.get_seq_length() == 0 and int(layer.keys.max()) == 0
    with pytest.raises(ValueError):           # FP8 handles with q_len > 1: not something update ever returns
        hf.fp8_decode_attention(module, torch.zeros(1, h_q, 2, d, dtype=torch.bfloat16, device=cuda_device),
                                layer.keys, layer.values)


def test_decode_update_rejects_overflow_on_the_host(pkg, cuda_device):
    """A full cache refuses the next token before anything is launched (the reference's host guard,
    runner/model/decode_runner.py:323-332): host length and device counter stay where they were."""
    hf = import_module("qwen38-5080_b200.hf")
    layer = hf.FP8StaticAttentionLayer(4, h_q=8)
    k = torch.ones(1, 8, 4, 128, dtype=torch.bfloat16, device=cuda_device)
    layer.update(k, k)
    assert layer.get_seq_length() == 4
    one = torch.ones(1, 8, 1, 128, dtype=torch.bfloat16, device=cuda_device)
    with pytest.raises(ValueError):
        layer.update(one, one)
    assert layer.get_seq_length() == 4 and int(layer.cumulative_length) == 4 and layer.check_status() == 0


class _PaddedReferenceLayer:
    """What the reference checks its static cache against (runner/model/padded_reference.py:35-44):
    a growing cache that, for a decode step, is padded to the capacity — here holding what an FP8
    cache holds, i.e. every appended row quantised with the layer's scales and dequantised again."""

    def __init__(self, capacity, k_scale, v_scale):
        self.capacity, self.ks, self.vs = capacity, k_scale.view(1, -1, 1, 1), v_scale.view(1, -1, 1, 1)
        self.k = self.v = self.k_bytes = None

    def _round_trip(self, x, s):
        b = (x.float() / s).clamp(-448, 448).to(torch.float8_e4m3fn)
        return b.view(torch.uint8), (b.float() * s).to(torch.bfloat16)

    def update(self, k, v):
        kb, kd = self._round_trip(k, self.ks)
        _, vd = self._round_trip(v, self.vs)
        self.k = kd if self.k is None else torch.cat([self.k, kd], dim=2)
        self.v = vd if self.v is None else torch.cat([self.v, vd], dim=2)
        self.k_bytes = kb if self.k_bytes is None else torch.cat([self.k_bytes, kb], dim=2)
        if k.shape[2] != 1:
            return self.k, self.v
        pad = self.capacity - self.k.shape[2]
        return torch.nn.functional.pad(self.k, (0, 0, 0, pad)), torch.nn.functional.pad(self.v, (0, 0, 0, pad))


class _OneLayerCache:
    """past_key_values stand-in for the stock path: hands update() to one layer object."""

    def __init__(self, layer):
        self.layer = layer

    def update(self, k, v, layer_idx, *a, **kw):
        return self.layer.update(k, v)


@pytest.mark.parametrize("heads", [(40, 8, 128), (24, 4, 256)])
@pytest.mark.parametrize("fuse_append", [False, True])
def test_real_attention_module_runs_through_the_shim(pkg, cuda_device, heads, fuse_append):
    """Qwen3_5Attention.forward, random weights, one full-attention layer: prefill of 37 tokens, then
    8 decode steps.  The module runs with config._attn_implementation = register()'s name and an
    FP8StaticAdapterCache as past_key_values, and again with "eager" over the dequantised, padded
    reference cache and the capacity-length mask; what reaches o_proj (attention * sigmoid(gate)) and
    the block's output are compared; the cache bytes are the quantisation of the module's own keys."""
    hf = import_module("qwen38-5080_b200.hf")
    from transformers.models.qwen3_5.configuration_qwen3_5 import Qwen3_5TextConfig
    from transformers.models.qwen3_5.modeling_qwen3_5 import Qwen3_5Attention, Qwen3_5TextRotaryEmbedding
    h_q, h_kv, d = heads
    hidden, cap, prefix, steps = 512, 256, 37, 8
    cfg = Qwen3_5TextConfig(vocab_size=64, hidden_size=hidden, intermediate_size=hidden, num_hidden_layers=1,
                            num_attention_heads=h_q, num_key_value_heads=h_kv, head_dim=d, layer_types=["full_attention"],
                            max_position_embeddings=4096)
    torch.manual_seed(7)
    attn = Qwen3_5Attention(cfg, 0).to(device=cuda_device, dtype=torch.bfloat16).eval()
    rotary = Qwen3_5TextRotaryEmbedding(cfg).to(cuda_device)
    name = hf.register()
    g = torch.Generator().manual_seed(3)
    xs = [torch.randn(1, prefix, hidden, generator=g).to(torch.bfloat16).to(cuda_device)] + \
         [torch.randn(1, 1, hidden, generator=g).to(torch.bfloat16).to(cuda_device) for _ in range(steps)]
    captured = []
    hook = attn.o_proj.register_forward_pre_hook(lambda mod, args: captured.append(args[0].detach().clone()))

    def positions(start, n):
        pos = torch.arange(start, start + n, device=cuda_device).view(1, 1, n).expand(3, 1, n)
        return rotary(xs[0], pos)

    def masks(start, n):
        if n == 1:            # the capacity-length decode mask (static_cache.py:79-82): slots > start are hidden
            m = torch.zeros(1, 1, 1, cap, dtype=torch.bfloat16, device=cuda_device)
            m[..., start + 1:] = torch.finfo(torch.bfloat16).min
            return m
        m = torch.full((n, n), torch.finfo(torch.bfloat16).min, dtype=torch.bfloat16, device=cuda_device).triu(1)
        return m.view(1, 1, n, n)

    # calibration pass: scales from the keys / values the module produces for the prefix
    class _Record:
        def update(self, k, v, layer_idx, *a, **kw):
            self.k, self.v = k, v
            return k, v
    rec = _Record()
    cfg._attn_implementation = "eager"
    with torch.no_grad():
        attn(xs[0], positions(0, prefix), masks(0, prefix), past_key_values=rec)
    ks = rec.k.float().abs().amax(dim=(0, 2, 3)) / 448 * 1.5
    vs = rec.v.float().abs().amax(dim=(0, 2, 3)) / 448 * 1.5
    captured.clear()

    # the stock path over the padded reference cache
    ref_layer = _PaddedReferenceLayer(cap, ks, vs)
    ref_cache = _OneLayerCache(ref_layer)
    ref_out, pos = [], 0
    with torch.no_grad():
        for x in xs:
            n = x.shape[1]
            ref_out.append(attn(x, positions(pos, n), masks(pos, n), past_key_values=ref_cache)[0])
            pos += n
    ref_in = list(captured)
    captured.clear()

    # the library behind the same module: attention function by name, FP8 layers behind a Cache container
    cfg._attn_implementation = name
    cache = hf.build_fp8_static_cache(cfg, cap, k_scales=[ks], v_scales=[vs], fuse_append=fuse_append)
    assert hf.preallocate_kv(cache, cfg, batch_size=1, device=cuda_device) == 2 * h_kv * cap * d
    layer = cache.layers[0]
    assert layer.cumulative_length.dim() == 0 and hf.cache_layout_gate(cache.layers)
    before = dict(hf.COUNTERS)
    our_out, pos = [], 0
    with torch.no_grad():
        for x in xs:
            n = x.shape[1]
            assert cache.get_mask_sizes(n, 0) == ((cap, 0) if n == 1 else (pos + n, 0))
            our_out.append(attn(x, positions(pos, n), masks(pos, n), past_key_values=cache)[0])
            pos += n
    torch.cuda.synchronize()
    hook.remove()
    our_in = list(captured)
    assert cache.check_status() == 0 and cache.get_seq_length() == prefix + steps
    assert int(layer.cumulative_length) == prefix + steps
    # wiring: every decode step went through the library, nothing fell back
    delta = {k: hf.COUNTERS[k] - before[k] for k in hf.COUNTERS}
    assert delta["fused_decode_calls"] == steps and delta["decode_fallbacks"] == 0
    assert delta["prefill_attention_calls"] == 1 and delta["bulk_appends"] == 1
    assert delta["fused_step_calls"] == (steps if fuse_append else 0) and delta["appends"] == (0 if fuse_append else steps)
    # cache bytes: the quantisation of the module's own rotated keys, bit for bit
    assert torch.equal(layer.keys[:, :, :prefix + steps], ref_layer.k_bytes)
    for i, (a, b) in enumerate(zip(our_in, ref_in)):
        diff = (a.float() - b.float()).abs().max().item()
        cos = torch.nn.functional.cosine_similarity(a.float().flatten(), b.float().flatten(), dim=0).item()
        assert diff <= TOL_MAX_ABS and cos >= TOL_COSINE, ("o_proj input", i, diff, cos)
    for i, (a, b) in enumerate(zip(our_out, ref_out)):
        cos = torch.nn.functional.cosine_similarity(a.float().flatten(), b.float().flatten(), dim=0).item()
        assert cos >= 0.999, ("block output", i, cos)
    cache.reset()
    assert cache.get_seq_length() == 0 and int(layer.cumulative_length) == 0
