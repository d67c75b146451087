"""GPU parity of the FP8 quantize-and-append: bit-exact against the oracle (torch's e4m3 cast)."""
import pytest
import torch

pytestmark = pytest.mark.gpu

SCALES = [1.0, 2.0 ** -7, 3.0 ** -3, 0.0094, 4.5 / 448, 1e-30, 1e30, 448.0]


def test_exhaustive_bf16_known_answer(pkg, oracle, cuda_device):
    """Every bf16 bit pattern x 8 scales through the append kernel == torch's clamp + cast."""
    n_layers, h_kv, d, cap = len(SCALES), 512, 128, 4
    bits = torch.arange(0, 65536, dtype=torch.int32).to(torch.int16).view(torch.bfloat16)
    x = bits.view(1, 1, h_kv, d).expand(n_layers, 1, h_kv, d).contiguous()
    scale = torch.tensor(SCALES, dtype=torch.float32).view(-1, 1).expand(n_layers, h_kv).contiguous()
    kc = torch.full((n_layers, 1, h_kv, cap, d), 0xAB, dtype=torch.uint8, device=cuda_device)
    vc = torch.full_like(kc, 0xCD)
    pos = torch.tensor([2], dtype=torch.int32, device=cuda_device)
    status = torch.zeros(1, dtype=torch.int32, device=cuda_device)
    pkg.kv_quant_append(x.to(cuda_device), x.to(cuda_device), kc, vc, scale.to(cuda_device), scale.to(cuda_device),
                        pos, h_q=h_kv, advance=True, status=status)
    torch.cuda.synchronize()
    want = oracle.quantize_e4m3(x, scale.view(n_layers, 1, h_kv, 1))
    nan_in = torch.isnan(x.float())
    for name, cache, sentinel in (("k", kc, 0xAB), ("v", vc, 0xCD)):
        got = cache[:, :, :, 2].cpu()
        assert torch.equal(got[~nan_in], want[~nan_in]), f"{name}: {(got != want)[~nan_in].sum().item()} bytes differ"
        assert bool(((got[nan_in] & 0x7F) == 0x7F).all())          # NaN in -> NaN byte
        assert torch.equal(got[nan_in] >> 7, (x.view(torch.int16)[nan_in] < 0).to(torch.uint8))   # sign kept
        others = cache[:, :, :, [0, 1, 3]].cpu()
        assert bool((others == sentinel).all()), "append wrote outside its slot"
    assert pos.item() == 3 and status.item() == 0


def test_append_matches_oracle_on_benchmark_distribution(pkg, oracle, cuda_device):
    """N(0,1) K/V, per-(layer, head) absmax/448 scales, ragged positions, two appends in a row."""
    n_layers, batch, h_q, h_kv, d, cap = 3, 4, 40, 8, 128, 64
    g = torch.Generator().manual_seed(0)
    hist = torch.randn(n_layers, batch, h_kv, 32, d, generator=g).to(torch.bfloat16)
    ks = hist.float().abs().amax(dim=(1, 3, 4)) / 448
    vs = ks * 1.25
    kc = torch.zeros(n_layers, batch, h_kv, cap, d, dtype=torch.uint8, device=cuda_device)
    vc = torch.zeros_like(kc)
    pos0 = [0, 5, 31, 62]
    pos = torch.tensor(pos0, dtype=torch.int32, device=cuda_device)
    status = torch.zeros(1, dtype=torch.int32, device=cuda_device)
    for step in range(2):
        k_new = (torch.randn(n_layers, batch, h_kv, d, generator=g) * 1.5).to(torch.bfloat16)  # some values saturate
        v_new = torch.randn(n_layers, batch, h_kv, d, generator=g).to(torch.bfloat16)
        pkg.kv_quant_append(k_new.to(cuda_device), v_new.to(cuda_device), kc, vc, ks.to(cuda_device), vs.to(cuda_device),
                            pos, h_q=h_q, advance=True, status=status)
        torch.cuda.synchronize()
        wk = oracle.quantize_e4m3(k_new, ks.view(n_layers, 1, h_kv, 1))
        wv = oracle.quantize_e4m3(v_new, vs.view(n_layers, 1, h_kv, 1))
        for b in range(batch):
            assert torch.equal(kc[:, b, :, pos0[b] + step].cpu(), wk[:, b])
            assert torch.equal(vc[:, b, :, pos0[b] + step].cpu(), wv[:, b])
    assert pos.cpu().tolist() == [p + 2 for p in pos0] and status.item() == 0


def test_append_at_capacity_sets_status_and_writes_nothing(pkg, cuda_device):
    n_layers, batch, h_kv, d, cap = 2, 2, 8, 128, 16
    kc = torch.full((n_layers, batch, h_kv, cap, d), 0x11, dtype=torch.uint8, device=cuda_device)
    vc = kc.clone()
    sc = torch.ones(n_layers, h_kv, device=cuda_device)
    pos = torch.tensor([cap, 3], dtype=torch.int32, device=cuda_device)
    status = torch.zeros(1, dtype=torch.int32, device=cuda_device)
    x = torch.ones(n_layers, batch, h_kv, d, dtype=torch.bfloat16, device=cuda_device)
    pkg.kv_quant_append(x, x, kc, vc, sc, sc, pos, h_q=40, advance=True, status=status)
    torch.cuda.synchronize()
    assert status.item() & pkg._lib.STATUS_POS_AT_CAPACITY
    assert bool((kc[:, 0] == 0x11).all()) and bool((vc[:, 0] == 0x11).all())   # full sequence untouched
    assert bool((kc[:, 1, :, 3] == 0x38).all())                               # 1.0 -> 0x38
    assert pos.cpu().tolist() == [cap, 4]                                     # full sequence not advanced


def test_per_token_scale_mode(pkg, oracle, cuda_device):
    """The reference's own granularity: scale per (token, head) computed by the kernel."""
    n_layers, batch, h_q, h_kv, d, cap = 2, 2, 24, 4, 256, 8
    g = torch.Generator().manual_seed(3)
    k_new = torch.randn(n_layers, batch, h_kv, d, generator=g).to(torch.bfloat16)
    v_new = torch.randn(n_layers, batch, h_kv, d, generator=g).to(torch.bfloat16)
    k_new[0, 0, 1] = 0   # an all-zero head row: scale 0, bytes 0
    kc = torch.full((n_layers, batch, h_kv, cap, d), 0x55, dtype=torch.uint8, device=cuda_device)
    vc = kc.clone()
    ks = torch.zeros(n_layers, batch, cap, h_kv, device=cuda_device)
    vs = torch.zeros_like(ks)
    pos = torch.tensor([1, 6], dtype=torch.int32, device=cuda_device)
    status = torch.zeros(1, dtype=torch.int32, device=cuda_device)
    pkg.kv_quant_append(k_new.to(cuda_device), v_new.to(cuda_device), kc, vc, ks, vs, pos, h_q=h_q, advance=False,
                        status=status)
    torch.cuda.synchronize()
    for layer in range(n_layers):
        for b, p in enumerate([1, 6]):
            for src, cache, sc in ((k_new, kc, ks), (v_new, vc, vs)):
                x = src[layer, b].view(1, h_kv, 1, d)
                s = oracle.token_scales(x)                       # [1,1,h_kv]
                assert torch.equal(sc[layer, b, p].cpu(), s.view(h_kv))
                assert torch.equal(cache[layer, b, :, p].cpu(), oracle.quantize_per_token(x, s).view(h_kv, d))
    assert pos.cpu().tolist() == [1, 6]


def test_bulk_append_dequant_and_calibration(pkg, oracle, cuda_device):
    """Prefill-side path: calibrate scales on the device, append 128 tokens, read them back dequantised."""
    n_layers, batch, h_q, h_kv, d, cap, n_tok = 2, 2, 40, 8, 128, 256, 128
    g = torch.Generator().manual_seed(7)
    k = torch.randn(n_layers, batch, h_kv, n_tok, d, generator=g).to(torch.bfloat16)
    v = torch.randn(n_layers, batch, h_kv, n_tok, d, generator=g).to(torch.bfloat16)
    cache = pkg.FP8StaticCache(n_layers, batch, h_q, h_kv, d, cap, device=cuda_device)
    cache.prefill(k.to(cuda_device), v.to(cuda_device), calibrate=True)
    torch.cuda.synchronize()
    ks = k.float().abs().amax(dim=(1, 3, 4)) / 448
    vs = v.float().abs().amax(dim=(1, 3, 4)) / 448
    assert torch.equal(cache.k_scale.cpu(), ks) and torch.equal(cache.v_scale.cpu(), vs)
    wk = oracle.quantize_e4m3(k, ks.view(n_layers, 1, h_kv, 1, 1))
    assert torch.equal(cache.k_cache[:, :, :, :n_tok].cpu(), wk)
    assert bool((cache.k_cache[:, :, :, n_tok:] == 0).all())
    assert cache.seq_pos.cpu().tolist() == [n_tok] * batch
    deq = pkg.dequant_prefix(cache.k_cache, cache.k_scale, n_tok, h_q=h_q)
    assert torch.equal(deq.cpu(), oracle.dequantize(wk, ks.view(n_layers, 1, h_kv, 1, 1)))
    with pytest.raises(ValueError):
        cache.require_capacity(cap)   # host-side capacity guard, before any launch
