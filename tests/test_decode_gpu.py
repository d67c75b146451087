"""GPU parity of the decode attention (both kernel variants) against the oracle and the
reference's golden outputs.  Tolerance: max abs err <= 2e-2 and cosine >= 0.9999 against the
reference's padded torch attention on the same seeded inputs."""
import numpy as np
import pytest
import torch

from helpers import TOL_COSINE, TOL_MAX_ABS, assert_parity, build_case, run_decode

pytestmark = pytest.mark.gpu
VARIANTS = ["simt", "mma", "umma2"]


def unsupported(pkg, variant, h_q, h_kv):
    """Every kernel serves query groups of up to 8 heads (the library's limit); kept as the one place
    where a variant's shape restrictions would be written down for the tests below."""
    return h_q // h_kv > 8


def _golden_case(oracle, m, fill_byte=0):
    q, k, v = oracle.make_inputs(m["seed"], m["h_q"], m["h_kv"], m["d"], m["length"])
    sk, sv = oracle.head_scales(k), oracle.head_scales(v)
    cap, L = m["capacity"], m["length"]
    kc = torch.full((1, 1, m["h_kv"], cap, m["d"]), fill_byte, dtype=torch.uint8)
    vc = torch.full_like(kc, fill_byte)
    kc[0, :, :, :L] = oracle.quantize_per_head(k, sk)
    vc[0, :, :, :L] = oracle.quantize_per_head(v, sv)
    return {"q": q.view(1, 1, m["h_q"], m["d"]).contiguous(), "k_cache": kc, "v_cache": vc,
            "k_scale": sk.view(1, -1), "v_scale": sv.view(1, -1), "lens": [L], "capacity": cap}


@pytest.mark.parametrize("variant", VARIANTS)
def test_golden_parity_with_the_reference(pkg, oracle, golden, cuda_device, variant):
    """Every fixture made by the reference's own eager_attention / fp64_reference."""
    data, meta = golden
    for name, m in meta.items():
        if unsupported(pkg, variant, m["h_q"], m["h_kv"]):
            continue
        case = _golden_case(oracle, m)
        out, status = run_decode(pkg, case, cuda_device, variant)
        assert status == 0
        ref = torch.from_numpy(data[f"{name}/out_bf16_bits"].view(np.int16)).view(torch.bfloat16).view(1, 1, m["h_q"], m["d"])
        assert_parity(oracle, out, ref, f"{variant}:{name}")
        # the reference's own acceptance rule: no farther from fp64 than 2x the baseline is
        f64 = torch.from_numpy(data[f"{name}/out_fp64_as_f32"]).view(1, 1, m["h_q"], m["d"]).double()
        d_out = (out.double() - f64).norm().item()
        d_ref = (ref.double() - f64).norm().item()
        assert d_out <= 2.0 * d_ref + 1e-3, (variant, name, d_out, d_ref)


@pytest.mark.parametrize("variant", VARIANTS)
def test_length_sweep_against_oracle(pkg, oracle, cuda_device, variant):
    """Boundary lengths of the reference's check list, two layers each."""
    for L in (1, 2, 15, 16, 17, 63, 64, 65, 127, 128, 129, 300, 513, 1023, 1024):
        case = build_case(oracle, 2, 1, 40, 8, 128, [L], 1024, seed=100 + L)
        out, status = run_decode(pkg, case, cuda_device, variant)
        ref = oracle.decode_step_reference(case["q"], case["k_cache"], case["v_cache"], case["k_scale"],
                                           case["v_scale"], case["lens"], 1024)
        assert status == 0
        assert_parity(oracle, out, ref, f"{variant}:L={L}")


@pytest.mark.parametrize("variant", VARIANTS)
def test_one_short_of_and_exactly_a_full_8192_cache(pkg, oracle, cuda_device, variant):
    """Depth 8191 and 8192 in capacity 8192 (the reference's check list names 8191): the last tile is
    one token short of full, then full; NaN bytes in the one free slot."""
    for L in (8191, 8192):
        case = build_case(oracle, 1, 1, 40, 8, 128, [L], 8192, seed=400 + L, fill_byte=0xFF)
        out, status = run_decode(pkg, case, cuda_device, variant)
        clean_k, clean_v = case["k_cache"].clone(), case["v_cache"].clone()
        clean_k[:, :, :, L:] = 0
        clean_v[:, :, :, L:] = 0
        ref = oracle.decode_step_reference(case["q"], clean_k, clean_v, case["k_scale"], case["v_scale"], [L], 8192)
        assert status == 0
        assert_parity(oracle, out, ref, f"{variant}:L={L}")


@pytest.mark.parametrize("variant", VARIANTS)
def test_single_token_is_exactly_the_value_row(pkg, oracle, cuda_device, variant):
    """L=1: softmax weight is 1, so out == bf16(dequantised V row) for every query head."""
    case = build_case(oracle, 1, 1, 40, 8, 128, [1], 64, seed=9)
    out, _ = run_decode(pkg, case, cuda_device, variant)
    v = case["v_cache"][0, 0, :, 0].view(torch.float8_e4m3fn).float() * case["v_scale"][0].view(-1, 1)
    assert torch.equal(out[0, 0], v.to(torch.bfloat16).repeat_interleave(5, dim=0))


@pytest.mark.parametrize("variant", VARIANTS)
@pytest.mark.parametrize("fill", [0x7F, 0xFF, 0x7E, 0x3C])
def test_fill_isolation(pkg, oracle, cuda_device, variant, fill):
    """Slots beyond the valid length may hold anything (NaN patterns, max finite, ordinary
    values): the result is bit-identical to the zero-filled cache (scripts/m3_check.py:313-326)."""
    for L, cap in ((300, 1024), (513, 1024), (65, 128), (1, 64)):
        base = build_case(oracle, 2, 1, 40, 8, 128, [L], cap, seed=5, fill_byte=0)
        dirty = build_case(oracle, 2, 1, 40, 8, 128, [L], cap, seed=5, fill_byte=fill)
        a, _ = run_decode(pkg, base, cuda_device, variant)
        b, _ = run_decode(pkg, dirty, cuda_device, variant)
        assert torch.equal(a.view(torch.int16), b.view(torch.int16)), (variant, hex(fill), L)
        assert bool(torch.isfinite(b.float()).all())


@pytest.mark.parametrize("variant", VARIANTS)
def test_repeat_and_reset_are_bitwise_stable(pkg, oracle, cuda_device, variant):
    case = build_case(oracle, 4, 2, 40, 8, 128, [700, 333], 1024, seed=21)
    dev = {k: (v.to(cuda_device) if isinstance(v, torch.Tensor) else v) for k, v in case.items()}
    shape = pkg.make_shape(40, dev["k_cache"], dev["v_cache"], dev["k_scale"])
    ws = pkg.Workspace(shape, cuda_device, variant=variant)
    seq = torch.tensor(case["lens"], dtype=torch.int32, device=cuda_device)
    outs = []
    for i in range(4):
        if i == 2:   # poison half of the partial area: what an earlier launch left there must never be taken for a partial
            ws.buf[: ws.nbytes // 2].fill_(0x7F)
        if i == 3:
            ws.init()
        outs.append(pkg.decode_attention(dev["q"], dev["k_cache"], dev["v_cache"], dev["k_scale"], dev["v_scale"], seq,
                                         workspace=ws).clone())
    torch.cuda.synchronize()
    for o in outs[1:]:
        assert torch.equal(o.view(torch.int16), outs[0].view(torch.int16))
    assert ws.read_status() == 0


def test_split_counts_agree(pkg, oracle, cuda_device):
    """Any split / CTA count gives the oracle's answer; all of them agree within tolerance."""
    case = build_case(oracle, 2, 1, 40, 8, 128, [1000], 1024, seed=33)
    ref = oracle.decode_step_reference(case["q"], case["k_cache"], case["v_cache"], case["k_scale"], case["v_scale"],
                                       case["lens"], 1024)
    outs = []
    for variant, counts in (("simt", [1, 2, 3, 4, 7, 8, 16]), ("mma", [1, 2, 3, 16, 37, 148, 296, 500, 2000]),
                            ("umma2", [1, 5, 148, 296, 1000])):
        for n in counts:
            out, status = run_decode(pkg, case, cuda_device, variant, num_splits=n)
            assert status == 0
            assert_parity(oracle, out, ref, f"{variant}:{n}")
            outs.append(out)
    for o in outs[1:]:
        assert (o.float() - outs[0].float()).abs().max().item() <= 2.0 ** -7


@pytest.mark.parametrize("variant", ["mma", "umma2"])
@pytest.mark.parametrize("h_q,h_kv,d", [(5, 1, 128), (8, 1, 128), (6, 1, 256), (10, 2, 128)])
def test_one_pair_spread_over_the_whole_grid(pkg, oracle, cuda_device, variant, h_q, h_kv, d):
    """A single layer with one or two KV heads and a long cache: every CTA of the persistent grid owns a piece of the
    same (layer, kv head) pair, so the owner of the last piece collects dozens of partials (several rounds of the
    split-K hand-over), for every accumulator width the kernels have (groups of 5, 6 and 8 heads; head_dim 128 and
    256); twice on one workspace, plus a forced grid larger than the device holds at once."""
    L, cap = 8000, 8192
    case = build_case(oracle, 1, 1, h_q, h_kv, d, [L], cap, seed=77)
    ref = oracle.decode_step_reference(case["q"], case["k_cache"], case["v_cache"], case["k_scale"], case["v_scale"],
                                       case["lens"], cap)
    dev = {k: (v.to(cuda_device) if isinstance(v, torch.Tensor) else v) for k, v in case.items()}
    shape = pkg.make_shape(h_q, dev["k_cache"], dev["v_cache"], dev["k_scale"])
    seq = torch.tensor([L], dtype=torch.int32, device=cuda_device)
    for n in (0, 1000):
        ws = pkg.Workspace(shape, cuda_device, variant=variant, num_splits=n)
        outs = [pkg.decode_attention(dev["q"], dev["k_cache"], dev["v_cache"], dev["k_scale"], dev["v_scale"], seq,
                                     workspace=ws).clone() for _ in range(2)]
        torch.cuda.synchronize()
        assert ws.read_status() == 0
        assert_parity(oracle, outs[0].cpu(), ref, f"{variant} {h_q}/{h_kv}/{d} ctas {ws.num_splits}")
        assert torch.equal(outs[0].view(torch.int16), outs[1].view(torch.int16))
        assert int(ws.buf.max()) == 0, "a launch leaves its workspace zeroed"


@pytest.mark.parametrize("variant", VARIANTS)
def test_reference_model_shape(pkg, oracle, cuda_device, variant):
    """The reference's own head shape: 24 q / 4 kv heads (group 6), head_dim 256."""
    case = build_case(oracle, 2, 1, 24, 4, 256, [513], 1024, seed=41)
    if unsupported(pkg, variant, 24, 4):
        with pytest.raises(pkg.B200AttnError):
            run_decode(pkg, case, cuda_device, variant)
        case = build_case(oracle, 2, 1, 20, 4, 256, [513], 1024, seed=41)   # group 5, same head_dim
    out, status = run_decode(pkg, case, cuda_device, variant)
    ref = oracle.decode_step_reference(case["q"], case["k_cache"], case["v_cache"], case["k_scale"], case["v_scale"],
                                       case["lens"], 1024)
    assert status == 0
    assert_parity(oracle, out, ref, variant)


@pytest.mark.parametrize("variant", VARIANTS)
@pytest.mark.parametrize("h_q,h_kv", [(8, 8), (16, 8), (64, 8), (3, 1)])
def test_other_group_sizes(pkg, oracle, cuda_device, variant, h_q, h_kv):
    case = build_case(oracle, 1, 2, h_q, h_kv, 128, [200, 77], 256, seed=51)
    if unsupported(pkg, variant, h_q, h_kv):
        with pytest.raises(pkg.B200AttnError):
            run_decode(pkg, case, cuda_device, variant)
        return
    out, _ = run_decode(pkg, case, cuda_device, variant)
    ref = oracle.decode_step_reference(case["q"], case["k_cache"], case["v_cache"], case["k_scale"], case["v_scale"],
                                       case["lens"], 256)
    assert_parity(oracle, out, ref, f"{variant}:{h_q}/{h_kv}")


@pytest.mark.parametrize("variant", VARIANTS)
def test_ragged_batch_with_empty_and_full_sequences(pkg, oracle, cuda_device, variant):
    lens = [0, 1, 512, 64, 300, 0, 129]
    case = build_case(oracle, 3, len(lens), 40, 8, 128, lens, 512, seed=61, fill_byte=0x7F)
    out, status = run_decode(pkg, case, cuda_device, variant)
    ref = oracle.decode_step_reference(case["q"], case["k_cache"], case["v_cache"], case["k_scale"], case["v_scale"],
                                       lens, 512)
    assert status == 0
    assert_parity(oracle, out, ref, variant)
    assert bool((out[:, 0] == 0).all()) and bool((out[:, 5] == 0).all())   # empty sequences -> zeros


@pytest.mark.parametrize("variant", ["mma", "umma2"])
def test_batched_ragged_decode_steps_bs16(pkg, oracle, cuda_device, variant):
    """The batched configuration in miniature: bs=16 ragged depths (seeded), 8 layers, two decode
    steps with a fused one-token append per sequence; bytes bit-exact, outputs within tolerance."""
    n_layers, batch, h_q, h_kv, d, cap = 8, 16, 40, 8, 128, 1100
    g = torch.Generator().manual_seed(0)
    depths = torch.randint(64, 1025, (batch,), generator=g).tolist()
    case = build_case(oracle, n_layers, batch, h_q, h_kv, d, depths, cap, seed=300)
    cache = pkg.FP8StaticCache(n_layers, batch, h_q, h_kv, d, cap, device=cuda_device, variant=variant)
    cache.k_cache.copy_(case["k_cache"]); cache.v_cache.copy_(case["v_cache"])
    cache.set_scales(case["k_scale"], case["v_scale"])
    cache.seq_pos.copy_(torch.tensor(depths, dtype=torch.int32))
    cache.host_len = list(depths)
    kc, vc = case["k_cache"].clone(), case["v_cache"].clone()
    for step in range(2):
        q = torch.randn(n_layers, batch, h_q, d, generator=g).to(torch.bfloat16)
        kn = torch.randn(n_layers, batch, h_kv, d, generator=g).to(torch.bfloat16)
        vn = torch.randn(n_layers, batch, h_kv, d, generator=g).to(torch.bfloat16)
        out = cache.step(q.to(cuda_device), kn.to(cuda_device), vn.to(cuda_device))
        torch.cuda.synchronize()
        wk = oracle.quantize_e4m3(kn, case["k_scale"].view(n_layers, 1, h_kv, 1))
        wv = oracle.quantize_e4m3(vn, case["v_scale"].view(n_layers, 1, h_kv, 1))
        for b in range(batch):
            kc[:, b, :, depths[b] + step] = wk[:, b]
            vc[:, b, :, depths[b] + step] = wv[:, b]
        assert torch.equal(cache.k_cache.cpu(), kc) and torch.equal(cache.v_cache.cpu(), vc)
        lens = [x + step + 1 for x in depths]
        ref = oracle.decode_step_reference(q, kc, vc, case["k_scale"], case["v_scale"], lens, cap)
        assert_parity(oracle, out.cpu(), ref, f"{variant}: step {step}")
    assert cache.seq_pos.cpu().tolist() == [x + 2 for x in depths] and cache.workspace.read_status() == 0


@pytest.mark.parametrize("variant", VARIANTS)
def test_large_query_magnitudes(pkg, oracle, cuda_device, variant):
    """Queries far outside f16 range (1e6 and 1e-6 scales per head) still match the oracle."""
    case = build_case(oracle, 1, 1, 40, 8, 128, [257], 512, seed=71)
    scale = torch.ones(40, 1)
    scale[::3] = 3e4
    scale[1::3] = 1e-5
    case["q"] = (case["q"].float() * scale).to(torch.bfloat16)
    out, _ = run_decode(pkg, case, cuda_device, variant)
    ref = oracle.decode_step_reference(case["q"], case["k_cache"], case["v_cache"], case["k_scale"], case["v_scale"],
                                       case["lens"], 512)
    assert bool(torch.isfinite(out.float()).all())
    # huge scores make the softmax one-hot; a flipped argmax between near-ties is legitimate, so
    # compare only heads whose reference is not one-hot-degenerate
    keep = [h for h in range(40) if h % 3 != 0]
    assert_parity(oracle, out[:, :, keep], ref[:, :, keep], variant)


@pytest.mark.parametrize("variant", VARIANTS)
def test_length_beyond_capacity_is_clamped_and_flagged(pkg, oracle, cuda_device, variant):
    case = build_case(oracle, 1, 1, 40, 8, 128, [128], 128, seed=81)
    ok, _ = run_decode(pkg, case, cuda_device, variant)
    case["lens"] = [500]
    out, status = run_decode(pkg, case, cuda_device, variant)
    assert status & pkg._lib.STATUS_LEN_OVER_CAP
    assert torch.equal(out.view(torch.int16), ok.view(torch.int16))


@pytest.mark.parametrize("variant", ["mma", "umma2"])
def test_gated_output_fusion(pkg, oracle, cuda_device, variant):
    """attn_output * sigmoid(gate) with two separate bf16 roundings, fused into the output store."""
    lens = [513, 64]
    case = build_case(oracle, 3, 2, 40, 8, 128, lens, 1024, seed=91)
    g = torch.Generator().manual_seed(5)
    gate = (torch.randn(3, 2, 40, 128, generator=g) * 2).to(torch.bfloat16)
    dev = {k: (v.to(cuda_device) if isinstance(v, torch.Tensor) else v) for k, v in case.items()}
    shape = pkg.make_shape(40, dev["k_cache"], dev["v_cache"], dev["k_scale"])
    ws = pkg.Workspace(shape, cuda_device, variant=variant)
    seq = torch.tensor(lens, dtype=torch.int32, device=cuda_device)
    plain = pkg.decode_attention(dev["q"], dev["k_cache"], dev["v_cache"], dev["k_scale"], dev["v_scale"], seq, workspace=ws).cpu()
    gated = pkg.decode_attention(dev["q"], dev["k_cache"], dev["v_cache"], dev["k_scale"], dev["v_scale"], seq, workspace=ws,
                                 gate=gate.to(cuda_device)).cpu()
    want = plain * torch.sigmoid(gate)          # torch: sigmoid rounds to bf16, the product rounds to bf16
    diff = (gated.float() - want.float()).abs()
    ulp = want.float().abs().clamp_min(2.0 ** -20) * 2.0 ** -7
    assert float((diff > ulp).float().mean()) == 0.0            # never more than one bf16 step apart
    assert float((gated != want).float().mean()) < 1e-3         # and bit-identical but for rare rounding ties
    ref = oracle.decode_step_reference(case["q"], case["k_cache"], case["v_cache"], case["k_scale"], case["v_scale"], lens, 1024)
    assert_parity(oracle, gated, ref * torch.sigmoid(gate), variant)


def test_per_token_scale_mode_decode(pkg, oracle, cuda_device):
    """The reference's frozen scale layout [capacity, kv_heads] per layer (SIMT kernel)."""
    n_layers, h_q, h_kv, d, L, cap = 2, 24, 4, 256, 300, 512
    q = torch.zeros(n_layers, 1, h_q, d, dtype=torch.bfloat16)
    kc = torch.zeros(n_layers, 1, h_kv, cap, d, dtype=torch.uint8)
    vc = torch.zeros_like(kc)
    ks = torch.zeros(n_layers, 1, cap, h_kv)
    vs = torch.zeros_like(ks)
    for layer in range(n_layers):
        qq, k, v = oracle.make_inputs(90 + layer, h_q, h_kv, d, L)
        q[layer, 0] = qq.view(h_q, d)
        sk, sv = oracle.token_scales(k), oracle.token_scales(v)
        ks[layer, :, :L], vs[layer, :, :L] = sk, sv
        kc[layer, :, :, :L] = oracle.quantize_per_token(k, sk)
        vc[layer, :, :, :L] = oracle.quantize_per_token(v, sv)
    case = {"q": q, "k_cache": kc, "v_cache": vc, "k_scale": ks, "v_scale": vs, "lens": [L], "capacity": cap}
    out, status = run_decode(pkg, case, cuda_device, "auto")
    ref = oracle.decode_step_reference(q, kc, vc, ks, vs, [L], cap)
    assert status == 0
    assert_parity(oracle, out, ref, "per-token")


def test_per_token_scales_on_the_tensor_cores(pkg, oracle, cuda_device):
    """The per-token scale layout through the all-tcgen05 kernel (each softmax thread applies its
    token's K and V scales): parity with the oracle on a ragged batch, agreement with the SIMT
    kernel, and the decode step — one launch with the all-tcgen05 kernel, which computes the new rows'
    scales itself, against append kernel + attention + position kernel with the SIMT kernel: cache bytes,
    scales and positions identical, over several steps (lengths cross a tile boundary)."""
    n_layers, batch, h_q, h_kv, d, cap = 2, 3, 40, 8, 128, 640
    lens = [300, 1, 513]
    q = torch.zeros(n_layers, batch, h_q, d, dtype=torch.bfloat16)
    kc = torch.full((n_layers, batch, h_kv, cap, d), 0xFF, dtype=torch.uint8)     # NaN patterns beyond the lengths
    vc = torch.full_like(kc, 0xFF)
    ks = torch.full((n_layers, batch, cap, h_kv), float("nan"))
    vs = torch.full_like(ks, float("nan"))
    for layer in range(n_layers):
        for b, L in enumerate(lens):
            qq, k, v = oracle.make_inputs(300 + 10 * layer + b, h_q, h_kv, d, L)
            q[layer, b] = qq.view(h_q, d)
            sk, sv = oracle.token_scales(k), oracle.token_scales(v)
            ks[layer, b, :L], vs[layer, b, :L] = sk[0], sv[0]
            kc[layer, b, :, :L] = oracle.quantize_per_token(k, sk)[0]
            vc[layer, b, :, :L] = oracle.quantize_per_token(v, sv)[0]
    case = {"q": q, "k_cache": kc, "v_cache": vc, "k_scale": ks, "v_scale": vs, "lens": lens, "capacity": cap}
    ref = oracle.decode_step_reference(q, torch.where(kc == 0xFF, torch.zeros_like(kc), kc), torch.where(vc == 0xFF, torch.zeros_like(vc), vc),
                                       torch.nan_to_num(ks), torch.nan_to_num(vs), lens, cap)
    outs = {}
    for variant in ("simt", "umma2"):
        outs[variant], status = run_decode(pkg, case, cuda_device, variant)
        assert status == 0
        assert not torch.isnan(outs[variant].float()).any(), variant
        assert_parity(oracle, outs[variant], ref, f"per-token {variant}")
    m = oracle.error_metrics(outs["umma2"], outs["simt"])
    assert m["max_abs"] <= 2.0 ** -6 and m["cosine"] >= 0.9999, m
    with pytest.raises(pkg.B200AttnError):        # the mma.sync kernel has no per-token path
        run_decode(pkg, case, cuda_device, "mma")
    # the decode step with per-token scales
    caches = {}
    for variant in ("simt", "umma2"):
        c = pkg.FP8StaticCache(n_layers, batch, h_q, h_kv, d, cap, device=cuda_device, variant=variant, scale_mode="per_token")
        c.k_cache.copy_(torch.where(kc == 0xFF, torch.zeros_like(kc), kc))
        c.v_cache.copy_(torch.where(vc == 0xFF, torch.zeros_like(vc), vc))
        c.k_scale.copy_(torch.nan_to_num(ks))
        c.v_scale.copy_(torch.nan_to_num(vs))
        c.seq_pos.copy_(torch.tensor(lens, dtype=torch.int32))
        caches[variant] = c
    g = torch.Generator().manual_seed(77)
    kn = torch.randn(n_layers, batch, h_kv, d, generator=g).to(torch.bfloat16).to(cuda_device)
    vn = torch.randn(n_layers, batch, h_kv, d, generator=g).to(torch.bfloat16).to(cuda_device)
    a, u = caches["simt"], caches["umma2"]
    for step in range(3):
        kn_s, vn_s = torch.roll(kn, step, dims=-1), torch.roll(vn, step, dims=-1)
        if step == 2:
            kn_s = kn_s.clone()
            kn_s[:, 1, 3] = 0                  # an all-zero key row: scale 0, zero bytes
        step_out = {v: caches[v].step(q.to(cuda_device), kn_s, vn_s, count=False).cpu() for v in caches}
        torch.cuda.synchronize()
        assert torch.equal(a.k_cache, u.k_cache) and torch.equal(a.v_cache, u.v_cache), f"step {step}: cache bytes"
        assert torch.equal(a.k_scale, u.k_scale) and torch.equal(a.v_scale, u.v_scale), f"step {step}: scales"
        assert torch.equal(a.seq_pos, u.seq_pos) and u.seq_pos.cpu().tolist() == [x + step + 1 for x in lens]
        assert a.workspace.read_status() == 0 and u.workspace.read_status() == 0
        want_s = oracle.token_scales(kn_s.cpu().transpose(0, 1).reshape(batch, n_layers * h_kv, 1, d))     # [B, 1, n*h]
        for b, L in enumerate(lens):
            assert torch.equal(u.k_scale[:, b, L + step].cpu().flatten(), want_s[b, 0]), f"step {step}: scales of sequence {b} vs the oracle"
        ref2 = oracle.decode_step_reference(q, u.k_cache.cpu(), u.v_cache.cpu(), u.k_scale.cpu(), u.v_scale.cpu(),
                                            [x + step + 1 for x in lens], cap)
        assert_parity(oracle, step_out["umma2"], ref2, f"per-token step {step}")
    assert float(u.k_scale[0, 1, lens[1] + 2, 3]) == 0.0 and int(u.k_cache[0, 1, 3, lens[1] + 2].max()) == 0


@pytest.mark.parametrize("variant", VARIANTS)
def test_decode_steps_and_cuda_graph_replay(pkg, oracle, cuda_device, variant):
    """Append + attend + advance, eagerly and under CUDA-graph replay: the graph advances the
    device-side position by itself, replays are bit-identical to eager steps, capture itself
    does not advance the cache (runner/model/graph_runner.py:127-198 in the reference)."""
    n_layers, batch, h_q, h_kv, d, cap, depth, steps = 4, 2, 40, 8, 128, 256, 100, 6
    g = torch.Generator().manual_seed(11)
    k0 = torch.randn(n_layers, batch, h_kv, depth, d, generator=g).to(torch.bfloat16)
    v0 = torch.randn(n_layers, batch, h_kv, depth, d, generator=g).to(torch.bfloat16)
    qs = torch.randn(steps, n_layers, batch, h_q, d, generator=g).to(torch.bfloat16).to(cuda_device)
    kn = torch.randn(steps, n_layers, batch, h_kv, d, generator=g).to(torch.bfloat16).to(cuda_device)
    vn = torch.randn(steps, n_layers, batch, h_kv, d, generator=g).to(torch.bfloat16).to(cuda_device)

    def fresh():
        c = pkg.FP8StaticCache(n_layers, batch, h_q, h_kv, d, cap, device=cuda_device, variant=variant)
        c.prefill(k0.to(cuda_device), v0.to(cuda_device), calibrate=True)
        return c

    eager = fresh()
    eager_out = [eager.step(qs[i], kn[i], vn[i]).clone() for i in range(steps)]
    torch.cuda.synchronize()
    assert eager.seq_pos.cpu().tolist() == [depth + steps] * batch

    # oracle for the last step: the cache now holds depth+steps tokens
    ref = oracle.decode_step_reference(qs[-1].cpu(), eager.k_cache.cpu(), eager.v_cache.cpu(), eager.k_scale.cpu(),
                                       eager.v_scale.cpu(), [depth + steps] * batch, cap)
    assert_parity(oracle, eager_out[-1].cpu(), ref, f"{variant}:eager last step")
    # appended bytes are bit-exact
    want = oracle.quantize_e4m3(kn[-1].cpu(), eager.k_scale.cpu().view(n_layers, 1, h_kv, 1))
    assert torch.equal(eager.k_cache[:, :, :, depth + steps - 1].cpu(), want)

    graphed = fresh()
    q_buf, k_buf, v_buf = qs[0].clone(), kn[0].clone(), vn[0].clone()
    out_buf = torch.empty_like(q_buf)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):   # warm-up on a side stream advances the cache: undo it afterwards
        graphed.step(q_buf, k_buf, v_buf, out=out_buf, count=False)
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    assert graphed.seq_pos.cpu().tolist() == [depth + 1] * batch
    graphed.seq_pos.fill_(depth)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        graphed.step(q_buf, k_buf, v_buf, out=out_buf, count=False)
    torch.cuda.synchronize()
    assert graphed.seq_pos.cpu().tolist() == [depth] * batch      # capture records, does not run
    for i in range(steps):
        q_buf.copy_(qs[i]); k_buf.copy_(kn[i]); v_buf.copy_(vn[i])
        graph.replay()
        torch.cuda.synchronize()
        assert torch.equal(out_buf.view(torch.int16), eager_out[i].view(torch.int16)), f"replay {i}"
    assert graphed.seq_pos.cpu().tolist() == [depth + steps] * batch
    assert torch.equal(graphed.k_cache, eager.k_cache) and torch.equal(graphed.v_cache, eager.v_cache)
    assert graphed.workspace.read_status() == 0

    # reset keeps addresses and reproduces the run (static_cache.py:161-164)
    ptr = graphed.k_cache.data_ptr()
    graphed.reset()
    graphed.prefill(k0.to(cuda_device), v0.to(cuda_device), calibrate=True)
    q_buf.copy_(qs[0]); k_buf.copy_(kn[0]); v_buf.copy_(vn[0])
    graph.replay()
    torch.cuda.synchronize()
    assert graphed.k_cache.data_ptr() == ptr
    assert torch.equal(out_buf.view(torch.int16), eager_out[0].view(torch.int16))


def test_full_size_properties(pkg, oracle, cuda_device):
    """64 layers x depth 8192 (the headline configuration): size-independent properties.
    (a) both kernel variants agree; (b) a value cache that is constant per head comes back as
    that constant whatever the keys are (softmax weights sum to one); (c) two layers are
    spot-checked against the oracle."""
    n_layers, h_q, h_kv, d, cap = 64, 40, 8, 128, 8192
    g = torch.Generator(device=cuda_device).manual_seed(0)

    def rand_bytes():
        x = torch.randn(n_layers, 1, h_kv, cap, d, generator=g, device=cuda_device, dtype=torch.bfloat16)
        return (x.float() / (4.5 / 448)).clamp(-448, 448).to(torch.float8_e4m3fn).view(torch.uint8)

    kc, vc = rand_bytes(), rand_bytes()
    ks = torch.full((n_layers, h_kv), 4.5 / 448, device=cuda_device)
    vs = ks.clone()
    q = torch.randn(n_layers, 1, h_q, d, generator=g, device=cuda_device, dtype=torch.bfloat16)
    seq = torch.tensor([cap], dtype=torch.int32, device=cuda_device)
    shape = pkg.make_shape(h_q, kc, vc, ks)
    outs = {}
    for variant in VARIANTS:
        ws = pkg.Workspace(shape, cuda_device, variant=variant)
        outs[variant] = pkg.decode_attention(q, kc, vc, ks, vs, seq, workspace=ws)
        torch.cuda.synchronize()
        assert ws.read_status() == 0
    for variant in ("mma", "umma2"):
        m = oracle.error_metrics(outs[variant].cpu(), outs["simt"].cpu())
        assert m["max_abs"] <= 2.0 ** -7 and m["cosine"] >= 0.99999, (variant, m)
    for layer in (0, 63):
        ref = oracle.decode_step_reference(q[layer:layer + 1].cpu(), kc[layer:layer + 1].cpu(), vc[layer:layer + 1].cpu(),
                                           ks[layer:layer + 1].cpu(), vs[layer:layer + 1].cpu(), [cap], cap)
        for variant in ("mma", "umma2"):      # umma2 is what the default kernel choice runs at this size
            assert_parity(oracle, outs[variant][layer:layer + 1].cpu(), ref, f"{variant} layer {layer}")
    const = torch.arange(h_kv, device=cuda_device).view(1, 1, h_kv, 1, 1).expand_as(vc)
    vconst = (0x30 + const).to(torch.uint8).contiguous()            # e4m3 0x30.. = 0.5, 0.5625, ...
    want = (vconst[0, 0, :, 0, 0].cpu().view(torch.float8_e4m3fn).float() * (4.5 / 448)).repeat_interleave(5)
    for variant in ("mma", "umma2"):
        ws = pkg.Workspace(shape, cuda_device, variant=variant)
        out = pkg.decode_attention(q, kc, vconst, ks, vs, seq, workspace=ws).cpu().float()
        assert (out - want.view(1, 1, h_q, 1)).abs().max().item() <= 2.0 ** -8 * want.max().item(), variant


def _random_cache_bytes(shape, gen, device, sigma_over_max=4.5):
    """e4m3 bytes of N(0,1) values quantised with scale sigma_over_max/448, made on the device."""
    x = torch.randn(shape, generator=gen, device=device, dtype=torch.bfloat16)
    return (x.float() / (sigma_over_max / 448)).clamp(-448, 448).to(torch.float8_e4m3fn).view(torch.uint8)


def test_long_context_size_against_the_oracle(pkg, oracle, cuda_device):
    """The long-context configuration at its own size: 64 layers, depth 32768 in capacity 33024, the
    kernel the default choice picks; layers 0 and 63 against the oracle, then one fused decode step
    (depth 32769) whose appended bytes must be the oracle's, layer 63 against the oracle again."""
    n_layers, h_q, h_kv, d, depth, cap = 64, 40, 8, 128, 32768, 33024
    g = torch.Generator(device=cuda_device).manual_seed(3)
    cache = pkg.FP8StaticCache(n_layers, 1, h_q, h_kv, d, cap, device=cuda_device)
    assert cache.workspace.resolved == "umma2"
    for layer in range(n_layers):      # layer by layer: the bf16 staging stays small
        cache.k_cache[layer, :, :, :depth] = _random_cache_bytes((1, h_kv, depth, d), g, cuda_device)
        cache.v_cache[layer, :, :, :depth] = _random_cache_bytes((1, h_kv, depth, d), g, cuda_device)
    cache.k_cache[:, :, :, depth:] = 0xFF          # NaN patterns in the free slots
    cache.v_cache[:, :, :, depth:] = 0xFF
    cache.k_scale.fill_(4.5 / 448)
    cache.v_scale.fill_(4.5 / 448)
    cache.seq_pos.fill_(depth)
    cache.host_len = [depth]
    q = torch.randn(n_layers, 1, h_q, d, generator=g, device=cuda_device, dtype=torch.bfloat16)
    kn = torch.randn(n_layers, 1, h_kv, d, generator=g, device=cuda_device, dtype=torch.bfloat16)
    vn = torch.randn(n_layers, 1, h_kv, d, generator=g, device=cuda_device, dtype=torch.bfloat16)
    out = cache.attend(q)
    torch.cuda.synchronize()
    assert cache.workspace.read_status() == 0
    ks, vs = cache.k_scale.cpu(), cache.v_scale.cpu()

    def check(result, layer, length, what):
        kb, vb = cache.k_cache[layer:layer + 1].cpu(), cache.v_cache[layer:layer + 1].cpu()
        kb[:, :, :, length:] = 0
        vb[:, :, :, length:] = 0
        ref = oracle.decode_step_reference(q[layer:layer + 1].cpu(), kb, vb, ks[layer:layer + 1], vs[layer:layer + 1], [length], cap)
        assert_parity(oracle, result[layer:layer + 1].cpu(), ref, what)

    for layer in (0, 63):
        check(out, layer, depth, f"depth {depth} layer {layer}")
    out2 = cache.step(q, kn, vn)
    torch.cuda.synchronize()
    assert cache.workspace.read_status() == 0 and cache.seq_pos.cpu().tolist() == [depth + 1]
    want_k = oracle.quantize_e4m3(kn.cpu(), ks.view(n_layers, 1, h_kv, 1))
    want_v = oracle.quantize_e4m3(vn.cpu(), vs.view(n_layers, 1, h_kv, 1))
    assert torch.equal(cache.k_cache[:, :, :, depth].cpu(), want_k) and torch.equal(cache.v_cache[:, :, :, depth].cpu(), want_v)
    check(out2, 63, depth + 1, f"fused step at depth {depth + 1} layer 63")


def test_batched_ragged_size_against_the_oracle(pkg, oracle, cuda_device):
    """The batched configuration at its own depths: bs = 16, depths randint(1024, 16385) with seed 0,
    capacity 16640 (2.1 M token rows per layer), 4 layers, the default kernel choice.  One fused decode
    step: every sequence of two layers against the oracle, appended bytes bit-exact for all layers."""
    n_layers, batch, h_q, h_kv, d, cap = 4, 16, 40, 8, 128, 16640
    depths = torch.randint(1024, 16384 + 1, (batch,), generator=torch.Generator().manual_seed(0)).tolist()
    g = torch.Generator(device=cuda_device).manual_seed(4)
    cache = pkg.FP8StaticCache(n_layers, batch, h_q, h_kv, d, cap, device=cuda_device)
    assert cache.workspace.resolved == "umma2"
    cache.k_cache.fill_(0xFF)                     # NaN patterns beyond every sequence's depth
    cache.v_cache.fill_(0xFF)
    for layer in range(n_layers):
        for b, L in enumerate(depths):
            cache.k_cache[layer, b, :, :L] = _random_cache_bytes((h_kv, L, d), g, cuda_device)
            cache.v_cache[layer, b, :, :L] = _random_cache_bytes((h_kv, L, d), g, cuda_device)
    cache.k_scale.fill_(4.5 / 448)
    cache.v_scale.fill_(4.5 / 448)
    cache.seq_pos.copy_(torch.tensor(depths, dtype=torch.int32))
    cache.host_len = list(depths)
    q = torch.randn(n_layers, batch, h_q, d, generator=g, device=cuda_device, dtype=torch.bfloat16)
    kn = torch.randn(n_layers, batch, h_kv, d, generator=g, device=cuda_device, dtype=torch.bfloat16)
    vn = torch.randn(n_layers, batch, h_kv, d, generator=g, device=cuda_device, dtype=torch.bfloat16)
    out = cache.step(q, kn, vn)
    torch.cuda.synchronize()
    assert cache.workspace.read_status() == 0
    assert cache.seq_pos.cpu().tolist() == [x + 1 for x in depths]
    ks, vs = cache.k_scale.cpu(), cache.v_scale.cpu()
    want_k = oracle.quantize_e4m3(kn.cpu(), ks.view(n_layers, 1, h_kv, 1))
    want_v = oracle.quantize_e4m3(vn.cpu(), vs.view(n_layers, 1, h_kv, 1))
    for b, L in enumerate(depths):
        assert torch.equal(cache.k_cache[:, b, :, L].cpu(), want_k[:, b]), f"appended K bytes of sequence {b}"
        assert torch.equal(cache.v_cache[:, b, :, L].cpu(), want_v[:, b]), f"appended V bytes of sequence {b}"
    for layer in (0, n_layers - 1):
        kb, vb = cache.k_cache[layer:layer + 1].cpu(), cache.v_cache[layer:layer + 1].cpu()
        for b, L in enumerate(depths):
            kb[:, b, :, L + 1:] = 0
            vb[:, b, :, L + 1:] = 0
        ref = oracle.decode_step_reference(q[layer:layer + 1].cpu(), kb, vb, ks[layer:layer + 1], vs[layer:layer + 1],
                                           [x + 1 for x in depths], cap)
        for b in range(batch):
            assert_parity(oracle, out[layer:layer + 1, b:b + 1].cpu(), ref[:, b:b + 1], f"layer {layer} sequence {b} depth {depths[b] + 1}")


def test_all_zero_head_stays_finite(pkg, oracle, cuda_device):
    """A KV head that is zero everywhere: calibration gives it scale 1 (not 0), its appended bytes are
    0, the attention output of its query heads is exactly 0 and nothing turns into NaN; a zero scale
    handed in by the caller gives zero bytes too, in the append kernel and in the fused step."""
    n_layers, h_q, h_kv, d, cap, depth = 2, 40, 8, 128, 256, 130
    g = torch.Generator().manual_seed(12)
    k0 = torch.randn(n_layers, 1, h_kv, depth, d, generator=g).to(torch.bfloat16)
    v0 = torch.randn(n_layers, 1, h_kv, depth, d, generator=g).to(torch.bfloat16)
    k0[:, :, 3] = 0
    v0[:, :, 3] = 0
    q = torch.randn(n_layers, 1, h_q, d, generator=g).to(torch.bfloat16).to(cuda_device)
    kn = torch.randn(n_layers, 1, h_kv, d, generator=g).to(torch.bfloat16)
    vn = torch.randn(n_layers, 1, h_kv, d, generator=g).to(torch.bfloat16)
    kn[:, :, 3] = 0
    vn[:, :, 3] = 0
    for variant in VARIANTS:
        c = pkg.FP8StaticCache(n_layers, 1, h_q, h_kv, d, cap, device=cuda_device, variant=variant)
        c.prefill(k0.to(cuda_device), v0.to(cuda_device), calibrate=True)
        assert c.k_scale[:, 3].cpu().tolist() == [1.0, 1.0] and c.v_scale[:, 3].cpu().tolist() == [1.0, 1.0]
        assert torch.equal(c.k_scale.cpu()[0], oracle.head_scales(k0[0]))
        out = c.step(q, kn.to(cuda_device), vn.to(cuda_device)).cpu()
        torch.cuda.synchronize()
        assert int(c.k_cache[:, :, 3].max()) == 0 and int(c.v_cache[:, :, 3].max()) == 0
        assert bool(torch.isfinite(out.float()).all()) and bool((out[:, :, 15:20] == 0).all()), variant
        ref = oracle.decode_step_reference(q.cpu(), c.k_cache.cpu(), c.v_cache.cpu(), c.k_scale.cpu(), c.v_scale.cpu(), [depth + 1], cap)
        assert_parity(oracle, out, ref, f"{variant}: zero head")
        # a zero scale from the caller: zero bytes, not NaN bytes
        c.k_scale[:, 5] = 0
        c.step(q, kn.to(cuda_device), vn.to(cuda_device))
        torch.cuda.synchronize()
        assert int(c.k_cache[:, :, 5, depth + 1].max()) == 0, variant


def test_fused_step_equals_separate_launches(pkg, oracle, cuda_device):
    """The stream-K kernels do a decode step in ONE launch (new rows quantised by the CTA that owns
    the pair's last tile, positions advanced by the last CTA to finish).  Against the separate
    append / attention / position launches of the SIMT variant: cache bytes and positions identical, outputs in tolerance;
    ragged lengths that cross a tile boundary, and a sequence already at capacity (flagged, neither
    written nor advanced)."""
    n_layers, batch, h_q, h_kv, d, cap, steps = 3, 4, 40, 8, 128, 256, 4
    lens = [126, 1, 200, cap - 2]          # 126 -> crosses the 128-token tile; cap-2 -> fills up, then refuses
    g = torch.Generator().manual_seed(23)
    k0 = torch.randn(n_layers, batch, h_kv, cap, d, generator=g).to(torch.bfloat16).to(cuda_device)
    v0 = torch.randn(n_layers, batch, h_kv, cap, d, generator=g).to(torch.bfloat16).to(cuda_device)
    qs = torch.randn(steps, n_layers, batch, h_q, d, generator=g).to(torch.bfloat16).to(cuda_device)
    kn = torch.randn(steps, n_layers, batch, h_kv, d, generator=g).to(torch.bfloat16).to(cuda_device)
    vn = torch.randn(steps, n_layers, batch, h_kv, d, generator=g).to(torch.bfloat16).to(cuda_device)
    caches = {}
    for variant in ("simt", "mma", "umma2"):
        c = pkg.FP8StaticCache(n_layers, batch, h_q, h_kv, d, cap, device=cuda_device, variant=variant)
        c.set_scales(pkg.calibrate_scales(k0, cap), pkg.calibrate_scales(v0, cap))
        # ragged prefill: every sequence gets its own prefix; garbage (0xFF = NaN) beyond it
        c.k_cache.fill_(0xFF)
        c.v_cache.fill_(0xFF)
        full = pkg.FP8StaticCache(n_layers, batch, h_q, h_kv, d, cap, device=cuda_device, variant="mma")
        full.set_scales(c.k_scale, c.v_scale)
        full.prefill(k0, v0)
        for b, L in enumerate(lens):
            c.k_cache[:, b, :, :L] = full.k_cache[:, b, :, :L]
            c.v_cache[:, b, :, :L] = full.v_cache[:, b, :, :L]
        c.seq_pos.copy_(torch.tensor(lens, dtype=torch.int32))
        caches[variant] = c
    for i in range(steps):
        outs = {v: caches[v].step(qs[i], kn[i], vn[i], count=False).clone() for v in caches}
        torch.cuda.synchronize()
        a = caches["simt"]
        want_pos = [min(L + i + 1, cap) for L in lens]
        full_already = lens[3] + i >= cap
        ref = oracle.decode_step_reference(qs[i].cpu(), a.k_cache.cpu(), a.v_cache.cpu(), a.k_scale.cpu(), a.v_scale.cpu(),
                                           want_pos, cap)
        for fused in ("mma", "umma2"):
            u = caches[fused]
            assert torch.equal(a.k_cache, u.k_cache) and torch.equal(a.v_cache, u.v_cache), f"step {i} {fused}: cache bytes differ"
            assert a.seq_pos.cpu().tolist() == u.seq_pos.cpu().tolist() == want_pos, f"step {i} {fused}"
            st_a, st_u = int(a.status.cpu().view(-1)[0]), int(u.status.cpu().view(-1)[0])
            assert bool(st_u & pkg._lib.STATUS_POS_AT_CAPACITY) == full_already and bool(st_a & pkg._lib.STATUS_POS_AT_CAPACITY) == full_already
            m = oracle.error_metrics(outs[fused].cpu(), outs["simt"].cpu())
            assert m["max_abs"] <= 2.0 ** -6 and m["cosine"] >= 0.9999, (i, fused, m)
            assert_parity(oracle, outs[fused].cpu(), ref, f"fused step {i} {fused}")
        for c in caches.values():
            c.workspace.status.zero_()


def test_random_shapes_against_the_oracle(pkg, oracle, cuda_device):
    """Seeded random geometries: layers, batch, heads, group size, head_dim, capacity, CTA count and
    ragged lengths that hit the awkward places (0, 1, one token short of / exactly / one token past
    a tile, full capacity), NaN bytes beyond every length; every tensor-core kernel that takes the
    shape against the oracle, and the one-launch step against the three-launch step."""
    import os
    rng = np.random.default_rng(int(os.environ.get("B200ATTN_TEST_SEED", "20260")))   # another seed: another set of geometries
    for trial in range(int(os.environ.get("B200ATTN_TEST_TRIALS", "14"))):
        d = 256 if trial % 5 == 4 else 128
        h_kv = int(rng.choice([1, 2, 4, 8]))
        group = int(rng.integers(1, 6)) if trial % 3 else int(rng.integers(1, 9))
        n_layers, batch = int(rng.integers(1, 5)), int(rng.integers(1, 6))
        cap = int(rng.choice([128, 192, 640, 1100]))
        special = [0, 1, 127, 128, 129, 255, 256, 257, cap - 1, cap]
        lens = [int(min(cap, rng.choice(special) if rng.random() < 0.6 else rng.integers(0, cap + 1))) for _ in range(batch)]
        if not any(lens):
            lens[0] = 1
        case = build_case(oracle, n_layers, batch, h_kv * group, h_kv, d, lens, cap, seed=1000 + trial, fill_byte=0xFF)
        clean = dict(case)
        clean["k_cache"] = case["k_cache"].clone()
        clean["v_cache"] = case["v_cache"].clone()
        for b, L in enumerate(lens):
            clean["k_cache"][:, b, :, L:] = 0
            clean["v_cache"][:, b, :, L:] = 0
        ref = oracle.decode_step_reference(case["q"], clean["k_cache"], clean["v_cache"], case["k_scale"], case["v_scale"], lens, cap)
        for b, L in enumerate(lens):
            if L == 0:
                ref[:, b] = 0          # an empty sequence has no attention output: defined as zeros
        what = f"trial {trial}: layers {n_layers} batch {batch} h_kv {h_kv} group {group} d {d} cap {cap} lens {lens}"
        n_ctas = int(rng.choice([0, 0, 7, 148, 333]))
        for variant in ("mma", "umma2"):
            if unsupported(pkg, variant, h_kv * group, h_kv):
                continue
            out, status = run_decode(pkg, case, cuda_device, variant, num_splits=n_ctas)
            assert status == 0, (what, variant)
            assert not torch.isnan(out.float()).any(), (what, variant)
            assert_parity(oracle, out, ref, f"{what} {variant} ctas {n_ctas}")
        if max(lens) < cap:
            # one decode step, fused launch vs append + attention + position kernels
            g = torch.Generator().manual_seed(trial)
            kn = torch.randn(n_layers, batch, h_kv, d, generator=g).to(torch.bfloat16).to(cuda_device)
            vn = torch.randn(n_layers, batch, h_kv, d, generator=g).to(torch.bfloat16).to(cuda_device)
            res = {}
            for variant in ("simt", "mma", "umma2"):
                c = pkg.FP8StaticCache(n_layers, batch, h_kv * group, h_kv, d, cap, device=cuda_device, variant=variant)
                c.set_scales(case["k_scale"].to(cuda_device), case["v_scale"].to(cuda_device))
                c.k_cache.copy_(case["k_cache"])
                c.v_cache.copy_(case["v_cache"])
                c.seq_pos.copy_(torch.tensor(lens, dtype=torch.int32))
                out = c.step(case["q"].to(cuda_device), kn, vn, count=False)
                torch.cuda.synchronize()
                res[variant] = (out.cpu(), c.k_cache.cpu(), c.v_cache.cpu(), c.seq_pos.cpu(), int(c.status.cpu().view(-1)[0]))
            a = res["simt"]
            for fused in ("mma", "umma2"):
                u = res[fused]
                assert a[4] == 0 and u[4] == 0, (what, fused)
                assert torch.equal(a[1], u[1]) and torch.equal(a[2], u[2]) and torch.equal(a[3], u[3]), (what, fused)
                m = oracle.error_metrics(u[0], a[0])
                assert m["max_abs"] <= 2.0 ** -6 and m["cosine"] >= 0.9999, (what, fused, m)


def test_peer_barrier_wait_is_bounded(pkg, cuda_device):
    """The cross-GPU barrier gives up after its 1 s budget when a peer never arrives (here: a second
    flag buffer that nobody writes), reports it in the status word, and leaves the context usable."""
    import ctypes
    import time
    lib = pkg._lib.lib()
    mine = torch.zeros(64, dtype=torch.int32, device=cuda_device)
    silent_peer = torch.zeros(64, dtype=torch.int32, device=cuda_device)   # stands in for a rank that never arrives
    status = torch.zeros(1, dtype=torch.int32, device=cuda_device)
    flags = (ctypes.c_void_p * 8)(mine.data_ptr(), silent_peer.data_ptr())
    t0 = time.perf_counter()
    rc = lib.b200attn_peer_barrier(flags, 0, 2, status.data_ptr(), torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    assert rc == 0
    assert status.item() & pkg._lib.STATUS_WAIT_TIMEOUT
    assert 0.5 < dt < 5.0, dt
    assert silent_peer[0].item() == 1          # our arrival was posted to the peer's buffer
    # a world of one completes at once, and the device still works
    status.zero_()
    solo = (ctypes.c_void_p * 8)(mine.data_ptr())
    assert lib.b200attn_peer_barrier(solo, 0, 1, status.data_ptr(), torch.cuda.current_stream().cuda_stream) == 0
    torch.cuda.synchronize()
    assert status.item() == 0
    assert float((torch.ones(8, device=cuda_device) * 2).sum()) == 16.0


def test_in_launch_barrier_wait_is_bounded(pkg, oracle, cuda_device):
    """The arrive-and-wait inside the attention launch (tensor-parallel decode step, all-tcgen05
    kernel): with a peer that never arrives — a second flag buffer that nobody writes — the last CTA
    gives up after its 1 s budget, the status word says so, both gathered buffers hold this rank's
    heads all the same, the cache and the positions are advanced, and the context stays usable."""
    import ctypes
    import time
    n_layers, batch, h_q, h_kv, d, cap, lens = 2, 1, 20, 4, 128, 256, [130]
    case = build_case(oracle, n_layers, batch, h_q, h_kv, d, lens, cap, seed=3)
    dev = cuda_device
    c = pkg.FP8StaticCache(n_layers, batch, h_q, h_kv, d, cap, device=dev, variant="umma2")
    c.set_scales(case["k_scale"].to(dev), case["v_scale"].to(dev))
    c.k_cache.copy_(case["k_cache"])
    c.v_cache.copy_(case["v_cache"])
    c.seq_pos.copy_(torch.tensor(lens, dtype=torch.int32))
    g = torch.Generator().manual_seed(4)
    kn = torch.randn(n_layers, batch, h_kv, d, generator=g).to(torch.bfloat16).to(dev)
    vn = torch.randn(n_layers, batch, h_kv, d, generator=g).to(torch.bfloat16).to(dev)
    full = [torch.full((n_layers, batch, 2 * h_q, d), float("nan"), dtype=torch.bfloat16, device=dev) for _ in range(2)]
    mine = torch.zeros(64, dtype=torch.int32, device=dev)
    silent_peer = torch.zeros(64, dtype=torch.int32, device=dev)     # stands in for a rank that never arrives
    peers = pkg._lib.B200AttnPeerOut(2, 0, 2 * h_q, 0, (ctypes.c_void_p * 8)(full[0].data_ptr(), full[1].data_ptr()))
    flags = (ctypes.c_void_p * 8)(mine.data_ptr(), silent_peer.data_ptr())
    q = case["q"].to(dev)
    ws = c.workspace
    t0 = time.perf_counter()
    rc = pkg._lib.lib().b200attn_append_decode_peers(
        ctypes.byref(c.shape), ctypes.byref(peers), q.data_ptr(), kn.data_ptr(), vn.data_ptr(), c.k_cache.data_ptr(),
        c.v_cache.data_ptr(), c.k_scale.data_ptr(), c.v_scale.data_ptr(), c.seq_pos.data_ptr(), 1, d ** -0.5,
        pkg._lib.VARIANTS["umma2"], ws.num_splits, ws.buf.data_ptr(), ws.nbytes, flags, ws.status.data_ptr(),
        torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    assert rc == 0
    assert ws.read_status() == pkg._lib.STATUS_WAIT_TIMEOUT
    assert 0.5 < dt < 5.0, dt
    assert silent_peer[0].item() == 1 and c.seq_pos.cpu().tolist() == [131]
    ref = oracle.decode_step_reference(case["q"], c.k_cache.cpu(), c.v_cache.cpu(), case["k_scale"], case["v_scale"], [131], cap)
    for buf in full:
        assert_parity(oracle, buf[:, :, :h_q].cpu(), ref, "gathered buffer")
        assert torch.isnan(buf[:, :, h_q:].float()).all()          # the other rank's heads: untouched
    assert float((torch.ones(8, device=dev) * 2).sum()) == 16.0


def test_packet_wait_is_bounded(pkg, oracle, cuda_device):
    """Tensor-parallel step in packet mode with a peer that never sends (a staging buffer nobody writes): every CTA's
    wait for the other rank's packets runs out after its 1 s budget, the status word says so, this rank's own heads are
    in its gathered tensor and in the 'peer's' staging all the same (as packets carrying step number 1), the cache and
    the positions are advanced, the step counter is 1 and the context stays usable."""
    import ctypes
    import time
    L = pkg._lib
    n_layers, batch, h_q, h_kv, d, cap, lens = 2, 1, 20, 4, 128, 256, [130]
    case = build_case(oracle, n_layers, batch, h_q, h_kv, d, lens, cap, seed=3)
    dev = cuda_device
    for variant in ("mma", "umma2"):
        c = pkg.FP8StaticCache(n_layers, batch, h_q, h_kv, d, cap, device=dev, variant=variant)
        c.set_scales(case["k_scale"].to(dev), case["v_scale"].to(dev))
        c.k_cache.copy_(case["k_cache"])
        c.v_cache.copy_(case["v_cache"])
        c.seq_pos.copy_(torch.tensor(lens, dtype=torch.int32))
        g = torch.Generator().manual_seed(4)
        kn = torch.randn(n_layers, batch, h_kv, d, generator=g).to(torch.bfloat16).to(dev)
        vn = torch.randn(n_layers, batch, h_kv, d, generator=g).to(torch.bfloat16).to(dev)
        nbytes = L.lib().b200attn_peer_staging_bytes(ctypes.byref(c.shape), 2)
        assert nbytes == 2 * 2 * n_layers * batch * h_q * d // 2 * 8
        mine = torch.zeros(nbytes // 8, dtype=torch.int64, device=dev)
        silent_peer = torch.zeros_like(mine)                         # stands in for a rank that never sends
        full = torch.full((n_layers, batch, 2 * h_q, d), float("nan"), dtype=torch.bfloat16, device=dev)
        step = torch.zeros(1, dtype=torch.int32, device=dev)
        out = (ctypes.c_void_p * 8)()
        out[0] = full.data_ptr()
        peers = L.B200AttnPeerOut(2, 0, 2 * h_q, L.GATHER_PACKETS, out, (ctypes.c_void_p * 8)(),
                                  (ctypes.c_void_p * 8)(mine.data_ptr(), silent_peer.data_ptr()), step.data_ptr())
        q = case["q"].to(dev)
        ws = c.workspace
        t0 = time.perf_counter()
        rc = L.lib().b200attn_append_decode_peers(
            ctypes.byref(c.shape), ctypes.byref(peers), q.data_ptr(), kn.data_ptr(), vn.data_ptr(), c.k_cache.data_ptr(),
            c.v_cache.data_ptr(), c.k_scale.data_ptr(), c.v_scale.data_ptr(), c.seq_pos.data_ptr(), 1, d ** -0.5,
            L.VARIANTS[variant], ws.num_splits, ws.buf.data_ptr(), ws.nbytes, None, ws.status.data_ptr(),
            torch.cuda.current_stream().cuda_stream)
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        assert rc == 0
        assert ws.read_status() == L.STATUS_WAIT_TIMEOUT, variant
        assert 0.5 < dt < 5.0, dt
        assert c.seq_pos.cpu().tolist() == [131] and int(step.item()) == 1
        ref = oracle.decode_step_reference(case["q"], c.k_cache.cpu(), c.v_cache.cpu(), case["k_scale"], case["v_scale"], [131], cap)
        assert_parity(oracle, full[:, :, :h_q].cpu(), ref, f"{variant}: own heads of the gathered tensor")
        assert torch.isnan(full[:, :, h_q:].float()).all()            # the other rank's heads: untouched
        slot = nbytes // 8 // 4                                      # [2 parities][2 senders][slot] packets
        sent = silent_peer.view(2, 2, slot)[1, 0]                    # step 1 is odd; this rank is sender 0
        assert bool(((sent >> 32) == 1).all()), "every packet carries the step number"
        vals = (sent & 0xFFFFFFFF).to(torch.int32).view(torch.bfloat16).view(n_layers, batch, h_q, d)
        assert torch.equal(vals.view(torch.int16), full[:, :, :h_q].contiguous().view(torch.int16))
        assert int(silent_peer.view(2, 2, slot)[0].abs().max()) == 0 and int(mine.abs().max()) == 0
        # barrier flags and packets do not mix
        flags = (ctypes.c_void_p * 8)(mine.data_ptr(), silent_peer.data_ptr())
        rc = L.lib().b200attn_append_decode_peers(
            ctypes.byref(c.shape), ctypes.byref(peers), q.data_ptr(), kn.data_ptr(), vn.data_ptr(), c.k_cache.data_ptr(),
            c.v_cache.data_ptr(), c.k_scale.data_ptr(), c.v_scale.data_ptr(), c.seq_pos.data_ptr(), 1, d ** -0.5,
            L.VARIANTS[variant], ws.num_splits, ws.buf.data_ptr(), ws.nbytes, flags, ws.status.data_ptr(),
            torch.cuda.current_stream().cuda_stream)
        assert rc == L.ERR_SHAPE
        assert float((torch.ones(8, device=dev) * 2).sum()) == 16.0


def test_reset_lifecycle_sequences(pkg, oracle, cuda_device):
    """The reset gates of the reference's check list (scripts/m3_check.py: A -> B -> A and short -> long -> short on one
    cache object against fresh caches): after an in-place reset a run reproduces, bit for bit, what a fresh cache gives,
    whatever ran before it; addresses never change; stale bytes of a longer earlier run stay invisible."""
    n_layers, batch, h_q, h_kv, d, cap = 3, 2, 40, 8, 128, 384
    g = torch.Generator().manual_seed(31)
    runs = {}
    for name, depth, steps in (("A", 100, 5), ("B", 260, 9), ("short", 17, 3), ("long", 300, 40)):
        runs[name] = {"k0": torch.randn(n_layers, batch, h_kv, depth, d, generator=g).to(torch.bfloat16).to(cuda_device),
                      "v0": torch.randn(n_layers, batch, h_kv, depth, d, generator=g).to(torch.bfloat16).to(cuda_device),
                      "q": torch.randn(steps, n_layers, batch, h_q, d, generator=g).to(torch.bfloat16).to(cuda_device),
                      "kn": torch.randn(steps, n_layers, batch, h_kv, d, generator=g).to(torch.bfloat16).to(cuda_device),
                      "vn": torch.randn(steps, n_layers, batch, h_kv, d, generator=g).to(torch.bfloat16).to(cuda_device)}

    def play(cache, run):
        cache.prefill(run["k0"], run["v0"], calibrate=True)
        outs = [cache.step(run["q"][i], run["kn"][i], run["vn"][i]).clone() for i in range(run["q"].shape[0])]
        torch.cuda.synchronize()
        assert cache.workspace.read_status() == 0
        return outs

    for variant in ("mma", "umma2"):
        fresh = {}
        for name, run in runs.items():
            fresh[name] = play(pkg.FP8StaticCache(n_layers, batch, h_q, h_kv, d, cap, device=cuda_device, variant=variant), run)
        one = pkg.FP8StaticCache(n_layers, batch, h_q, h_kv, d, cap, device=cuda_device, variant=variant)
        ptrs = (one.k_cache.data_ptr(), one.v_cache.data_ptr(), one.seq_pos.data_ptr())
        for name in ("A", "B", "A", "short", "long", "short"):
            one.reset()
            got = play(one, runs[name])
            assert (one.k_cache.data_ptr(), one.v_cache.data_ptr(), one.seq_pos.data_ptr()) == ptrs
            for i, (a, b) in enumerate(zip(got, fresh[name])):
                assert torch.equal(a.view(torch.int16), b.view(torch.int16)), (variant, name, i)


def test_canary_words_around_every_buffer_the_kernels_write(pkg, oracle, cuda_device):
    """Every buffer a launch may write — output, workspace (partials, CTA counter), status word, cache,
    positions — sits between guard regions filled with a pattern; lengths 1..160 (every position inside and across
    the 64- and 128-token tiles) x several CTA counts, attention alone and the fused step, both tensor-core kernels:
    the guards must come back untouched and the results must match the oracle.  (Stand-in for a memory checker.)"""
    n_layers, h_q, h_kv, d, cap, guard = 2, 40, 8, 128, 192, 4096
    dev = cuda_device

    class Guarded:
        def __init__(self, nbytes):
            self.nbytes = (nbytes + 255) // 256 * 256
            self.raw = torch.full((self.nbytes + 2 * guard,), 0xA5, dtype=torch.uint8, device=dev)
            self.body = self.raw[guard:guard + self.nbytes]

        def view(self, dtype, shape):
            n = int(torch.tensor(shape).prod()) * torch.empty(0, dtype=dtype).element_size()
            return self.body[:n].view(dtype).view(shape)

        def intact(self, used_bytes):
            tail = self.raw[guard + used_bytes:]
            return bool((self.raw[:guard] == 0xA5).all()) and bool((tail == 0xA5).all())

    g = torch.Generator().manual_seed(77)
    kn = torch.randn(n_layers, 1, h_kv, d, generator=g).to(torch.bfloat16).to(dev)
    vn = torch.randn(n_layers, 1, h_kv, d, generator=g).to(torch.bfloat16).to(dev)
    for L in list(range(1, 161, 3)) + [63, 64, 65, 127, 128, 129, 160]:
        case = build_case(oracle, n_layers, 1, h_q, h_kv, d, [L], cap, seed=500 + L, fill_byte=0xFF)
        clean_k, clean_v = case["k_cache"].clone(), case["v_cache"].clone()
        clean_k[:, :, :, L:] = 0
        clean_v[:, :, :, L:] = 0
        ref = oracle.decode_step_reference(case["q"], clean_k, clean_v, case["k_scale"], case["v_scale"], [L], cap)
        for variant, ctas in (("mma", 0), ("mma", 5), ("mma", 37), ("umma2", 0), ("umma2", 3), ("umma2", 148)):
            cache_bytes = n_layers * h_kv * cap * d
            gk, gv = Guarded(cache_bytes), Guarded(cache_bytes)
            kc, vc = gk.view(torch.uint8, (n_layers, 1, h_kv, cap, d)), gv.view(torch.uint8, (n_layers, 1, h_kv, cap, d))
            kc.copy_(case["k_cache"]); vc.copy_(case["v_cache"])
            ks, vs = case["k_scale"].to(dev), case["v_scale"].to(dev)
            shape = pkg.make_shape(h_q, kc, vc, ks)
            n = ctas or pkg.pick_splits(shape, variant=variant)
            ws_bytes = pkg.workspace_bytes(shape, n, variant)
            gw, go, gs, gp = Guarded(ws_bytes), Guarded(n_layers * h_q * d * 2), Guarded(4), Guarded(4)
            ws = pkg.Workspace(shape, dev, variant=variant, num_splits=n)
            ws.buf, ws.nbytes = gw.body[:ws_bytes], ws_bytes           # the library's workspace, between guards
            ws.status = gs.view(torch.int32, (1,))
            ws.status.zero_()
            ws.init()
            out = go.view(torch.bfloat16, (n_layers, 1, h_q, d))
            pos = gp.view(torch.int32, (1,))
            pos.fill_(L)
            q = case["q"].to(dev)
            pkg.decode_attention(q, kc, vc, ks, vs, pos, workspace=ws, out=out)
            torch.cuda.synchronize()
            what = f"L={L} {variant} ctas={n}"
            assert ws.read_status() == 0, what
            assert_parity(oracle, out.cpu(), ref, what)
            if L < cap:
                pkg.append_decode(q, kn, vn, kc, vc, ks, vs, pos, workspace=ws, out=out)
                torch.cuda.synchronize()
                assert ws.read_status() == 0 and int(pos.item()) == L + 1, what
            for name, gd, used in (("k cache", gk, cache_bytes), ("v cache", gv, cache_bytes), ("workspace", gw, ws_bytes),
                                   ("output", go, n_layers * h_q * d * 2), ("status", gs, 4), ("positions", gp, 4)):
                assert gd.intact(used), f"{what}: guard words of the {name} overwritten"
