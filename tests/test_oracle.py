"""CPU tests: the oracle against the reference's golden outputs and against torch's e4m3 cast."""
import ctypes
import hashlib

import numpy as np
import pytest
import torch


def _sha(t):
    return hashlib.sha256(t.contiguous().view(torch.uint8).numpy().tobytes()).hexdigest()


def _all_bf16():
    bits = torch.arange(0, 65536, dtype=torch.int32).to(torch.int16)
    return bits.view(torch.bfloat16)


SCALES = [1.0, 2.0 ** -7, 3.0 ** -3, 0.0094, 4.5 / 448, 1e-30, 1e30, 448.0, 0.1]


def test_numpy_e4m3_matches_torch_cast_exhaustive(oracle):
    """Every bf16 pattern x several scales: bit-level restatement == torch float8_e4m3fn cast."""
    x = _all_bf16()
    for s in SCALES:
        y = (x.float() / s).clamp(-448, 448)
        want = y.to(torch.float8_e4m3fn).view(torch.uint8).numpy()
        got = oracle.e4m3_bytes_from_f32(y.numpy())
        finite = ~torch.isnan(y).numpy()
        assert np.array_equal(got[finite], want[finite]), f"scale {s}"
        # NaN inputs: NaN byte with the sign kept
        assert np.all((got[~finite] & 0x7F) == 0x7F) and np.all((want[~finite] & 0x7F) == 0x7F)


def test_numpy_e4m3_unclamped_edges(oracle):
    """Overflow / rounding-edge list without the clamp (what the cast itself does)."""
    vals = torch.tensor([448.0, 449.0, 464.0, 465.0, 479.9, 480.0, 1e9, float("inf"), -464.0, -480.0,
                         2.0 ** -9, 2.0 ** -10, 1.5 * 2.0 ** -10, 2.0 ** -10 + 2.0 ** -20, 0.0, -0.0,
                         2.0 ** -6, 2.0 ** -6 - 2.0 ** -12, 0.0175, 7 * 2.0 ** -9 + 2.0 ** -10])
    want = vals.to(torch.float8_e4m3fn).view(torch.uint8).numpy()
    got = oracle.e4m3_bytes_from_f32(vals.numpy())
    assert np.array_equal(got, want)


def test_c_oracle_e4m3_matches_torch_exhaustive():
    from oracle import build as ob
    lib = ob.load()
    x = _all_bf16()
    xb = x.view(torch.int16).numpy().view(np.uint16).copy()
    for s in SCALES:
        want = (x.float() / s).clamp(-448, 448).to(torch.float8_e4m3fn).view(torch.uint8).numpy()
        got = np.zeros(65536, dtype=np.uint8)
        lib.oracle_quantize(xb.ctypes.data_as(ctypes.POINTER(ctypes.c_uint16)), ctypes.c_float(s),
                            got.ctypes.data_as(ctypes.POINTER(ctypes.c_uint8)), 65536)
        nan = torch.isnan(x.float() / s).numpy()
        assert np.array_equal(got[~nan], want[~nan]), f"scale {s}"
        assert np.all((got[nan] & 0x7F) == 0x7F)
    # and the byte -> float table
    allb = torch.arange(256, dtype=torch.int32).to(torch.uint8)
    ref = allb.view(torch.float8_e4m3fn).float().numpy()
    for b in range(256):
        v = lib.oracle_e4m3_to_f32(b)
        assert (np.isnan(v) and np.isnan(ref[b])) or v == ref[b]


def _rebuild(oracle, m):
    q, k, v = oracle.make_inputs(m["seed"], m["h_q"], m["h_kv"], m["d"], m["length"])
    sk, sv = oracle.head_scales(k), oracle.head_scales(v)
    kb, vb = oracle.quantize_per_head(k, sk), oracle.quantize_per_head(v, sv)
    return q, kb, vb, sk, sv


def test_golden_inputs_rebuild(oracle, golden):
    """The seeded inputs and the quantised bytes are the ones the fixtures were made from."""
    data, meta = golden
    for name, m in meta.items():
        if m["length"] > 2048:
            continue
        q, kb, vb, sk, sv = _rebuild(oracle, m)
        assert _sha(q) == m["sha_q"], name
        assert _sha(kb) == m["sha_k_bytes"], name
        assert _sha(vb) == m["sha_v_bytes"], name
        assert np.array_equal(sk.numpy(), data[f"{name}/k_scale"])
        assert np.array_equal(sv.numpy(), data[f"{name}/v_scale"])


def test_oracle_matches_reference_golden(oracle, golden):
    """padded_fp8_reference == the reference's eager_attention output; fp64 likewise."""
    data, meta = golden
    torch.set_num_threads(1)
    for name, m in meta.items():
        if m["length"] > 2048:
            continue
        q, kb, vb, sk, sv = _rebuild(oracle, m)
        out = oracle.padded_fp8_reference(q, kb, vb, sk, sv, m["capacity"])
        want = torch.from_numpy(data[f"{name}/out_bf16_bits"].view(np.int16)).view(torch.bfloat16)
        diff = (out.float() - want.float()).abs().max().item()
        # same torch build + thread count -> bitwise; another CPU may differ by a bf16 ulp
        assert diff <= 2.0 ** -8 * max(1.0, want.float().abs().max().item()), (name, diff)
        out64 = oracle.fp64_fp8_reference(q, kb, vb, sk, sv)
        want64 = torch.from_numpy(data[f"{name}/out_fp64_as_f32"])
        # the reference's fp64 runs over bf16-rounded dequantised K/V, ours over exact dequant
        tol = 2.0 ** -7 * max(1.0, want64.abs().max().item())
        assert (out64.float() - want64).abs().max().item() < tol, name


def test_oracle_bitwise_on_this_host(oracle, golden):
    """Diagnostic made a gate where it is stable: on the host that generated the fixtures
    (same torch build), the restatement is bit-identical to the reference."""
    data, meta = golden
    torch.set_num_threads(1)
    name = "b40x8x128_L513_c1024_s0"
    m = meta[name]
    q, kb, vb, sk, sv = _rebuild(oracle, m)
    out = oracle.padded_fp8_reference(q, kb, vb, sk, sv, m["capacity"])
    got = out.view(torch.int16).numpy().view(np.uint16)
    frac = float((got != data[f"{name}/out_bf16_bits"]).mean())
    assert frac <= 0.02, frac


def test_c_oracle_attention_close_to_torch_oracle(oracle):
    from oracle import build as ob
    lib = ob.load()
    h_q, h_kv, d, length, cap = 10, 2, 128, 77, 96
    q, k, v = oracle.make_inputs(5, h_q, h_kv, d, length)
    sk, sv = oracle.head_scales(k), oracle.head_scales(v)
    kb, vb = oracle.quantize_per_head(k, sk), oracle.quantize_per_head(v, sv)
    want = oracle.padded_fp8_reference(q, kb, vb, sk, sv, cap).view(h_q, d)
    kc = torch.zeros(1, 1, h_kv, cap, d, dtype=torch.uint8)
    vc = torch.zeros_like(kc)
    kc[0, :, :, :length] = kb
    vc[0, :, :, :length] = vb
    out = np.zeros((h_q, d), dtype=np.uint16)
    P = ctypes.POINTER
    qb = q.view(h_q, d).view(torch.int16).numpy().view(np.uint16).copy()
    seq = np.array([length], dtype=np.int32)
    rc = lib.oracle_decode_attention(1, 1, h_q, h_kv, d, cap, 0, qb.ctypes.data_as(P(ctypes.c_uint16)),
                                     kc.numpy().ctypes.data_as(P(ctypes.c_uint8)), vc.numpy().ctypes.data_as(P(ctypes.c_uint8)),
                                     sk.numpy().ctypes.data_as(P(ctypes.c_float)), sv.numpy().ctypes.data_as(P(ctypes.c_float)),
                                     seq.ctypes.data_as(P(ctypes.c_int)), ctypes.c_float(d ** -0.5),
                                     out.ctypes.data_as(P(ctypes.c_uint16)))
    assert rc == 0
    got = torch.from_numpy(out.view(np.int16)).view(torch.bfloat16)
    m = oracle.error_metrics(got, want)
    assert m["max_abs"] <= 4e-3 and m["cosine"] >= 0.99999, m


def test_degenerate_softmax_cases(oracle):
    """L=1 -> out equals the dequantised V row; identical keys -> mean of V."""
    h_q, h_kv, d = 10, 2, 128
    q, k, v = oracle.make_inputs(1, h_q, h_kv, d, 1)
    sk, sv = oracle.head_scales(k), oracle.head_scales(v)
    kb, vb = oracle.quantize_per_head(k, sk), oracle.quantize_per_head(v, sv)
    out = oracle.padded_fp8_reference(q, kb, vb, sk, sv, 64).view(h_q, d)
    vd = oracle.dequantize(vb, sv.view(1, -1, 1, 1))[0, :, 0]
    assert torch.equal(out, vd.repeat_interleave(h_q // h_kv, dim=0))
    q, k, v = oracle.make_inputs(2, h_q, h_kv, d, 8)
    k[:] = k[:, :, :1]
    sk, sv = oracle.head_scales(k), oracle.head_scales(v)
    kb, vb = oracle.quantize_per_head(k, sk), oracle.quantize_per_head(v, sv)
    out = oracle.padded_fp8_reference(q, kb, vb, sk, sv, 64).view(h_q, d).float()
    mean = oracle.dequantize(vb, sv.view(1, -1, 1, 1))[0].float().mean(dim=1).repeat_interleave(h_q // h_kv, dim=0)
    assert (out - mean).abs().max().item() < 2e-2


def test_per_token_quantisation_roundtrip(oracle):
    """The reference's own scale granularity: round trip within its recorded accuracy
    (nrmse 0.0261, cosine 0.99966 in docs/journal/2026-10-23-phase2-r3-coordinator.md:194-195)."""
    _, k, _ = oracle.make_inputs(0, 24, 4, 256, 513)
    s = oracle.token_scales(k)
    kb = oracle.quantize_per_token(k, s)
    kd = oracle.dequantize(kb, s.permute(0, 2, 1).unsqueeze(-1))
    m = oracle.error_metrics(kd, k)
    assert 0.02 < m["nrmse"] < 0.03 and m["cosine"] > 0.9995, m


def _bf16(data, key, shape):
    return torch.from_numpy(data[key].view(np.int16).copy()).view(torch.bfloat16).view(*shape)


def producer_case(data, name, m):
    b, h_q, h_kv, d, r = m["batch"], m["h_q"], m["h_kv"], m["d"], m["rotary_dim"]
    return {"q_raw": _bf16(data, f"{name}/q_raw", (b, h_q, 1, d)), "k_raw": _bf16(data, f"{name}/k_raw", (b, h_kv, 1, d)),
            "wq": _bf16(data, f"{name}/wq", (d,)), "wk": _bf16(data, f"{name}/wk", (d,)),
            "cos": _bf16(data, f"{name}/cos", (b, 1, r)), "sin": _bf16(data, f"{name}/sin", (b, 1, r)),
            "q_out": _bf16(data, f"{name}/q_out", (b, h_q, 1, d)), "k_out": _bf16(data, f"{name}/k_out", (b, h_kv, 1, d))}


def test_producer_oracle_matches_the_model_code(oracle, producer_golden):
    """q_norm / k_norm + partial rotary embedding: the restatement equals, bit for bit, what the
    third-party model code the reference runs produced for the committed fixtures."""
    data, meta = producer_golden
    names = [n for n in meta if n != "transformers"]
    assert len(names) >= 4
    for name in names:
        m = meta[name]
        c = producer_case(data, name, m)
        q, k = oracle.producer_reference(c["q_raw"], c["k_raw"], c["wq"], c["wk"], m["eps"], c["cos"], c["sin"])
        assert torch.equal(q.view(torch.int16), c["q_out"].view(torch.int16)), name
        assert torch.equal(k.view(torch.int16), c["k_out"].view(torch.int16)), name
        # the pass-through dims really pass through, the rotated ones really change
        r = m["rotary_dim"]
        normed = oracle.qk_norm(c["q_raw"], c["wq"], m["eps"])
        assert torch.equal(q[..., r:], normed[..., r:])
        assert not torch.equal(q[..., :r], normed[..., :r])
