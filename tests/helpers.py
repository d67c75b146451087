"""Shared builders for the GPU parity tests (inputs on the CPU via the oracle, then uploaded)."""
import torch

TOL_MAX_ABS = 2e-2     # bf16 tolerance of the benchmark: max abs err <= 2e-2
TOL_COSINE = 0.9999    # and cosine >= 0.9999, against the reference's padded torch attention


def build_case(oracle, n_layers, batch, h_q, h_kv, d, lens, capacity, seed, fill_byte=0):
    """Quantised caches for ragged lengths `lens`; per-(layer, kv head) scales over the whole layer."""
    q = torch.zeros(n_layers, batch, h_q, d, dtype=torch.bfloat16)
    kc = torch.full((n_layers, batch, h_kv, capacity, d), fill_byte, dtype=torch.uint8)
    vc = torch.full((n_layers, batch, h_kv, capacity, d), fill_byte, dtype=torch.uint8)
    ks = torch.zeros(n_layers, h_kv)
    vs = torch.zeros(n_layers, h_kv)
    for layer in range(n_layers):
        raw = []
        for b in range(batch):
            qq, k, v = oracle.make_inputs(seed + 131 * layer + 7 * b, h_q, h_kv, d, max(int(lens[b]), 1))
            raw.append((qq, k[:, :, :lens[b]], v[:, :, :lens[b]]))
        nonempty = [r for r in raw if r[1].shape[2] > 0]
        ks[layer] = torch.stack([oracle.head_scales(r[1]) for r in nonempty]).amax(0) if nonempty else 1.0
        vs[layer] = torch.stack([oracle.head_scales(r[2]) for r in nonempty]).amax(0) if nonempty else 1.0
        for b, (qq, k, v) in enumerate(raw):
            q[layer, b] = qq.view(h_q, d)
            if lens[b]:
                kc[layer, b, :, :lens[b]] = oracle.quantize_per_head(k, ks[layer])[0]
                vc[layer, b, :, :lens[b]] = oracle.quantize_per_head(v, vs[layer])[0]
    return {"q": q, "k_cache": kc, "v_cache": vc, "k_scale": ks, "v_scale": vs, "lens": list(map(int, lens)),
            "capacity": capacity}


def run_decode(pkg, case, device, variant="auto", num_splits=0):
    """Upload a case and run the library's decode through the C-ABI; returns (out_cpu, status)."""
    dev = {k: (v.to(device) if isinstance(v, torch.Tensor) else v) for k, v in case.items()}
    shape = pkg.make_shape(case["q"].shape[2], dev["k_cache"], dev["v_cache"], dev["k_scale"])
    ws = pkg.Workspace(shape, device, variant=variant, num_splits=num_splits)
    seq_len = torch.tensor(case["lens"], dtype=torch.int32, device=device)
    out = pkg.decode_attention(dev["q"], dev["k_cache"], dev["v_cache"], dev["k_scale"], dev["v_scale"], seq_len,
                               workspace=ws)
    torch.cuda.synchronize()
    return out.cpu(), ws.read_status()


def assert_parity(oracle, out, ref, what=""):
    m = oracle.error_metrics(out, ref)
    assert m["max_abs"] <= TOL_MAX_ABS and m["cosine"] >= TOL_COSINE, (what, m)
    return m
