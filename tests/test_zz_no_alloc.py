"""The allocation-free decode entry point (b200attn_decode_static), driven through the C-ABI.

Hosts whose device memory belongs to a framework pool, or whose step cannot tolerate an
allocation, call this instead of b200attn_decode: the split-K scratch sits in a fixed array
inside the library.  It must give what the workspace-taking entry point gives — checked here on
two calls in a row (the second call sees the scratch the first one left behind) — and must refuse
requests that do not fit.  Kept last in collection order so a failure here cannot hide others.
"""
import ctypes

import pytest
import torch

from helpers import TOL_COSINE, TOL_MAX_ABS, build_case

pytestmark = pytest.mark.gpu


def _call_static(lib, shape, dev, seq, scale, num_splits, out, status):
    return lib.b200attn_decode_static(ctypes.byref(shape), dev["q"].data_ptr(), dev["k_cache"].data_ptr(),
                                      dev["v_cache"].data_ptr(), dev["k_scale"].data_ptr(), dev["v_scale"].data_ptr(),
                                      seq.data_ptr(), 0, scale, num_splits, out.data_ptr(), status.data_ptr(),
                                      torch.cuda.current_stream().cuda_stream)


def test_static_scratch_entry_point_matches_workspace_entry_point(pkg, oracle, cuda_device):
    lib = pkg._lib.lib()
    assert lib.b200attn_static_scratch_bytes() == 8 << 20
    for lens, cap, n_layers in (([700, 333], 1024, 4), ([1000], 1024, 16)):
        case = build_case(oracle, n_layers, len(lens), 40, 8, 128, lens, cap, seed=7)
        dev = {k: (v.to(cuda_device) if isinstance(v, torch.Tensor) else v) for k, v in case.items()}
        shape = pkg.make_shape(40, dev["k_cache"], dev["v_cache"], dev["k_scale"])
        seq = torch.tensor(lens, dtype=torch.int32, device=cuda_device)
        ws = pkg.Workspace(shape, cuda_device, variant="mma")
        want = pkg.decode_attention(dev["q"], dev["k_cache"], dev["v_cache"], dev["k_scale"], dev["v_scale"], seq,
                                    workspace=ws)                                   # the existing entry point
        status = torch.zeros(1, dtype=torch.int32, device=cuda_device)
        for call in range(2):                                                       # two calls in a row
            out = torch.full_like(want, float("nan"))
            rc = _call_static(lib, shape, dev, seq, 128 ** -0.5, ws.num_splits, out, status)
            assert rc == 0, lib.b200attn_error_string(rc)
            torch.cuda.synchronize()
            assert status.item() == 0
            m = oracle.error_metrics(out.cpu(), want.cpu())
            assert m["max_abs"] <= TOL_MAX_ABS and m["cosine"] >= TOL_COSINE, (call, m)
            assert torch.equal(out.view(torch.int16), want.view(torch.int16)), f"call {call}: same kernel, same split -> same bits"
        # default split count (0) is accepted as well
        out = torch.empty_like(want)
        assert _call_static(lib, shape, dev, seq, 128 ** -0.5, 0, out, status) == 0
        torch.cuda.synchronize()
        m = oracle.error_metrics(out.cpu(), want.cpu())
        assert m["max_abs"] <= TOL_MAX_ABS and m["cosine"] >= TOL_COSINE, m


def test_static_scratch_holds_the_long_cache_grid(pkg, oracle, cuda_device):
    """444 CTAs (three per SM: the grid of the mma.sync kernel on a long cache of the benchmark's head shape) fit the
    fixed scratch; split pairs, so the partials go through it."""
    lib = pkg._lib.lib()
    lens, cap, n_layers = [8000], 8192, 8
    case = build_case(oracle, n_layers, 1, 40, 8, 128, lens, cap, seed=11)
    dev = {k: (v.to(cuda_device) if isinstance(v, torch.Tensor) else v) for k, v in case.items()}
    shape = pkg.make_shape(40, dev["k_cache"], dev["v_cache"], dev["k_scale"])
    seq = torch.tensor(lens, dtype=torch.int32, device=cuda_device)
    ref = oracle.decode_step_reference(case["q"], case["k_cache"], case["v_cache"], case["k_scale"], case["v_scale"], lens, cap)
    status = torch.zeros(1, dtype=torch.int32, device=cuda_device)
    for call in range(2):
        out = torch.full((n_layers, 1, 40, 128), float("nan"), dtype=torch.bfloat16, device=cuda_device)
        rc = _call_static(lib, shape, dev, seq, 128 ** -0.5, 444, out, status)
        assert rc == 0, lib.b200attn_error_string(rc)
        torch.cuda.synchronize()
        assert status.item() == 0
        m = oracle.error_metrics(out.cpu(), ref)
        assert m["max_abs"] <= TOL_MAX_ABS and m["cosine"] >= TOL_COSINE, (call, m)


def test_static_scratch_rejects_what_does_not_fit(pkg, cuda_device):
    """Refusals happen on the host, before the shared scratch is touched or anything is launched.  The
    pointers are real (small) tensors all the same: should the order of the checks ever change, the
    test gets a wrong return code rather than a kernel running on invented addresses."""
    lib = pkg._lib.lib()
    big = pkg.B200AttnShape(64, 16, 40, 8, 128, 1024, 0, 0, 0, 0)
    buf = torch.zeros(4096, dtype=torch.uint8, device=cuda_device)
    a = buf.data_ptr()
    rc = lib.b200attn_decode_static(ctypes.byref(big), a, a, a, a, a, a, 0, 0.1, 4000, a, a, None)
    assert rc == pkg._lib.ERR_TOO_LARGE
    assert b"8 MiB" in lib.b200attn_error_string(rc)
    assert lib.b200attn_decode_static(None, a, a, a, a, a, a, 0, 0.1, 0, a, a, None) == pkg._lib.ERR_NULL
    small = pkg.B200AttnShape(1, 1, 40, 8, 128, 64, 0, 0, 0, 0)
    assert lib.b200attn_decode_static(ctypes.byref(small), a + 4, a, a, a, a, a, 0, 0.1, 0, a, a, None) == pkg._lib.ERR_ALIGN
    assert lib.b200attn_decode_static(ctypes.byref(small), a, a, a, a, a, a, 0, 0.1, -2, a, a, None) == pkg._lib.ERR_SPLITS
    torch.cuda.synchronize()
    assert int(buf.max()) == 0
