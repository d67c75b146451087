"""CPU tests of the C-ABI: the library loads, exports every declared symbol, and validates
arguments on the host before any launch (no compute call needs a GPU here)."""
import ctypes
import re
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]


def declared_symbols():
    text = (ROOT / "include" / "b200attn.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(b200attn_\w+)\s*\(", text)))


def test_header_declares_the_expected_entry_points():
    syms = declared_symbols()
    for name in ("b200attn_kv_quant_append", "b200attn_decode", "b200attn_append_decode", "b200attn_pick_splits",
                 "b200attn_workspace_bytes", "b200attn_version"):
        assert name in syms


def test_library_exports_every_declared_symbol(pkg):
    lib = pkg._lib.lib()
    for name in declared_symbols():
        assert hasattr(lib, name), f"{name} declared in include/b200attn.h but not exported"
        assert name in pkg._lib.PROTOTYPES, f"{name} has no ctypes prototype"
    assert lib.b200attn_version() == 100


def _shape(pkg, **kw):
    base = dict(n_layers=64, batch=1, h_q=40, h_kv=8, head_dim=128, capacity=8192, scale_mode=0, reserved=0,
                k_layer_stride=0, v_layer_stride=0)
    base.update(kw)
    return pkg.B200AttnShape(**base)


def test_pick_splits_and_workspace_are_pure_host_functions(pkg):
    lib = pkg._lib.lib()
    s = _shape(pkg)
    n = lib.b200attn_pick_splits(ctypes.byref(s), 8192, 148, pkg._lib.VARIANT_MMA)
    assert n > 0 and n % 148 == 0          # persistent grid: a multiple of the SM count
    n1 = lib.b200attn_pick_splits(ctypes.byref(s), 8192, 148, pkg._lib.VARIANT_SIMT)
    assert 1 <= n1 <= 256
    short = _shape(pkg, n_layers=1)
    assert lib.b200attn_pick_splits(ctypes.byref(short), 64, 148, pkg._lib.VARIANT_SIMT) == 1
    out = ctypes.c_size_t(0)
    assert lib.b200attn_workspace_bytes(ctypes.byref(s), n, pkg._lib.VARIANT_MMA, ctypes.byref(out)) == 0
    assert out.value >= n * 2 * 5 * 128 * 4 + 64 * 8 * 4
    assert lib.b200attn_workspace_bytes(ctypes.byref(s), n1, pkg._lib.VARIANT_SIMT, ctypes.byref(out)) == 0
    assert out.value == 64 * 8 * n1 * (5 * 128 + 16) * 4


@pytest.mark.parametrize("kw,code", [
    (dict(head_dim=96), "ERR_SHAPE"), (dict(h_q=41), "ERR_SHAPE"), (dict(h_q=72), "ERR_SHAPE"),
    (dict(capacity=0), "ERR_SHAPE"), (dict(scale_mode=3), "ERR_SHAPE"), (dict(reserved=1), "ERR_SHAPE"),
    (dict(k_layer_stride=8), "ERR_SHAPE"), (dict(k_layer_stride=8192 * 8 * 128 + 8), "ERR_ALIGN"),
])
def test_bad_shapes_are_rejected_on_the_host(pkg, kw, code):
    lib = pkg._lib.lib()
    s = _shape(pkg, **kw)
    assert lib.b200attn_pick_splits(ctypes.byref(s), 128, 148, 0) == getattr(pkg._lib, code)


def test_null_and_misaligned_arguments_launch_nothing(pkg):
    """All of these return before the first CUDA call, so they run without a GPU."""
    lib = pkg._lib.lib()
    L = pkg._lib
    s = _shape(pkg)
    a = 0x10000  # fake, aligned, never dereferenced: validation fails first
    assert lib.b200attn_decode(None, a, a, a, a, a, a, 0, 0.1, 0, 0, a, 1 << 30, a, a, None) == L.ERR_NULL
    assert lib.b200attn_decode(ctypes.byref(s), None, a, a, a, a, a, 0, 0.1, 0, 0, a, 1 << 30, a, a, None) == L.ERR_NULL
    assert lib.b200attn_decode(ctypes.byref(s), a + 4, a, a, a, a, a, 0, 0.1, 0, 0, a, 1 << 30, a, a, None) == L.ERR_ALIGN
    assert lib.b200attn_decode(ctypes.byref(s), a, a, a, a, a, a, 0, 0.1, 7, 0, a, 1 << 30, a, a, None) == L.ERR_VARIANT
    assert lib.b200attn_decode(ctypes.byref(s), a, a, a, a, a, a, 0, 0.1, 0, 296, a, 16, a, a, None) == L.ERR_WORKSPACE
    assert lib.b200attn_decode(ctypes.byref(s), a, a, a, a, a, a, 0, 0.1, 0, -3, a, 1 << 30, a, a, None) == L.ERR_SPLITS
    assert lib.b200attn_kv_quant_append(ctypes.byref(s), None, a, a, a, a, a, a, 1, a, None) == L.ERR_NULL
    assert lib.b200attn_kv_quant_append_bulk(ctypes.byref(s), 9000, a, a, a, a, a, a, a, 1, a, None) == L.ERR_CAPACITY
    tok = _shape(pkg, scale_mode=1)   # per-token scales: the SIMT and all-tcgen05 kernels, not the mma.sync ones
    assert lib.b200attn_decode(ctypes.byref(tok), a, a, a, a, a, a, 0, 0.1, L.VARIANT_MMA, 0, a, 1 << 30, a, a, None) == L.ERR_SHAPE
    assert b"aligned" in lib.b200attn_error_string(L.ERR_ALIGN)


def test_python_wrappers_refuse_cpu_tensors(pkg):
    import torch
    kc = torch.zeros(1, 1, 8, 64, 128, dtype=torch.uint8)
    sc = torch.ones(1, 8)
    shape = pkg.make_shape(40, kc, kc, sc)
    assert (shape.n_layers, shape.h_kv, shape.capacity, shape.scale_mode) == (1, 8, 64, 0)
    with pytest.raises(ValueError):
        pkg.kv_quant_append(torch.zeros(1, 1, 8, 128, dtype=torch.bfloat16), torch.zeros(1, 1, 8, 128, dtype=torch.bfloat16),
                            kc, kc, sc, sc, torch.zeros(1, dtype=torch.int32), status=torch.zeros(1, dtype=torch.int32))


def test_kernel_choice_is_a_pure_host_function(pkg):
    """b200attn_resolve_variant: what AUTO stands for on a shape, explicit requests echoed or refused."""
    lib, L = pkg._lib.lib(), pkg._lib
    r = lambda shape, v=0: lib.b200attn_resolve_variant(ctypes.byref(shape), v)   # noqa: E731
    assert r(_shape(pkg)) == L.VARIANT_UMMA2                                   # the benchmark shape, depth 8192
    assert r(_shape(pkg, capacity=32768 + 256)) == L.VARIANT_UMMA2
    assert r(_shape(pkg, capacity=1024)) == L.VARIANT_MMA                       # short cache
    assert r(_shape(pkg, n_layers=1, capacity=2048)) == L.VARIANT_MMA           # too few tiles per CTA
    assert r(_shape(pkg, h_q=24, h_kv=4, head_dim=256)) == L.VARIANT_UMMA2      # the reference model's shape: group 6, head_dim 256
    assert r(_shape(pkg, scale_mode=1)) == L.VARIANT_UMMA2                      # per-token scales, long cache
    assert r(_shape(pkg, scale_mode=1, capacity=512)) == L.VARIANT_SIMT         # per-token scales, short cache
    assert r(_shape(pkg, h_q=8, h_kv=1, batch=16, capacity=16640)) == L.VARIANT_UMMA2   # group 8
    # KV-head shards of the benchmark shape: a half keeps the all-tcgen05 kernel, a quarter and an eighth (55 and 28 tiles
    # per SM) do not, unless their scales are per token (the mma.sync kernel does not take those); an eighth at depth
    # 32768 keeps it
    assert r(_shape(pkg, h_q=20, h_kv=4)) == L.VARIANT_UMMA2
    assert r(_shape(pkg, h_q=10, h_kv=2)) == L.VARIANT_MMA
    assert r(_shape(pkg, h_q=5, h_kv=1)) == L.VARIANT_MMA
    assert r(_shape(pkg, h_q=5, h_kv=1, scale_mode=1)) == L.VARIANT_UMMA2
    assert r(_shape(pkg, h_q=5, h_kv=1, capacity=32768 + 256)) == L.VARIANT_UMMA2
    one = _shape(pkg, h_q=5, h_kv=1)
    assert lib.b200attn_pick_splits(ctypes.byref(one), 8192, 148, 0) == 296     # two CTAs per SM for the small shard
    assert lib.b200attn_pick_splits(ctypes.byref(_shape(pkg)), 8192, 148, L.VARIANT_MMA) == 444
    for v in (L.VARIANT_SIMT, L.VARIANT_MMA, L.VARIANT_UMMA2):
        assert r(_shape(pkg), v) == v
    assert r(_shape(pkg, h_q=48, h_kv=8), L.VARIANT_UMMA2) == L.VARIANT_UMMA2   # group 6
    assert r(_shape(pkg, scale_mode=1), L.VARIANT_MMA) == L.ERR_SHAPE
    assert r(_shape(pkg), 9) == L.ERR_VARIANT
    assert r(_shape(pkg, head_dim=96)) == L.ERR_SHAPE
    # the workspace follows the resolved kernel: one CTA per SM for the all-tcgen05 kernel
    s = _shape(pkg)
    n = lib.b200attn_pick_splits(ctypes.byref(s), 8192, 148, 0)
    assert n == 148
    out = ctypes.c_size_t(0)
    assert lib.b200attn_workspace_bytes(ctypes.byref(s), n, 0, ctypes.byref(out)) == 0
    assert out.value >= n * 2 * (5 * 128 + 16) * 4 + (64 * 8 + 1) * 4


def test_step_and_producer_entry_points_validate_before_launching(pkg):
    lib, L = pkg._lib.lib(), pkg._lib
    s = _shape(pkg)
    a = 0x10000  # fake, aligned, never dereferenced: validation fails first
    # b200attn_append_decode: NULL new rows with the one-launch kernel, bad variant
    assert lib.b200attn_append_decode(ctypes.byref(s), a, None, a, a, a, a, a, a, 1, 0.1, 0, 0, a, 1 << 30, a, a, None) == L.ERR_NULL
    assert lib.b200attn_append_decode(ctypes.byref(s), a, a, a, a, a, a, a, a, 1, 0.1, 0, 0, a, 16, a, a, None) == L.ERR_WORKSPACE
    assert lib.b200attn_append_decode(ctypes.byref(s), a, a, a, a, a, a, a, a, 1, 0.1, 0, 0, a, 1 << 30, None, a, None) == L.ERR_NULL
    # b200attn_append_decode_peers: peers missing, wrong head total, NULL peer buffer, NULL flag
    peers = L.B200AttnPeerOut(2, 0, 80, 0, (ctypes.c_void_p * 8)(a, a))
    args = (a, a, a, a, a, a, a, a, 1, 0.1, 0, 0, a, 1 << 30)
    assert lib.b200attn_append_decode_peers(ctypes.byref(s), None, *args, None, a, None) == L.ERR_NULL
    bad_total = L.B200AttnPeerOut(2, 0, 40, 0, (ctypes.c_void_p * 8)(a, a))
    assert lib.b200attn_append_decode_peers(ctypes.byref(s), ctypes.byref(bad_total), *args, None, a, None) == L.ERR_SHAPE
    hole = L.B200AttnPeerOut(2, 0, 80, 0, (ctypes.c_void_p * 8)(a, None))
    assert lib.b200attn_append_decode_peers(ctypes.byref(s), ctypes.byref(hole), *args, None, a, None) == L.ERR_NULL
    flags = (ctypes.c_void_p * 8)(a, None)
    assert lib.b200attn_append_decode_peers(ctypes.byref(s), ctypes.byref(peers), *args, flags, a, None) == L.ERR_NULL
    # b200attn_qk_norm_rope_append: NULL input, rotary_dim not a whole number of lanes / too large, misaligned
    pargs = lambda **kw: [kw.get("q", a), a, a, a, a, ctypes.c_float(kw.get("eps", 1e-6)), a, a, kw.get("r", 64), kw.get("qo", a), None,  # noqa: E731
                          a, a, a, a, a, 1, a, None]
    assert lib.b200attn_qk_norm_rope_append(ctypes.byref(s), *pargs(q=None)) == L.ERR_NULL
    assert lib.b200attn_qk_norm_rope_append(ctypes.byref(s), *pargs(r=12)) == L.ERR_SHAPE
    assert lib.b200attn_qk_norm_rope_append(ctypes.byref(s), *pargs(r=136)) == L.ERR_SHAPE
    assert lib.b200attn_qk_norm_rope_append(ctypes.byref(s), *pargs(eps=float("nan"))) == L.ERR_SHAPE
    assert lib.b200attn_qk_norm_rope_append(ctypes.byref(s), *pargs(qo=a + 8)) == L.ERR_ALIGN
