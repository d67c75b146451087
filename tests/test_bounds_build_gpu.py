"""The index-checking build (python qwen38-5080_b200/build.py --bounds; loaded when B200ATTN_BOUNDS=1): the same
kernels with their index computations checked on the device.  A sweep over every length 1..160 (each position in and
across the 64- and 128-token tiles), several CTA counts, attention alone and the fused step, ragged batches and the
tensor-parallel output paths with local stand-ins for the peers must never raise B200ATTN_STATUS_BOUNDS, and the
results must be the regular build's.  Runs in a child process: the flavour is chosen when the package is imported."""
import os
import subprocess
import sys
from pathlib import Path

import pytest

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parents[1]

SWEEP = r'''
import ctypes, importlib, sys
sys.path.insert(0, "ROOT"); sys.path.insert(0, "ROOT/tests")
import torch
from oracle import ref_attention as oracle
from helpers import build_case, assert_parity
pkg = importlib.import_module("qwen38-5080_b200")
L = pkg._lib
assert L.lib().b200attn_bounds_checked() == 1
dev = torch.device("cuda:0")
n_layers, h_q, h_kv, d, cap = 2, 40, 8, 128, 192
g = torch.Generator().manual_seed(1)
launches = 0
for length in range(1, 161):
    batch = 1 if length % 5 else 3
    lens = [length] if batch == 1 else [length, max(1, length // 2), 0]
    case = build_case(oracle, n_layers, batch, h_q, h_kv, d, lens, cap, seed=900 + length, fill_byte=0xFF)
    devc = {k: (v.to(dev) if isinstance(v, torch.Tensor) else v) for k, v in case.items()}
    ref = None
    if length % 16 == 1:
        ck, cv = case["k_cache"].clone(), case["v_cache"].clone()
        for b, n in enumerate(lens):
            ck[:, b, :, n:] = 0; cv[:, b, :, n:] = 0
        ref = oracle.decode_step_reference(case["q"], ck, cv, case["k_scale"], case["v_scale"], lens, cap)
    kn = torch.randn(n_layers, batch, h_kv, d, generator=g).to(torch.bfloat16).to(dev)
    vn = torch.randn(n_layers, batch, h_kv, d, generator=g).to(torch.bfloat16).to(dev)
    for variant, ctas in (("mma", 0), ("mma", 37), ("umma2", 0), ("umma2", 5)):
        shape = pkg.make_shape(h_q, devc["k_cache"], devc["v_cache"], devc["k_scale"])
        ws = pkg.Workspace(shape, dev, variant=variant, num_splits=ctas)
        seq = torch.tensor(lens, dtype=torch.int32, device=dev)
        out = pkg.decode_attention(devc["q"], devc["k_cache"], devc["v_cache"], devc["k_scale"], devc["v_scale"], seq, workspace=ws)
        kc, vc, pos = devc["k_cache"].clone(), devc["v_cache"].clone(), seq.clone()
        pkg.append_decode(devc["q"], kn, vn, kc, vc, devc["k_scale"], devc["v_scale"], pos, workspace=ws)
        torch.cuda.synchronize()
        launches += 2
        st = ws.read_status()
        assert st & L.STATUS_BOUNDS == 0 and st == 0, (length, variant, ctas, st)
        if ref is not None:
            for b, n in enumerate(lens):
                if n == 0: ref[:, b] = 0
            assert_parity(oracle, out.cpu(), ref, f"L={length} {variant} {ctas}")
# tensor-parallel output paths with local buffers standing in for the peers (rank 0 of 2)
case = build_case(oracle, n_layers, 1, 20, 4, d, [150], cap, seed=7)
devc = {k: (v.to(dev) if isinstance(v, torch.Tensor) else v) for k, v in case.items()}
shape = pkg.make_shape(20, devc["k_cache"], devc["v_cache"], devc["k_scale"])
seq = torch.tensor([150], dtype=torch.int32, device=dev)
for variant in ("mma", "umma2"):
    ws = pkg.Workspace(shape, dev, variant=variant)
    nbytes = L.lib().b200attn_peer_staging_bytes(ctypes.byref(shape), 2)
    mine = torch.zeros(nbytes // 8, dtype=torch.int64, device=dev); other = torch.zeros_like(mine)
    slot = nbytes // 8 // 4
    mine.view(2, 2, slot)[1, 1] = (1 << 32)                      # the "other rank's" packets of step 1: zeros carrying the step number
    full = torch.zeros(n_layers, 1, 40, d, dtype=torch.bfloat16, device=dev)
    step = torch.zeros(1, dtype=torch.int32, device=dev)
    outp = (ctypes.c_void_p * 8)(); outp[0] = full.data_ptr()
    peers = L.B200AttnPeerOut(2, 0, 40, L.GATHER_PACKETS, outp, (ctypes.c_void_p * 8)(),
                              (ctypes.c_void_p * 8)(mine.data_ptr(), other.data_ptr()), step.data_ptr())
    rc = L.lib().b200attn_decode_peers(ctypes.byref(shape), ctypes.byref(peers), devc["q"].data_ptr(), devc["k_cache"].data_ptr(),
                                       devc["v_cache"].data_ptr(), devc["k_scale"].data_ptr(), devc["v_scale"].data_ptr(), seq.data_ptr(), 0,
                                       d ** -0.5, L.VARIANTS[variant], ws.num_splits, ws.buf.data_ptr(), ws.nbytes, ws.status.data_ptr(),
                                       torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert rc == 0 and ws.read_status() == 0 and int(step.item()) == 1, (variant, rc, ws.read_status())
    launches += 1
print("bounds sweep ok:", launches, "launches")
'''.replace("ROOT", str(ROOT))


def test_index_checking_build_stays_silent(cuda_device):
    env = dict(os.environ, B200ATTN_BOUNDS="1")
    res = subprocess.run([sys.executable, "-c", SWEEP], capture_output=True, text=True, env=env, timeout=1200)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-4000:]
    assert "bounds sweep ok" in res.stdout
