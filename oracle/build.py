"""Compile the plain-C oracle (oracle/ref_attention.c) into oracle/libref_attention.so.

Test infrastructure only.  The reference is a pure-Python project (no C/C++ sources), so there
is nothing to compile into oracle/_ref/; this builds the C restatement and nothing else.
"""
from __future__ import annotations

import ctypes
import os
import shutil
import subprocess
from pathlib import Path

HERE = Path(__file__).resolve().parent
SRC = HERE / "ref_attention.c"
LIB = HERE / "libref_attention.so"


def build(force: bool = False) -> Path:
    if LIB.exists() and not force and LIB.stat().st_mtime >= SRC.stat().st_mtime:
        return LIB
    gcc = shutil.which("gcc")
    if gcc is None:
        raise RuntimeError("gcc not found: cannot build the C oracle")
    tmp = LIB.with_suffix(".so.tmp")
    base = [gcc, "-O2", "-fPIC", "-shared", "-std=c11", "-fno-fast-math", str(SRC), "-lm", "-o", str(tmp)]
    res = subprocess.run(base[:1] + ["-fopenmp"] + base[1:], capture_output=True, text=True)
    if res.returncode:  # no OpenMP runtime: build single-threaded
        res = subprocess.run(base, capture_output=True, text=True)
    if res.returncode:
        raise RuntimeError("C oracle build failed:\n" + res.stderr)
    os.replace(tmp, LIB)
    return LIB


def load() -> ctypes.CDLL:
    lib = ctypes.CDLL(str(build()))
    u8p, u16p, f32p, i32p = (ctypes.POINTER(t) for t in (ctypes.c_uint8, ctypes.c_uint16, ctypes.c_float, ctypes.c_int))
    lib.oracle_f32_to_e4m3.restype, lib.oracle_f32_to_e4m3.argtypes = ctypes.c_uint8, [ctypes.c_float]
    lib.oracle_e4m3_to_f32.restype, lib.oracle_e4m3_to_f32.argtypes = ctypes.c_float, [ctypes.c_uint8]
    lib.oracle_quantize.restype, lib.oracle_quantize.argtypes = None, [u16p, ctypes.c_float, u8p, ctypes.c_long]
    lib.oracle_decode_attention.restype = ctypes.c_int
    lib.oracle_decode_attention.argtypes = [ctypes.c_int] * 7 + [u16p, u8p, u8p, f32p, f32p, i32p, ctypes.c_float, u16p]
    return lib


if __name__ == "__main__":
    print(build(force=True))
