"""Build libb200attn.so in-tree with nvcc for sm_100a (cross-compiles without a GPU).

    python qwen38-5080_b200/build.py [-v] [--bounds]

--bounds builds libb200attn_bounds.so instead: the same sources with -DB200ATTN_BOUNDS=1, in which
the kernels check the indices of their global-memory accesses (cache rows, copy coordinates, partial
slots and their owners, output and packet positions) and report a violation as B200ATTN_STATUS_BOUNDS in the
status word (never a trap).  Setting B200ATTN_BOUNDS=1 in the environment makes the package load it.
"""
from __future__ import annotations

import fcntl
import hashlib
import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
CSRC = PKG_DIR / "csrc"
LIB_PATH = PKG_DIR / "libb200attn.so"
STAMP_PATH = PKG_DIR / "libb200attn.so.hash"
BOUNDS_LIB_PATH = PKG_DIR / "libb200attn_bounds.so"


def lib_path(bounds: bool = False) -> Path:
    return BOUNDS_LIB_PATH if bounds else LIB_PATH


def stamp_path(bounds: bool = False) -> Path:
    return Path(str(lib_path(bounds)) + ".hash")
SOURCES = ["api.cu", "append.cu", "decode_simt.cu", "decode_mma.cu", "decode_umma2.cu", "static_scratch.cu", "peer_barrier.cu", "producer.cu"]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
    "--cudart", "static",
]


def find_nvcc() -> str:
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        raise RuntimeError("nvcc not found: the CUDA library cannot be built")
    return nvcc


def sources() -> list[Path]:
    return [CSRC / s for s in SOURCES if (CSRC / s).exists()]


def source_hash() -> str:
    """Hash of everything the library is compiled from; the build bakes it into the library
    (b200attn_source_hash) so that a loader can tell a stale binary from a current one."""
    h = hashlib.sha256()
    deps = sorted(CSRC.glob("*.cu")) + sorted(CSRC.glob("*.cuh")) + [PKG_DIR.parent / "include" / "b200attn.h"]
    for d in deps:
        h.update(d.name.encode())
        h.update(d.read_bytes())
    return h.hexdigest()[:16]


def built_hash(bounds: bool = False) -> str | None:
    """The source hash recorded beside the library by the build that made it."""
    stamp, lib = stamp_path(bounds), lib_path(bounds)
    return stamp.read_text().strip() if stamp.exists() and lib.exists() else None


def needs_build(bounds: bool = False) -> bool:
    return built_hash(bounds) != source_hash()


def build(verbose: bool = False, force: bool = False, bounds: bool = False) -> Path:
    """Compile every .cu of csrc/ into libb200attn.so (bounds: the index-checking flavour,
    libb200attn_bounds.so).  Returns the library path.  Concurrent callers (the ranks of a
    multi-process run) are serialised by a file lock; the later ones find the library up to date."""
    if not force and not needs_build(bounds):
        return lib_path(bounds)
    with open(PKG_DIR / ".build.lock", "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        if not force and not needs_build(bounds):
            return lib_path(bounds)
        return _build_locked(verbose, bounds)


def _build_locked(verbose: bool, bounds: bool) -> Path:
    nvcc = find_nvcc()
    digest = source_hash()
    objs = []
    build_dir = PKG_DIR / ("build_bounds" if bounds else "build")
    build_dir.mkdir(exist_ok=True)
    LIB_PATH, STAMP_PATH = lib_path(bounds), stamp_path(bounds)
    procs = []
    for src in sources():
        obj = build_dir / (src.stem + ".o")
        cmd = [nvcc, *NVCC_FLAGS, f'-DB200ATTN_SOURCE_HASH="{digest}"', "-c", str(src), "-o", str(obj)]
        if bounds:
            cmd.insert(1, "-DB200ATTN_BOUNDS=1")
        if verbose:
            cmd += ["-Xptxas", "-v"]
        procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
        objs.append(obj)
    for src, proc in procs:
        out, _ = proc.communicate()
        if verbose or proc.returncode:
            sys.stderr.write(out)
        if proc.returncode:
            raise RuntimeError(f"nvcc failed on {src.name}")
    tmp = LIB_PATH.with_suffix(".so.tmp")
    cmd = [nvcc, "-shared", "--cudart", "static", "-o", str(tmp), *map(str, objs)]
    res = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if res.returncode:
        sys.stderr.write(res.stdout)
        raise RuntimeError(f"link of {LIB_PATH.name} failed")
    os.replace(tmp, LIB_PATH)
    STAMP_PATH.write_text(digest + "\n")
    return LIB_PATH


if __name__ == "__main__":
    print(build(verbose="-v" in sys.argv, force=True, bounds="--bounds" in sys.argv))
