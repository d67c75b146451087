"""ctypes binding of libb200attn.so (the C-ABI declared in include/b200attn.h).

The library is the product: there is no Python or CPU fallback.  If the shared object is
missing and cannot be built, importing the ops fails loudly.
"""
from __future__ import annotations

import ctypes
import os
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
# B200ATTN_BOUNDS=1: the index-checking build of the same sources (build.py --bounds), for chasing a memory error
BOUNDS = os.environ.get("B200ATTN_BOUNDS") == "1"
LIB_PATH = PKG_DIR / ("libb200attn_bounds.so" if BOUNDS else "libb200attn.so")

c_void_p, c_int, c_float, c_size_t, c_ll = ctypes.c_void_p, ctypes.c_int, ctypes.c_float, ctypes.c_size_t, ctypes.c_longlong

# host-side error codes / status bits / variants (include/b200attn.h)
OK = 0
ERR_NULL, ERR_SHAPE, ERR_ALIGN, ERR_WORKSPACE, ERR_SPLITS, ERR_CUDA, ERR_CAPACITY, ERR_VARIANT, ERR_TOO_LARGE = range(-1, -10, -1)
STATUS_POS_AT_CAPACITY, STATUS_LEN_OVER_CAP, STATUS_WAIT_TIMEOUT, STATUS_LEN_NEGATIVE, STATUS_BOUNDS = 1, 2, 4, 8, 16
VARIANT_AUTO, VARIANT_SIMT, VARIANT_MMA, VARIANT_UMMA2 = 0, 1, 2, 4
VARIANTS = {"auto": VARIANT_AUTO, "simt": VARIANT_SIMT, "mma": VARIANT_MMA, "umma2": VARIANT_UMMA2}
SCALE_PER_HEAD, SCALE_PER_TOKEN = 0, 1
GATHER_STORES, GATHER_STORES_2BUF, GATHER_PACKETS = 1, 2, 3


class B200AttnShape(ctypes.Structure):
    _fields_ = [
        ("n_layers", c_int), ("batch", c_int), ("h_q", c_int), ("h_kv", c_int), ("head_dim", c_int),
        ("capacity", c_int), ("scale_mode", c_int), ("reserved", c_int),
        ("k_layer_stride", c_ll), ("v_layer_stride", c_ll),
    ]


class B200AttnPeerOut(ctypes.Structure):
    _fields_ = [("n_peers", c_int), ("rank", c_int), ("h_q_total", c_int), ("mode", c_int),
                ("out", c_void_p * 8), ("out_alt", c_void_p * 8), ("staging", c_void_p * 8), ("step", c_void_p)]


# name -> (restype, argtypes); every symbol include/b200attn.h declares
PROTOTYPES = {
    "b200attn_version": (c_int, []),
    "b200attn_bounds_checked": (c_int, []),
    "b200attn_source_hash": (ctypes.c_char_p, []),
    "b200attn_error_string": (ctypes.c_char_p, [c_int]),
    "b200attn_last_cuda_error": (c_int, []),
    "b200attn_pick_splits": (c_int, [ctypes.POINTER(B200AttnShape), c_int, c_int, c_int]),
    "b200attn_resolve_variant": (c_int, [ctypes.POINTER(B200AttnShape), c_int]),
    "b200attn_workspace_bytes": (c_int, [ctypes.POINTER(B200AttnShape), c_int, c_int, ctypes.POINTER(c_size_t)]),
    "b200attn_workspace_init": (c_int, [c_void_p, c_size_t, c_void_p]),
    "b200attn_kv_quant_append": (c_int, [ctypes.POINTER(B200AttnShape), c_void_p, c_void_p, c_void_p, c_void_p,
                                         c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p]),
    "b200attn_kv_quant_append_bulk": (c_int, [ctypes.POINTER(B200AttnShape), c_int, c_void_p, c_void_p, c_void_p,
                                              c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p]),
    "b200attn_decode": (c_int, [ctypes.POINTER(B200AttnShape), c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                c_void_p, c_int, c_float, c_int, c_int, c_void_p, c_size_t, c_void_p, c_void_p,
                                c_void_p]),
    "b200attn_decode_gated": (c_int, [ctypes.POINTER(B200AttnShape), c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                      c_void_p, c_void_p, c_int, c_float, c_int, c_int, c_void_p, c_size_t, c_void_p,
                                      c_void_p, c_void_p]),
    "b200attn_decode_peers": (c_int, [ctypes.POINTER(B200AttnShape), ctypes.POINTER(B200AttnPeerOut), c_void_p, c_void_p,
                                      c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_float, c_int, c_int, c_void_p,
                                      c_size_t, c_void_p, c_void_p]),
    "b200attn_peer_staging_bytes": (c_size_t, [ctypes.POINTER(B200AttnShape), c_int]),
    "b200attn_peer_barrier": (c_int, [ctypes.POINTER(c_void_p), c_int, c_int, c_void_p, c_void_p]),
    "b200attn_decode_static": (c_int, [ctypes.POINTER(B200AttnShape), c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                       c_void_p, c_int, c_float, c_int, c_void_p, c_void_p, c_void_p]),
    "b200attn_static_scratch_bytes": (c_size_t, []),
    "b200attn_append_decode": (c_int, [ctypes.POINTER(B200AttnShape), c_void_p, c_void_p, c_void_p, c_void_p,
                                       c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_float, c_int, c_int,
                                       c_void_p, c_size_t, c_void_p, c_void_p, c_void_p]),
    "b200attn_append_decode_peers": (c_int, [ctypes.POINTER(B200AttnShape), ctypes.POINTER(B200AttnPeerOut), c_void_p, c_void_p,
                                             c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_float, c_int,
                                             c_int, c_void_p, c_size_t, ctypes.POINTER(c_void_p), c_void_p, c_void_p]),
    "b200attn_qk_norm_rope_append": (c_int, [ctypes.POINTER(B200AttnShape), c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                             c_float, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
                                             c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p]),
    "b200attn_dequant_prefix": (c_int, [ctypes.POINTER(B200AttnShape), c_int, c_void_p, c_ll, c_void_p, c_void_p,
                                        c_void_p]),
    "b200attn_calibrate_scales": (c_int, [ctypes.POINTER(B200AttnShape), c_int, c_void_p, c_void_p, c_void_p]),
}

_lib = None


class B200AttnError(ValueError):
    """A host-side argument error reported by the library (nothing was launched)."""

    def __init__(self, code: int, where: str):
        self.code = code
        msg = lib().b200attn_error_string(code).decode()
        if code == ERR_CUDA:
            msg += f" (cudaError {lib().b200attn_last_cuda_error()})"
        super().__init__(f"{where}: {msg} [{code}]")


def lib() -> ctypes.CDLL:
    """Load the library, building it first when it is absent or was compiled from other sources than
    the ones beside it (the hash the build baked in is compared with the sources' hash)."""
    global _lib
    if _lib is not None:
        return _lib
    from . import build as _build
    want = _build.source_hash()
    if _build.needs_build(BOUNDS) or os.environ.get("B200ATTN_REBUILD") == "1":
        _build.build(force=os.environ.get("B200ATTN_REBUILD") == "1", bounds=BOUNDS)   # raises if nvcc is missing: no fallback
    if not LIB_PATH.exists():
        raise RuntimeError(f"{LIB_PATH} is missing: build it with `python {PKG_DIR / 'build.py'}`")
    handle = ctypes.CDLL(str(LIB_PATH))
    for name, (res, args) in PROTOTYPES.items():
        fn = getattr(handle, name)  # AttributeError if the build lost a symbol
        fn.restype, fn.argtypes = res, args
    have = handle.b200attn_source_hash().decode()
    if have != want:
        raise RuntimeError(f"{LIB_PATH} was built from other sources (library {have}, sources {want}): rebuild it with "
                           f"`python {PKG_DIR / 'build.py'}`")
    _lib = handle
    return _lib


def check(code: int, where: str) -> int:
    if code < 0:
        raise B200AttnError(code, where)
    return code
