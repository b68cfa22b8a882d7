"""ctypes binding of libbob_sm100.so (the C ABI declared in include/bob_sm100.h).

There is no fallback: if the library is missing or a call fails, an exception is raised.
"""

from __future__ import annotations

import ctypes
import os
import threading
from pathlib import Path

_PKG = Path(__file__).resolve().parent
_LIB_PATH = Path(os.environ.get("BOB_SM100_LIB", _PKG / "libbob_sm100.so"))

FP16, BF16 = 0, 1
STAGE_FWD, STAGE_BWD1, STAGE_BWD2 = 0, 1, 2

_vp = ctypes.c_void_p


class Geom(ctypes.Structure):
    """Mirror of `bob_sm100_geom`."""

    _fields_ = [
        ("B", ctypes.c_int32), ("Hq", ctypes.c_int32), ("Hkv", ctypes.c_int32),
        ("Nq", ctypes.c_int32), ("Nk", ctypes.c_int32), ("D", ctypes.c_int32),
        ("dtype", ctypes.c_int32), ("is_causal", ctypes.c_int32), ("window", ctypes.c_int32),
        ("device", ctypes.c_int32),
        ("q_offset", ctypes.c_int64), ("k_offset", ctypes.c_int64),
        ("scale", ctypes.c_float), ("reserved", ctypes.c_int32),
        ("q_strides", ctypes.c_int64 * 3), ("k_strides", ctypes.c_int64 * 3),
        ("v_strides", ctypes.c_int64 * 3), ("out_strides", ctypes.c_int64 * 3),
        ("do_strides", ctypes.c_int64 * 3), ("dq_strides", ctypes.c_int64 * 3),
        ("uq_strides", ctypes.c_int64 * 3), ("uk_strides", ctypes.c_int64 * 3),
        ("uv_strides", ctypes.c_int64 * 3),
    ]


# every symbol include/bob_sm100.h declares: name -> (restype, argtypes)
SYMBOLS = {
    "bob_sm100_version": (ctypes.c_int, []),
    "bob_sm100_error_string": (ctypes.c_char_p, [ctypes.c_int]),
    "bob_sm100_workspace_bytes": (ctypes.c_size_t, [ctypes.c_int, ctypes.POINTER(Geom)]),
    "bob_sm100_kernel_launches": (ctypes.c_int, [ctypes.c_int, ctypes.POINTER(Geom)]),
    "bob_sm100_read_status": (ctypes.c_int, [_vp, _vp]),
    "bob_sm100_last_status": (ctypes.c_int, [ctypes.c_int]),
    "bob_sm100_fwd": (ctypes.c_int, [ctypes.POINTER(Geom)] + [_vp] * 7),
    "bob_sm100_bwd1": (ctypes.c_int, [ctypes.POINTER(Geom)] + [_vp] * 13),
    "bob_sm100_bwd2": (ctypes.c_int, [ctypes.POINTER(Geom)] + [_vp] * 18),
    "bob_sm100_bwd2_part": (ctypes.c_int, [ctypes.c_int, ctypes.POINTER(Geom)] + [_vp] * 18),
    "bob_sm100_noalloc_max_rows": (ctypes.c_size_t, []),
    "bob_sm100_noalloc_read_status": (ctypes.c_int, [ctypes.c_int, _vp]),
    "bob_sm100_bwd2_noalloc": (ctypes.c_int, [ctypes.POINTER(Geom)] + [_vp] * 17),
    "bob_sm100_timeout_selftest": (ctypes.c_int, [_vp, _vp]),
    "bob_sm100_selftest": (ctypes.c_int, [_vp, _vp, ctypes.c_int, _vp, _vp, _vp]),
}

_lib = None
_lock = threading.Lock()


class BobSm100Error(RuntimeError):
    pass


def load():
    """Load the shared library once; raise if it is absent or lacks a declared symbol."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is not None:
            return _lib
        if not _LIB_PATH.exists():
            raise BobSm100Error(
                f"{_LIB_PATH} not found: build it with `python -m flashbob_b200.build` "
                "(needs nvcc); the CUDA route has no fallback")
        lib = ctypes.CDLL(str(_LIB_PATH))
        for name, (res, args) in SYMBOLS.items():
            if not hasattr(lib, name):
                raise BobSm100Error(f"{_LIB_PATH} does not export {name}")
            fn = getattr(lib, name)
            fn.restype = res
            fn.argtypes = args
        _lib = lib
    return _lib


def check(rc: int, what: str) -> None:
    if rc != 0:
        msg = load().bob_sm100_error_string(rc).decode()
        raise BobSm100Error(f"{what} failed with code {rc}: {msg}")
