"""The shared library builds for sm_100a, loads without a GPU and exports every declared symbol."""

import ctypes
import re
from pathlib import Path

import pytest
import torch

from flashbob_b200 import _lib, build

ROOT = Path(__file__).resolve().parents[1]


def _declared_symbols():
    text = (ROOT / "include" / "bob_sm100.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(bob_sm100_[a-z0-9_]+)\s*\(", text)))


def test_library_builds_and_exports_every_declared_symbol():
    lib_path = build.build_library()
    assert lib_path.exists()
    lib = ctypes.CDLL(str(lib_path))
    declared = _declared_symbols()
    assert declared, "no declarations found in include/bob_sm100.h"
    for name in declared:
        assert hasattr(lib, name), f"{name} declared but not exported"
    assert set(declared) == set(_lib.SYMBOLS), "ctypes binding and header disagree"


def test_host_only_entry_points():
    lib = _lib.load()
    assert lib.bob_sm100_version() >= 100
    assert lib.bob_sm100_error_string(0) == b"ok"
    assert b"head dimension" in lib.bob_sm100_error_string(-4)
    g = _lib.Geom()
    g.B, g.Hq, g.Hkv, g.Nq, g.Nk, g.D = 2, 8, 2, 1000, 1000, 64
    fwd = lib.bob_sm100_workspace_bytes(_lib.STAGE_FWD, ctypes.byref(g))
    bwd2 = lib.bob_sm100_workspace_bytes(_lib.STAGE_BWD2, ctypes.byref(g))
    assert fwd == 256
    assert bwd2 >= 256 + 2 * 2 * 8 * 1000 * 4 and bwd2 % 256 == 0


def test_geometry_struct_matches_the_header_layout():
    # 10 int32, 2 int64, float + int32, 9 x 3 int64
    assert ctypes.sizeof(_lib.Geom) == 40 + 16 + 8 + 9 * 24


def test_cuda_route_has_no_fallback(monkeypatch, tmp_path):
    """With the library missing, loading raises instead of silently computing elsewhere."""
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "_LIB_PATH", tmp_path / "absent.so")
    with pytest.raises(_lib.BobSm100Error, match="no fallback"):
        _lib.load()


def test_kernel_wrappers_refuse_cpu_tensors():
    from flashbob_b200 import ops

    t = torch.zeros(1, 1, 16, 64, dtype=torch.bfloat16)
    with pytest.raises(ValueError, match="CUDA"):
        ops.attention_forward(t, t, t, is_causal=True, window_size=0, q_offset=0, k_offset=0, scale=None)
