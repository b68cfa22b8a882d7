"""Public surface and CPU numerics of the operator.
Mirrors the reference's unit tests (reference: tests/unit/test_public_api.py:17-75) with the
materialized reference function replaced by the oracle and the committed golden fixtures."""

import ast
import subprocess
import sys
from pathlib import Path

import numpy as np
import torch

import bob
import flashbob_b200
from oracle import bob_oracle as O

ROOT = Path(__file__).resolve().parents[1]
GOLDEN = Path(__file__).parent / "golden"


def _second_grad(op, q, k, v, dO, bars, **kw):
    q, k, v, dO = (t.detach().clone().requires_grad_(True) for t in (q, k, v, dO))
    out = op(q, k, v, **kw)
    first = torch.autograd.grad(out, (q, k, v), dO, create_graph=True)
    return (out, *first, *torch.autograd.grad(first, (q, k, v, dO), bars))


def test_public_surface_contains_exactly_one_operator():
    assert bob.__all__ == ["sdpa_bob"]
    assert flashbob_b200.__all__ == ["sdpa_bob"]
    assert callable(bob.sdpa_bob) and bob.sdpa_bob is flashbob_b200.sdpa_bob


def test_importing_the_package_imports_no_attention_library_and_no_oracle():
    probe = subprocess.run(
        [sys.executable, "-c",
         "import sys; import bob; "
         "print(any(m in sys.modules for m in ('flash_attn', 'triton', 'flashinfer', 'oracle', "
         "'oracle.bob_oracle')))"],
        capture_output=True, text=True, check=True, cwd=ROOT)
    assert probe.stdout.strip() == "False"


def test_product_sources_never_reference_the_oracle():
    for path in (ROOT / "flashbob_b200").rglob("*"):
        if path.suffix in (".py", ".cu", ".cuh", ".h"):
            assert "oracle" not in path.read_text(), path


def _golden_case(name):
    z = np.load(GOLDEN / f"{name}.npz", allow_pickle=True)
    meta = ast.literal_eval(str(z["meta"]))
    g = torch.Generator().manual_seed(meta["seed"])
    q_shape, kv_shape = (1, meta["hq"], meta["nq"], meta["d"]), (1, meta["hkv"], meta["nk"], meta["d"])
    r = lambda s: torch.randn(s, dtype=torch.float32, generator=g)
    t = (r(q_shape), r(kv_shape), r(kv_shape), r(q_shape), r(q_shape), r(kv_shape), r(kv_shape))
    return z, meta, t


def test_cpu_square_second_gradient_matches_reference_fixture():
    z, meta, (q, k, v, dO, bq, bk, bv) = _golden_case("unit_square")
    got = _second_grad(bob.sdpa_bob, q, k, v, dO, (bq, bk, bv), **meta["kw"])
    for n, t in zip(O.OUTPUT_NAMES, got):
        torch.testing.assert_close(t, torch.from_numpy(z[f"op32_{n}"]), rtol=2e-5, atol=2e-5)
        torch.testing.assert_close(t.double(), torch.from_numpy(z[f"ref64_{n}"]), rtol=2e-5, atol=2e-5)


def test_cpu_rectangular_second_gradient_matches_reference_fixture():
    z, meta, (q, k, v, dO, bq, bk, bv) = _golden_case("unit_rect")
    got = _second_grad(bob.sdpa_bob, q, k, v, dO, (bq, bk, bv), **meta["kw"])
    for n, t in zip(O.OUTPUT_NAMES, got):
        torch.testing.assert_close(t, torch.from_numpy(z[f"op32_{n}"]), rtol=2e-5, atol=2e-5)
        torch.testing.assert_close(t.double(), torch.from_numpy(z[f"ref64_{n}"]), rtol=2e-5, atol=2e-5)


def test_cpu_window_and_offsets_match_fixtures():
    for name in ("window", "rect", "rect_offsets", "causal", "noncausal"):
        z, meta, (q, k, v, dO, bq, bk, bv) = _golden_case(name)
        got = _second_grad(bob.sdpa_bob, q, k, v, dO, (bq, bk, bv), **meta["kw"])
        for n, t in zip(O.OUTPUT_NAMES, got):
            ref = torch.from_numpy(z[f"op32_{n}"])
            assert (t - ref).abs().max().item() <= 1e-5 * max(1.0, ref.abs().max().item()), (name, n)


def test_config0_cpu_chain_within_1e5_relative_of_fp64():
    """The CPU benchmark configuration: fp32 MHA B=1 H=2 S=128 D=64 causal, scale 1/8."""
    z = np.load(GOLDEN / "config0_chain.npz")
    g = torch.Generator().manual_seed(0)
    q, k, v = (torch.randn((1, 2, 128, 64), dtype=torch.float32, generator=g) for _ in range(3))
    got = O.loss_chain(bob.sdpa_bob, q, k, v, is_causal=True, scale=1 / 8.0)
    for n in ("out", "dq", "dk", "dv", "ddq", "ddk", "ddv"):
        m = O.error_metrics(got[n], torch.from_numpy(z[f"math64_{n}"]))
        assert m["max_abs_rel"] <= 1e-5 and m["l2_rel"] <= 1e-5, (n, m)


def test_right_aligned_default_offset():
    q = torch.randn(1, 1, 3, 8)
    k, v = torch.randn(1, 1, 7, 8), torch.randn(1, 1, 7, 8)
    a = bob.sdpa_bob(q, k, v, is_causal=True)
    b = bob.sdpa_bob(q, k, v, is_causal=True, q_offset=4)
    c = bob.sdpa_bob(q, k, v, is_causal=True, q_offset=14, k_offset=10)
    torch.testing.assert_close(a, b)
    torch.testing.assert_close(a, c)
    ref = O.attention_dense(q, k, v, is_causal=True, q_offset=4)
    torch.testing.assert_close(a, ref, rtol=1e-5, atol=1e-6)
