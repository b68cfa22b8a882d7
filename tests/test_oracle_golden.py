"""The CPU oracle against fixtures produced by the reference's own functions.

Fixtures: tests/golden/*.npz (made by tests/golden/make_golden.py with the reference imported).
`ref64_*`  = the reference's materialized attention differentiated twice in fp64,
`math64_*` = the fp64 entry points under the reference operator,
`op32_*`   = the reference operator itself on CPU fp32 tensors.
"""

import ast
from pathlib import Path

import numpy as np
import pytest
import torch

from oracle import bob_oracle as O

GOLDEN = Path(__file__).parent / "golden"
CASES = ["unit_square", "unit_rect", "causal", "noncausal", "window", "gqa", "mqa", "rect",
         "rect_offsets"]


def _load(name):
    z = np.load(GOLDEN / f"{name}.npz", allow_pickle=True)
    meta = ast.literal_eval(str(z["meta"]))
    return z, meta


def _inputs(meta, dtype):
    q_shape = (1, meta["hq"], meta["nq"], meta["d"])
    kv_shape = (1, meta["hkv"], meta["nk"], meta["d"])
    g = torch.Generator().manual_seed(meta["seed"])
    r = lambda s: torch.randn(s, dtype=torch.float32, generator=g).to(dtype)
    return r(q_shape), r(kv_shape), r(kv_shape), r(q_shape), r(q_shape), r(kv_shape), r(kv_shape)


@pytest.mark.parametrize("name", CASES)
def test_autograd_oracle_matches_reference_fp64(name):
    z, meta = _load(name)
    q, k, v, dO, bq, bk, bv = _inputs(meta, torch.float64)
    got = O.second_order_autograd(q, k, v, dO, bq, bk, bv, **meta["kw"])
    for n in O.OUTPUT_NAMES:
        torch.testing.assert_close(got[n], torch.from_numpy(z[f"ref64_{n}"]), rtol=1e-11, atol=1e-12)
        if f"math64_{n}" in z:
            torch.testing.assert_close(got[n], torch.from_numpy(z[f"math64_{n}"]), rtol=1e-11, atol=1e-12)


@pytest.mark.parametrize("name", CASES)
def test_closed_form_oracle_matches_reference_fp64(name):
    z, meta = _load(name)
    q, k, v, dO, bq, bk, bv = _inputs(meta, torch.float64)
    got = O.bob_closed_form(q, k, v, dO, bq, bk, bv, **meta["kw"]).outputs()
    for n in O.OUTPUT_NAMES:
        torch.testing.assert_close(got[n], torch.from_numpy(z[f"ref64_{n}"]), rtol=1e-10, atol=1e-12)


@pytest.mark.parametrize("name", [c for c in CASES if c not in ("gqa", "mqa")])
def test_cpu_route_restatement_matches_reference_operator_fp32(name):
    """fp32 CPU tolerance of the task: 1e-5 relative (to the largest reference magnitude)."""
    z, meta = _load(name)
    q, k, v, dO, bq, bk, bv = _inputs(meta, torch.float32)
    q, k, v, dO = (t.requires_grad_(True) for t in (q, k, v, dO))
    out = O.reference_cpu_route(q, k, v, **meta["kw"])
    first = torch.autograd.grad(out, (q, k, v), dO, create_graph=True)
    second = torch.autograd.grad(first, (q, k, v, dO), (bq, bk, bv))
    for n, t in zip(O.OUTPUT_NAMES, (out, *first, *second)):
        ref = torch.from_numpy(z[f"op32_{n}"])
        assert (t.detach() - ref).abs().max().item() <= 1e-5 * max(1.0, ref.abs().max().item()), n


def test_closed_form_with_undefined_tangents():
    q, k, v, dO, uQ = O.seeded_inputs(5, (1, 2, 20, 8), (1, 2, 20, 8), torch.float64, n_extra_q=2)
    geom = dict(is_causal=True)
    a = O.bob_closed_form(q, k, v, dO, uQ, None, None, **geom).outputs()
    b = O.second_order_autograd(q, k, v, dO, uQ, None, None, **geom)
    for n in O.OUTPUT_NAMES:
        torch.testing.assert_close(a[n], b[n], rtol=1e-10, atol=1e-12)


def test_rows_without_keys_give_zeros():
    # queries that sit before every key: no attending key, output and gradients are zero
    q, k, v, dO, uQ = O.seeded_inputs(2, (1, 1, 6, 8), (1, 1, 4, 8), torch.float64, n_extra_q=2)
    uK, uV = O.seeded_inputs(3, (1, 1, 6, 8), (1, 1, 4, 8), torch.float64)[1:]
    r = O.bob_closed_form(q, k, v, dO, uQ, uK, uV, is_causal=True, q_offset=0, k_offset=3)
    assert torch.isinf(r.lse[0, 0, :3]).all() and (r.out[0, 0, :3] == 0).all()
    assert all(torch.isfinite(x).all() for x in r.outputs().values())
    ag = O.second_order_autograd(q, k, v, dO, uQ, uK, uV, is_causal=True, q_offset=0, k_offset=3)
    for n in O.OUTPUT_NAMES:
        torch.testing.assert_close(r.outputs()[n], ag[n], rtol=1e-10, atol=1e-12)


def test_config0_chain_matches_reference_operator():
    """The CPU benchmark configuration: MHA fp32 B=1 H=2 S=128 D=64 causal, loss chain."""
    z = np.load(GOLDEN / "config0_chain.npz")
    g = torch.Generator().manual_seed(0)
    q, k, v = (torch.randn((1, 2, 128, 64), dtype=torch.float32, generator=g) for _ in range(3))
    got = O.loss_chain(O.reference_cpu_route, q, k, v, is_causal=True, scale=1 / 8.0)
    got64 = O.loss_chain(O.attention_dense, q.double(), k.double(), v.double(), is_causal=True,
                         scale=1 / 8.0)
    for n in ("out", "dq", "dk", "dv", "ddq", "ddk", "ddv"):
        ref32, ref64 = torch.from_numpy(z[f"op32_{n}"]), torch.from_numpy(z[f"math64_{n}"])
        assert O.error_metrics(got[n], ref32)["max_abs_rel"] <= 1e-5, n
        assert O.error_metrics(got[n], ref64)["max_abs_rel"] <= 1e-5, n        # fp32 vs fp64
        assert O.error_metrics(got64[n], ref64)["max_abs_rel"] <= 1e-10, n


def test_chain_reenters_first_backward():
    """(ddq, ddk, ddv) = (Qbar, Kbar, Vbar) + first backward with cotangent (2/numel) dObar."""
    q, k, v = O.seeded_inputs(7, (1, 2, 24, 8), (1, 2, 24, 8), torch.float64)
    kw = dict(is_causal=True)
    chain = O.loss_chain(O.attention_dense, q, k, v, **kw)
    n_q, n_k = q.numel(), k.numel()
    dO = 2 * chain["out"] / n_q
    uQ, uK, uV = 2 * chain["dq"] / n_q, 2 * chain["dk"] / n_k, 2 * chain["dv"] / n_k
    r = O.bob_closed_form(q, k, v, dO, uQ, uK, uV, **kw)
    again = O.bob_closed_form(q, k, v, 2 * r.dObar / n_q, None, None, None, **kw)
    for name, bar, g in (("ddq", r.Qbar, again.dQ), ("ddk", r.Kbar, again.dK), ("ddv", r.Vbar, again.dV)):
        torch.testing.assert_close(chain[name], bar + g, rtol=1e-9, atol=1e-20)


def test_unmasked_pair_count():
    assert O.unmasked_pairs(128, 128, is_causal=True) == 8256
    assert O.unmasked_pairs(1024, 1024, is_causal=True) == 524800
    assert O.unmasked_pairs(4096, 4096, is_causal=True) == 8390656
    assert O.unmasked_pairs(128, 512, is_causal=True, window_size=256) == 32768
    assert O.unmasked_pairs(128, 512, is_causal=True, window_size=256, q_offset=1000, k_offset=616) == 32768
    m = O.valid_mask(13, 29, is_causal=True, window_size=5, q_offset=20, k_offset=3)
    assert int(m.sum()) == O.unmasked_pairs(13, 29, is_causal=True, window_size=5, q_offset=20, k_offset=3)


def test_streamed_closed_form_equals_the_dense_closed_form():
    """The row-blocked, head-by-head evaluation used for the largest configuration is the same
    function as the dense closed form (which is pinned against the reference above)."""
    cases = [((2, 4, 70, 16), (2, 2, 70, 16), dict(is_causal=True)),
             ((1, 2, 33, 16), (1, 1, 90, 16), dict(is_causal=True, window_size=20)),
             ((1, 3, 40, 8), (1, 3, 40, 8), dict()),
             ((1, 2, 96, 16), (1, 2, 64, 16), dict(is_causal=True, q_offset=0, k_offset=40))]
    for qs, ks, kw in cases:
        q, k, v, dO, uQ = O.seeded_inputs(1, qs, ks, torch.float64, n_extra_q=2)
        uK, uV = O.seeded_inputs(2, qs, ks, torch.float64)[1:]
        a = O.bob_closed_form(q, k, v, dO, uQ, uK, uV, **kw)
        b = O.bob_closed_form_streamed(q, k, v, dO, uQ, uK, uV, row_block=16, **kw)
        for n in O.OUTPUT_NAMES + ("alpha", "ecirc", "delta"):
            torch.testing.assert_close(getattr(b, n), getattr(a, n), rtol=1e-11, atol=1e-11)
        fin = torch.isfinite(a.lse)
        assert torch.equal(torch.isfinite(b.lse), fin)
        torch.testing.assert_close(b.lse[fin], a.lse[fin], rtol=1e-12, atol=1e-12)


def test_sharded_loss_chain_with_global_mean_counts_equals_the_full_chain():
    """Evaluating the benchmark's loss chain on one KV group with the FULL tensors' element counts in
    the means gives that group's slice of the full chain, Hessian-vector product included."""
    q, k, v = O.seeded_inputs(7, (1, 4, 24, 8), (1, 2, 24, 8), torch.float64)
    gq, gk, gv = O.seeded_inputs(8, (1, 4, 24, 8), (1, 2, 24, 8), torch.float64)
    full = O.loss_chain(O.attention_dense, q, k, v, hvp_directions=(gq, gk, gv), is_causal=True)
    for hk in range(2):
        hs = slice(2 * hk, 2 * hk + 2)
        part = O.loss_chain(O.attention_dense, q[:, hs], k[:, hk:hk + 1], v[:, hk:hk + 1],
                            hvp_directions=(gq[:, hs], gk[:, hk:hk + 1], gv[:, hk:hk + 1]),
                            mean_counts=(q.numel(), k.numel()), is_causal=True)
        for n in ("ddq", "hvq", "dq"):
            torch.testing.assert_close(part[n], full[n][:, hs], rtol=1e-10, atol=1e-18)
        for n in ("ddk", "ddv", "hvk", "hvv", "dk", "dv"):
            torch.testing.assert_close(part[n], full[n][:, hk:hk + 1], rtol=1e-10, atol=1e-18)
