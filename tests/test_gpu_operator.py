"""GPU tests of the public operator and its autograd chain (drop-in behaviour)."""

import pytest
import torch

import bob
from flashbob_b200 import interface
from oracle import bob_oracle as O

pytestmark = pytest.mark.gpu
BF16, FP16 = torch.bfloat16, torch.float16


def _second_grad(op, q, k, v, dO, bars, **kw):
    q, k, v, dO = (t.detach().clone().requires_grad_(True) for t in (q, k, v, dO))
    out = op(q, k, v, **kw)
    first = torch.autograd.grad(out, (q, k, v), dO, create_graph=True)
    second = torch.autograd.grad(first, (q, k, v, dO), bars)
    return (out, *first, *second)


@pytest.mark.parametrize(
    ("shape", "kwargs"),
    [
        ((2, 2, 64, 64, 64), {"is_causal": True}),
        ((2, 2, 48, 48, 128), {"is_causal": False}),
        ((2, 2, 64, 64, 64), {"is_causal": True, "window_size": 16}),
        ((8, 2, 64, 64, 64), {"is_causal": True}),
        ((8, 1, 64, 64, 64), {"is_causal": True}),
        ((2, 2, 32, 64, 64), {"is_causal": True, "window_size": 32, "q_offset": 32, "k_offset": 0}),
        ((4, 4, 130, 130, 32), {"is_causal": True, "scale": 0.3}),
    ],
)
def test_second_gradient_through_autograd_matches_oracle(shape, kwargs):
    """Mirror of the reference's CUDA acceptance test
    (reference: tests/cuda/test_attention_correctness.py:33-53)."""
    hq, hkv, nq, nk, d = shape
    q, k, v, dO, bq = O.seeded_inputs(0, (1, hq, nq, d), (1, hkv, nk, d), BF16, n_extra_q=2)
    bk, bv = O.seeded_inputs(1, (1, hq, nq, d), (1, hkv, nk, d), BF16)[1:]
    ref = O.second_order_autograd(q, k, v, dO, bq, bk, bv, **kwargs)
    c = lambda t: t.cuda()
    got = _second_grad(bob.sdpa_bob, c(q), c(k), c(v), c(dO), (c(bq), c(bk), c(bv)), **kwargs)
    for n, t in zip(O.OUTPUT_NAMES, got):
        assert t.dtype == BF16 and t.is_contiguous() and t.is_cuda
        torch.testing.assert_close(t.double().cpu(), ref[n], rtol=0.08, atol=0.08)
        assert O.error_metrics(t, ref[n])["l2_rel"] < 6e-3, n


def test_only_query_tangent_defined():
    q, k, v, dO, bq = O.seeded_inputs(0, (1, 2, 64, 64), (1, 2, 64, 64), BF16, n_extra_q=2)
    ref = O.second_order_autograd(q, k, v, dO, bq, None, None, is_causal=True)
    qd, kd, vd, dOd = (t.cuda().requires_grad_(True) for t in (q, k, v, dO))
    out = bob.sdpa_bob(qd, kd, vd, is_causal=True)
    first = torch.autograd.grad(out, (qd, kd, vd), dOd, create_graph=True)
    got = torch.autograd.grad((first[0] * bq.cuda()).sum(), (qd, kd, vd, dOd))
    for n, t in zip(("Qbar", "Kbar", "Vbar", "dObar"), got):
        torch.testing.assert_close(t.double().cpu(), ref[n], rtol=0.08, atol=0.08)
        assert O.error_metrics(t, ref[n])["l2_rel"] < 6e-3, n


def test_first_gradient_without_graph_takes_the_plain_path():
    """create_graph=False: the first backward runs alone and its result carries no graph
    (reference: src/bob/sdpa.py:338-353)."""
    q, k, v, dO = O.seeded_inputs(3, (2, 4, 200, 64), (2, 2, 200, 64), BF16, n_extra_q=1)
    ref = O.bob_closed_form(q, k, v, dO, None, None, None, is_causal=True)
    qd, kd, vd = (t.cuda().requires_grad_(True) for t in (q, k, v))
    out = bob.sdpa_bob(qd, kd, vd, is_causal=True)
    grads = torch.autograd.grad(out, (qd, kd, vd), dO.cuda())
    for n, t in zip(("dQ", "dK", "dV"), grads):
        assert not t.requires_grad
        assert O.error_metrics(t, getattr(ref, n))["l2_rel"] < 6e-3, n
    out = bob.sdpa_bob(qd, kd, vd, is_causal=True)
    out.backward(dO.cuda())
    assert O.error_metrics(qd.grad, ref.dQ)["l2_rel"] < 6e-3


def _chain_case(dtype, q_shape, kv_shape, seed, **kw):
    q, k, v = O.seeded_inputs(seed, q_shape, kv_shape, dtype)
    ref = O.loss_chain(O.attention_dense, q.double(), k.double(), v.double(), **kw)
    return (q, k, v), ref


def test_config1_loss_chain_bf16_mha():
    """B=2 H=8 S=1024 D=64 causal bf16; L1 = mean(out^2), L2 = sum of mean(grad^2); second grads
    equal (Qbar, Kbar, Vbar) plus a re-entered first backward.  Magnitudes are ~1e-15, so the
    comparison is relative to the largest reference value."""
    (q, k, v), ref = _chain_case(BF16, (2, 8, 1024, 64), (2, 8, 1024, 64), 1, is_causal=True)
    got = O.loss_chain(bob.sdpa_bob, q.cuda(), k.cuda(), v.cuda(), is_causal=True)
    for n in ("out", "dq", "dk", "dv", "ddq", "ddk", "ddv"):
        m = O.error_metrics(got[n], ref[n])
        assert m["l2_rel"] < 2e-2 and m["max_abs_rel"] < 4e-2, (n, m)


def test_config3_fp16_rectangular_window_two_offset_conventions():
    """B=4 H=16 Nq=128 Nk=512 D=128 fp16 causal window 256: right-aligned default (q_offset 384)
    and explicit offsets (1000, 616) describe the same geometry and must agree bit for bit.
    Explicit N(0,1) cotangents (the literal fp16 loss chain underflows to zero second grads)."""
    qs, ks = (4, 16, 128, 128), (4, 16, 512, 128)
    q, k, v, dO, bq = O.seeded_inputs(3, qs, ks, FP16, n_extra_q=2)
    bk, bv = O.seeded_inputs(4, qs, ks, FP16)[1:]
    c = lambda t: t.cuda()
    a = _second_grad(bob.sdpa_bob, c(q), c(k), c(v), c(dO), (c(bq), c(bk), c(bv)), is_causal=True, window_size=256)
    b = _second_grad(bob.sdpa_bob, c(q), c(k), c(v), c(dO), (c(bq), c(bk), c(bv)), is_causal=True, window_size=256,
                     q_offset=1000, k_offset=616)
    for x, y in zip(a, b):
        assert torch.equal(x, y)
    sl = slice(0, 1)   # oracle on one batch element (fp64, materialized)
    ref = O.second_order_autograd(q[sl], k[sl], v[sl], dO[sl], bq[sl], bk[sl], bv[sl], is_causal=True,
                                  window_size=256, q_offset=384, k_offset=0)
    for n, t in zip(O.OUTPUT_NAMES, a):
        m = O.error_metrics(t[sl], ref[n])
        assert m["l2_rel"] < 1e-3 and m["max_abs_rel"] < 4e-3, (n, m)


def test_config3_literal_fp16_chain_is_degenerate_like_the_reference():
    """The literal fp16 chain: dO = 2*out/numel is subnormal in fp16, the squared first gradients
    flush to zero, L2 == 0 and the second gradients are exactly zero (the reference's own fp16
    path does the same); with fp32 loss arithmetic the chain is finite."""
    q, k, v = O.seeded_inputs(3, (4, 16, 128, 128), (4, 16, 512, 128), FP16)
    got = O.loss_chain(bob.sdpa_bob, q.cuda(), k.cuda(), v.cuda(), is_causal=True, window_size=256)
    for n in ("ddq", "ddk", "ddv"):
        assert got[n].float().abs().max().item() == 0.0
    got = O.loss_chain(bob.sdpa_bob, q.cuda(), k.cuda(), v.cuda(), fp32_losses=True, is_causal=True,
                       window_size=256)
    assert all(torch.isfinite(got[n].float()).all() for n in ("ddq", "ddk", "ddv"))


def test_widened_grouped_heads_behind_the_switch():
    q = torch.randn(1, 4, 96, 64, device="cuda", dtype=BF16)
    k = torch.randn(1, 2, 160, 64, device="cuda", dtype=BF16)
    with pytest.raises(NotImplementedError, match="rectangular"):
        bob.sdpa_bob(q, k, k, is_causal=True)
    with pytest.raises(NotImplementedError, match="window"):
        bob.sdpa_bob(q, k[:, :, :96], k[:, :, :96], is_causal=True, window_size=8)
    with pytest.raises(TypeError, match="bfloat16"):
        bob.sdpa_bob(q.half(), k[:, :, :96].half(), k[:, :, :96].half(), is_causal=True)
    interface.ALLOW_WIDENED_GQA = True
    try:
        dO, uQ = torch.randn_like(q), torch.randn_like(q)
        uK, uV = torch.randn_like(k), torch.randn_like(k)
        kw = dict(is_causal=True, window_size=50)
        got = _second_grad(bob.sdpa_bob, q, k, k.clone(), dO, (uQ, uK, uV), **kw)
        ref = O.second_order_autograd(q.cpu(), k.cpu(), k.cpu(), dO.cpu(), uQ.cpu(), uK.cpu(), uV.cpu(), **kw)
        for n, t in zip(O.OUTPUT_NAMES, got):
            assert O.error_metrics(t, ref[n])["l2_rel"] < 6e-3, n
    finally:
        interface.ALLOW_WIDENED_GQA = False


def test_second_backward_is_linear_in_the_tangents_at_full_size():
    """Size-independent property at the headline configuration (GQA 32/8, S=4096, D=64):
    bwd2(u1 + u2) == bwd2(u1) + bwd2(u2) up to 16-bit rounding, and one KV group of the full
    problem matches the fp64 oracle."""
    from flashbob_b200 import ops
    B, Hq, Hkv, N, D = 1, 32, 8, 4096, 64
    q, k, v, dO, u1 = O.seeded_inputs(2, (B, Hq, N, D), (B, Hkv, N, D), BF16, n_extra_q=2)
    k1, v1 = O.seeded_inputs(1002, (B, Hq, N, D), (B, Hkv, N, D), BF16)[1:]
    geom = dict(is_causal=True, window_size=0, q_offset=0, k_offset=0, scale=None)
    c = lambda t: t.cuda()
    qd, kd, vd, dOd = map(c, (q, k, v, dO))
    out, lse = ops.attention_forward(qd, kd, vd, **geom)
    dQ, dK, dV, delta, pk = ops.attention_first_backward(qd, kd, vd, out, lse, dOd, **geom)
    run = lambda a, b, cc: ops.attention_second_backward(qd, kd, vd, out, lse, delta, pk, dOd, dQ, a, b, cc, **geom)
    full = run(c(u1), c(k1), c(v1))
    parts_q = run(c(u1), None, None)
    parts_kv = run(None, c(k1), c(v1))
    for n, f, a, b in zip(("Qbar", "Kbar", "Vbar", "dObar"), full, parts_q, parts_kv):
        m = O.error_metrics(a.float() + b.float(), f.float())
        assert m["l2_rel"] < 8e-3, (n, m)
    # one KV group (4 query heads) against fp64
    hk = 5
    hs = slice(hk * 4, hk * 4 + 4)
    ref = O.bob_closed_form(q[:, hs], k[:, hk:hk + 1], v[:, hk:hk + 1], dO[:, hs], u1[:, hs],
                            k1[:, hk:hk + 1], v1[:, hk:hk + 1], **geom)
    got = dict(out=out[:, hs], dQ=dQ[:, hs], dK=dK[:, hk:hk + 1], dV=dV[:, hk:hk + 1], Qbar=full[0][:, hs],
               Kbar=full[1][:, hk:hk + 1], Vbar=full[2][:, hk:hk + 1], dObar=full[3][:, hs])
    for n in O.OUTPUT_NAMES:
        m = O.error_metrics(got[n], getattr(ref, n))
        assert m["l2_rel"] < 6e-3 and m["max_abs_rel"] < 3e-2, (n, m)


def test_config2_loss_chain_and_hessian_vector_product_through_the_operator():
    """bf16 GQA B=1 Hq=32 Hkv=8 S=4096 D=64 causal through `bob.sdpa_bob`: the literal two-level chain
    (L1 = mean(out^2), L2 = sum of mean(grad^2)) AND the Hessian-vector product of L1 with N(0,1)
    directions (the pattern of the reference's examples/hessian_vector_product.py:54-61), against
    the fp64 oracle evaluated KV group by KV group with the full tensors' element counts in the
    means.  Values are ~1e-17, so errors are relative; the bf16 loss arithmetic (squares and means of
    bf16 tensors) is part of what is compared."""
    B, Hq, Hkv, N, D = 1, 32, 8, 4096, 64
    G = Hq // Hkv
    q, k, v = O.seeded_inputs(2, (B, Hq, N, D), (B, Hkv, N, D), BF16)
    gq, gk, gv = O.seeded_inputs(1002, (B, Hq, N, D), (B, Hkv, N, D), BF16)
    got = O.loss_chain(bob.sdpa_bob, q.cuda(), k.cuda(), v.cuda(), hvp_directions=(gq.cuda(), gk.cuda(), gv.cuda()),
                       is_causal=True)
    got = {n: t.float().cpu() for n, t in got.items()}
    counts = (q.numel(), k.numel())
    worst = {}
    for hk in range(Hkv):
        hs, ks = slice(hk * G, hk * G + G), slice(hk, hk + 1)
        ref = O.loss_chain(O.attention_dense, q[:, hs].double(), k[:, ks].double(), v[:, ks].double(),
                           hvp_directions=(gq[:, hs].double(), gk[:, ks].double(), gv[:, ks].double()),
                           mean_counts=counts, is_causal=True)
        for n in ("out", "dq", "ddq", "hvq"):
            m = O.error_metrics(got[n][:, hs], ref[n])
            worst[n] = max(worst.get(n, 0.0), m["l2_rel"])
        for n in ("dk", "dv", "ddk", "ddv", "hvk", "hvv"):
            m = O.error_metrics(got[n][:, ks], ref[n])
            worst[n] = max(worst.get(n, 0.0), m["l2_rel"])
    # first-order quantities carry one level of bf16 rounding, second-order ones two levels plus
    # the bf16 loss arithmetic between them
    for n in ("out", "dq", "dk", "dv"):
        assert worst[n] < 8e-3, (n, worst)
    for n in ("ddq", "ddk", "ddv", "hvq", "hvk", "hvv"):
        assert worst[n] < 2e-2, (n, worst)
