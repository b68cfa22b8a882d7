"""GPU parity: the CUDA kernels, called through the C ABI, against the fp64 CPU oracle.

Tolerances.  The kernels round the same quantities to 16 bits as the reference's CUDA route does
(derived operands, saved `out` and first-order `dQ`), so every output carries a relative L2 error
of a few 1e-3 in bf16 (a few 1e-4 in fp16) against fp64.  Bars used here, per output tensor:
bf16  l2_rel <= 6e-3, max_abs <= 2e-2 * max|ref|;  fp16  l2_rel <= 1e-3, max_abs <= 4e-3 * max|ref|;
and the reference's own acceptance test, assert_close(rtol=atol=0.08)
(reference: tests/cuda/test_attention_correctness.py:53).
"""

import ast
import ctypes
from pathlib import Path

import numpy as np
import pytest
import torch

from flashbob_b200 import _lib, ops
from oracle import bob_oracle as O

pytestmark = pytest.mark.gpu
GOLDEN = Path(__file__).parent / "golden"
BF16, FP16 = torch.bfloat16, torch.float16
BARS = {BF16: (6e-3, 2e-2), FP16: (1e-3, 4e-3)}


def _check(name, got, ref, dtype):
    if ref.abs().max().item() == 0:
        # an exactly-zero expectation (e.g. one key: dS = P (dP - delta) = 0) is met only up to the
        # 16-bit rounding of the saved `out` that delta is formed from
        assert got.float().abs().max().item() <= 0.08, name
        return
    m = O.error_metrics(got, ref)
    l2, mx = BARS[dtype]
    assert torch.isfinite(got.float()).all(), name
    assert m["l2_rel"] <= l2, (name, m)
    assert m["max_abs_rel"] <= mx, (name, m)
    torch.testing.assert_close(got.double().cpu(), ref.double(), rtol=0.08, atol=0.08)


def _run_kernels(q, k, v, dO, uQ, uK, uV, geom):
    c = lambda t: None if t is None else t.cuda()
    qd, kd, vd, dOd, uQd, uKd, uVd = map(c, (q, k, v, dO, uQ, uK, uV))
    out, lse = ops.attention_forward(qd, kd, vd, **geom)
    dQ, dK, dV, delta, pk = ops.attention_first_backward(qd, kd, vd, out, lse, dOd, **geom)
    Qb, Kb, Vb, dOb = ops.attention_second_backward(qd, kd, vd, out, lse, delta, pk, dOd, dQ, uQd, uKd,
                                                    uVd, **geom)
    return dict(out=out, dQ=dQ, dK=dK, dV=dV, Qbar=Qb, Kbar=Kb, Vbar=Vb, dObar=dOb), lse, delta


def _geom(Nq, Nk, **kw):
    causal = kw.get("is_causal", False)
    return dict(is_causal=causal, window_size=kw.get("window_size", 0),
                q_offset=O.infer_q_offset(Nq, Nk, kw.get("q_offset"), kw.get("k_offset", 0), causal),
                k_offset=kw.get("k_offset", 0), scale=kw.get("scale"))


def test_tensor_core_plumbing_known_answer():
    lib = _lib.load()
    for dtype in (BF16, FP16):
        g = torch.Generator().manual_seed(0)
        a = torch.randn(128, 64, generator=g).to(dtype).cuda()
        b = torch.randn(64, 64, generator=g).to(dtype).cuda()
        out = torch.zeros(8, 128, 64, device="cuda")
        st = torch.zeros(1, dtype=torch.int32, device="cuda")
        rc = lib.bob_sm100_selftest(a.data_ptr(), b.data_ptr(), int(dtype == BF16), out.data_ptr(),
                                    st.data_ptr(), torch.cuda.current_stream().cuda_stream)
        torch.cuda.synchronize()
        assert rc == 0 and st.item() == 0
        ab_t, ab = a.double() @ b.double().T, a.double() @ b.double()
        torch.testing.assert_close(out[0].double(), ab_t, rtol=1e-5, atol=1e-4)
        torch.testing.assert_close(out[1].double(), ab, rtol=1e-5, atol=1e-4)
        torch.testing.assert_close(out[2].double(), ab_t, rtol=1e-5, atol=1e-4)
        for i in (3, 4, 7):
            torch.testing.assert_close(out[i].double(), ab_t, rtol=1e-5, atol=1e-4)
        for i in (5, 6):
            torch.testing.assert_close(out[i].double(), ab, rtol=1e-5, atol=1e-4)


def test_bounded_wait_gives_up_and_reports():
    """Failure detection without a fault: a wait that nothing completes runs out after ~0.5 s of SM
    cycles, the kernel records a status and returns, and the context keeps working."""
    lib = _lib.load()
    st = torch.zeros(1, dtype=torch.int32, device="cuda")
    assert lib.bob_sm100_timeout_selftest(st.data_ptr(), torch.cuda.current_stream().cuda_stream) == 0
    torch.cuda.synchronize()
    assert st.item() == 77
    assert float((torch.ones(4, device="cuda") * 2).sum()) == 8.0      # context still usable
    lib.bob_sm100_last_status(torch.cuda.current_device())             # the self-test also reports there: clear it


CASES = {
    # name: (B, Hq, Hkv, Nq, Nk, D, dtype, kwargs)
    "causal64": (1, 2, 2, 64, 64, 64, BF16, dict(is_causal=True)),
    "noncausal48_d128": (1, 2, 2, 48, 48, 128, BF16, dict()),
    "window16": (1, 2, 2, 64, 64, 64, BF16, dict(is_causal=True, window_size=16)),
    "gqa": (1, 8, 2, 64, 64, 64, BF16, dict(is_causal=True)),
    "mqa": (1, 8, 1, 64, 64, 64, BF16, dict(is_causal=True)),
    "rect_w32": (1, 2, 2, 32, 64, 64, BF16, dict(is_causal=True, window_size=32, q_offset=32, k_offset=0)),
    "ragged_causal": (2, 3, 3, 301, 301, 64, BF16, dict(is_causal=True, scale=0.2)),
    "ragged_noncausal_rect": (1, 2, 2, 77, 203, 64, BF16, dict()),
    "window_long": (1, 2, 2, 700, 700, 64, BF16, dict(is_causal=True, window_size=130)),
    "gqa_ragged": (2, 6, 2, 333, 333, 64, BF16, dict(is_causal=True)),
    "d32": (1, 2, 2, 100, 100, 32, BF16, dict(is_causal=True)),
    "d128_causal": (1, 2, 2, 384, 384, 128, BF16, dict(is_causal=True)),
    "d128_gqa": (1, 4, 1, 260, 260, 128, BF16, dict(is_causal=True)),
    "fp16_causal": (1, 2, 2, 200, 200, 64, FP16, dict(is_causal=True)),
    "fp16_rect_d128": (2, 3, 3, 128, 512, 128, FP16, dict(is_causal=True, window_size=256)),
    "large_offsets": (1, 2, 2, 128, 512, 64, BF16, dict(is_causal=True, window_size=256, q_offset=1000, k_offset=616)),
    "tiny": (1, 1, 1, 1, 1, 32, BF16, dict(is_causal=True)),
    "one_query_many_keys": (1, 2, 2, 1, 500, 64, BF16, dict(is_causal=True)),
    "keyless_rows": (1, 2, 2, 96, 64, 64, BF16, dict(is_causal=True, q_offset=0, k_offset=40)),
}


@pytest.mark.parametrize("name", list(CASES))
def test_all_eight_outputs_match_oracle(name):
    B, Hq, Hkv, Nq, Nk, D, dtype, kw = CASES[name]
    q, k, v, dO, uQ = O.seeded_inputs(11, (B, Hq, Nq, D), (B, Hkv, Nk, D), dtype, n_extra_q=2)
    uK, uV = O.seeded_inputs(12, (B, Hq, Nq, D), (B, Hkv, Nk, D), dtype)[1:]
    geom = _geom(Nq, Nk, **kw)
    ref = O.bob_closed_form(q, k, v, dO, uQ, uK, uV, **geom)
    got, lse, delta = _run_kernels(q, k, v, dO, uQ, uK, uV, geom)
    fin = torch.isfinite(ref.lse)
    assert torch.equal(torch.isfinite(lse.cpu()), fin)
    torch.testing.assert_close(lse.cpu().double()[fin], ref.lse[fin], rtol=1e-5, atol=1e-5)
    for n in O.OUTPUT_NAMES:
        _check(f"{name}:{n}", got[n], getattr(ref, n), dtype)


@pytest.mark.parametrize("causal", [True, False])
@pytest.mark.parametrize("D", [64, 128])
def test_forward_when_the_row_maximum_keeps_growing(causal, D):
    """Scores that grow along the keys by ~14 (log2 units) per 128 keys: every tile raises the running
    maximum past the forward's rescaling threshold, so the accumulator in tensor memory is rescaled
    tile after tile and the two pointwise groups end with very different references."""
    B, H, N = 1, 2, 640
    g = torch.Generator().manual_seed(5)
    q = 0.05 * torch.randn(B, H, N, D, generator=g)
    k = 0.05 * torch.randn(B, H, N, D, generator=g)
    q[..., 0] = 4.0
    k[..., 0] = 0.15 * torch.arange(N, dtype=torch.float32) * (8.0 / D ** 0.5) ** -1 * 1.0
    v = torch.randn(B, H, N, D, generator=g)
    dO, uQ, uK, uV = (torch.randn(B, H, N, D, generator=g) for _ in range(4))
    q, k, v, dO, uQ, uK, uV = (t.to(BF16) for t in (q, k, v, dO, uQ, uK, uV))
    geom = _geom(N, N, is_causal=causal)
    ref = O.bob_closed_form(q, k, v, dO, uQ, uK, uV, **geom)
    got, lse, _ = _run_kernels(q, k, v, dO, uQ, uK, uV, geom)
    # the maximum really moves: the lse of late rows is far above that of early rows
    assert (ref.lse[..., -1] - ref.lse[..., 0]).min().item() > 20.0 or not causal
    torch.testing.assert_close(lse.cpu().double(), ref.lse, rtol=1e-5, atol=2e-5)
    # out and dV (= P^T dO) are free of cancellation; with keys this large the other gradients are
    # differences of big rounded terms and say nothing about the forward
    for n in ("out", "dV"):
        _check(f"growing:{n}", got[n], getattr(ref, n), BF16)
    for n in O.OUTPUT_NAMES:
        assert torch.isfinite(got[n].float()).all(), n


@pytest.mark.parametrize("missing", [("k", "v"), ("q",), ("q", "k"), ("v",), ("q", "v")])
def test_undefined_tangents(missing):
    """Undefined tangents switch products off; results equal the oracle with those tangents zero
    (reference: tests/cuda/test_attention_correctness.py:56-76, src/bob/sdpa.py:177-180)."""
    B, Hq, Hkv, Nq, Nk, D = 1, 4, 2, 150, 150, 64
    q, k, v, dO, uQ = O.seeded_inputs(21, (B, Hq, Nq, D), (B, Hkv, Nk, D), BF16, n_extra_q=2)
    uK, uV = O.seeded_inputs(22, (B, Hq, Nq, D), (B, Hkv, Nk, D), BF16)[1:]
    uQ = None if "q" in missing else uQ
    uK = None if "k" in missing else uK
    uV = None if "v" in missing else uV
    geom = _geom(Nq, Nk, is_causal=True)
    ref = O.bob_closed_form(q, k, v, dO, uQ, uK, uV, **geom)
    got, _, _ = _run_kernels(q, k, v, dO, uQ, uK, uV, geom)
    for n in ("Qbar", "Kbar", "Vbar", "dObar"):
        r = getattr(ref, n)
        if r.abs().max() == 0:
            assert got[n].float().abs().max().item() == 0, n
        else:
            _check(f"{missing}:{n}", got[n], r, BF16)


@pytest.mark.parametrize("name", ["causal", "noncausal", "window", "gqa", "mqa", "rect"])
def test_golden_geometries_of_the_reference_cuda_tests(name):
    """Shapes and seeds of the reference's CUDA acceptance test, inputs rounded to bf16."""
    z = np.load(GOLDEN / f"{name}.npz", allow_pickle=True)
    meta = ast.literal_eval(str(z["meta"]))
    q_shape = (1, meta["hq"], meta["nq"], meta["d"])
    kv_shape = (1, meta["hkv"], meta["nk"], meta["d"])
    g = torch.Generator().manual_seed(meta["seed"])
    r = lambda s: torch.randn(s, dtype=torch.float32, generator=g).to(BF16)
    q, k, v, dO, uQ, uK, uV = r(q_shape), r(kv_shape), r(kv_shape), r(q_shape), r(q_shape), r(kv_shape), r(kv_shape)
    geom = _geom(meta["nq"], meta["nk"], **meta["kw"])
    got, _, _ = _run_kernels(q, k, v, dO, uQ, uK, uV, geom)
    ref = O.bob_closed_form(q, k, v, dO, uQ, uK, uV, **geom)
    for n in O.OUTPUT_NAMES:
        _check(f"{name}:{n}", got[n], getattr(ref, n), BF16)
        # the unrounded fp64 golden differs only by input rounding: loose sanity bound
        gold = torch.from_numpy(z[f"ref64_{n}"])
        assert O.error_metrics(got[n], gold)["l2_rel"] < 0.05, n


def test_strided_inputs_are_read_in_place():
    """[B, N, H, D] storage viewed as [B, H, N, D] goes to the kernels without a copy."""
    B, H, N, D = 2, 4, 160, 64
    q, k, v, dO, uQ = O.seeded_inputs(31, (B, H, N, D), (B, H, N, D), BF16, n_extra_q=2)
    uK, uV = O.seeded_inputs(32, (B, H, N, D), (B, H, N, D), BF16)[1:]
    geom = _geom(N, N, is_causal=True)
    ref = O.bob_closed_form(q, k, v, dO, uQ, uK, uV, **geom)
    tr = lambda t: t.cuda().transpose(1, 2).contiguous().transpose(1, 2)   # same values, BNHD storage
    qd, kd, vd, dOd, uQd, uKd, uVd = map(tr, (q, k, v, dO, uQ, uK, uV))
    assert not qd.is_contiguous() and ops._tma_ready(qd) is qd
    out, lse = ops.attention_forward(qd, kd, vd, **geom)
    dQ, dK, dV, delta, pk = ops.attention_first_backward(qd, kd, vd, out, lse, dOd, **geom)
    res = ops.attention_second_backward(qd, kd, vd, out, lse, delta, pk, dOd, dQ, uQd, uKd, uVd, **geom)
    for n, t in zip(O.OUTPUT_NAMES, (out, dQ, dK, dV, *res)):
        _check(f"strided:{n}", t, getattr(ref, n), BF16)
    # a layout the kernels cannot address (odd row stride) is copied, not rejected
    odd = torch.randn(B, H, N, D + 1, device="cuda").to(BF16)[..., :D]
    assert ops._tma_ready(odd) is not odd


def test_c_abi_rejects_bad_arguments_on_the_host():
    lib = _lib.load()
    g = _lib.Geom()
    g.B, g.Hq, g.Hkv, g.Nq, g.Nk, g.D = 1, 2, 2, 64, 64, 64
    g.dtype, g.is_causal, g.window, g.device, g.scale = _lib.BF16, 1, 0, 0, 0.125
    for f in (g.q_strides, g.k_strides, g.v_strides):
        f[0], f[1], f[2] = 2 * 64 * 64, 64 * 64, 64
    t = torch.zeros(1, 2, 64, 64, dtype=BF16, device="cuda")
    lse = torch.zeros(1, 2, 64, device="cuda")
    ws = torch.zeros(1024, dtype=torch.uint8, device="cuda")
    vp = lambda x: ctypes.c_void_p(x.data_ptr())
    call = lambda: lib.bob_sm100_fwd(ctypes.byref(g), vp(t), vp(t), vp(t), vp(t), vp(lse), vp(ws), None)
    assert call() == 0
    assert lib.bob_sm100_fwd(ctypes.byref(g), None, vp(t), vp(t), vp(t), vp(lse), vp(ws), None) == -1
    g.D = 72
    assert call() == -4
    g.D = 64
    g.Hkv = 3
    assert call() == -2
    g.Hkv = 2
    g.window, g.is_causal = 4, 0
    assert call() == -2
    g.window, g.is_causal = 0, 1
    g.q_strides[2] = 65
    assert call() == -5
    g.q_strides[2] = 64
    assert lib.bob_sm100_fwd(ctypes.byref(g), vp(t), vp(t), vp(t), vp(t), vp(lse), None, None) == -6
    # misaligned pointers are refused on the host instead of faulting on the device: inputs read by
    # TMA, results written with 16-byte stores, pk read as float4 (16 bytes), fp32 statistics (4 bytes)
    off = lambda x, n: ctypes.c_void_p(x.data_ptr() + n)
    assert lib.bob_sm100_fwd(ctypes.byref(g), off(t, 2), vp(t), vp(t), vp(t), vp(lse), vp(ws), None) == -10
    assert lib.bob_sm100_fwd(ctypes.byref(g), vp(t), vp(t), vp(t), off(t, 8), vp(lse), vp(ws), None) == -10
    assert lib.bob_sm100_fwd(ctypes.byref(g), vp(t), vp(t), vp(t), vp(t), off(lse, 2), vp(ws), None) == -10
    for f in (g.out_strides, g.do_strides, g.dq_strides, g.uq_strides, g.uk_strides, g.uv_strides):
        f[0], f[1], f[2] = 2 * 64 * 64, 64 * 64, 64
    pk = torch.zeros(1, 2, 64, 64, device="cuda")
    bwd1 = lambda dq, dk, dv, dl, pk_: lib.bob_sm100_bwd1(ctypes.byref(g), vp(t), vp(t), vp(t), vp(t), vp(lse), vp(t),
                                                          dq, dk, dv, dl, pk_, vp(ws), None)
    assert bwd1(off(t, 8), vp(t), vp(t), vp(lse), vp(pk)) == -10
    assert bwd1(vp(t), vp(t), off(t, 4), vp(lse), vp(pk)) == -10
    assert bwd1(vp(t), vp(t), vp(t), off(lse, 1), vp(pk)) == -10
    assert bwd1(vp(t), vp(t), vp(t), vp(lse), off(pk, 8)) == -10
    ws2 = torch.zeros(lib.bob_sm100_workspace_bytes(_lib.STAGE_BWD2, ctypes.byref(g)), dtype=torch.uint8, device="cuda")
    bwd2 = lambda qb, kb, vb, dob, pk_: lib.bob_sm100_bwd2(ctypes.byref(g), vp(t), vp(t), vp(t), vp(t), vp(lse), vp(lse),
                                                           pk_, vp(t), vp(t), vp(t), vp(t), vp(t), qb, kb, vb, dob,
                                                           vp(ws2), None)
    assert bwd2(vp(t), vp(t), vp(t), off(t, 8), vp(pk)) == -10
    assert bwd2(vp(t), off(t, 2), vp(t), vp(t), vp(pk)) == -10
    assert bwd2(vp(t), vp(t), vp(t), vp(t), off(pk, 4)) == -10
    assert lib.bob_sm100_bwd2_part(4, ctypes.byref(g), *([vp(t)] * 4), vp(lse), vp(lse), vp(pk), *([vp(t)] * 9),
                                   vp(ws2), None) == -2
    torch.cuda.synchronize()
    assert b"stride" in lib.bob_sm100_error_string(-5)
    assert b"aligned" in lib.bob_sm100_error_string(-10)


@pytest.mark.parametrize("D", [16, 48, 80, 96, 112])
def test_head_dims_between_the_operator_s_three(D):
    """The C ABI takes any head dim that is a multiple of 16 up to 128 (the operator itself admits
    32, 64 and 128): TMA zero-fills the padding columns and the stores skip them."""
    B, Hq, Hkv, N = 1, 4, 2, 150
    q, k, v, dO, uQ = O.seeded_inputs(70 + D, (B, Hq, N, D), (B, Hkv, N, D), BF16, n_extra_q=2)
    uK, uV = O.seeded_inputs(170 + D, (B, Hq, N, D), (B, Hkv, N, D), BF16)[1:]
    geom = _geom(N, N, is_causal=True)
    ref = O.bob_closed_form(q, k, v, dO, uQ, uK, uV, **geom)
    got, lse, _ = _run_kernels(q, k, v, dO, uQ, uK, uV, geom)
    torch.testing.assert_close(lse.cpu().double(), ref.lse, rtol=1e-5, atol=1e-5)
    for n in O.OUTPUT_NAMES:
        _check(f"d{D}:{n}", got[n], getattr(ref, n), BF16)


def test_a_give_up_is_visible_without_synchronising_per_call():
    """A kernel that gives up on a bounded wait also writes its code to a page-locked host word; the
    next call on the device (or `ops.check_device_status`) raises.  The run-out is the library's own
    self-test kernel (a wait that nothing completes), nothing faults."""
    lib = _lib.load()
    dev = torch.cuda.current_device()
    t = torch.zeros(1, 2, 64, 64, dtype=BF16, device="cuda")
    geom = _geom(64, 64, is_causal=True)
    ops.attention_forward(t, t, t, **geom)                  # sets up the device's status word
    torch.cuda.synchronize()
    assert lib.bob_sm100_last_status(dev) == 0
    st = torch.zeros(1, dtype=torch.int32, device="cuda")
    assert lib.bob_sm100_timeout_selftest(st.data_ptr(), torch.cuda.current_stream().cuda_stream) == 0
    torch.cuda.synchronize()
    assert st.item() == 77
    with pytest.raises(_lib.BobSm100Error, match="77"):
        ops.check_device_status()
    assert lib.bob_sm100_last_status(dev) == 0              # reading clears it
    ops.attention_forward(t, t, t, **geom)                  # and later calls are unaffected


@pytest.mark.parametrize("shape", [(8, 12, 12, 1024, 64), (1, 32, 8, 2048, 64), (2, 8, 2, 1024, 128), (2, 16, 4, 2048, 128)])
def test_repeated_calls_are_bit_identical(shape):
    """Every stage returns the same bits for the same inputs, however the work items were dealt to the
    CTAs of a persistent launch (more items than SMs in all shapes but the third): an item is computed by
    one CTA, and which pointwise group sums which of its tiles depends on the item alone."""
    B, Hq, Hkv, N, D = shape
    g = torch.Generator().manual_seed(7)
    r = lambda h: torch.randn(B, h, N, D, generator=g).to(BF16).cuda()
    q, k, v, dO, uQ, uK, uV = r(Hq), r(Hkv), r(Hkv), r(Hq), r(Hq), r(Hkv), r(Hkv)
    geom = _geom(N, N, is_causal=True)
    first = ops.attention_forward(q, k, v, **geom)
    for _ in range(4):
        again = ops.attention_forward(q, k, v, **geom)
        assert all(torch.equal(a, b) for a, b in zip(first, again))
    out, lse = first
    b1 = ops.attention_first_backward(q, k, v, out, lse, dO, **geom)
    for _ in range(3):
        again = ops.attention_first_backward(q, k, v, out, lse, dO, **geom)
        assert all(torch.equal(a, b) for a, b in zip(b1, again))
    dQ, _, _, delta, pk = b1
    b2 = ops.attention_second_backward(q, k, v, out, lse, delta, pk, dO, dQ, uQ, uK, uV, **geom)
    for _ in range(3):
        again = ops.attention_second_backward(q, k, v, out, lse, delta, pk, dO, dQ, uQ, uK, uV, **geom)
        assert all(torch.equal(a, b) for a, b in zip(b2, again))


def test_the_three_stages_replay_from_a_cuda_graph(monkeypatch):
    """Launch-bound callers (many small per-layer calls, reference: examples/hessian_vector_product.py:54-61)
    can record the calls once: after one eager call per device (which creates the library's host-visible
    status word) the C-ABI entry points only enqueue work on the given stream - a memset of the status
    block and the kernels - so a stream capture takes them, and a replay returns the eager call's bits."""
    # (the test suite turns on the per-call status read-back, which waits for the stream: not inside a capture)
    monkeypatch.setattr(ops, "_CHECK_STATUS", False)
    B, Hq, Hkv, N, D = 2, 12, 12, 512, 64
    g = torch.Generator().manual_seed(11)
    r = lambda h: torch.randn(B, h, N, D, generator=g).to(BF16).cuda()
    q, k, v, dO, uQ, uK, uV = r(Hq), r(Hkv), r(Hkv), r(Hq), r(Hq), r(Hkv), r(Hkv)
    geom = _geom(N, N, is_causal=True)

    def stages():
        out, lse = ops.attention_forward(q, k, v, **geom)
        dQ, dK, dV, delta, pk = ops.attention_first_backward(q, k, v, out, lse, dO, **geom)
        return (out, dQ, dK, dV) + ops.attention_second_backward(q, k, v, out, lse, delta, pk, dO, dQ, uQ, uK, uV, **geom)

    eager = [t.clone() for t in stages()]
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        recorded = stages()
    for _ in range(2):
        for t in recorded:
            t.zero_()
        graph.replay()
        torch.cuda.synchronize()
        assert all(torch.equal(a, b) for a, b in zip(recorded, eager))
    ops.check_device_status()
