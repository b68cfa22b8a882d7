"""The workspace-free second backward (`bob_sm100_bwd2_noalloc`) against the regular entry point.

Some hosts cannot hand a scratch buffer to a call - they run where allocator calls are forbidden
or they do not own an allocator at all - so this entry point keeps its scratch inside the library.
The test drives both entry points through the C ABI on the same inputs, twice in a row (the
built-in scratch keeps the previous call's contents), and expects identical results; it also
checks that a problem larger than the built-in scratch is refused on the host.
This file sorts last on purpose: a `-x` run has exercised every other test before it starts.
"""

import ctypes

import pytest
import torch

from flashbob_b200 import _lib, ops
from oracle import bob_oracle as O

pytestmark = pytest.mark.gpu


def _vp(t):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def _setup(seed, B, Hq, Hkv, N, D):
    dtype = torch.bfloat16
    q, k, v, dO, uQ = O.seeded_inputs(seed, (B, Hq, N, D), (B, Hkv, N, D), dtype, n_extra_q=2)
    uK, uV = O.seeded_inputs(seed + 1, (B, Hq, N, D), (B, Hkv, N, D), dtype)[1:]
    t = {n: x.cuda() for n, x in dict(q=q, k=k, v=v, dO=dO, uQ=uQ, uK=uK, uV=uV).items()}
    geom = dict(is_causal=True, window_size=0, q_offset=0, k_offset=0, scale=None)
    t["out"], t["lse"] = ops.attention_forward(t["q"], t["k"], t["v"], **geom)
    t["dQ"], _, _, t["delta"], t["pk"] = ops.attention_first_backward(
        t["q"], t["k"], t["v"], t["out"], t["lse"], t["dO"], **geom)
    g = ops._geom(t["q"], t["k"], **geom)
    for field, name in ((g.q_strides, "q"), (g.k_strides, "k"), (g.v_strides, "v"), (g.out_strides, "out"),
                        (g.do_strides, "dO"), (g.dq_strides, "dQ"), (g.uq_strides, "uQ"),
                        (g.uk_strides, "uK"), (g.uv_strides, "uV")):
        ops._set_strides(field, t[name])
    return t, g


def _results(t):
    return [torch.full_like(t[n], float("nan")) for n in ("q", "k", "k", "q")]   # Qbar, Kbar, Vbar, dObar


def _call(lib, fn_name, g, t, res, ws=None):
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    args = [ctypes.byref(g)] + [_vp(t[n]) for n in ("q", "k", "v", "out", "lse", "delta", "pk", "dO", "dQ",
                                                    "uQ", "uK", "uV")] + [_vp(r) for r in res]
    if ws is not None:
        args.append(_vp(ws))
    args.append(stream)
    return getattr(lib, fn_name)(*args)


def test_noalloc_second_backward_matches_regular_entry_point_twice():
    lib = _lib.load()
    for round_, (seed, shape) in enumerate(((40, (2, 4, 2, 300, 64)), (50, (1, 8, 8, 520, 128)))):
        t, g = _setup(seed, *shape)
        ws = torch.empty(lib.bob_sm100_workspace_bytes(_lib.STAGE_BWD2, ctypes.byref(g)), dtype=torch.uint8,
                         device="cuda")
        ref = _results(t)
        assert _call(lib, "bob_sm100_bwd2", g, t, ref, ws) == 0
        torch.cuda.synchronize()
        assert lib.bob_sm100_read_status(_vp(ws), None) == 0
        first, second = _results(t), _results(t)
        before = torch.cuda.memory_allocated()
        assert _call(lib, "bob_sm100_bwd2_noalloc", g, t, first) == 0     # two calls in a row on the
        assert _call(lib, "bob_sm100_bwd2_noalloc", g, t, second) == 0    # same stream share the scratch
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == before
        assert lib.bob_sm100_noalloc_read_status(torch.cuda.current_device(), None) == 0
        for got in (first, second):
            for name, a, b in zip(("Qbar", "Kbar", "Vbar", "dObar"), got, ref):
                assert torch.isfinite(a.float()).all(), (round_, name)
                torch.testing.assert_close(a.float(), b.float(), rtol=0.0, atol=0.0, msg=f"{round_}:{name}")


def test_noalloc_refuses_problems_beyond_its_scratch():
    lib = _lib.load()
    assert lib.bob_sm100_noalloc_max_rows() == 1 << 20
    t, g = _setup(60, 1, 2, 2, 64, 64)
    g.Nq = (1 << 20)          # 2 heads x 2^20 rows: twice the limit; refused before anything is read
    rc = _call(lib, "bob_sm100_bwd2_noalloc", g, t, _results(t))
    assert rc == -12
    assert b"built-in scratch" in lib.bob_sm100_error_string(rc)
    torch.cuda.synchronize()
