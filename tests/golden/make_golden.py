"""Generate the golden fixtures in this directory from the reference implementation.

Run where the reference checkout is available:

    python tests/golden/make_golden.py /path/to/reference

It imports the reference's own CPU code (`bob.sdpa_bob` on CPU tensors,
`bob.attention.sdpa_math`, `bob.kernels.rectangular.sdpa_math_rect`,
`benchmarks.attention.attention_reference`) and records, for seeded inputs, the eight outputs
of the two-level gradient protocol.  The seeds and shapes are those of the reference's own
tests (tests/unit/test_public_api.py:36-75, tests/cuda/test_attention_correctness.py:33-53)
plus the small benchmark configuration.  The fixtures are small `.npz` files; the tests read
them without the reference being present.
"""

import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
NAMES = ("out", "dQ", "dK", "dV", "Qbar", "Kbar", "Vbar", "dObar")


def second_grad(op, q, k, v, dO, bars, **kw):
    q, k, v, dO = (t.detach().clone().requires_grad_(True) for t in (q, k, v, dO))
    out = op(q, k, v, **kw)
    first = torch.autograd.grad(out, (q, k, v), dO, create_graph=True)
    second = torch.autograd.grad(first, (q, k, v, dO), bars)
    return [t.detach() for t in (out, *first, *second)]


def draw(seed, q_shape, kv_shape, dtype):
    g = torch.Generator().manual_seed(seed)
    r = lambda s: torch.randn(s, dtype=torch.float32, generator=g).to(dtype)
    # order: q, k, v, dO, barQ, barK, barV
    return r(q_shape), r(kv_shape), r(kv_shape), r(q_shape), r(q_shape), r(kv_shape), r(kv_shape)


def main(ref_root: str) -> None:
    sys.path[:0] = [str(Path(ref_root) / "src"), str(Path(ref_root))]
    import bob
    from bob.attention import sdpa_math
    from bob.kernels.rectangular import sdpa_math_rect
    from benchmarks.attention import attention_reference

    cases = {
        # name: (Hq, Hkv, Nq, Nk, D, kwargs, seed)
        "unit_square": (2, 2, 5, 5, 4, dict(is_causal=True, scale=0.7), 0),
        "unit_rect": (2, 2, 3, 6, 4, dict(is_causal=True, window_size=4, q_offset=3, k_offset=0), 1),
        "causal": (2, 2, 64, 64, 64, dict(is_causal=True), 0),
        "noncausal": (2, 2, 48, 48, 128, dict(is_causal=False), 0),
        "window": (2, 2, 64, 64, 64, dict(is_causal=True, window_size=16), 0),
        "gqa": (8, 2, 64, 64, 64, dict(is_causal=True), 0),
        "mqa": (8, 1, 64, 64, 64, dict(is_causal=True), 0),
        "rect": (2, 2, 32, 64, 64, dict(is_causal=True, window_size=32, q_offset=32, k_offset=0), 0),
        "rect_offsets": (2, 2, 24, 40, 32, dict(is_causal=True, window_size=20, q_offset=1000,
                                                k_offset=984), 3),
    }
    for name, (hq, hkv, nq, nk, d, kw, seed) in cases.items():
        q_shape, kv_shape = (1, hq, nq, d), (1, hkv, nk, d)
        store = {}
        # (1) fp64 ground truth from the reference's materialized reference function
        t64 = draw(seed, q_shape, kv_shape, torch.float64)
        vals = second_grad(attention_reference, *t64[:4], t64[4:], **kw)
        for n, x in zip(NAMES, vals):
            store[f"ref64_{n}"] = x.numpy()
        # (2) the operator's own CPU route in fp32 (MHA only: the CPU route rejects GQA)
        if hq == hkv:
            t32 = draw(seed, q_shape, kv_shape, torch.float32)
            vals = second_grad(bob.sdpa_bob, *t32[:4], t32[4:], **kw)
            for n, x in zip(NAMES, vals):
                store[f"op32_{n}"] = x.numpy()
            # (3) the fp64 entry points under the operator (it rejects fp64 itself)
            rect = nq != nk or kw.get("q_offset", 0) != kw.get("k_offset", 0)
            if rect:
                fn = lambda q, k, v: sdpa_math_rect(
                    q, k, v, q_offset=kw["q_offset"], k_offset=kw["k_offset"],
                    is_causal=kw["is_causal"], window_size=kw.get("window_size", 0),
                    scale=kw.get("scale"))
            else:
                fn = lambda q, k, v: sdpa_math(q, k, v, is_causal=kw["is_causal"],
                                               scale=kw.get("scale"),
                                               window_size=kw.get("window_size", 0))
            vals = second_grad(fn, *t64[:4], t64[4:])
            for n, x in zip(NAMES, vals):
                store[f"math64_{n}"] = x.numpy()
        store["meta"] = np.array(repr(dict(hq=hq, hkv=hkv, nq=nq, nk=nk, d=d, kw=kw, seed=seed)))
        np.savez_compressed(HERE / f"{name}.npz", **store)
        print(name, {k: v.shape for k, v in store.items() if k.startswith("ref64")})

    # The small benchmark configuration: MHA fp32, B=1, H=2, S=128, D=64, causal, loss chain.
    g = torch.Generator().manual_seed(0)
    shape = (1, 2, 128, 64)
    q, k, v = (torch.randn(shape, dtype=torch.float32, generator=g) for _ in range(3))

    def chain(op, q, k, v, **kw):
        q, k, v = (t.detach().clone().requires_grad_(True) for t in (q, k, v))
        out = op(q, k, v, **kw)
        L1 = out.square().mean()
        dq, dk, dv = torch.autograd.grad(L1, (q, k, v), create_graph=True)
        L2 = dq.square().mean() + dk.square().mean() + dv.square().mean()
        return [t.detach() for t in (out, dq, dk, dv, *torch.autograd.grad(L2, (q, k, v)))]

    names = ("out", "dq", "dk", "dv", "ddq", "ddk", "ddv")
    store = {}
    for n, x in zip(names, chain(bob.sdpa_bob, q, k, v, is_causal=True, scale=1 / 8.0)):
        store[f"op32_{n}"] = x.numpy()
    for n, x in zip(names, chain(sdpa_math, q.double(), k.double(), v.double(), is_causal=True,
                                 scale=1 / 8.0)):
        store[f"math64_{n}"] = x.numpy()
    np.savez_compressed(HERE / "config0_chain.npz", **store)
    print("config0_chain", {k: float(np.abs(v).max()) for k, v in store.items()})


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: python make_golden.py <checkout of the reference project>")
    main(sys.argv[1])
