#!/usr/bin/env python
"""Runs the UNMODIFIED reference (`bob` from baseline/_ref, installed there with pip from the
reference checkout) through its own public operator and prints one JSON object.

This file imports nothing of this repository: no kernels, no host wrappers, no oracle.  It is meant
to run as a child process whose `sys.path` starts with baseline/_ref, so that `import bob` is the
reference and not this repository's alias package of the same name.

Modes
  cpu    the reference's CPU route (`bob.sdpa_bob` on CPU tensors = PyTorch math attention with stock
         autograd, reference: src/bob/sdpa.py:457-465) timed on the host cores: second
         `autograd.grad` (with respect to q, k, v and the first cotangent) of ONE KV head of the
         workload with `--heads` of its query heads, for `--kv-heads` KV heads one after the other.
         The reference's CPU route refuses grouped heads, so each query head is one multi-head call
         on the shared K/V and autograd sums the key-side gradients.
  cuda   the reference's CUDA route (cuDNN forward / first backward + its Triton second backward)
         on the current GPU: first-call time (autotune), warm times of forward, forward + first
         backward, second backward and the whole loss chain, and per-tensor errors of all eight
         outputs against the reference's own fp64 CPU path (`bob.attention.sdpa_math`) on one KV
         group.  With --save the eight outputs of that KV group are written to a file.
"""

from __future__ import annotations

import argparse
import json
import os
import sys
import time
from pathlib import Path

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE / "_ref"))

import torch  # noqa: E402


def _import_reference():
    import bob

    if "_ref" not in str(Path(bob.__file__).resolve()):
        raise RuntimeError(f"`bob` resolved to {bob.__file__}, not to baseline/_ref")
    return bob


def _seeded(seed, shapes, dtype):
    g = torch.Generator().manual_seed(int(seed))
    return [torch.randn(s, dtype=torch.float32, generator=g).to(dtype) for s in shapes]


def causal_pairs(n):
    return n * (n + 1) // 2


def mode_cpu(a):
    bob = _import_reference()
    torch.set_num_threads(a.threads or os.cpu_count() or 1)
    N, D, H, M = a.seq, a.dim, a.heads, a.kv_heads
    times = []
    for i in range(a.warmup + a.steps):
        step = 0.0
        for kv in range(M):
            # one KV head at a time: the graph of the first gradients (untimed) is rebuilt for each, so
            # that only one head group's materialized score tensors are alive at once
            q, dO, uQ = _seeded(10 * kv, [(1, H, N, D)] * 3, torch.float32)
            k, v, uK, uV = _seeded(10 * kv + 1, [(1, 1, N, D)] * 4, torch.float32)
            q, k, v, dO = (t.requires_grad_(True) for t in (q, k, v, dO))
            out = torch.cat([bob.sdpa_bob(q[:, h:h + 1], k, v, is_causal=True) for h in range(H)], dim=1)
            first = torch.autograd.grad(out, (q, k, v), dO, create_graph=True)
            t0 = time.perf_counter()
            torch.autograd.grad(first, (q, k, v, dO), (uQ, uK, uV))
            step += time.perf_counter() - t0
            del out, first
        if i >= a.warmup:
            times.append(step)
    print(json.dumps({"mode": "cpu", "seconds": times, "flops_per_step": 12 * 2 * causal_pairs(N) * D * H * M,
                      "threads": torch.get_num_threads(), "heads": H, "kv_heads": M, "seq": N, "dim": D,
                      "what": "bob.sdpa_bob CPU route (math attention, stock autograd), fp32"}))


def _second(op, q, k, v, dO, bars, **kw):
    q, k, v, dO = (t.detach().clone().requires_grad_(True) for t in (q, k, v, dO))
    out = op(q, k, v, **kw)
    first = torch.autograd.grad(out, (q, k, v), dO, create_graph=True)
    second = torch.autograd.grad(first, (q, k, v, dO), bars)
    return (out, *first, *second)


def _err(actual, expected):
    a, e = actual.detach().double().cpu(), expected.detach().double().cpu()
    d = a - e
    return {"l2_rel": d.norm().item() / e.norm().item(), "max_abs_rel": d.abs().max().item() / e.abs().max().item()}


def _time(fn, n=10, warm=3):
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(n):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / n


NAMES = ("out", "dQ", "dK", "dV", "Qbar", "Kbar", "Vbar", "dObar")


def mode_cuda(a):
    bob = _import_reference()
    from bob.attention import sdpa_math

    dt = {"bf16": torch.bfloat16, "fp16": torch.float16}[a.dtype]
    B, Hq, Hkv, Nq, Nk, D = a.batch, a.hq, a.hkv, a.seq, a.seq_k or a.seq, a.dim
    G = Hq // Hkv
    kw = dict(is_causal=True)
    if a.window:
        kw["window_size"] = a.window
    q, k, v, dO, bq = _seeded(a.seed, [(B, Hq, Nq, D), (B, Hkv, Nk, D), (B, Hkv, Nk, D), (B, Hq, Nq, D), (B, Hq, Nq, D)], dt)
    _, bk, bv = _seeded(a.seed + 1000, [(B, Hq, Nq, D), (B, Hkv, Nk, D), (B, Hkv, Nk, D)], dt)
    c = lambda t: t.cuda()
    qd, kd, vd, dOd, bars = c(q), c(k), c(v), c(dO), (c(bq), c(bk), c(bv))
    t0 = time.time()
    got = _second(bob.sdpa_bob, qd, kd, vd, dOd, bars, **kw)
    torch.cuda.synchronize()
    first_call = time.time() - t0
    res = {"mode": "cuda", "shape": {"B": B, "Hq": Hq, "Hkv": Hkv, "Nq": Nq, "Nk": Nk, "D": D, "dtype": a.dtype, **kw},
           "first_call_s": first_call, "torch": torch.__version__}
    try:
        import triton
        res["triton"] = triton.__version__
    except Exception:  # pragma: no cover
        pass
    # errors of KV group `a.group` of batch 0 against the reference's own fp64 CPU path
    hk = a.group
    hs = slice(hk * G, hk * G + G)
    rq, rdO, rbq = (t[:1, hs].double() for t in (q, dO, bq))
    rk, rv, rbk, rbv = (t[:1, hk:hk + 1].double().repeat_interleave(G, dim=1) for t in (k, v, bk, bv))
    if Nq == Nk:
        op64 = lambda x, y, z: sdpa_math(x, y, z, is_causal=True, window_size=a.window)
    else:
        from bob.kernels.rectangular import sdpa_math_rect
        op64 = lambda x, y, z: sdpa_math_rect(x, y, z, q_offset=Nk - Nq, k_offset=0, is_causal=True,
                                              window_size=a.window, scale=None)
    ref = _second(op64, rq, rk, rv, rdO, (rbq, rbk, rbv))
    red = lambda t: t.reshape(1, 1, G, Nk, D).sum(2)          # expanded KV heads back to the one KV head
    ref = [t if i in (0, 1, 4, 7) else red(t) for i, t in enumerate(ref)]
    pick = lambda i, t: t[:1, hs] if i in (0, 1, 4, 7) else t[:1, hk:hk + 1]
    res["errors_vs_fp64"] = {n: _err(pick(i, got[i]), ref[i]) for i, n in enumerate(NAMES)}
    if a.save:
        torch.save({"outputs": {n: pick(i, got[i]).cpu() for i, n in enumerate(NAMES)}, "group": hk, "seed": a.seed}, a.save)
    if a.time:
        unit = 2 * (causal_pairs(Nq) if Nq == Nk and not a.window else 0) * D * B * Hq
        qg, kg, vg, dOg = (t.detach().clone().requires_grad_(True) for t in (qd, kd, vd, dOd))
        out = bob.sdpa_bob(qg, kg, vg, **kw)
        first = torch.autograd.grad(out, (qg, kg, vg), dOg, create_graph=True)
        t_fwd = _time(lambda: bob.sdpa_bob(qg, kg, vg, **kw))
        t_fb = _time(lambda: torch.autograd.grad(bob.sdpa_bob(qg, kg, vg, **kw), (qg, kg, vg), dOg, create_graph=True))
        t_b2 = _time(lambda: torch.autograd.grad(first, (qg, kg, vg, dOg), bars, retain_graph=True))

        def chain():
            o = bob.sdpa_bob(qg, kg, vg, **kw)
            dq, dk, dv = torch.autograd.grad(o.float().square().mean(), (qg, kg, vg), create_graph=True)
            L2 = dq.float().square().mean() + dk.float().square().mean() + dv.float().square().mean()
            return torch.autograd.grad(L2, (qg, kg, vg))

        t_chain = _time(chain, n=5, warm=2)
        res["ms"] = {"forward": t_fwd, "forward_plus_first_backward": t_fb, "second_backward": t_b2, "chain": t_chain}
        if unit:
            res["tflops"] = {"forward_2u": 2 * unit / t_fwd / 1e9, "second_backward_12u": 12 * unit / t_b2 / 1e9,
                             "chain_24u": 24 * unit / t_chain / 1e9}
    print(json.dumps(res))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--mode", choices=["cpu", "cuda"], required=True)
    ap.add_argument("--seq", type=int, default=4096)
    ap.add_argument("--seq-k", type=int, default=0)
    ap.add_argument("--dim", type=int, default=64)
    ap.add_argument("--heads", type=int, default=1, help="cpu mode: query heads of the one KV head")
    ap.add_argument("--kv-heads", type=int, default=1, help="cpu mode: KV heads per step, one after the other")
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=1)
    ap.add_argument("--threads", type=int, default=0)
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--hq", type=int, default=32)
    ap.add_argument("--hkv", type=int, default=8)
    ap.add_argument("--window", type=int, default=0)
    ap.add_argument("--dtype", default="bf16")
    ap.add_argument("--seed", type=int, default=2)
    ap.add_argument("--group", type=int, default=0)
    ap.add_argument("--save", default="")
    ap.add_argument("--time", action="store_true")
    a = ap.parse_args()
    (mode_cpu if a.mode == "cpu" else mode_cuda)(a)


if __name__ == "__main__":
    main()
