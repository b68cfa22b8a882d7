"""Attention micro-benchmark with a correctness check, flag-compatible with the reference's
`python -m benchmarks.attention` (reference: benchmarks/attention/__main__.py:193-222 for the flags,
:53-189 for the flow, benchmarks/attention/__init__.py:93-117 for the two-level protocol,
benchmarks/harness.py:239-279 for the timing method).

    python -m flashbob_b200.attention_bench --mode gqa --h 32 --h-kv 8 --n 4096 --d 64 --csv out.csv

Backends: `bob` (this library's `sdpa_bob`) and `math` (materialized attention in plain PyTorch,
differentiated by stock autograd).  With `--check` every output of `bob` (out, dQ, dK, dV and, for
`--order second`, Qbar, Kbar, Vbar, dObar) is compared with `math` on the same seeded inputs.
One CSV row per backend: geometry, status, median / p20 / p80 milliseconds of one forward + first
(+ second) gradient evaluation, peak memory, per-output errors, algorithmic TFLOP/s.
"""

from __future__ import annotations

import argparse
import csv
import math
import statistics
import time
from pathlib import Path

import torch

from .interface import sdpa_bob

OUTPUTS = ("out", "dQ", "dK", "dV", "Qbar", "Kbar", "Vbar", "dObar")
_DTYPES = {"bf16": torch.bfloat16, "fp16": torch.float16, "fp32": torch.float32}


def math_attention(q, k, v, *, is_causal=False, scale=None, window_size=0, q_offset=None, k_offset=0):
    """Materialized softmax(QK^T) V with absolute-position masking; grouped heads by repetition."""
    n_q, n_k = q.shape[-2], k.shape[-2]
    reps = q.shape[1] // k.shape[1]
    if reps > 1:
        k, v = k.repeat_interleave(reps, 1), v.repeat_interleave(reps, 1)
    tau = q.shape[-1] ** -0.5 if scale is None else scale
    logits = (q @ k.transpose(-1, -2)) * tau
    if is_causal:
        q0 = (k_offset + max(0, n_k - n_q)) if q_offset is None else q_offset
        gap = (torch.arange(n_q, device=q.device) + q0)[:, None] - (torch.arange(n_k, device=q.device) + k_offset)
        keep = gap >= 0
        if window_size:
            keep &= gap < window_size
        logits = logits.masked_fill(~keep, -math.inf)
    elif window_size:
        raise NotImplementedError("window_size>0 requires is_causal=True")
    return torch.softmax(logits, -1).to(v.dtype) @ v


BACKENDS = {"bob": sdpa_bob, "math": math_attention}


def _draw(args, dtype, device):
    if args.mode == "square":
        hq, hkv, m, n = args.h, args.h, args.n, args.n
    elif args.mode == "gqa":
        hq, hkv, m, n = args.h, args.h_kv, args.n, args.n
    else:
        hq, hkv, m, n = args.h, args.h, args.m, args.n_kv
    gen = torch.Generator(device=device).manual_seed(args.seed)
    rnd = lambda *shape, grad=False: torch.randn(*shape, dtype=dtype, device=device, generator=gen,
                                                 requires_grad=grad)
    qs, ks = (args.b, hq, m, args.d), (args.b, hkv, n, args.d)
    leaves = (rnd(*qs, grad=True), rnd(*ks, grad=True), rnd(*ks, grad=True), rnd(*qs, grad=True))
    bars = (rnd(*qs), rnd(*ks), rnd(*ks))
    return (hq, hkv, m, n), leaves, bars


def _evaluate(op, leaves, bars, order, kwargs):
    q, k, v, g = leaves
    out = op(q, k, v, **kwargs)
    first = torch.autograd.grad(out, (q, k, v), g, create_graph=(order == "second"))
    vals = (out, *first)
    if order == "second":
        vals += torch.autograd.grad(first, (q, k, v, g), bars)
    return {n: t.detach() for n, t in zip(OUTPUTS, vals)}


def _pairs(m, n, kwargs):
    if not kwargs["is_causal"]:
        return m * n
    q0 = kwargs["q_offset"] if kwargs["q_offset"] is not None else kwargs["k_offset"] + max(0, n - m)
    d, w, total = q0 - kwargs["k_offset"], kwargs["window_size"], 0
    for i in range(m):
        hi, lo = min(n - 1, i + d), (max(0, i + d - w + 1) if w else 0)
        total += max(0, hi - lo + 1)
    return total


def _time(fn, warmup, iters, device):
    for _ in range(warmup):
        fn()
    ms = []
    if device.type == "cuda":
        torch.cuda.synchronize(device)
        torch.cuda.reset_peak_memory_stats(device)
        for _ in range(iters):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(); fn(); b.record(); b.synchronize()
            ms.append(a.elapsed_time(b))
        peak = torch.cuda.max_memory_allocated(device) / 2**20
    else:
        for _ in range(iters):
            t0 = time.perf_counter(); fn(); ms.append((time.perf_counter() - t0) * 1e3)
        peak = float("nan")
    ms.sort()
    pick = lambda f: ms[min(len(ms) - 1, int(f * len(ms)))]
    return {"ms": statistics.median(ms), "ms_p20": pick(0.2), "ms_p80": pick(0.8), "peak_mib": peak}


def run(args) -> list[dict]:
    dev = torch.device(("cuda" if torch.cuda.is_available() else "cpu") if args.device == "auto" else args.device)
    dtype = _DTYPES[args.dtype]
    kwargs = dict(is_causal=args.causal, scale=args.scale, window_size=args.window, q_offset=args.q_offset,
                  k_offset=args.k_offset)
    (hq, hkv, m, n), _, _ = _draw(args, dtype, dev)
    if kwargs["q_offset"] is None and args.mode == "rect":
        kwargs["q_offset"] = args.k_offset + (n - m)
    names = OUTPUTS[: 8 if args.order == "second" else 4]
    unit = 2 * _pairs(m, n, kwargs) * args.d * args.b * hq
    flops = unit * (2 + 5 + (12 if args.order == "second" else 0))
    truth = None
    if args.check:
        _, leaves, bars = _draw(args, dtype, dev)
        truth = _evaluate(math_attention, leaves, bars, args.order, kwargs)
    rows = []
    for name in args.backends:
        row = dict(mode=args.mode, backend=name, order=args.order, B=args.b, H_Q=hq, H_KV=hkv, M=m, N=n, D=args.d,
                   causal=args.causal, window=args.window, dtype=args.dtype, status="pending", error=None)
        try:
            _, leaves, bars = _draw(args, dtype, dev)
            if truth is not None:
                got = _evaluate(BACKENDS[name], leaves, bars, args.order, kwargs)
                for o in names:
                    a, b = got[o].float(), truth[o].float()
                    row[f"{o}_max_abs"] = float((a - b).abs().max())
                    row[f"{o}_l2_rel"] = float((a - b).norm() / b.norm().clamp_min(1e-30))
                    torch.testing.assert_close(a, b, atol=args.atol, rtol=args.rtol,
                                               msg=f"{name} {o} failed the correctness check")
            row.update(_time(lambda: _evaluate(BACKENDS[name], leaves, bars, args.order, kwargs), args.warmup,
                             args.iters, dev))
            row["tflops"] = flops / (row["ms"] * 1e-3) / 1e12
            row["status"] = "ok"
        except torch.OutOfMemoryError as err:
            row["status"], row["error"] = "oom", " ".join(str(err).split())[:200]
        rows.append(row)
    base = next((r["ms"] for r in rows if r["backend"] == "math" and r["status"] == "ok"), None)
    for r in rows:
        r["speedup_vs_math"] = base / r["ms"] if base and r["status"] == "ok" else None
        shown = f"{r['ms']:.3f} ms  {r['tflops']:.1f} TFLOP/s" if r["status"] == "ok" else r["status"]
        print(f"{r['mode']:>6} {r['backend']:>5} B={r['B']} H={hq}/{hkv} M={m} N={n} D={args.d} {shown}")
    if args.csv:
        path = Path(args.csv)
        path.parent.mkdir(parents=True, exist_ok=True)
        cols = list(dict.fromkeys(c for r in rows for c in r))
        with path.open("w", newline="") as fh:
            w = csv.DictWriter(fh, fieldnames=cols)
            w.writeheader(); w.writerows(rows)
    return rows


def build_parser() -> argparse.ArgumentParser:
    p = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    p.add_argument("--mode", choices=("square", "gqa", "rect"), default="square")
    p.add_argument("--backends", nargs="+", choices=tuple(BACKENDS), default=("math", "bob"))
    p.add_argument("--order", choices=("first", "second"), default="second")
    p.add_argument("--b", type=int, default=1)
    p.add_argument("--h", type=int, default=8, help="query heads; also key heads outside GQA")
    p.add_argument("--h-kv", type=int, default=2)
    p.add_argument("--n", type=int, default=512, help="square sequence length")
    p.add_argument("--m", type=int, default=128, help="rectangular query length")
    p.add_argument("--n-kv", type=int, default=512, help="rectangular key/value length")
    p.add_argument("--d", type=int, default=64)
    p.add_argument("--causal", action=argparse.BooleanOptionalAction, default=True)
    p.add_argument("--window", type=int, default=0)
    p.add_argument("--q-offset", type=int)
    p.add_argument("--k-offset", type=int, default=0)
    p.add_argument("--scale", type=float)
    p.add_argument("--dtype", choices=tuple(_DTYPES), default="bf16")
    p.add_argument("--device", choices=("auto", "cpu", "cuda"), default="cuda")
    p.add_argument("--warmup", type=int, default=10)
    p.add_argument("--iters", type=int, default=50)
    p.add_argument("--seed", type=int, default=0)
    p.add_argument("--check", action=argparse.BooleanOptionalAction, default=True)
    p.add_argument("--atol", type=float, default=0.08)
    p.add_argument("--rtol", type=float, default=0.08)
    p.add_argument("--csv")
    return p


def main(argv=None) -> None:
    run(build_parser().parse_args(argv))


if __name__ == "__main__":
    main()
