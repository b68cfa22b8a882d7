"""Hessian-vector products over the parameters of a small transformer, through `sdpa_bob`.

What a second-order optimiser or a curvature probe does with the operator: `Hv = d/dtheta (dL/dtheta . v)`
needs the first gradients kept in the graph, so every attention layer is evaluated forward, backward
with `create_graph=True`, and backward once more.  PyTorch's fused attention kernels have no second
backward; its math backend has one but materializes the `[B, H, N, N]` score matrix.  This module
times one such step per sequence length for both and reports latency, peak memory and how far the two
`Hv` results are apart (reference: examples/hessian_vector_product.py:22-92 for the measured step and
its flags, benchmarks/models/language_model_benchmark.py:625-646 for the step inside its model
benchmark).

    python -m flashbob_b200.hvp_bench --seq-lens 1024 4096 --dim 768 --heads 12 --layers 4
"""

from __future__ import annotations

import argparse
import csv
import statistics
import sys

import torch
import torch.nn as nn
import torch.nn.functional as F

from .interface import sdpa_bob


def math_attention(q, k, v, *, is_causal=False, scale=None):
    """Materialized attention in plain tensor operations: differentiable any number of times,
    O(N^2) memory.  Grouped heads are expanded."""
    g = q.shape[1] // k.shape[1]
    if g > 1:
        k, v = k.repeat_interleave(g, dim=1), v.repeat_interleave(g, dim=1)
    s = (q @ k.transpose(-1, -2)) * (q.shape[-1] ** -0.5 if scale is None else scale)
    if is_causal:
        n_q, n_k = s.shape[-2:]
        keep = torch.ones(n_q, n_k, dtype=torch.bool, device=s.device).tril(n_k - n_q)
        s = s.masked_fill(~keep, float("-inf"))
    return torch.softmax(s.float(), dim=-1).to(q.dtype) @ v


class Layer(nn.Module):
    """Pre-norm attention + MLP block; `kv_heads < heads` gives grouped-query attention."""

    def __init__(self, dim: int, heads: int, kv_heads: int, attention):
        super().__init__()
        if dim % heads or heads % kv_heads:
            raise ValueError("dim must be a multiple of heads, heads a multiple of kv_heads")
        self.heads, self.kv_heads, self.hd, self.attention = heads, kv_heads, dim // heads, attention
        self.norm1, self.norm2 = nn.LayerNorm(dim), nn.LayerNorm(dim)
        self.q = nn.Linear(dim, dim, bias=False)
        self.kv = nn.Linear(dim, 2 * kv_heads * self.hd, bias=False)
        self.o = nn.Linear(dim, dim, bias=False)
        self.up, self.down = nn.Linear(dim, 4 * dim), nn.Linear(4 * dim, dim)

    def forward(self, x):
        b, n, _ = x.shape
        h = self.norm1(x)
        q = self.q(h).view(b, n, self.heads, self.hd).transpose(1, 2)
        k, v = (t.view(b, n, self.kv_heads, self.hd).transpose(1, 2) for t in self.kv(h).chunk(2, dim=-1))
        y = self.attention(q, k, v, is_causal=True)
        x = x + self.o(y.transpose(1, 2).reshape(b, n, -1))
        return x + self.down(F.gelu(self.up(self.norm2(x))))


def hvp(model: nn.Module, x: torch.Tensor, directions):
    """`Hv` of the mean-square output with respect to every parameter, `v` given per parameter."""
    params = list(model.parameters())
    loss = model(x).float().square().mean()
    grads = torch.autograd.grad(loss, params, create_graph=True)
    inner = sum((g.float() * d).sum() for g, d in zip(grads, directions))
    return torch.autograd.grad(inner, params)


BACKENDS = {"math": math_attention, "bob": sdpa_bob}


def measure(backend: str, seq_len: int, args, device, dtype):
    torch.manual_seed(0)
    model = nn.Sequential(*[Layer(args.dim, args.heads, args.kv_heads or args.heads, BACKENDS[backend])
                            for _ in range(args.layers)]).to(device=device, dtype=dtype)
    x = torch.randn(args.batch, seq_len, args.dim, device=device, dtype=dtype)
    directions = [torch.randn_like(p, dtype=torch.float32) for p in model.parameters()]
    step = lambda: hvp(model, x, directions)
    for _ in range(args.warmup):
        step()
    cuda = device.type == "cuda"
    if cuda:
        torch.cuda.synchronize(device)
        torch.cuda.reset_peak_memory_stats(device)
    times = []
    result = None
    for _ in range(args.iters):
        if cuda:
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            result = step()
            e1.record()
            e1.synchronize()
            times.append(e0.elapsed_time(e1))
        else:
            import time
            t0 = time.perf_counter()
            result = step()
            times.append((time.perf_counter() - t0) * 1e3)
    peak = torch.cuda.max_memory_allocated(device) / 2**20 if cuda else float("nan")
    flat = torch.cat([r.detach().float().flatten() for r in result]).cpu()
    return statistics.median(times), peak, flat


def run(args) -> list[dict]:
    device = torch.device(args.device)
    dtype = {"bf16": torch.bfloat16, "fp16": torch.float16, "fp32": torch.float32}[args.dtype]
    rows = []
    for n in args.seq_lens:
        row = {"N": n, "batch": args.batch, "dim": args.dim, "heads": args.heads,
               "kv_heads": args.kv_heads or args.heads, "layers": args.layers, "dtype": args.dtype}
        flats = {}
        for name in ("math", "bob"):
            try:
                ms, peak, flats[name] = measure(name, n, args, device, dtype)
                row[f"{name}_ms"], row[f"{name}_MiB"] = ms, peak
            except torch.OutOfMemoryError:
                row[f"{name}_ms"], row[f"{name}_MiB"] = None, None
            if device.type == "cuda":
                torch.cuda.empty_cache()
        if len(flats) == 2:
            row["hv_l2_rel"] = ((flats["bob"] - flats["math"]).norm() / flats["math"].norm()).item()
        if row.get("math_ms") and row.get("bob_ms"):
            row["speedup"] = row["math_ms"] / row["bob_ms"]
        rows.append(row)
    return rows


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--seq-lens", nargs="+", type=int, default=[512, 1024, 2048, 4096])
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--dim", type=int, default=512)
    ap.add_argument("--heads", type=int, default=8)
    ap.add_argument("--kv-heads", type=int, default=0, help="fewer than --heads: grouped-query attention")
    ap.add_argument("--layers", type=int, default=2)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--dtype", default="bf16", choices=["bf16", "fp16", "fp32"])
    ap.add_argument("--device", default="cuda")
    ap.add_argument("--csv", default="")
    return ap


def main(argv=None) -> None:
    args = build_parser().parse_args(argv)
    if args.device == "cuda" and not torch.cuda.is_available():
        raise SystemExit("no CUDA device (use --device cpu --dtype fp32 for a functional run)")
    rows = run(args)
    cols = ["N", "batch", "dim", "heads", "kv_heads", "layers", "dtype", "math_ms", "math_MiB", "bob_ms", "bob_MiB",
            "speedup", "hv_l2_rel"]
    fmt = lambda v: "" if v is None else (f"{v:.4g}" if isinstance(v, float) else str(v))
    print(" ".join(f"{c:>9}" for c in cols))
    for r in rows:
        print(" ".join(f"{fmt(r.get(c)):>9}" for c in cols))
    if args.csv:
        with open(args.csv, "w", newline="") as fh:
            w = csv.DictWriter(fh, fieldnames=cols)
            w.writeheader()
            for r in rows:
                w.writerow({c: r.get(c) for c in cols})


if __name__ == "__main__":
    main(sys.argv[1:])
