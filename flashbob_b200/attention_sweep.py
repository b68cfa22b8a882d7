"""A bounded replay of the reference's attention sweeps through this library's micro-benchmark.

    python -m flashbob_b200.attention_sweep --csv sweep.csv [--full]

The reference's `benchmarks/reproduce.sh attention` target (reference: benchmarks/reproduce.sh:63-107)
sweeps multi-head attention at head dims 32 / 64 / 128 up to 262 144 tokens, grouped heads 24/8 at
head dim 128, multi-query 8/1 at head dim 64 and a 256 x 4096 rectangle with a 512-token window, each
case through `python -m benchmarks.attention` with the flags that `flashbob_b200.attention_bench`
also takes.  This script runs the same cases (a subset of the lengths by default, all of them with
--full) through `attention_bench.run` and writes every row into one CSV.  Cases too large for a
materialized comparison run with `--no-check`, as in the reference.
"""

from __future__ import annotations

import argparse
import csv
from pathlib import Path

from . import attention_bench


def cases(full: bool):
    sq = lambda n, d, check=True: (f"mha-d{d}-n{n}", ["--mode", "square", "--n", str(n), "--d", str(d)], check)
    out = []
    for n in ((256, 512, 1024, 2048, 4096, 8192, 16384) if full else (1024, 4096, 16384)):
        out.append(sq(n, 64))
    for d in (32, 128):
        out.append(sq(4096, d))
    for n in ((256, 512, 1024, 2048) if full else (2048,)):
        out.append(sq(n, 128))
    for n in ((32768, 65536, 131072, 262144) if full else (32768, 131072)):
        out.append(sq(n, 64, check=False))
    for n in ((8192, 16384, 32768, 65536) if full else (16384,)):
        out.append(sq(n, 128, check=False))
    for n in ((256, 512, 1024, 2048, 4096) if full else (1024, 4096)):
        out.append((f"gqa-n{n}", ["--mode", "gqa", "--h", "24", "--h-kv", "8", "--n", str(n), "--d", "128"], True))
        out.append((f"mqa-n{n}", ["--mode", "gqa", "--h", "8", "--h-kv", "1", "--n", str(n), "--d", "64"], True))
    out.append(("rectangular", ["--mode", "rect", "--m", "256", "--n-kv", "4096", "--window", "512", "--d", "64"], True))
    return out


def main(argv=None) -> None:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--csv", required=True)
    ap.add_argument("--full", action="store_true", help="every length of the reference's sweep")
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--iters", type=int, default=10)
    a = ap.parse_args(argv)
    rows = []
    parser = attention_bench.build_parser()
    for name, flags, check in cases(a.full):
        extra = ["--backends", "math", "bob", "--check"] if check else ["--backends", "bob", "--no-check"]
        args = parser.parse_args(flags + extra + ["--warmup", str(a.warmup), "--iters", str(a.iters)])
        for r in attention_bench.run(args):
            rows.append({"case": name, **r})
    cols = list(dict.fromkeys(c for r in rows for c in r))
    path = Path(a.csv)
    path.parent.mkdir(parents=True, exist_ok=True)
    with path.open("w", newline="") as fh:
        w = csv.DictWriter(fh, fieldnames=cols)
        w.writeheader()
        w.writerows(rows)


if __name__ == "__main__":
    main()
