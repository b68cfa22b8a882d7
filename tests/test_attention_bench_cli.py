"""The micro-benchmark CLI: flags, CSV columns and the built-in correctness check."""

import csv

import pytest

from flashbob_b200 import attention_bench as ab


def test_cli_runs_on_cpu_and_writes_the_expected_columns(tmp_path):
    out = tmp_path / "rows.csv"
    rows = ab.run(ab.build_parser().parse_args(
        ["--device", "cpu", "--dtype", "fp32", "--n", "24", "--h", "2", "--d", "8", "--warmup", "0", "--iters", "2",
         "--atol", "2e-5", "--rtol", "2e-5", "--csv", str(out)]))
    assert [r["backend"] for r in rows] == ["math", "bob"] and all(r["status"] == "ok" for r in rows)
    with out.open() as fh:
        cols = csv.DictReader(fh).fieldnames
    for c in ("mode", "backend", "order", "B", "H_Q", "H_KV", "M", "N", "D", "causal", "window", "dtype", "status",
              "ms", "Qbar_max_abs", "dObar_l2_rel", "speedup_vs_math", "tflops"):
        assert c in cols, c


def test_cli_rect_window_on_cpu():
    rows = ab.run(ab.build_parser().parse_args(
        ["--device", "cpu", "--dtype", "fp32", "--mode", "rect", "--m", "6", "--n-kv", "14", "--window", "5", "--h", "2",
         "--d", "8", "--warmup", "0", "--iters", "1", "--atol", "2e-5", "--rtol", "2e-5"]))
    assert all(r["status"] == "ok" for r in rows)


@pytest.mark.gpu
@pytest.mark.parametrize("argv", [
    ["--mode", "square", "--n", "256", "--d", "64"],
    ["--mode", "gqa", "--h", "8", "--h-kv", "2", "--n", "256", "--d", "64"],
    ["--mode", "gqa", "--h", "8", "--h-kv", "1", "--n", "256", "--d", "64"],
    ["--mode", "rect", "--m", "128", "--n-kv", "256", "--window", "128", "--d", "64"],
    ["--mode", "square", "--n", "300", "--d", "32", "--dtype", "fp16"],
    ["--mode", "square", "--n", "256", "--d", "128", "--no-causal"],
])
def test_cli_check_on_gpu(argv):
    """The bounded operator checks of the reference's reproduce driver
    (reference: benchmarks/reproduce.sh:52-61), all eight outputs at atol = rtol = 0.08."""
    rows = ab.run(ab.build_parser().parse_args(argv + ["--warmup", "1", "--iters", "3"]))
    assert all(r["status"] == "ok" for r in rows)


def test_sweep_lists_the_reference_cases():
    """The sweep driver covers the case families of the reference's sweep (reference:
    benchmarks/reproduce.sh:63-107) and every flag list parses with the CLI's own parser."""
    from flashbob_b200 import attention_sweep

    full = attention_sweep.cases(full=True)
    names = [n for n, _, _ in full]
    assert len(full) == 7 + 2 + 4 + 4 + 4 + 10 + 1
    for expect in ("mha-d64-n256", "mha-d32-n4096", "mha-d128-n4096", "mha-d64-n262144", "mha-d128-n65536", "gqa-n4096",
                   "mqa-n256", "rectangular"):
        assert expect in names
    parser = ab.build_parser()
    for _, flags, check in full:
        args = parser.parse_args(flags + (["--check"] if check else ["--no-check"]))
        assert args.d in (32, 64, 128)
    assert not dict((n, c) for n, _, c in full)["mha-d64-n32768"]      # too large to materialize: unchecked
    subset = [n for n, _, _ in attention_sweep.cases(full=False)]
    assert set(subset) <= set(names) and "rectangular" in subset
