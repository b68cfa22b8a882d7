"""The model-level Hessian-vector-product benchmark: flags, and agreement of the two attention
backends on a tiny model (CPU: `sdpa_bob`'s math route; GPU: the CUDA kernels)."""

import pytest

from flashbob_b200 import hvp_bench as hb


def _args(*extra):
    return hb.build_parser().parse_args(["--seq-lens", "48", "--dim", "32", "--heads", "4", "--layers", "2",
                                         "--warmup", "0", "--iters", "1", *extra])


def test_cpu_run_agrees_with_materialized_attention():
    rows = hb.run(_args("--device", "cpu", "--dtype", "fp32"))
    assert len(rows) == 1 and rows[0]["hv_l2_rel"] < 1e-4
    # grouped heads are a CUDA-only feature of the operator, as in the reference
    with pytest.raises(NotImplementedError):
        hb.run(_args("--device", "cpu", "--dtype", "fp32", "--kv-heads", "2"))


@pytest.mark.gpu
@pytest.mark.parametrize("extra", [[], ["--kv-heads", "2"]])
def test_gpu_run_agrees_with_materialized_attention(extra):
    """bf16 on the GPU: Hv over all parameters of a two-layer model, CUDA kernels against materialized
    attention evaluated in bf16 as well; both carry 16-bit rounding, so the bar is a few per cent."""
    args = hb.build_parser().parse_args(["--seq-lens", "256", "--dim", "256", "--heads", "4", "--layers", "2",
                                         "--warmup", "1", "--iters", "2", *extra])
    rows = hb.run(args)
    assert rows[0]["bob_ms"] > 0 and rows[0]["hv_l2_rel"] < 0.05
