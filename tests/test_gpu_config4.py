"""Parity of the head-dim-128, group-8 kernels that the multi-GPU scaling configuration runs
(bf16 GQA B=8 Hq=64 Hkv=8 S=8192 D=128 causal, sharded by (batch, KV head) units).

At head dim 128 the kernels run one CTA per work item with 32-wide swept tiles; the configuration
puts many items on every SM and sums eight query heads per KV head inside the column-owned CTAs.
Two checks against the fp64 oracle, all eight outputs each:
  * a medium case (S=2048) evaluated by the dense closed form, and
  * one full (batch, KV head) unit of the configuration (8 query heads, S=8192) evaluated one query
    head at a time and a block of rows at a time, key-side results summed over the heads
    (the reference's ground truth for grouped heads is the same materialized attention with
    repeated KV heads: benchmarks/attention/__init__.py:20-55; its grouped launcher for this shape
    is src/bob/kernels/gqa.py:540-718).
"""

import pytest
import torch

from flashbob_b200 import ops, sharding
from oracle import bob_oracle as O

pytestmark = pytest.mark.gpu
BF16 = torch.bfloat16
GEOM = dict(is_causal=True, window_size=0, q_offset=0, k_offset=0, scale=None)
# per-output bars for bf16: relative L2 and max-abs relative to the largest reference value
L2_BAR, MAX_BAR = 4e-3, 1.2e-2


def _kernels(q, k, v, dO, uQ, uK, uV):
    c = lambda t: t.cuda()
    qd, kd, vd, dOd = map(c, (q, k, v, dO))
    out, lse = ops.attention_forward(qd, kd, vd, **GEOM)
    dQ, dK, dV, delta, pk = ops.attention_first_backward(qd, kd, vd, out, lse, dOd, **GEOM)
    Qb, Kb, Vb, dOb = ops.attention_second_backward(qd, kd, vd, out, lse, delta, pk, dOd, dQ, c(uQ), c(uK), c(uV),
                                                    **GEOM)
    ops.check_device_status()
    return dict(out=out, dQ=dQ, dK=dK, dV=dV, Qbar=Qb, Kbar=Kb, Vbar=Vb, dObar=dOb), lse


def _compare(got, lse, ref, tag):
    torch.testing.assert_close(lse.cpu().double(), ref.lse, rtol=1e-5, atol=2e-5)
    for n in O.OUTPUT_NAMES:
        m = O.error_metrics(got[n], getattr(ref, n))
        assert torch.isfinite(got[n].float()).all(), (tag, n)
        assert m["l2_rel"] <= L2_BAR and m["max_abs_rel"] <= MAX_BAR, (tag, n, m)


def test_head_dim_128_group_8_many_items_per_sm():
    B, Hq, Hkv, N, D = 2, 16, 2, 2048, 128       # 2 x 16 x 16 = 512 row items, 64 column items of 8 heads
    q, k, v, dO, uQ = O.seeded_inputs(41, (B, Hq, N, D), (B, Hkv, N, D), BF16, n_extra_q=2)
    uK, uV = O.seeded_inputs(42, (B, Hq, N, D), (B, Hkv, N, D), BF16)[1:]
    got, lse = _kernels(q, k, v, dO, uQ, uK, uV)
    ref = O.bob_closed_form_streamed(q, k, v, dO, uQ, uK, uV, **GEOM)
    _compare(got, lse, ref, "d128_g8_s2048")


def test_one_unit_of_the_scaling_configuration():
    """Unit (b=3, kv-head=5) of B=8 Hq=64 Hkv=8 S=8192 D=128, drawn from a seed of its own (units are
    independent, so a unit can be checked alone) and run through the kernels as a batch of one unit
    with H_KV = 1, the shape a rank of the sharded benchmark sees."""
    B, Hq, Hkv, N, D = 8, 64, 8, 8192, 128
    G = Hq // Hkv
    unit = 3 * Hkv + 5
    assert unit in sharding.unit_range(B * Hkv, 8, 3)            # rank 3 of 8 owns it
    q, k, v, dO, uQ = O.seeded_inputs(4000 + unit, (1, G, N, D), (1, 1, N, D), BF16, n_extra_q=2)
    uK, uV = O.seeded_inputs(5000 + unit, (1, G, N, D), (1, 1, N, D), BF16)[1:]
    got, lse = _kernels(q, k, v, dO, uQ, uK, uV)
    ref = O.bob_closed_form_streamed(q, k, v, dO, uQ, uK, uV, **GEOM)
    _compare(got, lse, ref, "config4_unit")
