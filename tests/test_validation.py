"""Argument contract of the public operator, raised before any launch.
Mirrors the reference's unit tests (reference: tests/unit/test_attention_validation.py:14-56)."""

import pytest
import torch

from bob import sdpa_bob


def _inputs():
    return tuple(torch.randn(1, 2, 4, 8) for _ in range(3))


@pytest.mark.parametrize(
    ("kwargs", "message"),
    [
        ({"scale": 0.0}, "scale"),
        ({"scale": float("nan")}, "scale"),
        ({"scale": True}, "scale"),
        ({"scale": "1"}, "scale"),
        ({"window_size": -1}, "window"),
        ({"window_size": 1.5}, "window"),
        ({"window_size": True}, "window"),
        ({"is_causal": False, "window_size": 2}, "causal"),
        ({"is_causal": 1}, "causal"),
        ({"q_offset": -1}, "offset"),
        ({"q_offset": 1.5}, "offset"),
        ({"k_offset": True}, "offset"),
        ({"k_offset": -3}, "offset"),
    ],
)
def test_invalid_scalar_arguments_fail_at_the_public_boundary(kwargs, message):
    with pytest.raises((TypeError, ValueError, NotImplementedError), match=message):
        sdpa_bob(*_inputs(), **kwargs)


def test_exception_types():
    q, k, v = _inputs()
    with pytest.raises(TypeError):
        sdpa_bob(q, k, v, window_size=1.5)
    with pytest.raises(ValueError):
        sdpa_bob(q, k, v, is_causal=True, window_size=-1)
    with pytest.raises(NotImplementedError):
        sdpa_bob(q, k, v, window_size=2)
    with pytest.raises(ValueError):
        sdpa_bob(q, k, v, scale=float("inf"))
    with pytest.raises(TypeError):
        sdpa_bob(q.numpy(), k, v)
    with pytest.raises(ValueError, match="rank"):
        sdpa_bob(q[0], k, v)
    with pytest.raises(TypeError, match="dtype"):
        sdpa_bob(q.double(), k.double(), v.double())
    with pytest.raises(ValueError, match="batch"):
        sdpa_bob(torch.randn(2, 2, 4, 8), k, v)
    with pytest.raises(ValueError, match="head dimension"):
        sdpa_bob(torch.randn(1, 2, 4, 16), k, v)
    with pytest.raises(ValueError, match="positive"):
        sdpa_bob(torch.randn(1, 2, 0, 8), k, v)


def test_mismatched_key_and_value_shapes_are_rejected():
    q, k, _ = _inputs()
    with pytest.raises(ValueError, match="shape"):
        sdpa_bob(q, k, torch.randn(1, 2, 5, 8))


def test_mixed_input_dtypes_are_rejected():
    q, k, v = _inputs()
    with pytest.raises(ValueError, match="dtype"):
        sdpa_bob(q, k.double(), v)


def test_query_heads_must_be_divisible_by_key_heads():
    q, k = torch.randn(1, 3, 4, 8), torch.randn(1, 2, 4, 8)
    with pytest.raises(ValueError, match="divisible"):
        sdpa_bob(q, k, torch.randn_like(k))


def test_cpu_gqa_reports_the_unsupported_route():
    q, k = torch.randn(1, 4, 4, 8), torch.randn(1, 2, 4, 8)
    with pytest.raises(NotImplementedError, match="CUDA"):
        sdpa_bob(q, k, torch.randn_like(k), is_causal=True)


def test_forward_mode_and_functorch_are_rejected():
    import torch.autograd.forward_ad as fwAD

    q, k, v = _inputs()
    with fwAD.dual_level():
        dual = fwAD.make_dual(q, torch.ones_like(q))
        with pytest.raises(NotImplementedError, match="forward-mode"):
            sdpa_bob(dual, k, v)
    with pytest.raises(NotImplementedError, match="torch.func"):
        torch.func.grad(lambda x: sdpa_bob(x, k, v).sum())(q)
