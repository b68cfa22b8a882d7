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


def test_grouped_head_rejections_come_in_the_reference_order():
    """Double violations: the reference refuses a rectangle first (src/bob/sdpa.py:429-433), then CPU
    tensors, then a dtype other than bf16, then a window, then a group above 32
    (src/bob/sdpa.py:129-137)."""
    q4, k2 = torch.randn(1, 4, 4, 8), torch.randn(1, 2, 6, 8)
    with pytest.raises(NotImplementedError, match="rectangular"):      # CPU and rectangular
        sdpa_bob(q4, k2, torch.randn_like(k2), is_causal=True)
    k2 = torch.randn(1, 2, 4, 8)
    with pytest.raises(NotImplementedError, match="CUDA"):             # CPU, fp32 and windowed
        sdpa_bob(q4, k2, torch.randn_like(k2), is_causal=True, window_size=2)
    q66, k1 = torch.randn(1, 66, 4, 8), torch.randn(1, 1, 4, 8)
    with pytest.raises(NotImplementedError, match="CUDA"):             # CPU and group 66
        sdpa_bob(q66, k1, torch.randn_like(k1), is_causal=True)


def test_grouped_head_rejection_order_with_fake_cuda_tensors(monkeypatch):
    """The CUDA-side order (dtype before window before group size), checked on the CPU by calling the
    check itself with tensors that claim to be on a GPU."""
    from flashbob_b200 import interface

    class _Fake:
        def __init__(self, heads, dtype):
            self.shape, self.dtype, self.is_cuda = (1, heads, 4, 64), dtype, True

    with pytest.raises(TypeError, match="bfloat16"):                   # fp16, windowed, group 64
        interface._check_grouped(_Fake(64, torch.float16), _Fake(1, torch.float16), window=2, rectangular=False)
    with pytest.raises(NotImplementedError, match="sliding"):          # bf16, windowed, group 64
        interface._check_grouped(_Fake(64, torch.bfloat16), _Fake(1, torch.bfloat16), window=2, rectangular=False)
    with pytest.raises(NotImplementedError, match="up to 32"):
        interface._check_grouped(_Fake(64, torch.bfloat16), _Fake(1, torch.bfloat16), window=0, rectangular=False)
    with pytest.raises(NotImplementedError, match="rectangular"):
        interface._check_grouped(_Fake(64, torch.float16), _Fake(1, torch.float16), window=2, rectangular=True)
    interface._check_grouped(_Fake(8, torch.bfloat16), _Fake(2, torch.bfloat16), window=0, rectangular=False)


def test_hf_attention_interface_refuses_masks_and_dropout():
    """An explicit mask means a padded batch, which an operator without a bias cannot honour
    (reference: examples/huggingface_backend.py:45-53)."""
    from flashbob_b200 import adapters

    q, k, v = _inputs()
    mask = torch.zeros(1, 1, 4, 4)
    with pytest.raises(NotImplementedError, match="padded"):
        adapters.hf_attention_interface(None, q, k, v, mask)
    with pytest.raises(NotImplementedError, match="dropout"):
        adapters.hf_attention_interface(None, q, k, v, None, dropout=0.1)
    out, weights = adapters.hf_attention_interface(None, q, k, v, None, scaling=0.5)
    assert weights is None and out.shape == (1, 4, 2, 8) and out.is_contiguous()
    ref = torch.softmax((q @ k.transpose(-1, -2)) * 0.5 + torch.full((4, 4), float("-inf")).triu(1), -1) @ v
    torch.testing.assert_close(out, ref.transpose(1, 2), rtol=1e-5, atol=1e-5)
