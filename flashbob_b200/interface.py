"""The public operator `sdpa_bob` and its two-level autograd chain, hosted on libbob_sm100.so.

Drop-in for the reference operator (reference: src/bob/sdpa.py:387-468): same signature, same
exceptions raised before any launch (reference: src/bob/sdpa.py:21-137, pinned by
tests/unit/test_attention_validation.py:14-56), same offset and window inference
(reference: src/bob/sdpa.py:371-384, src/bob/attention.py:93-102) and the same autograd
protocol (reference: src/bob/sdpa.py:239-368):

  * `SDPAWithBoB.forward` runs the forward kernel and keeps (q, k, v, out, lse);
  * `SDPAWithBoB.backward` runs only the first backward when grad mode is off, otherwise it
    applies `BoBSecondOrder`, whose forward is the first backward and whose backward is the
    second backward returning gradients for (q, k, v, dO);
  * undefined incoming tangents arrive as None (`set_materialize_grads(False)`) and switch off
    the products they would feed.

CUDA tensors always go through the CUDA library: there is no fallback, a missing library raises.
CPU tensors take PyTorch's math attention with stock autograd, exactly as the reference's CPU
route does (reference: src/bob/sdpa.py:437-465).
"""

from __future__ import annotations

import math
import numbers
import operator as _operator

import torch
from torch.autograd import Function

from . import ops

__all__ = ["sdpa_bob"]

_CUDA_DTYPES = (torch.float16, torch.bfloat16)
_CPU_DTYPES = (torch.float16, torch.bfloat16, torch.float32)
_CUDA_HEAD_DIMS = (32, 64, 128)
_MAX_GROUP = 32

# The kernels handle grouped heads with any mask, length pair and 16-bit dtype.  The reference
# rejects grouped heads combined with a window, a rectangle or fp16; those rejections are kept
# unless this switch is turned on.
ALLOW_WIDENED_GQA = False


# --------------------------------------------------------------------------------------
# argument checks
# --------------------------------------------------------------------------------------
def _as_count(name: str, value, *, optional: bool = False):
    """A non-negative Python int from an int-like; bools and floats are rejected."""
    if value is None and optional:
        return None
    if isinstance(value, bool):
        raise TypeError(f"{name} must be an integer, got {value!r}")
    try:
        number = _operator.index(value)
    except TypeError:
        raise TypeError(f"{name} must be an integer, got {value!r}") from None
    if number < 0:
        raise ValueError(f"{name} must be >= 0, got {number}")
    return number


def _check_tensors(q, k, v) -> None:
    named = (("q", q), ("k", k), ("v", v))
    for name, t in named:
        if not isinstance(t, torch.Tensor):
            raise TypeError(f"{name} must be a torch.Tensor")
        if torch.autograd.forward_ad.unpack_dual(t).tangent is not None:
            raise NotImplementedError(
                "forward-mode AD is unsupported; differentiate with reverse mode "
                "(torch.autograd.grad twice) instead")
        if t.ndim != 4:
            raise ValueError(f"{name} must have rank 4 [B, H, N, D], got shape {tuple(t.shape)}")
    shapes = f"q={tuple(q.shape)} k={tuple(k.shape)} v={tuple(v.shape)}"
    if min(min(t.shape) for _, t in named) <= 0:
        raise ValueError(f"every dimension of q, k and v must be positive, got {shapes}")
    if tuple(v.shape) != tuple(k.shape):
        raise ValueError(f"v shape {tuple(v.shape)} must equal k shape {tuple(k.shape)}")
    if q.shape[0] != k.shape[0]:
        raise ValueError(f"q, k and v must share the batch size, got {shapes}")
    if q.shape[3] != k.shape[3]:
        raise ValueError(f"q, k and v must share the head dimension, got {shapes}")
    if q.shape[1] % k.shape[1] != 0:
        raise ValueError(
            f"query heads H_Q={q.shape[1]} must be divisible by KV heads H_KV={k.shape[1]}")
    if not (q.device == k.device == v.device):
        raise ValueError(f"q, k and v must be on one device, got {q.device}, {k.device}, {v.device}")
    if not (q.dtype == k.dtype == v.dtype):
        raise ValueError(f"q, k and v must share one dtype, got {q.dtype}, {k.dtype}, {v.dtype}")
    allowed = _CUDA_DTYPES if q.is_cuda else _CPU_DTYPES
    if q.dtype not in allowed:
        raise TypeError(
            f"q, k and v dtype must be one of {', '.join(map(str, allowed))}; got {q.dtype}")
    if q.is_cuda and q.shape[3] not in _CUDA_HEAD_DIMS:
        raise ValueError(f"CUDA head dimension D must be one of {_CUDA_HEAD_DIMS}, got {q.shape[3]}")


def _check_scalars(is_causal, scale, window_size, q_offset, k_offset):
    if not isinstance(is_causal, bool):
        raise TypeError(f"is_causal must be bool, got {type(is_causal).__name__}")
    window = _as_count("window_size", window_size)
    if window > 0 and not is_causal:
        raise NotImplementedError("window_size>0 requires is_causal=True")
    q_off = _as_count("q_offset", q_offset, optional=True)
    k_off = _as_count("k_offset", k_offset)
    if scale is not None:
        if isinstance(scale, bool) or not isinstance(scale, numbers.Real):
            raise TypeError(f"scale must be a finite positive number, got {scale!r}")
        if not math.isfinite(float(scale)) or float(scale) <= 0.0:
            raise ValueError(f"scale must be a finite positive number, got {scale!r}")
    return window, q_off, k_off


def _check_grouped(q, k, *, window: int, rectangular: bool) -> None:
    """Rejections for grouped heads, in the reference's order: a rectangle is refused first
    (reference: src/bob/sdpa.py:429-433), then CPU tensors, a dtype other than bf16, a window and a
    group larger than 32 (reference: src/bob/sdpa.py:129-137).  With ALLOW_WIDENED_GQA only the CPU
    and group-size limits remain."""
    if rectangular and not ALLOW_WIDENED_GQA:
        raise NotImplementedError("FlashBoB GQA/MQA does not support rectangular attention")
    if not q.is_cuda:
        raise NotImplementedError("FlashBoB GQA/MQA requires CUDA")
    if not ALLOW_WIDENED_GQA:
        if q.dtype != torch.bfloat16:
            raise TypeError("FlashBoB GQA/MQA requires bfloat16")
        if window > 0:
            raise NotImplementedError("FlashBoB GQA/MQA does not support sliding windows")
    if q.shape[1] // k.shape[1] > _MAX_GROUP:
        raise NotImplementedError(f"FlashBoB GQA/MQA supports grouping factors up to {_MAX_GROUP}")


def _resolve_q_offset(n_q: int, n_k: int, q_offset, k_offset: int, is_causal: bool) -> int:
    """Explicit offset wins; a causal rectangle defaults to right alignment."""
    if q_offset is not None:
        return q_offset
    if is_causal and n_q != n_k:
        return k_offset + max(0, n_k - n_q)
    return k_offset


# --------------------------------------------------------------------------------------
# CPU route
# --------------------------------------------------------------------------------------
def _cpu_math_attention(q, k, v, *, is_causal, window, q_offset, k_offset, scale, rectangular):
    """PyTorch math attention; windows and rectangles become an additive 0 / -inf bias."""
    import torch.nn.functional as F
    from torch.nn.attention import SDPBackend, sdpa_kernel

    n_q, n_k = q.shape[2], k.shape[2]
    flag = is_causal and not rectangular and window == 0
    bias = None
    if is_causal and not flag:
        dist = (torch.arange(n_q, device=q.device) + q_offset)[:, None] \
            - (torch.arange(n_k, device=q.device) + k_offset)[None, :]
        keep = dist >= 0
        if window > 0:
            keep &= dist < window
        bias = torch.zeros(keep.shape, dtype=q.dtype, device=q.device).masked_fill(~keep, -math.inf)
    with sdpa_kernel(SDPBackend.MATH):
        return F.scaled_dot_product_attention(q, k, v, attn_mask=bias, dropout_p=0.0,
                                              is_causal=flag, scale=scale)


# --------------------------------------------------------------------------------------
# autograd chain
# --------------------------------------------------------------------------------------
class BoBSecondOrder(Function):
    """First backward as a differentiable function of (q, k, v, dO); its backward is the
    second backward (gradients for q, k, v and dO)."""

    @staticmethod
    def forward(ctx, q, k, v, dO, out, lse, q_offset, k_offset, is_causal, window_size, scale):
        ctx.set_materialize_grads(False)
        geom = dict(is_causal=is_causal, window_size=window_size, q_offset=q_offset,
                    k_offset=k_offset, scale=scale)
        dQ, dK, dV, delta, pk = ops.attention_first_backward(q, k, v, out, lse, dO, **geom)
        ctx.save_for_backward(q, k, v, out, lse, dO, dQ, delta, pk)
        ctx.geom = geom
        return dQ, dK, dV

    @staticmethod
    def backward(ctx, uQ, uK, uV):
        q, k, v, out, lse, dO, dQ, delta, pk = ctx.saved_tensors
        if uQ is None and uK is None and uV is None:
            return (None,) * 11
        Qbar, Kbar, Vbar, dObar = ops.attention_second_backward(
            q, k, v, out, lse, delta, pk, dO, dQ, uQ, uK, uV, **ctx.geom)
        return (Qbar, Kbar, Vbar, dObar, None, None, None, None, None, None, None)


class SDPAWithBoB(Function):
    """Attention forward whose backward is itself differentiable once more."""

    @staticmethod
    def forward(ctx, q, k, v, q_offset, k_offset, is_causal, window_size, scale):
        # An undefined cotangent (the second differentiation of leaf-cotangent protocols reaches this
        # node with nothing to propagate) must not be turned into a tensor of zeros and pushed
        # through a pointless first backward.
        ctx.set_materialize_grads(False)
        q_offset = 0 if q_offset is None else int(q_offset)
        k_offset = 0 if k_offset is None else int(k_offset)
        geom = dict(is_causal=is_causal, window_size=window_size, q_offset=q_offset,
                    k_offset=k_offset, scale=scale)
        out, lse = ops.attention_forward(q, k, v, **geom)
        ctx.save_for_backward(q, k, v, out, lse)
        ctx.geom = geom
        return out

    @staticmethod
    def backward(ctx, dO):
        if dO is None:
            return (None,) * 8
        q, k, v, out, lse = ctx.saved_tensors
        g = ctx.geom
        if not torch.is_grad_enabled():
            dQ, dK, dV, _, _ = ops.attention_first_backward(q, k, v, out, lse, dO,
                                                            for_second_order=False, **g)
        else:
            dQ, dK, dV = BoBSecondOrder.apply(q, k, v, dO, out, lse, g["q_offset"], g["k_offset"],
                                              g["is_causal"], g["window_size"], g["scale"])
        return dQ, dK, dV, None, None, None, None, None


# --------------------------------------------------------------------------------------
# public operator
# --------------------------------------------------------------------------------------
def sdpa_bob(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, *, is_causal: bool = False,
             scale: float | None = None, window_size: int = 0, q_offset: int | None = None,
             k_offset: int = 0) -> torch.Tensor:
    """Scaled dot-product attention that can be differentiated twice by reverse mode.

    q is [B, H_Q, N_Q, D]; k and v are [B, H_KV, N_KV, D] with H_Q a multiple of H_KV.  Query row
    i sits at absolute position q_offset + i and key row j at k_offset + j; `is_causal` keeps keys
    at positions <= the query's, `window_size` w > 0 further keeps only the last w of them.  With
    `q_offset=None` a causal call with N_Q != N_KV is right-aligned.  CUDA tensors must be fp16 or
    bf16 with D in {32, 64, 128}; CPU tensors (also fp32) use PyTorch's math attention.
    """
    if torch._C._are_functorch_transforms_active():
        raise NotImplementedError(
            "torch.func transforms are unsupported; differentiate with reverse mode "
            "(torch.autograd.grad twice) instead")
    _check_tensors(q, k, v)
    window, q_off, k_off = _check_scalars(is_causal, scale, window_size, q_offset, k_offset)
    n_q, n_k = q.shape[2], k.shape[2]
    q_off = _resolve_q_offset(n_q, n_k, q_off, k_off, is_causal)
    rectangular = n_q != n_k or q_off != k_off
    grouped = q.shape[1] != k.shape[1]

    # a window that already covers every causal key is no window
    if is_causal and window > 0:
        reach = (q_off - k_off + n_q) if rectangular else n_q
        if window >= reach:
            window = 0
    if grouped:
        _check_grouped(q, k, window=window, rectangular=rectangular)

    if not q.is_cuda:
        return _cpu_math_attention(q, k, v, is_causal=is_causal, window=window, q_offset=q_off,
                                   k_offset=k_off, scale=scale, rectangular=rectangular)
    return SDPAWithBoB.apply(q, k, v, q_off, k_off, is_causal, window, scale)
