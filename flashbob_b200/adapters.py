"""Caller-side adapters: other attention calling conventions on top of `sdpa_bob`.

They mirror what the reference's examples do around its operator
(reference: examples/flash_attn_drop_in.py:26-39 for the [batch, seq, heads, dim] layout,
examples/huggingface_backend.py:29-61 for the Hugging Face attention-interface signature), but
never copy: the kernels read `[B, N, H, D]` storage in place through strided TMA descriptors.
"""

from __future__ import annotations

import torch

from .interface import sdpa_bob


def flash_attn_layout(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, *, softmax_scale=None, causal=False,
                      window_size=(-1, -1)) -> torch.Tensor:
    """`flash_attn_func`-style call: q [B, Nq, Hq, D], k / v [B, Nk, Hkv, D] -> out [B, Nq, Hq, D].

    `window_size=(left, 0)` with left >= 0 means a causal sliding window of left + 1 keys.
    """
    left, right = window_size
    if right not in (-1, 0) or (left >= 0 and not causal):
        raise NotImplementedError("only causal (left, 0) windows are supported")
    window = left + 1 if left >= 0 else 0
    out = sdpa_bob(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), is_causal=causal,
                   scale=softmax_scale, window_size=window)
    return out.transpose(1, 2)


def hf_attention_interface(module, query, key, value, attention_mask=None, *, scaling=None, dropout=0.0,
                           is_causal=None, sliding_window=None, **_unused):
    """Hugging Face `AttentionInterface` signature: [B, H, N, D] tensors in, ([B, N, H, D], None) out.

    Masking is implicit only: causal with right alignment (a decode step with one query and a cache
    of N keys sees all of them), optionally limited to the last `sliding_window` keys.  An explicit
    `attention_mask` is refused, as the reference's entry point does
    (reference: examples/huggingface_backend.py:45-49): the operator takes no bias, so a padded
    batch would silently attend to pad tokens.  Dropout must be 0.
    """
    if attention_mask is not None:
        raise NotImplementedError(
            "sdpa_bob takes no attention bias, so padded batches are unsupported; "
            "pass attention_mask=None with an unpadded causal batch")
    if dropout:
        raise NotImplementedError("attention dropout is not supported")
    causal = bool(getattr(module, "is_causal", True)) if is_causal is None else bool(is_causal)
    window = int(sliding_window) if (sliding_window and causal) else 0
    out = sdpa_bob(query, key, value, is_causal=causal, scale=scaling, window_size=window)
    return out.transpose(1, 2).contiguous(), None
