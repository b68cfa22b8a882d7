"""Tensor-level wrappers of the three C-ABI stages (forward, first backward, second backward).

PyTorch is used only for device memory and streams; all arithmetic happens in libbob_sm100.so.
These functions replace the reference's front end and launchers:
`bob.attention.forward` / `first_backward` (reference: src/bob/attention.py:251-289),
`bob.kernels.rectangular.rect_forward` / `rect_first_backward`
(reference: src/bob/kernels/rectangular.py:220-253) and the three second-backward launchers
`square.bob_2pass`, `gqa.bob_gqa`, `rectangular.bob_2pass_rect`
(reference: src/bob/kernels/square.py:383-525, gqa.py:540-718, rectangular.py:628-777).
"""

from __future__ import annotations

import ctypes
import math
import os

import torch

from . import _lib

_CHECK_STATUS = os.environ.get("BOB_SM100_CHECK_STATUS", "0") not in ("", "0")



def _tma_ready(t: torch.Tensor) -> torch.Tensor:
    """Return `t` itself when the kernels can address it in place, else a contiguous copy.

    In-place addressing needs unit stride along the head dim, batch/head/row strides that are
    multiples of 8 elements (16 bytes) and a 16-byte aligned base.
    """
    if t.stride(-1) == 1 and all(s % 8 == 0 for s in t.stride()[:3]) and t.data_ptr() % 16 == 0 \
            and all(s > 0 or n == 1 for s, n in zip(t.stride()[:3], t.shape[:3])):
        return t
    return t.contiguous()


def _set_strides(field, t: torch.Tensor) -> None:
    s = t.stride()
    field[0], field[1], field[2] = s[0], s[1], s[2]


def _geom(q, k, *, is_causal, window_size, q_offset, k_offset, scale) -> _lib.Geom:
    B, Hq, Nq, D = q.shape
    Hkv, Nk = k.shape[1], k.shape[2]
    g = _lib.Geom()
    g.B, g.Hq, g.Hkv, g.Nq, g.Nk, g.D = B, Hq, Hkv, Nq, Nk, D
    g.dtype = _lib.BF16 if q.dtype == torch.bfloat16 else _lib.FP16
    g.is_causal = int(bool(is_causal))
    g.window = int(window_size)
    g.device = q.device.index if q.device.index is not None else torch.cuda.current_device()
    g.q_offset, g.k_offset = int(q_offset), int(k_offset)
    g.scale = float(scale) if scale is not None else 1.0 / math.sqrt(D)
    return g


def _ptr(t):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def _stream(device) -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)


def _workspace(stage: int, g: _lib.Geom, device) -> torch.Tensor:
    n = _lib.load().bob_sm100_workspace_bytes(stage, ctypes.byref(g))
    return torch.empty(n, dtype=torch.uint8, device=device)


def _finish(ws: torch.Tensor, device, what: str) -> None:
    """Raise if a kernel on this device gave up on a bounded wait.

    Default: a non-blocking look at the device's host-visible status word, which a kernel writes as
    it gives up - so a time-out of an earlier call surfaces here, at the latest one call late, without
    any synchronisation.  With BOB_SM100_CHECK_STATUS=1 the call's own status word is read back
    after waiting for the stream (exact attribution, one synchronisation per call).
    """
    lib = _lib.load()
    if _CHECK_STATUS:
        _lib.check(lib.bob_sm100_read_status(_ptr(ws), _stream(device)), f"{what} (device status)")
    index = device.index if device.index is not None else torch.cuda.current_device()
    st = lib.bob_sm100_last_status(index)
    if st:
        _lib.check(st, f"an earlier libbob_sm100 kernel on cuda:{index} (seen after {what}; its results are undefined)")


def check_device_status(device=None) -> None:
    """Raise if any libbob_sm100 kernel on `device` gave up on a bounded wait since the last check.
    Non-blocking; call it after a synchronisation point (for instance at the end of a training step)
    to be sure that every kernel launched before it is covered."""
    index = torch.cuda.current_device() if device is None else torch.device(device).index
    st = _lib.load().bob_sm100_last_status(index)
    if st:
        _lib.check(st, f"a libbob_sm100 kernel on cuda:{index}")


def _require_cuda_16bit(*tensors) -> None:
    for t in tensors:
        if t is None:
            continue
        if not t.is_cuda:
            raise ValueError("libbob_sm100 kernels take CUDA tensors only")
        if t.dtype not in (torch.float16, torch.bfloat16):
            raise TypeError(f"libbob_sm100 kernels take fp16 or bf16 tensors, got {t.dtype}")


def attention_forward(q, k, v, *, is_causal, window_size, q_offset, k_offset, scale):
    """out [B,Hq,Nq,D] (input dtype) and natural-log lse [B,Hq,Nq] (fp32)."""
    _require_cuda_16bit(q, k, v)
    lib = _lib.load()
    q, k, v = _tma_ready(q), _tma_ready(k), _tma_ready(v)
    g = _geom(q, k, is_causal=is_causal, window_size=window_size, q_offset=q_offset,
              k_offset=k_offset, scale=scale)
    _set_strides(g.q_strides, q); _set_strides(g.k_strides, k); _set_strides(g.v_strides, v)
    out = torch.empty(q.shape, dtype=q.dtype, device=q.device)
    lse = torch.empty(q.shape[:3], dtype=torch.float32, device=q.device)
    ws = _workspace(_lib.STAGE_FWD, g, q.device)
    with torch.cuda.device(q.device):
        rc = lib.bob_sm100_fwd(ctypes.byref(g), _ptr(q), _ptr(k), _ptr(v), _ptr(out), _ptr(lse),
                               _ptr(ws), _stream(q.device))
    _lib.check(rc, "bob_sm100_fwd")
    _finish(ws, q.device, "bob_sm100_fwd")
    return out, lse


def attention_first_backward(q, k, v, out, lse, dO, *, is_causal, window_size, q_offset, k_offset,
                             scale, for_second_order=True):
    """dQ, dK, dV (input dtype, contiguous), delta = rowsum(dO*out) [B,Hq,Nq] (fp32) and, when
    `for_second_order`, pk = softmax(S) K [B,Hq,Nq,D] (fp32) for the second backward (else None)."""
    _require_cuda_16bit(q, k, v, out, dO)
    lib = _lib.load()
    q, k, v, out, dO = (_tma_ready(t) for t in (q, k, v, out, dO))
    lse = lse.contiguous()
    g = _geom(q, k, is_causal=is_causal, window_size=window_size, q_offset=q_offset,
              k_offset=k_offset, scale=scale)
    _set_strides(g.q_strides, q); _set_strides(g.k_strides, k); _set_strides(g.v_strides, v)
    _set_strides(g.out_strides, out); _set_strides(g.do_strides, dO)
    dQ = torch.empty(q.shape, dtype=q.dtype, device=q.device)
    dK = torch.empty(k.shape, dtype=q.dtype, device=q.device)
    dV = torch.empty(k.shape, dtype=q.dtype, device=q.device)
    delta = torch.empty(q.shape[:3], dtype=torch.float32, device=q.device)
    pk = torch.empty(q.shape, dtype=torch.float32, device=q.device) if for_second_order else None
    ws = _workspace(_lib.STAGE_BWD1, g, q.device)
    with torch.cuda.device(q.device):
        rc = lib.bob_sm100_bwd1(ctypes.byref(g), _ptr(q), _ptr(k), _ptr(v), _ptr(out), _ptr(lse),
                                _ptr(dO), _ptr(dQ), _ptr(dK), _ptr(dV), _ptr(delta), _ptr(pk), _ptr(ws),
                                _stream(q.device))
    _lib.check(rc, "bob_sm100_bwd1")
    _finish(ws, q.device, "bob_sm100_bwd1")
    return dQ, dK, dV, delta, pk


def attention_second_backward(q, k, v, out, lse, delta, pk, dO, dQ, uQ, uK, uV, *, is_causal,
                              window_size, q_offset, k_offset, scale):
    """Qbar, Kbar, Vbar, dObar (input dtype, contiguous).  uQ/uK/uV may be None."""
    _require_cuda_16bit(q, k, v, out, dO, dQ, uQ, uK, uV)
    lib = _lib.load()
    q, k, v, out, dO, dQ = (_tma_ready(t) for t in (q, k, v, out, dO, dQ))
    uQ, uK, uV = (None if t is None else _tma_ready(t.to(q.dtype)) for t in (uQ, uK, uV))
    lse, delta, pk = lse.contiguous(), delta.contiguous(), pk.contiguous()
    g = _geom(q, k, is_causal=is_causal, window_size=window_size, q_offset=q_offset,
              k_offset=k_offset, scale=scale)
    for field, t in ((g.q_strides, q), (g.k_strides, k), (g.v_strides, v), (g.out_strides, out),
                     (g.do_strides, dO), (g.dq_strides, dQ), (g.uq_strides, uQ),
                     (g.uk_strides, uK), (g.uv_strides, uV)):
        if t is not None:
            _set_strides(field, t)
    Qbar = torch.empty(q.shape, dtype=q.dtype, device=q.device)
    dObar = torch.empty(q.shape, dtype=q.dtype, device=q.device)
    Kbar = torch.empty(k.shape, dtype=q.dtype, device=q.device)
    Vbar = torch.empty(k.shape, dtype=q.dtype, device=q.device)
    ws = _workspace(_lib.STAGE_BWD2, g, q.device)
    with torch.cuda.device(q.device):
        rc = lib.bob_sm100_bwd2(ctypes.byref(g), _ptr(q), _ptr(k), _ptr(v), _ptr(out), _ptr(lse),
                                _ptr(delta), _ptr(pk), _ptr(dO), _ptr(dQ), _ptr(uQ), _ptr(uK), _ptr(uV),
                                _ptr(Qbar), _ptr(Kbar), _ptr(Vbar), _ptr(dObar), _ptr(ws),
                                _stream(q.device))
    _lib.check(rc, "bob_sm100_bwd2")
    _finish(ws, q.device, "bob_sm100_bwd2")
    return Qbar, Kbar, Vbar, dObar
