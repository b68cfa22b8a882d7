"""CPU oracle for the second-order scaled-dot-product-attention path.  TEST INFRASTRUCTURE ONLY.

This module restates, on the CPU and in any floating dtype (fp64 for parity work), the
algorithm of the reference's `bob.sdpa_bob` path.  Nothing in the product package imports it;
it is used by the tests, by the smoke check and by the CPU-baseline leg of the benchmark.

Parity status: PINNED.  `tests/golden/*.npz` hold outputs of the reference's own functions
(`bob.sdpa_bob` on CPU, `bob.attention.sdpa_math`, `bob.kernels.rectangular.sdpa_math_rect`,
`benchmarks.attention.attention_reference`) on seeded inputs, produced by
`tests/golden/make_golden.py`; `tests/test_oracle_golden.py` checks every function here
against them.

Reference locations restated here (paths inside the reference project):
  * materialized attention, GQA by head repetition, absolute-position causal / window mask:
    benchmarks/attention/__init__.py:20-55
  * CPU route of the operator (math SDPA with an additive -inf bias for windows and
    rectangles): src/bob/attention.py:105-149, src/bob/kernels/rectangular.py:52-95
  * offset / window inference: src/bob/sdpa.py:371-384, src/bob/attention.py:93-102
  * closed-form second backward (row statistics alpha, E; outputs Qbar, Kbar, Vbar, dObar):
    src/bob/kernels/common.py:15-30, 512-612, 638-652, 695-786
  * two-level gradient protocol with explicit cotangents: benchmarks/attention/__init__.py:93-117,
    tests/cuda/test_attention_correctness.py:26-30
"""

from __future__ import annotations

import math
from dataclasses import dataclass

import torch

OUTPUT_NAMES = ("out", "dQ", "dK", "dV", "Qbar", "Kbar", "Vbar", "dObar")


# --------------------------------------------------------------------------------------
# geometry
# --------------------------------------------------------------------------------------
def infer_q_offset(q_len: int, k_len: int, q_offset, k_offset: int, is_causal: bool) -> int:
    """Right-aligned default for causal rectangles (src/bob/sdpa.py:371-377)."""
    if q_offset is not None:
        return int(q_offset)
    if is_causal and q_len != k_len:
        return int(k_offset) + max(0, k_len - q_len)
    return int(k_offset)


def valid_mask(q_len: int, k_len: int, *, is_causal: bool, window_size: int, q_offset: int,
               k_offset: int) -> torch.Tensor:
    """[q_len, k_len] bool: which (query, key) pairs attend.

    Non-causal: all.  Causal: key position <= query position (absolute).  Window w > 0:
    additionally query position - key position < w.
    """
    if not is_causal:
        if window_size:
            raise NotImplementedError("sliding windows require causal attention")
        return torch.ones(q_len, k_len, dtype=torch.bool)
    qi = torch.arange(q_len) + int(q_offset)
    kj = torch.arange(k_len) + int(k_offset)
    dist = qi[:, None] - kj[None, :]
    mask = dist >= 0
    if window_size:
        mask &= dist < int(window_size)
    return mask


def unmasked_pairs(q_len, k_len, *, is_causal, window_size=0, q_offset=None, k_offset=0) -> int:
    """Exact count of attending (query, key) pairs of ONE query head (the `A` of the FLOP
    convention: forward 2u, first backward 5u, second backward 12u with u = 2*A*D*B*Hq)."""
    q_offset = infer_q_offset(q_len, k_len, q_offset, k_offset, is_causal)
    if not is_causal:
        return q_len * k_len
    total = 0
    delta = q_offset - k_offset
    for i in range(q_len):
        hi = min(k_len - 1, i + delta)
        lo = max(0, i + delta - window_size + 1) if window_size else 0
        if hi >= lo:
            total += hi - lo + 1
    return total


# --------------------------------------------------------------------------------------
# forward
# --------------------------------------------------------------------------------------
def _expand_kv(x: torch.Tensor, groups: int) -> torch.Tensor:
    return x if groups == 1 else x.repeat_interleave(groups, dim=1)


def attention_dense(q, k, v, *, is_causal=False, scale=None, window_size=0, q_offset=None,
                    k_offset=0, return_lse=False):
    """Materialized attention in the dtype of the inputs.  Differentiable to any order.

    Rows with no attending key produce zeros (and lse = -inf) instead of NaN.
    """
    B, Hq, Nq, D = q.shape
    Hkv, Nk = k.shape[1], k.shape[2]
    if Hq % Hkv:
        raise ValueError("query heads must be divisible by key/value heads")
    q_offset = infer_q_offset(Nq, Nk, q_offset, k_offset, is_causal)
    scale = 1.0 / math.sqrt(D) if scale is None else float(scale)
    kx, vx = _expand_kv(k, Hq // Hkv), _expand_kv(v, Hq // Hkv)
    s = torch.matmul(q, kx.transpose(-1, -2)) * scale
    mask = valid_mask(Nq, Nk, is_causal=is_causal, window_size=window_size, q_offset=q_offset,
                      k_offset=k_offset).to(q.device)
    neg = torch.finfo(s.dtype).min
    s_m = torch.where(mask, s, torch.full_like(s, neg))
    m = s_m.max(dim=-1, keepdim=True).values.detach()
    e = torch.exp(s_m - m) * mask
    l = e.sum(dim=-1, keepdim=True)
    has = l > 0
    p = torch.where(has, e / torch.where(has, l, torch.ones_like(l)), torch.zeros_like(e))
    out = torch.matmul(p.to(v.dtype), vx)
    if return_lse:
        lse = torch.where(has, m + torch.log(torch.where(has, l, torch.ones_like(l))),
                          torch.full_like(l, -math.inf)).squeeze(-1)
        return out, lse
    return out


def reference_cpu_route(q, k, v, *, is_causal=False, scale=None, window_size=0, q_offset=None,
                        k_offset=0):
    """The reference operator's CPU route: PyTorch math SDPA, stock autograd.

    Square, no window -> `is_causal` flag; anything else -> additive bias of 0 / -inf built
    from absolute positions (src/bob/attention.py:124-149, src/bob/kernels/rectangular.py:76-95).
    MHA only, as in the reference (its CPU route rejects grouped heads).
    """
    import torch.nn.functional as F
    from torch.nn.attention import SDPBackend, sdpa_kernel

    Nq, Nk = q.shape[-2], k.shape[-2]
    q_offset = infer_q_offset(Nq, Nk, q_offset, k_offset, is_causal)
    rectangular = Nq != Nk or q_offset != k_offset
    if not rectangular and is_causal and window_size >= Nq:
        window_size = 0
    bias = None
    use_flag = is_causal and not rectangular and window_size == 0
    if is_causal and not use_flag:
        mask = valid_mask(Nq, Nk, is_causal=True, window_size=window_size, q_offset=q_offset,
                          k_offset=k_offset)
        bias = torch.zeros(mask.shape, dtype=q.dtype).masked_fill(~mask, float("-inf"))
    with sdpa_kernel(SDPBackend.MATH):
        return F.scaled_dot_product_attention(q, k, v, attn_mask=bias, dropout_p=0.0,
                                              is_causal=use_flag, scale=scale)


# --------------------------------------------------------------------------------------
# two-level gradients by autograd (ground truth)
# --------------------------------------------------------------------------------------
def second_order_autograd(q, k, v, dO, uQ, uK, uV, *, dtype=torch.float64, **geom):
    """All eight outputs by double backward through `attention_dense` in `dtype`.

    uQ/uK/uV may be None (undefined tangent: contributes nothing).  Returns a dict keyed by
    OUTPUT_NAMES (values detached, in `dtype`).
    """
    q, k, v, dO = (t.detach().to(dtype).requires_grad_(True) for t in (q, k, v, dO))
    out = attention_dense(q, k, v, **geom)
    dQ, dK, dV = torch.autograd.grad(out, (q, k, v), dO, create_graph=True)
    total = 0.0
    for g, u in ((dQ, uQ), (dK, uK), (dV, uV)):
        if u is not None:
            total = total + (g * u.detach().to(dtype)).sum()
    if isinstance(total, float):
        zeros = [torch.zeros_like(t) for t in (q, k, v, dO)]
        second = zeros
    else:
        second = torch.autograd.grad(total, (q, k, v, dO), allow_unused=True)
        second = [torch.zeros_like(t) if g is None else g for g, t in zip(second, (q, k, v, dO))]
    vals = (out, dQ, dK, dV, *second)
    return {n: t.detach() for n, t in zip(OUTPUT_NAMES, vals)}


# --------------------------------------------------------------------------------------
# closed-form restatement of the kernels' algebra (what each GPU kernel must produce)
# --------------------------------------------------------------------------------------
@dataclass
class DenseBoB:
    out: torch.Tensor
    lse: torch.Tensor      # [B, Hq, Nq] natural log
    delta: torch.Tensor    # [B, Hq, Nq] rowsum(dO * out)
    dQ: torch.Tensor
    dK: torch.Tensor
    dV: torch.Tensor
    alpha: torch.Tensor    # [B, Hq, Nq]
    ecirc: torch.Tensor    # [B, Hq, Nq]  (E = ecirc - alpha * delta)
    Qbar: torch.Tensor
    Kbar: torch.Tensor
    Vbar: torch.Tensor
    dObar: torch.Tensor

    def outputs(self):
        return {n: getattr(self, n) for n in OUTPUT_NAMES}


def bob_closed_form(q, k, v, dO, uQ, uK, uV, *, dtype=torch.float64, is_causal=False, scale=None,
                    window_size=0, q_offset=None, k_offset=0) -> DenseBoB:
    """Forward, first backward and second backward from explicit formulas (no autograd).

      S = t Q K^T (masked)   L = logsumexp S   P = exp(S - L)   O = P V
      delta = rowsum(dO * O)  dP = dO V^T  dS = P*(dP - delta)  dQ = t dS K  dK = t dS^T Q  dV = P^T dO
      F = t (uQ K^T + Q uK^T)  C = dO uV^T  alpha = rowsum(P*F)  T = C + F*(dP - delta)
      ecirc = rowsum(P*T)
      dObar = P uV + (P*F) V - alpha O
      Qbar  = t[(P*T) K + dS uK - ecirc (P K)] - alpha dQ
      Sbar  = P*(T - alpha (dP - delta) - ecirc)
      Kbar  = t[Sbar^T Q + dS^T uQ]        Vbar = (P*(F - alpha))^T dO
    dK, dV, Kbar, Vbar are summed over the query heads of a KV group.
    """
    B, Hq, Nq, D = q.shape
    Hkv, Nk = k.shape[1], k.shape[2]
    G = Hq // Hkv
    t = 1.0 / math.sqrt(D) if scale is None else float(scale)
    q_offset = infer_q_offset(Nq, Nk, q_offset, k_offset, is_causal)
    cv = lambda x, like: torch.zeros_like(like) if x is None else x.detach().to(dtype)
    q, k, v, dO = (x.detach().to(dtype) for x in (q, k, v, dO))
    uQ, uK, uV = cv(uQ, q), cv(uK, k), cv(uV, v)
    kx, vx, uKx, uVx = (_expand_kv(x, G) for x in (k, v, uK, uV))
    mask = valid_mask(Nq, Nk, is_causal=is_causal, window_size=window_size, q_offset=q_offset,
                      k_offset=k_offset)

    out, lse = attention_dense(q, k, v, is_causal=is_causal, scale=t, window_size=window_size,
                               q_offset=q_offset, k_offset=k_offset, return_lse=True)
    S = torch.matmul(q, kx.transpose(-1, -2)) * t
    lse_safe = torch.where(torch.isfinite(lse), lse, torch.zeros_like(lse))
    P = torch.exp(torch.where(mask, S - lse_safe[..., None], torch.full_like(S, -math.inf)))
    P = torch.where(torch.isfinite(lse)[..., None], P, torch.zeros_like(P))

    delta = (dO * out).sum(-1)
    dP = torch.matmul(dO, vx.transpose(-1, -2))
    dPs = dP - delta[..., None]
    dS = P * dPs
    dQ = t * torch.matmul(dS, kx)
    dKx = t * torch.matmul(dS.transpose(-1, -2), q)
    dVx = torch.matmul(P.transpose(-1, -2), dO)

    F = t * (torch.matmul(uQ, kx.transpose(-1, -2)) + torch.matmul(q, uKx.transpose(-1, -2)))
    C = torch.matmul(dO, uVx.transpose(-1, -2))
    alpha = (P * F).sum(-1)
    T = C + F * dPs
    ecirc = (P * T).sum(-1)
    dObar = torch.matmul(P, uVx) + torch.matmul(P * F, vx) - alpha[..., None] * out
    Qbar = t * (torch.matmul(P * T, kx) + torch.matmul(dS, uKx)
                - ecirc[..., None] * torch.matmul(P, kx)) - alpha[..., None] * dQ
    Sbar = P * (T - alpha[..., None] * dPs - ecirc[..., None])
    Kbarx = t * (torch.matmul(Sbar.transpose(-1, -2), q) + torch.matmul(dS.transpose(-1, -2), uQ))
    Vbarx = torch.matmul((P * (F - alpha[..., None])).transpose(-1, -2), dO)

    red = lambda x: x.reshape(B, Hkv, G, Nk, D).sum(2)
    return DenseBoB(out=out, lse=lse, delta=delta, dQ=dQ, dK=red(dKx), dV=red(dVx), alpha=alpha,
                    ecirc=ecirc, Qbar=Qbar, Kbar=red(Kbarx), Vbar=red(Vbarx), dObar=dObar)


def bob_closed_form_streamed(q, k, v, dO, uQ, uK, uV, *, dtype=torch.float64, is_causal=False,
                             scale=None, window_size=0, q_offset=None, k_offset=0, row_block=1024):
    """`bob_closed_form` for sequences whose [Nq, Nk] score matrices do not fit in memory at once.

    Same formulas, evaluated one query head at a time and `row_block` query rows at a time (every
    row statistic is local to its row, so a block of whole rows is self-contained); the key-side
    results dK, dV, Kbar, Vbar are accumulated over the row blocks and over the query heads of a KV
    group.  This is how the largest benchmark configuration is checked: one (batch, KV head) unit,
    one query head at a time (the score matrices of one head alone take 512 MiB each in fp64).
    """
    B, Hq, Nq, D = q.shape
    Hkv, Nk = k.shape[1], k.shape[2]
    G = Hq // Hkv
    t = 1.0 / math.sqrt(D) if scale is None else float(scale)
    q_offset = infer_q_offset(Nq, Nk, q_offset, k_offset, is_causal)
    cv = lambda x, like: torch.zeros_like(like) if x is None else x.detach().to(dtype)
    q, k, v, dO = (x.detach().to(dtype) for x in (q, k, v, dO))
    uQ, uK, uV = cv(uQ, q), cv(uK, k), cv(uV, v)
    zq = lambda: torch.zeros(B, Hq, Nq, D, dtype=dtype)
    zk = lambda: torch.zeros(B, Hkv, Nk, D, dtype=dtype)
    zs = lambda: torch.zeros(B, Hq, Nq, dtype=dtype)
    out, dQ, Qbar, dObar = zq(), zq(), zq(), zq()
    dK, dV, Kbar, Vbar = zk(), zk(), zk(), zk()
    lse, delta, alpha, ecirc = zs(), zs(), zs(), zs()
    kj = torch.arange(Nk) + int(k_offset)
    for b in range(B):
        for h in range(Hq):
            hk = h // G
            K_, V_, uK_, uV_ = k[b, hk], v[b, hk], uK[b, hk], uV[b, hk]
            for r0 in range(0, Nq, row_block):
                r1 = min(Nq, r0 + row_block)
                Q_, dO_, uQ_ = q[b, h, r0:r1], dO[b, h, r0:r1], uQ[b, h, r0:r1]
                if is_causal:
                    dist = (torch.arange(r0, r1) + int(q_offset))[:, None] - kj[None, :]
                    mask = dist >= 0
                    if window_size:
                        mask &= dist < int(window_size)
                else:
                    mask = torch.ones(r1 - r0, Nk, dtype=torch.bool)
                S = (Q_ @ K_.T) * t
                S = torch.where(mask, S, torch.full_like(S, -math.inf))
                m = S.max(dim=-1, keepdim=True).values
                has = torch.isfinite(m)
                m = torch.where(has, m, torch.zeros_like(m))
                e = torch.exp(S - m)
                l = e.sum(-1, keepdim=True)
                P = torch.where(has, e / torch.where(has, l, torch.ones_like(l)), torch.zeros_like(e))
                L = torch.where(has, m + torch.log(torch.where(has, l, torch.ones_like(l))),
                                torch.full_like(m, -math.inf)).squeeze(-1)
                O_ = P @ V_
                dl = (dO_ * O_).sum(-1)
                dPs = dO_ @ V_.T - dl[:, None]
                dS = P * dPs
                dQ_ = t * (dS @ K_)
                F = t * (uQ_ @ K_.T + Q_ @ uK_.T)
                C = dO_ @ uV_.T
                al = (P * F).sum(-1)
                T = C + F * dPs
                ec = (P * T).sum(-1)
                Sbar = P * (T - al[:, None] * dPs - ec[:, None])
                out[b, h, r0:r1], lse[b, h, r0:r1], delta[b, h, r0:r1] = O_, L, dl
                alpha[b, h, r0:r1], ecirc[b, h, r0:r1], dQ[b, h, r0:r1] = al, ec, dQ_
                dObar[b, h, r0:r1] = P @ uV_ + (P * F) @ V_ - al[:, None] * O_
                Qbar[b, h, r0:r1] = t * ((P * T) @ K_ + dS @ uK_ - ec[:, None] * (P @ K_)) - al[:, None] * dQ_
                dK[b, hk] += t * (dS.T @ Q_)
                dV[b, hk] += P.T @ dO_
                Kbar[b, hk] += t * (Sbar.T @ Q_ + dS.T @ uQ_)
                Vbar[b, hk] += (P * (F - al[:, None])).T @ dO_
    return DenseBoB(out=out, lse=lse, delta=delta, dQ=dQ, dK=dK, dV=dV, alpha=alpha, ecirc=ecirc,
                    Qbar=Qbar, Kbar=Kbar, Vbar=Vbar, dObar=dObar)


# --------------------------------------------------------------------------------------
# the benchmark's loss chain
# --------------------------------------------------------------------------------------
def loss_chain(op, q, k, v, *, fp32_losses=False, hvp_directions=None, mean_counts=None, **kwargs):
    """L1 = mean(out^2); first grads with create_graph; L2 = sum of mean(grad^2); second grads.

    Because dO depends on `out`, the second differentiation re-enters the first backward:
    (ddq, ddk, ddv) = (Qbar, Kbar, Vbar) + first_backward(cotangent = (2/numel) dObar).
    With `hvp_directions` = (gq, gk, gv) also returns the Hessian-vector product of L1.
    `mean_counts` = (numel of out and q, numel of k) replaces the means' denominators: a shard of
    (batch, KV head) units evaluated with the FULL tensors' element counts gives exactly the
    full chain's gradients for that shard (heads do not interact).
    """
    q, k, v = (t.detach().clone().requires_grad_(True) for t in (q, k, v))
    out = op(q, k, v, **kwargs)
    up = (lambda t: t.float()) if fp32_losses else (lambda t: t)
    if mean_counts is None:
        mean = lambda t, which: up(t).square().mean()
    else:
        mean = lambda t, which: up(t).square().sum() / mean_counts[which]
    L1 = mean(out, 0)
    dq, dk, dv = torch.autograd.grad(L1, (q, k, v), create_graph=True)
    L2 = mean(dq, 0) + mean(dk, 1) + mean(dv, 1)
    want_hvp = hvp_directions is not None
    ddq, ddk, ddv = torch.autograd.grad(L2, (q, k, v), retain_graph=want_hvp)
    res = {"out": out.detach(), "dq": dq.detach(), "dk": dk.detach(), "dv": dv.detach(),
           "ddq": ddq, "ddk": ddk, "ddv": ddv}
    if want_hvp:
        gq, gk, gv = hvp_directions
        inner = (up(dq) * up(gq)).sum() + (up(dk) * up(gk)).sum() + (up(dv) * up(gv)).sum()
        hq, hk, hv = torch.autograd.grad(inner, (q, k, v))
        res.update(hvq=hq, hvk=hk, hvv=hv)
    return res


# --------------------------------------------------------------------------------------
# seeded inputs and error metrics
# --------------------------------------------------------------------------------------
def seeded_inputs(seed, q_shape, kv_shape, dtype, *, n_extra_q=0, n_extra_kv=0):
    """q, k, v (then n_extra_q query-shaped and n_extra_kv key-shaped tensors) i.i.d. N(0,1)
    from a CPU generator in fp32, rounded to `dtype`."""
    g = torch.Generator().manual_seed(int(seed))
    draw = lambda shape: torch.randn(shape, dtype=torch.float32, generator=g).to(dtype)
    base = [draw(q_shape), draw(kv_shape), draw(kv_shape)]
    extra_q = [draw(q_shape) for _ in range(n_extra_q)]
    extra_kv = [draw(kv_shape) for _ in range(n_extra_kv)]
    return base + extra_q + extra_kv


def error_metrics(actual: torch.Tensor, expected: torch.Tensor) -> dict:
    a, e = actual.detach().double().cpu(), expected.detach().double().cpu()
    diff = (a - e)
    ref_max = e.abs().max().item()
    ref_l2 = e.norm().item()
    return {
        "max_abs": diff.abs().max().item(),
        "max_abs_rel": diff.abs().max().item() / ref_max if ref_max > 0 else float("nan"),
        "l2_rel": diff.norm().item() / ref_l2 if ref_l2 > 0 else float("nan"),
    }
