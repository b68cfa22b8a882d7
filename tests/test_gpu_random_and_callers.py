"""Randomised geometries against the oracle, and caller-level use: layout adapters and a
Hessian-vector product over the parameters of a small attention block."""

import random

import pytest
import torch

import bob
from flashbob_b200 import adapters, interface, ops
from oracle import bob_oracle as O

pytestmark = pytest.mark.gpu
BF16, FP16 = torch.bfloat16, torch.float16


def _random_case(rng):
    D = rng.choice([32, 64, 128])
    dtype = rng.choice([BF16, BF16, FP16])
    Hkv = rng.choice([1, 2, 3])
    G = rng.choice([1, 1, 2, 4])
    B = rng.choice([1, 2])
    Nq = rng.randint(1, 330)
    kind = rng.choice(["square", "square", "rect", "noncausal"])
    kw = {}
    if kind == "square":
        Nk = Nq
        kw = dict(is_causal=True)
        if rng.random() < 0.5:
            kw["window_size"] = rng.randint(1, Nq + 5)
    elif kind == "rect":
        Nk = rng.randint(1, 400)
        k_off = rng.choice([0, rng.randint(0, 2000)])
        kw = dict(is_causal=True, k_offset=k_off, q_offset=k_off + rng.randint(0, max(0, Nk - 1)))
        if rng.random() < 0.5:
            kw["window_size"] = rng.randint(1, 200)
    else:
        Nk = rng.randint(1, 400)
        kw = dict(is_causal=False)
    if rng.random() < 0.3:
        kw["scale"] = rng.uniform(0.05, 0.5)
    return B, Hkv * G, Hkv, Nq, Nk, D, dtype, kw


@pytest.mark.parametrize("seed", range(24))
def test_random_geometry_matches_oracle(seed):
    rng = random.Random(1234 + seed)
    B, Hq, Hkv, Nq, Nk, D, dtype, kw = _random_case(rng)
    q, k, v, dO, uQ = O.seeded_inputs(seed, (B, Hq, Nq, D), (B, Hkv, Nk, D), dtype, n_extra_q=2)
    uK, uV = O.seeded_inputs(seed + 500, (B, Hq, Nq, D), (B, Hkv, Nk, D), dtype)[1:]
    causal = kw.get("is_causal", False)
    geom = dict(is_causal=causal, window_size=kw.get("window_size", 0),
                q_offset=O.infer_q_offset(Nq, Nk, kw.get("q_offset"), kw.get("k_offset", 0), causal),
                k_offset=kw.get("k_offset", 0), scale=kw.get("scale"))
    ref = O.bob_closed_form(q, k, v, dO, uQ, uK, uV, **geom)
    c = lambda t: t.cuda()
    out, lse = ops.attention_forward(c(q), c(k), c(v), **geom)
    dQ, dK, dV, delta, pk = ops.attention_first_backward(c(q), c(k), c(v), out, lse, c(dO), **geom)
    Qb, Kb, Vb, dOb = ops.attention_second_backward(c(q), c(k), c(v), out, lse, delta, pk, c(dO), dQ, c(uQ), c(uK),
                                                    c(uV), **geom)
    got = dict(out=out, dQ=dQ, dK=dK, dV=dV, Qbar=Qb, Kbar=Kb, Vbar=Vb, dObar=dOb)
    l2_bar = 8e-3 if dtype == BF16 else 1.5e-3
    for n in O.OUTPUT_NAMES:
        r = getattr(ref, n)
        g = got[n]
        assert torch.isfinite(g.float()).all(), (n, geom)
        scale = r.abs().max().item()
        if scale == 0:
            assert g.float().abs().max().item() <= 0.08, (n, geom)
            continue
        m = O.error_metrics(g, r)
        # tiny tensors (a handful of elements) have noisy relative norms: bound the absolute error too
        assert m["l2_rel"] <= l2_bar or m["max_abs"] <= 0.02 * max(1.0, scale), (n, m, geom, (B, Hq, Hkv, Nq, Nk, D))


@pytest.mark.parametrize("seed", range(16))
def test_random_geometry_with_many_work_items(seed):
    """Shapes with several batch elements and heads, so that most launches have more work items than SMs
    and run persistently (every head dim the C ABI takes, grouped heads with windows and rectangles
    included); one (batch, KV group) slice of each is compared with the oracle."""
    rng = random.Random(99991 + seed)
    D = rng.choice([16, 32, 48, 64, 80, 96, 128])
    dtype = rng.choice([BF16, BF16, FP16])
    Hkv, G, B = rng.choice([2, 4, 6]), rng.choice([1, 2, 4, 8]), rng.choice([2, 4, 6])
    Nq = rng.randint(130, 720)
    kind = rng.choice(["square", "square", "window", "rect", "noncausal"])
    if kind in ("square", "window"):
        Nk, kw = Nq, dict(is_causal=True)
        if kind == "window":
            kw["window_size"] = rng.randint(1, Nq + 5)
    elif kind == "rect":
        Nk = rng.randint(130, 800)
        k_off = rng.choice([0, rng.randint(0, 2000)])
        kw = dict(is_causal=True, k_offset=k_off, q_offset=k_off + rng.randint(0, max(0, Nk - 1)))
        if rng.random() < 0.5:
            kw["window_size"] = rng.randint(1, 300)
    else:
        Nk, kw = rng.randint(130, 800), dict(is_causal=False)
    Hq = Hkv * G
    q, k, v, dO, uQ = O.seeded_inputs(seed, (B, Hq, Nq, D), (B, Hkv, Nk, D), dtype, n_extra_q=2)
    uK, uV = O.seeded_inputs(seed + 500, (B, Hq, Nq, D), (B, Hkv, Nk, D), dtype)[1:]
    causal = kw.get("is_causal", False)
    geom = dict(is_causal=causal, window_size=kw.get("window_size", 0),
                q_offset=O.infer_q_offset(Nq, Nk, kw.get("q_offset"), kw.get("k_offset", 0), causal),
                k_offset=kw.get("k_offset", 0), scale=None)
    c = lambda t: t.cuda()
    out, lse = ops.attention_forward(c(q), c(k), c(v), **geom)
    dQ, dK, dV, delta, pk = ops.attention_first_backward(c(q), c(k), c(v), out, lse, c(dO), **geom)
    Qb, Kb, Vb, dOb = ops.attention_second_backward(c(q), c(k), c(v), out, lse, delta, pk, c(dO), dQ, c(uQ), c(uK),
                                                    c(uV), **geom)
    got = dict(out=out, dQ=dQ, dK=dK, dV=dV, Qbar=Qb, Kbar=Kb, Vbar=Vb, dObar=dOb)
    b, hk = rng.randrange(B), rng.randrange(Hkv)
    hs = slice(hk * G, hk * G + G)
    kv = lambda t: t[b:b + 1, hk:hk + 1]
    qs = lambda t: t[b:b + 1, hs]
    ref = O.bob_closed_form(qs(q), kv(k), kv(v), qs(dO), qs(uQ), kv(uK), kv(uV), **geom)
    l2_bar = 8e-3 if dtype == BF16 else 1.5e-3
    for n in O.OUTPUT_NAMES:
        r = getattr(ref, n)
        g = qs(got[n]) if n in ("out", "dQ", "Qbar", "dObar") else kv(got[n])
        assert torch.isfinite(got[n].float()).all(), (n, geom)
        scale = r.abs().max().item()
        if scale == 0:
            continue
        m = O.error_metrics(g, r)
        assert m["l2_rel"] <= l2_bar or m["max_abs"] <= 0.02 * max(1.0, scale), (n, m, geom, (B, Hq, Hkv, Nq, Nk, D))


def test_flash_attn_layout_adapter_reads_bnhd_storage_in_place():
    B, N, Hq, Hkv, D = 2, 200, 4, 2, 64
    g = torch.Generator().manual_seed(5)
    r = lambda *s: torch.randn(*s, generator=g).to(BF16)
    q, k, v = r(B, N, Hq, D), r(B, N, Hkv, D), r(B, N, Hkv, D)
    out = adapters.flash_attn_layout(q.cuda(), k.cuda(), v.cuda(), causal=True)
    assert out.shape == (B, N, Hq, D)
    ref = O.attention_dense(q.transpose(1, 2).double(), k.transpose(1, 2).double(), v.transpose(1, 2).double(),
                            is_causal=True).transpose(1, 2)
    assert O.error_metrics(out, ref)["l2_rel"] < 6e-3
    win = adapters.flash_attn_layout(q[:, :, :2].cuda(), k[:, :, :2].cuda(), v[:, :, :2].cuda(), causal=True,
                                     window_size=(31, 0))
    ref = O.attention_dense(q[:, :, :2].transpose(1, 2).double(), k[:, :, :2].transpose(1, 2).double(),
                            v[:, :, :2].transpose(1, 2).double(), is_causal=True, window_size=32).transpose(1, 2)
    assert O.error_metrics(win, ref)["l2_rel"] < 6e-3


def test_hf_attention_interface_against_the_oracle():
    """The Hugging Face attention-interface signature (reference: examples/huggingface_backend.py:29-61):
    grouped heads through `num_key_value_groups`-style shapes, a sliding window, and a single-token
    decode step over a cache (right-aligned, so every cached key - or the last `sliding_window` of
    them - is visible).  Output layout [B, N, H, D], contiguous."""
    g = torch.Generator().manual_seed(9)
    r = lambda *s: torch.randn(*s, generator=g).to(BF16)

    class _Module:
        is_causal = True

    # grouped heads, prefill
    q, k, v = r(2, 8, 150, 64), r(2, 2, 150, 64), r(2, 2, 150, 64)
    out, w = adapters.hf_attention_interface(_Module(), q.cuda(), k.cuda(), v.cuda(), None, scaling=0.11)
    assert w is None and out.shape == (2, 150, 8, 64) and out.is_contiguous()
    ref = O.attention_dense(q.double(), k.double(), v.double(), is_causal=True, scale=0.11).transpose(1, 2)
    assert O.error_metrics(out, ref)["l2_rel"] < 6e-3
    # sliding window, prefill (multi-head: the reference supports windows without grouping)
    q, k, v = r(1, 4, 300, 64), r(1, 4, 300, 64), r(1, 4, 300, 64)
    out, _ = adapters.hf_attention_interface(_Module(), q.cuda(), k.cuda(), v.cuda(), None, sliding_window=64)
    ref = O.attention_dense(q.double(), k.double(), v.double(), is_causal=True, window_size=64).transpose(1, 2)
    assert O.error_metrics(out, ref)["l2_rel"] < 6e-3
    # single-token decode over a cache of 257 keys, with and without a window
    q, k, v = r(2, 4, 1, 64), r(2, 4, 257, 64), r(2, 4, 257, 64)
    for window in (0, 100):
        out, _ = adapters.hf_attention_interface(_Module(), q.cuda(), k.cuda(), v.cuda(), None,
                                                 sliding_window=window or None)
        assert out.shape == (2, 1, 4, 64)
        ref = O.attention_dense(q.double(), k.double(), v.double(), is_causal=True, window_size=window,
                                q_offset=256, k_offset=0).transpose(1, 2)
        assert O.error_metrics(out, ref)["l2_rel"] < 6e-3, window
    # second order through the adapter: gradients flow through the transposed, contiguous output
    q, k, v = (t.cuda().requires_grad_(True) for t in (r(1, 4, 96, 64), r(1, 2, 96, 64), r(1, 2, 96, 64)))
    out, _ = adapters.hf_attention_interface(_Module(), q, k, v, None)
    first = torch.autograd.grad(out.float().square().mean(), (q, k, v), create_graph=True)
    second = torch.autograd.grad(sum(f.float().square().sum() for f in first), (q, k, v))
    assert all(torch.isfinite(t.float()).all() and t.abs().max() > 0 for t in second)
    with pytest.raises(NotImplementedError, match="padded"):
        adapters.hf_attention_interface(_Module(), q, k, v, torch.zeros(1, 1, 96, 96, device="cuda"))


class _Block(torch.nn.Module):
    def __init__(self, dim, heads, kv_heads, attend):
        super().__init__()
        self.h, self.hk, self.d = heads, kv_heads, dim // heads
        self.wq = torch.nn.Linear(dim, heads * self.d, bias=False)
        self.wk = torch.nn.Linear(dim, kv_heads * self.d, bias=False)
        self.wv = torch.nn.Linear(dim, kv_heads * self.d, bias=False)
        self.wo = torch.nn.Linear(heads * self.d, dim, bias=False)
        self.attend = attend

    def forward(self, x):
        B, N, _ = x.shape
        q = self.wq(x).view(B, N, self.h, self.d).transpose(1, 2)
        k = self.wk(x).view(B, N, self.hk, self.d).transpose(1, 2)
        v = self.wv(x).view(B, N, self.hk, self.d).transpose(1, 2)
        o = self.attend(q, k, v)
        return x + self.wo(o.transpose(1, 2).reshape(B, N, self.h * self.d))


def test_hessian_vector_product_over_parameters_of_an_attention_block():
    """Hv = d/dtheta <grad L(theta), v>: the second differentiation runs through the second backward
    (grouped heads, strided q/k/v views) and the re-entered first backward."""
    torch.manual_seed(0)
    dim, heads, kv_heads, B, N = 256, 4, 2, 2, 160
    ref_block = _Block(dim, heads, kv_heads, lambda q, k, v: O.attention_dense(q, k, v, is_causal=True)).double()
    gpu_block = _Block(dim, heads, kv_heads, lambda q, k, v: bob.sdpa_bob(q, k, v, is_causal=True)).cuda().to(BF16)
    with torch.no_grad():
        for pr, pg in zip(ref_block.parameters(), gpu_block.parameters()):
            pr.copy_(pr.to(BF16).double())
            pg.copy_(pr.to(BF16))
    x = torch.randn(B, N, dim).to(BF16)
    vecs = [torch.randn_like(p).to(BF16) for p in ref_block.parameters()]

    def hvp(block, x, vecs):
        params = list(block.parameters())
        loss = block(x).float().square().mean() if x.is_cuda else block(x).square().mean()
        grads = torch.autograd.grad(loss, params, create_graph=True)
        inner = sum((g.float() * v.float()).sum() if x.is_cuda else (g * v).sum() for g, v in zip(grads, vecs))
        return torch.autograd.grad(inner, params)

    want = hvp(ref_block, x.double(), [v.double() for v in vecs])
    got = hvp(gpu_block, x.cuda(), [v.cuda() for v in vecs])
    for w, g in zip(want, got):
        m = O.error_metrics(g, w)
        assert m["l2_rel"] < 3e-2, m
