"""Batch x KV-head sharding: unit bookkeeping, and a 2-rank gloo run on CPU whose gathered shard
results equal the unsharded operator."""

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from flashbob_b200 import sharding


def test_unit_ranges_partition_the_units():
    for n in (1, 7, 8, 64):
        for w in (1, 2, 3, 4, 8):
            seen = []
            for r in range(w):
                seen += list(sharding.unit_range(n, w, r))
            assert seen == list(range(n))
    with pytest.raises(ValueError):
        sharding.unit_range(8, 2, 2)


def test_unit_views_do_not_copy_and_round_trip():
    q = torch.randn(2, 8, 5, 4)
    k = torch.randn(2, 2, 6, 4)
    uq, uk, uv = sharding.as_units(q, k, k)
    assert uq.shape == (4, 4, 5, 4) and uk.shape == (4, 1, 6, 4)
    assert uq.data_ptr() == q.data_ptr()
    assert torch.equal(sharding.from_units(uq, 2, 8), q)
    # unit u = (b, h_kv) holds query heads h_kv*G .. h_kv*G+G-1 of batch b
    assert torch.equal(uq[3], q[1, 4:8])
    assert torch.equal(sharding.from_units(uk, 2, 2), k)
    for bad in ((uq, 2, 4), (uq, 3, 8), (uk, 2, 8)):       # head counts / batch sizes that do not match the units
        with pytest.raises(ValueError):
            sharding.from_units(*bad)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, tmpdir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from bob import sdpa_bob

        g = torch.Generator().manual_seed(0)
        B, H, N, D = 3, 2, 12, 8               # 6 units over 2 ranks; MHA so the CPU route applies
        q, k, v = (torch.randn(B, H, N, D, generator=g) for _ in range(3))
        sq, sk, sv = (t.clone().requires_grad_(True) for t in sharding.shard(q, k, v, world, rank))
        out = sdpa_bob(sq, sk, sv, is_causal=True)
        # global denominators keep the mathematics independent of the sharding
        L1 = out.square().sum() / q.numel()
        dq, dk, dv = torch.autograd.grad(L1, (sq, sk, sv), create_graph=True)
        L2 = dq.square().sum() / q.numel() + dk.square().sum() / k.numel() + dv.square().sum() / v.numel()
        ddq, ddk, ddv = torch.autograd.grad(L2, (sq, sk, sv))
        gathered = [None] * world
        dist.all_gather_object(gathered, (ddq, ddk, ddv))
        if rank == 0:
            full = [torch.cat([g[i] for g in gathered], 0) for i in range(3)]
            torch.save([sharding.from_units(t, B, H) for t in full], os.path.join(tmpdir, "sharded.pt"))
    finally:
        dist.destroy_process_group()


def test_two_rank_sharded_chain_equals_unsharded(tmp_path):
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    sharded = torch.load(tmp_path / "sharded.pt")
    from bob import sdpa_bob

    g = torch.Generator().manual_seed(0)
    q, k, v = (torch.randn(3, 2, 12, 8, generator=g).requires_grad_(True) for _ in range(3))
    out = sdpa_bob(q, k, v, is_causal=True)
    L1 = out.square().mean()
    dq, dk, dv = torch.autograd.grad(L1, (q, k, v), create_graph=True)
    L2 = dq.square().mean() + dk.square().mean() + dv.square().mean()
    ref = torch.autograd.grad(L2, (q, k, v))
    for a, b in zip(sharded, ref):
        torch.testing.assert_close(a, b, rtol=1e-5, atol=1e-12)
