"""Batch x KV-head sharding of the operator across the GPUs of one node.

Every (batch, KV head) unit - its G query heads, its K/V head, all tangents and all outputs - is
independent of every other unit (the group reduction of dK, dV, Kbar, Vbar stays inside a unit),
so the units are dealt to the ranks in contiguous blocks and no collective touches the data path.
The reference has no counterpart (its only multi-GPU code is a data-parallel trainer).
"""

from __future__ import annotations

import torch


def unit_range(n_units: int, world_size: int, rank: int) -> range:
    """Contiguous block of units owned by `rank`; the first `n_units % world_size` ranks hold one
    extra unit."""
    if not (0 <= rank < world_size):
        raise ValueError(f"rank {rank} outside world of {world_size}")
    base, extra = divmod(n_units, world_size)
    start = rank * base + min(rank, extra)
    return range(start, start + base + (1 if rank < extra else 0))


def as_units(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor):
    """View [B, Hq, Nq, D] / [B, Hkv, Nk, D] tensors as per-unit batches:
    q -> [B*Hkv, G, Nq, D], k and v -> [B*Hkv, 1, Nk, D] (no copy for contiguous inputs)."""
    B, Hq, Nq, D = q.shape
    Hkv, Nk = k.shape[1], k.shape[2]
    if Hq % Hkv:
        raise ValueError(f"query heads H_Q={Hq} must be divisible by KV heads H_KV={Hkv}")
    G = Hq // Hkv
    return (q.reshape(B * Hkv, G, Nq, D), k.reshape(B * Hkv, 1, Nk, D), v.reshape(B * Hkv, 1, Nk, D))


def shard(q, k, v, world_size: int, rank: int):
    """This rank's units of (q, k, v), shaped for `sdpa_bob` (batch = units, H_KV = 1)."""
    uq, uk, uv = as_units(q, k, v)
    r = unit_range(uq.shape[0], world_size, rank)
    return uq[r.start:r.stop], uk[r.start:r.stop], uv[r.start:r.stop]


def from_units(x_units: torch.Tensor, B: int, heads: int) -> torch.Tensor:
    """Inverse of `as_units` for one tensor: [B*Hkv, h, N, D] -> [B, Hkv*h, N, D]."""
    U, h, N, D = x_units.shape
    if B <= 0 or U % B or heads != (U // B) * h:
        raise ValueError(f"{U} units of {h} heads do not form a [B={B}, H={heads}] tensor")
    return x_units.reshape(B, heads, N, D)
