"""Sharding of the two hot paths over the GPUs of one box: one process per GPU,
`torch.distributed` for the plumbing.

Both paths split into independent units with no collective on the data path:
the backward over (request, KV head) — the integer grids, the dQ reduction of
a GQA group and dK/dV are all confined to one unit, so a shard's gradients are
the 1-GPU run's bits — and the decode over requests (their pages, lengths and
references). The only exchange the cache format needs is an 8-bit V's scale at
prefill, which is the layer's: `shared_v_scale`. The reference is single-GPU
(no process group anywhere in it); this module is new.
"""

from __future__ import annotations

import math


def split_even(n_units: int, world: int, rank: int) -> range:
    """Rank `rank`'s contiguous share of `n_units`, sizes differing by at most one."""
    base, extra = divmod(n_units, world)
    lo = rank * base + min(rank, extra)
    return range(lo, lo + base + (1 if rank < extra else 0))


def backward_units(batch: int, n_kv_heads: int, world: int, rank: int):
    """(request, KV head) units of a dense backward for this rank, as
    `{request: (first KV head, one past last)}`. A KV head's G query heads stay
    together, so every reduction stays inside one rank."""
    out = {}
    for u in split_even(batch * n_kv_heads, world, rank):
        b, h = divmod(u, n_kv_heads)
        lo, hi = out.get(b, (h, h))
        out[b] = (min(lo, h), max(hi, h + 1))
    return out


def balance(costs, world: int):
    """Longest-processing-time partition of items with `costs` over `world`
    ranks: `parts[r]` lists the item indices of rank r, each in input order.
    Used with cost L for decode requests and L^2 for packed backward
    sequences."""
    order = sorted(range(len(costs)), key=lambda i: (-costs[i], i))
    load = [0.0] * world
    parts = [[] for _ in range(world)]
    for i in order:
        r = min(range(world), key=lambda j: (load[j], j))
        parts[r].append(i)
        load[r] += costs[i]
    return [sorted(p) for p in parts]


def v_scale_from_amax(amax: float, headroom: float = 2.0) -> float:
    """The prompt writer's rule for an 8-bit V's layer scale: the least power
    of two at or above amax * headroom / 448 (the device evaluates the same
    rule in fp32; for a power-of-two result the two agree)."""
    import numpy as np

    t = np.float32(np.float32(amax) * np.float32(headroom)) * np.float32(1.0 / 448.0)
    t = max(float(t), 1e-30)
    return 2.0 ** math.ceil(math.log2(t))


def shared_v_scale(v_local, headroom: float = 2.0, group=None) -> float:
    """One V scale for every shard of a layer: all-reduce (MAX) the shards'
    largest |v|, then apply the writer's rule. Pass the result as `v_scale=`
    to each rank's `FoldKVCache` so all shards encode V identically to a
    single-GPU prefill of the whole batch."""
    import torch
    import torch.distributed as dist

    amax = v_local.abs().amax().float().reshape(1)
    if dist.is_available() and dist.is_initialized():
        dist.all_reduce(amax, op=dist.ReduceOp.MAX, group=group)
    return v_scale_from_amax(float(amax), headroom)


def gather_rows(t, group=None):
    """All ranks' row blocks of `t` concatenated in rank order (equal shapes)."""
    import torch
    import torch.distributed as dist

    if not (dist.is_available() and dist.is_initialized()):
        return t
    out = [torch.empty_like(t) for _ in range(dist.get_world_size(group))]
    dist.all_gather(out, t.contiguous(), group=group)
    return torch.cat(out)
