"""Sharding of the hot path across the GPUs of one node.

Every (sequence, value head) pair is an independent recurrence, so the path partitions with no exchange
step: shard the batch (or whole GVA groups of heads) across ranks, run the same operators on each shard and,
only when results have to be compared with a single-device run, gather them.  Collectives are therefore
never on the data path; `gather_along` is for verification and result collection.  The reference has no
multi-device support beyond a per-call device guard (…/ops/ascendc/_runtime.py:153-174).
"""
from __future__ import annotations

from typing import Dict, Optional, Sequence, Tuple

import torch
import torch.distributed as dist


def shard_range(total: int, world: int, rank: int, granule: int = 1) -> Tuple[int, int]:
    """Contiguous [begin, end) of `total` items for `rank`, in multiples of `granule` (e.g. HV // HK value
    heads, so that a GVA group is never split: dq / dk need all value heads of a group)."""
    if total % granule:
        raise ValueError(f"total={total} is not a multiple of granule={granule}")
    units = total // granule
    base, rem = divmod(units, world)
    begin = rank * base + min(rank, rem)
    end = begin + base + (1 if rank < rem else 0)
    return begin * granule, end * granule


def shard_batch(tensors: Dict[str, Optional[torch.Tensor]], world: int, rank: int, dim: int = 0):
    """Slice every tensor of a step along the batch dimension."""
    out = {}
    for name, t in tensors.items():
        if t is None:
            out[name] = None
            continue
        b, e = shard_range(t.shape[dim], world, rank)
        out[name] = t.narrow(dim, b, e - b)
    return out


def shard_heads(q, k, v, g, beta, initial_state, world: int, rank: int):
    """Slice a GDN step by whole GVA groups: q,k [B,T,HK,K]; v [B,T,HV,V]; g,beta [B,T,HV]; state [N,HV,K,V]."""
    HK, HV = q.shape[2], v.shape[2]
    kb, ke = shard_range(HK, world, rank)
    rep = HV // HK
    vb, ve = kb * rep, ke * rep
    h0 = None if initial_state is None else initial_state[:, vb:ve]
    return q[:, :, kb:ke], k[:, :, kb:ke], v[:, :, vb:ve], g[:, :, vb:ve], beta[:, :, vb:ve], h0


def gather_along(t: torch.Tensor, dim: int, sizes: Optional[Sequence[int]] = None, group=None) -> torch.Tensor:
    """All-gather shards of possibly different extent along `dim` (verification / result collection only)."""
    world = dist.get_world_size(group)
    if world == 1:
        return t
    if sizes is None:
        mine = torch.tensor([t.shape[dim]], device=t.device, dtype=torch.int64)
        all_sizes = [torch.zeros_like(mine) for _ in range(world)]
        dist.all_gather(all_sizes, mine, group=group)
        sizes = [int(s.item()) for s in all_sizes]
    mx = max(sizes)
    pad_shape = list(t.shape)
    pad_shape[dim] = mx
    buf = t.new_zeros(pad_shape)
    buf.narrow(dim, 0, t.shape[dim]).copy_(t)
    outs = [torch.empty_like(buf) for _ in range(world)]
    dist.all_gather(outs, buf.contiguous(), group=group)
    return torch.cat([o.narrow(dim, 0, s) for o, s in zip(outs, sizes)], dim=dim)


def max_over_ranks(value: float, device, group=None) -> float:
    """Reduction used for timing: a multi-GPU step takes as long as its slowest rank."""
    t = torch.tensor([value], device=device, dtype=torch.float64)
    if dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    return float(t.item())
