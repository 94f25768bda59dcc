"""Sharding of independent domains across ranks and the one collective of the path.

Every input and every BaB subdomain is bounded independently, so the batch axis
is split into contiguous blocks (one per rank, weights replicated) and the only
exchange is an all-gather of the per-domain results: `[B_local, S]` fp32 lower
bounds and `[B_local]` int8 verdicts.  Works on any torch.distributed backend
(NCCL on the GPU box, gloo in the CPU tests).  The reference has no multi-device
code; this module is new.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Tuple

import torch
import torch.distributed as dist


_GATHER_BUFFERS: Dict[tuple, Tuple[torch.Tensor, torch.Tensor]] = {}


def shard_range(n: int, rank: int, world: int) -> Tuple[int, int]:
    """Contiguous block [start, stop) of `n` items owned by `rank`; blocks differ by at most one item."""
    if world <= 0 or not (0 <= rank < world):
        raise ValueError(f"bad rank/world: {rank}/{world}")
    base, extra = divmod(int(n), int(world))
    start = rank * base + min(rank, extra)
    return start, start + base + (1 if rank < extra else 0)


def shard_sizes(n: int, world: int) -> List[int]:
    return [shard_range(n, r, world)[1] - shard_range(n, r, world)[0] for r in range(world)]


def gather_domain_results(
    lower: torch.Tensor, verdict: torch.Tensor, n_total: int, group: Optional[dist.ProcessGroup] = None
) -> Tuple[torch.Tensor, torch.Tensor]:
    """All-gather per-domain lower bounds [B_local,S] and verdicts [B_local] (int8)
    into [n_total,S] / [n_total] on every rank, in global domain order."""
    if not dist.is_initialized() or dist.get_world_size(group) == 1:
        return lower, verdict
    world = dist.get_world_size(group)
    sizes = shard_sizes(n_total, world)
    pad = max(sizes)
    S = int(lower.shape[1])
    # ONE collective per step: bounds and verdict of a domain travel as one row of S + 1 floats, gathered into a
    # receive buffer that is kept between calls (keyed by shape, dtype and device).
    key = (world, pad, S, lower.dtype, str(lower.device))
    bufs = _GATHER_BUFFERS.get(key)
    if bufs is None:
        if len(_GATHER_BUFFERS) > 16:
            _GATHER_BUFFERS.clear()
        bufs = (torch.zeros(pad, S + 1, dtype=lower.dtype, device=lower.device),
                torch.empty(world * pad, S + 1, dtype=lower.dtype, device=lower.device))
        _GATHER_BUFFERS[key] = bufs
    send, recv = bufs
    n_local = int(lower.shape[0])
    send[:n_local, :S] = lower
    send[:n_local, S] = verdict.to(lower.dtype)
    dist.all_gather_into_tensor(recv, send, group=group)
    if all(s == pad for s in sizes):  # equal shards: the receive buffer already is the global order
        rows = recv
    else:
        rows = torch.cat([recv[r * pad : r * pad + sizes[r]] for r in range(world)], dim=0)
    return rows[:, :S].clone(), rows[:, S].to(torch.int8)
