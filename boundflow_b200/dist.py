"""Sharding of independent domains across ranks and the one collective of the path.

Every input and every BaB subdomain is bounded independently, so the batch axis
is split into contiguous blocks (one per rank, weights replicated) and the only
exchange is an all-gather of the per-domain results: `[B_local, S]` fp32 lower
bounds and `[B_local]` int8 verdicts.  Works on any torch.distributed backend
(NCCL on the GPU box, gloo in the CPU tests).  The reference has no multi-device
code; this module is new.
"""
from __future__ import annotations

from typing import List, Optional, Tuple

import torch
import torch.distributed as dist


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
    send_l = torch.zeros(pad, S, dtype=lower.dtype, device=lower.device)
    send_v = torch.zeros(pad, dtype=torch.int8, device=verdict.device)
    send_l[: lower.shape[0]] = lower
    send_v[: verdict.shape[0]] = verdict.to(torch.int8)
    recv_l = torch.empty(world * pad, S, dtype=lower.dtype, device=lower.device)
    recv_v = torch.empty(world * pad, dtype=torch.int8, device=verdict.device)
    dist.all_gather_into_tensor(recv_l, send_l, group=group)
    dist.all_gather_into_tensor(recv_v, send_v, group=group)
    out_l = torch.cat([recv_l[r * pad : r * pad + sizes[r]] for r in range(world)], dim=0)
    out_v = torch.cat([recv_v[r * pad : r * pad + sizes[r]] for r in range(world)], dim=0)
    return out_l, out_v
