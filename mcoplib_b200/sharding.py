"""Token sharding of the hot path across the GPUs of one node.

Rows are independent given the replicated small parameters, so every rank owns a contiguous token range,
runs the whole chain on it, and no collective is on the data path.  The per-expert counts / offsets of the
scatter are local to the rank's shard (experts are not sharded).  Results are gathered only to verify them.
"""
from __future__ import annotations

from typing import List, Tuple

import torch


def shard_range(tokens: int, rank: int, world: int) -> Tuple[int, int]:
    """Contiguous token range [t0, t1) of `rank`; the first `tokens % world` ranks hold one extra token."""
    if world < 1 or not (0 <= rank < world) or tokens < 0:
        raise ValueError(f"bad shard request tokens={tokens} rank={rank} world={world}")
    base, extra = divmod(tokens, world)
    t0 = rank * base + min(rank, extra)
    return t0, t0 + base + (1 if rank < extra else 0)


def gather_for_verification(local: torch.Tensor, tokens: int, group=None) -> torch.Tensor:
    """All-gathers per-token results (dim 0 = this rank's tokens) into the full tensor on every rank.
    Off the clock: used only by tests and verification runs.  Works on gloo (CPU) and nccl."""
    import torch.distributed as dist
    world = dist.get_world_size(group)
    sizes = [shard_range(tokens, r, world) for r in range(world)]
    longest = max(b - a for a, b in sizes)
    pad = torch.zeros((longest,) + tuple(local.shape[1:]), dtype=local.dtype, device=local.device)
    pad[: local.shape[0]] = local
    parts: List[torch.Tensor] = [torch.empty_like(pad) for _ in range(world)]
    dist.all_gather(parts, pad, group=group)
    return torch.cat([p[: b - a] for p, (a, b) in zip(parts, sizes)], dim=0)


def max_over_ranks(value: float, device, group=None) -> float:
    """Step time of a multi-GPU run: the maximum over ranks of the per-rank device time."""
    import torch.distributed as dist
    t = torch.tensor([value], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    return float(t[0])
