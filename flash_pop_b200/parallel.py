"""Splitting one retention problem over several GPUs.

Every (batch row, head) pair is an independent recurrence, so a problem shards with no exchange of data: batch
rows are dealt out contiguously, and when there are fewer rows than ranks the heads of a row are split as well
(strided head views are taken in place by the kernels, and the per-head decays are sliced alike).  Each rank runs
the single-GPU operator on its piece; concatenating the pieces gives the single-GPU result.  The only collective
a benchmark needs is the max of the per-rank times.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Sequence, Tuple


@dataclass(frozen=True)
class Shard:
    batch: slice
    heads: slice

    def take_seq(self, t):
        """View of a (B, T, H, d) activation owned by this shard."""
        return None if t is None else t[self.batch, :, self.heads]

    def take_state(self, t):
        """View of a (B, H, dk, dv) state owned by this shard."""
        return None if t is None else t[self.batch, self.heads]

    def take_decays(self, decays: Sequence[float]) -> Tuple[float, ...]:
        return tuple(decays[self.heads])


def partition(B: int, H: int, rank: int, world: int) -> Shard:
    """The piece of a (B rows, H heads) problem that `rank` of `world` owns (possibly empty)."""
    if not 0 <= rank < world:
        raise ValueError(f"rank {rank} outside world {world}")
    if B >= world:
        base, extra = divmod(B, world)
        start = rank * base + min(rank, extra)
        return Shard(slice(start, start + base + (1 if rank < extra else 0)), slice(0, H))
    # fewer rows than ranks: ranks_per_row ranks share one row and split its heads
    ranks_per_row = world // B if B > 0 else world
    row, part = divmod(rank, ranks_per_row)
    if B == 0 or row >= B:
        return Shard(slice(0, 0), slice(0, 0))
    parts = min(ranks_per_row, H)
    if part >= parts:
        return Shard(slice(row, row + 1), slice(0, 0))
    base, extra = divmod(H, parts)
    h0 = part * base + min(part, extra)
    return Shard(slice(row, row + 1), slice(h0, h0 + base + (1 if part < extra else 0)))


def max_over_ranks(value: float, device=None) -> float:
    """Max of a per-rank number (a device-measured time) over the default process group; identity without one."""
    import torch
    import torch.distributed as dist
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return float(value)
    t = torch.tensor([value], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())
