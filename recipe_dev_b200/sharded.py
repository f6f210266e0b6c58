"""Row-split LM head and expert-parallel MoE across the GPUs of one node.

One process per GPU; `torch.distributed` (NCCL on GPUs, gloo on CPU in the tests) carries the
one exchange each config has:

* LM head (lone_split of a large sum by rows, recipe.rs:21010-21020): rank r holds the contiguous
  rows [r * rows / world, (r + 1) * rows / world) of the table, computes its slice of the logits
  and the slices are all-gathered (Primitive::Exchange gather, recipe.rs:5386-5394).
* MoE bank: rank r holds the whole experts [r * E / world, (r + 1) * E / world); the router and the
  top-k are replicated; every rank adds up its own routed experts, rank 0 adds the shared expert,
  and the [hidden, tokens] outputs are all-reduced (sum). The reference slices every expert's rows
  across dies instead (recipe.rs:4764-4766) and sums the dies' planes in die order; the exchange
  has the same shape, the order of the cross-rank additions differs (within tolerance, not bit-equal).

Kernels only ever read local memory: the collective lands remote slices in local buffers.
The compute is passed in as callables so that the partition / exchange logic is testable on CPU.
"""
from __future__ import annotations

from typing import Callable, Sequence


def shard_range(total: int, world: int, rank: int) -> tuple[int, int]:
    """Contiguous share [first, first + count) of `total` units for `rank`; sizes differ by at most one."""
    if world <= 0 or not 0 <= rank < world:
        raise ValueError(f"rank {rank} outside a world of {world}")
    first = total * rank // world
    return first, total * (rank + 1) // world - first


def shard_sizes(total: int, world: int) -> list[int]:
    return [shard_range(total, world, r)[1] for r in range(world)]


def gather_rows(local, rows: int, dist, world: int, rank: int):
    """All-gathers the ranks' logit slices ([tokens, local_rows]) into [tokens, rows]."""
    import torch

    sizes = shard_sizes(rows, world)
    if local.shape[-1] != sizes[rank]:
        raise ValueError(f"rank {rank} holds {local.shape[-1]} rows, its share is {sizes[rank]}")
    if world == 1:
        return local
    tokens = local.shape[0]
    if len(set(sizes)) == 1:
        out = torch.empty((world * tokens, sizes[0]), dtype=local.dtype, device=local.device)
        dist.all_gather_into_tensor(out, local.contiguous())
        return out.view(world, tokens, sizes[0]).permute(1, 0, 2).reshape(tokens, rows)
    # uneven shares: every rank sends the widest share (its own padded), the padding is cut after the gather
    widest = max(sizes)
    padded = torch.zeros((tokens, widest), dtype=local.dtype, device=local.device)
    padded[:, : sizes[rank]] = local
    out = torch.empty((world * tokens, widest), dtype=local.dtype, device=local.device)
    dist.all_gather_into_tensor(out, padded)
    out = out.view(world, tokens, widest)
    return torch.cat([out[r, :, : sizes[r]] for r in range(world)], dim=-1)


class ShardedHead:
    """A row-split matrix: `compute(x) -> [tokens, local_rows]` on this rank's rows, then the gather."""

    def __init__(self, rows: int, compute: Callable, dist, world: int, rank: int):
        self.rows, self.compute, self.dist, self.world, self.rank = rows, compute, dist, world, rank
        self.first, self.count = shard_range(rows, world, rank)

    def __call__(self, x):
        return gather_rows(self.compute(x), self.rows, self.dist, self.world, self.rank)


class ShardedExperts:
    """An expert-parallel bank: `compute(x, routing, include_shared) -> [hidden, tokens]` over this
    rank's experts, then the all-reduce."""

    def __init__(self, experts: int, compute: Callable, dist, world: int, rank: int):
        self.experts, self.compute, self.dist, self.world, self.rank = experts, compute, dist, world, rank
        self.first, self.count = shard_range(experts, world, rank)

    def __call__(self, x, routing):
        y = self.compute(x, routing, self.rank == 0)
        if self.world > 1:
            self.dist.all_reduce(y)
        return y


def routed_bytes_per_rank(routing, experts: int, world: int, expert_bytes: int) -> Sequence[int]:
    """Weight bytes each rank streams for these routing weights ([experts, tokens]): the load balance of a step."""
    taken = (routing != 0).sum(dim=1) if hasattr(routing, "dim") else (routing != 0).sum(axis=1)
    out = []
    for r in range(world):
        first, count = shard_range(experts, world, r)
        out.append(int(taken[first:first + count].sum()) * expert_bytes)
    return out
