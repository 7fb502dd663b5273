"""Multi-GPU sharding of the GDN2 operators: independent (batch, head) shards.

Every (batch, head) pair is an independent recurrence and no kernel of the reference
communicates across them (its grids are products over batch x heads, e.g.
src/gdn2_sm120/chunk.py:895-1053), so the multi-GPU form is pure data parallelism:
one process per GPU, each rank owns a contiguous slice of the batch axis (or of the head
axis when the batch is smaller than the world), no collective on the compute path.
The only communication is the optional final gather of outputs / states and the
max-over-ranks reduction of device timings.  These helpers run on any
``torch.distributed`` backend (NCCL on GPUs, gloo in the CPU tests).
"""

from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.distributed as dist


@dataclass(frozen=True)
class Shard:
    axis: int        # 0 = batch axis, 2 = head axis of a [B, T, H, D] tensor
    start: int
    stop: int

    @property
    def size(self) -> int:
        return self.stop - self.start


def _even_split(total: int, parts: int, index: int) -> tuple[int, int]:
    base, extra = divmod(total, parts)
    start = index * base + min(index, extra)
    return start, start + base + (1 if index < extra else 0)


def plan(batch: int, heads: int, world_size: int, rank: int) -> Shard:
    """Slice owned by ``rank``: along batch when B >= world, else along heads."""

    if world_size <= 0 or not 0 <= rank < world_size:
        raise ValueError("rank must satisfy 0 <= rank < world_size")
    if batch >= world_size:
        return Shard(0, *_even_split(batch, world_size, rank))
    if heads >= world_size:
        return Shard(2, *_even_split(heads, world_size, rank))
    raise ValueError("fewer (batch, head) units than ranks along both axes")


def take(tensor: torch.Tensor | None, shard: Shard, *, is_state: bool = False):
    """Contiguous local slice of a sequence tensor [B,T,H,D] or a state [B,H,K,V]."""

    if tensor is None:
        return None
    axis = shard.axis if not is_state else (0 if shard.axis == 0 else 1)
    return tensor.narrow(axis, shard.start, shard.size).contiguous()


def gather(local: torch.Tensor, shard: Shard, world_size: int, *, is_state: bool = False,
           group=None) -> torch.Tensor:
    """All-gather equally sized shards back into the global tensor (every rank gets it).

    Every rank must hold a shard of the same shape: collectives over unequal buffers are undefined
    (NCCL) or fail (gloo).  The shard sizes are compared first -- one tiny collective -- and a
    ``ValueError`` is raised on every rank when they differ, before any data moves.  Batch-axis
    shards are gathered straight into the result (``all_gather_into_tensor``); head-axis shards
    need one concatenation."""

    axis = shard.axis if not is_state else (0 if shard.axis == 0 else 1)
    sizes = torch.zeros(world_size, dtype=torch.int64, device=local.device)
    sizes[dist.get_rank(group)] = shard.size
    dist.all_reduce(sizes, op=dist.ReduceOp.SUM, group=group)
    sizes = sizes.tolist()
    if len(set(sizes)) != 1:
        raise ValueError(
            f"gather needs equally sized shards but the ranks hold {sizes} units along axis {shard.axis}; "
            "choose a batch (or head count) divisible by the number of ranks"
        )
    local = local.contiguous()
    if axis == 0:
        full = torch.empty((local.shape[0] * world_size, *local.shape[1:]), dtype=local.dtype,
                           device=local.device)
        dist.all_gather_into_tensor(full, local, group=group)
        return full
    pieces = [torch.empty_like(local) for _ in range(world_size)]
    dist.all_gather(pieces, local, group=group)
    return torch.cat(pieces, dim=axis)


def max_over_ranks(value: float, device, group=None) -> float:
    """Max-reduce a per-rank scalar (device timings are reported as the slowest rank)."""

    box = torch.tensor([float(value)], device=device, dtype=torch.float64)
    if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(box, op=dist.ReduceOp.MAX, group=group)
    return float(box.item())


def sum_over_ranks(value: float, device, group=None) -> float:
    box = torch.tensor([float(value)], device=device, dtype=torch.float64)
    if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(box, op=dist.ReduceOp.SUM, group=group)
    return float(box.item())
