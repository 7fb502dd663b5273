"""World-size-2 CPU tests (gloo) of the multi-GPU host logic: partition of the (batch, head)
units, local slicing, the final gather and the max-over-ranks timing reduction.  The
operators themselves need no collective, so this is everything that runs between ranks."""

from __future__ import annotations

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from gdn2_sm120_b200 import shard


def test_plan_partitions_every_unit_exactly_once():
    for batch, heads, world in ((32, 32, 8), (4, 32, 8), (5, 3, 2), (1024, 32, 8), (3, 8, 4)):
        owned = []
        for rank in range(world):
            s = shard.plan(batch, heads, world, rank)
            assert s.axis == (0 if batch >= world else 2)
            owned.append((s.start, s.stop))
        total = batch if batch >= world else heads
        assert owned[0][0] == 0 and owned[-1][1] == total
        assert all(a[1] == b[0] for a, b in zip(owned, owned[1:]))
        sizes = [b - a for a, b in owned]
        assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        shard.plan(1, 1, 2, 0)
    with pytest.raises(ValueError):
        shard.plan(4, 4, 2, 2)


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, axis_case: str):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        gen = torch.Generator().manual_seed(0)  # every rank draws the same global tensors
        batch, heads = (4, 3) if axis_case == "batch" else (1, 4)
        seq = torch.randn(batch, 5, heads, 8, generator=gen)
        state = torch.randn(batch, heads, 8, 8, generator=gen)
        plan = shard.plan(batch, heads, world, rank)
        local_seq = shard.take(seq, plan)
        local_state = shard.take(state, plan, is_state=True)
        assert local_seq.is_contiguous() and local_state.is_contiguous()
        # an operator that treats (batch, head) units independently
        local_out = local_seq * 2.0 + local_state.sum(dim=(-1, -2))[:, None, :, None]
        want = seq * 2.0 + state.sum(dim=(-1, -2))[:, None, :, None]
        gathered = shard.gather(local_out, plan, world)
        gathered_state = shard.gather(local_state, plan, world, is_state=True)
        assert torch.equal(gathered, want)
        assert torch.equal(gathered_state, state)
        slowest = shard.max_over_ranks(10.0 + rank, torch.device("cpu"))
        assert slowest == 10.0 + (world - 1)
        assert shard.sum_over_ranks(1.0, torch.device("cpu")) == float(world)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("axis_case", ["batch", "heads"])
def test_two_rank_shard_gather_and_timing_reduction(axis_case):
    port = _free_port()
    mp.spawn(_worker, args=(2, port, axis_case), nprocs=2, join=True)


def _uneven_worker(rank: int, world: int, port: int):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        seq = torch.zeros(5, 2, 3, 8)  # 5 batch rows over 2 ranks: shards of 3 and 2
        plan = shard.plan(5, 3, world, rank)
        assert plan.size == (3 if rank == 0 else 2)
        with pytest.raises(ValueError, match="equally sized shards"):
            shard.gather(shard.take(seq, plan), plan, world)
        # the group is still usable afterwards: nothing was left half-done
        assert shard.sum_over_ranks(1.0, torch.device("cpu")) == float(world)
    finally:
        dist.destroy_process_group()


def test_gather_rejects_uneven_shards_on_every_rank():
    port = _free_port()
    mp.spawn(_uneven_worker, args=(2, port), nprocs=2, join=True)


def test_reductions_without_a_process_group_are_identity():
    assert shard.max_over_ranks(3.5, torch.device("cpu")) == 3.5
    assert shard.sum_over_ranks(3.5, torch.device("cpu")) == 3.5
