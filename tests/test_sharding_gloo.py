"""The N>1 host logic (lane plans, head gather, max-over-ranks timing) on CPU with gloo, world size 2."""

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from mlx_turboquant_b200 import sharding


def test_plan_by_sequence_covers_everything_once():
    for n_seq, world in ((64, 8), (16, 3), (7, 7), (9, 2)):
        seen = []
        for r in range(world):
            p = sharding.plan_lanes(n_seq, 8, world, r)
            assert (p.head_begin, p.head_end) == (0, 8)
            seen += list(range(p.seq_begin, p.seq_end))
        assert seen == list(range(n_seq))
        sizes = [sharding.plan_lanes(n_seq, 8, world, r).n_lanes for r in range(world)]
        assert max(sizes) - min(sizes) <= 8


def test_plan_by_head_when_sequences_are_fewer_than_ranks():
    lanes = set()
    for r in range(8):
        p = sharding.plan_lanes(1, 8, 8, r)
        assert (p.seq_begin, p.seq_end) == (0, 1) and p.n_lanes == 1
        lanes.add((p.seq_begin, p.head_begin))
    assert lanes == {(0, h) for h in range(8)}
    p = sharding.plan_lanes(2, 8, 8, 5)
    assert (p.seq_begin, p.head_begin, p.head_end) == (1, 2, 4)
    with pytest.raises(ValueError):
        sharding.plan_lanes(3, 8, 8, 0)
    with pytest.raises(ValueError):
        sharding.plan_lanes(1, 6, 4, 0)
    with pytest.raises(ValueError):
        sharding.plan_lanes(4, 8, 2, 2)


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        # head-split plan of one sequence with 8 KV heads / 32 query heads: each rank attends its own heads
        plan = sharding.plan_lanes(1, 8, world, rank)
        hq_per_kv = 4
        g = torch.Generator().manual_seed(7)
        full = torch.randn(1, 32, 1, 16, generator=g)                       # what one GPU would have produced
        local = full[:, plan.head_begin * hq_per_kv:plan.head_end * hq_per_kv]
        gathered = sharding.gather_heads(local)
        t = sharding.job_time_ms(10.0 + 5.0 * rank)
        ret[rank] = (bool(torch.equal(gathered, full)), t, plan.n_lanes)
    finally:
        dist.destroy_process_group()


def test_world_size_two_gloo():
    world, port = 2, _free_port()
    ctx = mp.get_context("spawn")
    ret = ctx.Manager().dict()
    procs = [ctx.Process(target=_worker, args=(r, world, port, ret)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    assert ret[0] == (True, 15.0, 4) and ret[1] == (True, 15.0, 4)


def test_job_time_without_process_group():
    assert sharding.job_time_ms(3.5) == 3.5
