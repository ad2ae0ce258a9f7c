"""Host-side logic of the row-sharded cast on CPU: the shard plan, and the amax
combination over a world_size-2 gloo group checked against the unsharded oracle."""

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle
from conftest import as_u8
from transformer_nuggets_b200.dist.sharded import combine_amax, combine_amax_bounded, plan_row_shards


@pytest.mark.parametrize("rows,world", [(131072, 8), (131072, 1), (1000, 4), (128, 8), (0, 2), (129, 2)])
def test_plan_row_shards(rows, world):
    plan = plan_row_shards(rows, world)
    assert len(plan) == world
    assert plan[0][0] == 0 and plan[-1][1] == rows
    for (a0, a1), (b0, b1) in zip(plan, plan[1:]):
        assert a1 == b0 and a0 <= a1
    for s, e in plan:
        assert s % 128 == 0
    sizes = [e - s for s, e in plan]
    assert max(sizes) - min(sizes) <= 128 or rows < 128 * world


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank, world, port):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        g = torch.Generator().manual_seed(77)
        x = torch.randn(512, 96, generator=g).to(torch.bfloat16)
        x[300] *= 1000.0  # the outlier row lives on the last rank only
        s, e = plan_row_shards(x.shape[0], world)[rank]
        local = x[s:e]
        amax = local.abs().max().float().reshape(1)
        combine_amax(amax, None)
        full_q, full_scale = oracle.fp8_dynamic_quant(x, torch.float8_e4m3fn)
        scale = (torch.tensor(448.0) / torch.clamp(amax, min=1e-12)).reshape(1)
        dummy = torch.zeros(1)
        q = oracle.fp8_scaled_quant(local, scale, dummy, torch.float8_e4m3fn, True)
        ok = torch.equal(scale, full_scale) and torch.equal(as_u8(q), as_u8(full_q[s:e]))
        q_ok = bool(ok)
    finally:
        dist.destroy_process_group()
    return q_ok


def _entry(rank, world, port, results):
    ok = _rank_main(rank, world, port)
    results[rank] = 1 if ok else 0


def test_gloo_two_ranks_match_unsharded_oracle():
    world = 2
    port = _free_port()
    results = mp.get_context("spawn").Manager().dict()
    mp.spawn(_entry, args=(world, port, results), nprocs=world, join=True)
    assert dict(results) == {0: 1, 1: 1}


def _late_entry(rank, world, port, results):
    import time

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    # phase 1: the last rank is one second late; the bounded combine still completes
    amax = torch.tensor([float(rank + 1)])
    if rank == world - 1:
        time.sleep(1.0)
    ok1 = combine_amax_bounded(amax, None, timeout_s=30.0)
    results[("late", rank)] = (ok1, amax.item())
    # phase 2: the last rank withholds its contribution; the others give up and report it
    if rank == world - 1:
        time.sleep(6.0)
    else:
        t0 = time.time()
        ok2 = combine_amax_bounded(torch.tensor([1.0]), None, timeout_s=2.0)
        results[("withheld", rank)] = (ok2, time.time() - t0 < 5.5)
    os._exit(0)  # the group is broken on purpose: leave without a collective shutdown


@pytest.mark.timeout(180)
@pytest.mark.parametrize("world", [2, 3])
def test_gloo_late_and_withheld_rank(world):
    port = _free_port()
    results = mp.get_context("spawn").Manager().dict()
    mp.spawn(_late_entry, args=(world, port, results), nprocs=world, join=True)
    got = dict(results)
    for r in range(world):
        assert got[("late", r)] == (True, float(world))
    for r in range(world - 1):
        assert got[("withheld", r)] == (False, True)
