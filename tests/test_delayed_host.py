"""Host-side logic of the delayed-scaling state on CPU: the oracle's update rule on known
answers, the per-tensor amax MAX-reduction over a world_size-2 gloo group, and the refusal
to build the state on a CPU device."""

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle
from transformer_nuggets_b200.fp8.delayed_scaling import DelayedScaling, combine_amaxes


def test_oracle_update_known_answers():
    hist = torch.tensor([[4.0, 2.0, 8.0], [0.0, 0.0, 0.0], [1.0, float("nan"), 3.0]])
    amax = torch.tensor([1.0, 0.0, 7.0])
    new, scale = oracle.delayed_scale_update(hist, amax, torch.float8_e4m3fn)
    assert new[0].tolist() == [1.0, 4.0, 2.0]  # the 8.0 was the oldest entry and is gone
    assert scale[0].item() == 448.0 / 4.0
    assert new[1].tolist() == [0.0, 0.0, 0.0] and scale[1].item() == torch.tensor(448.0) / torch.tensor(1e-12)
    assert new[2][0].item() == 7.0 and torch.isnan(new[2][2]) and torch.isnan(scale[2])
    _, scale52 = oracle.delayed_scale_update(hist[:1], amax[:1], torch.float8_e5m2)
    assert scale52[0].item() == 57344.0 / 4.0


def test_state_needs_a_cuda_device():
    with pytest.raises(ValueError):
        DelayedScaling(2, device="cpu")
    with pytest.raises(ValueError):
        DelayedScaling(1, history_len=2048, device="cuda")


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _entry(rank, world, port, results):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        amax = torch.tensor([1.0 + rank, 5.0 - 3 * rank, 0.0])
        combine_amaxes(amax, None)
        results[rank] = amax.tolist()
    finally:
        dist.destroy_process_group()


def test_gloo_two_ranks_agree_on_amaxes():
    world = 2
    port = _free_port()
    results = mp.get_context("spawn").Manager().dict()
    mp.spawn(_entry, args=(world, port, results), nprocs=world, join=True)
    assert dict(results) == {0: [2.0, 5.0, 0.0], 1: [2.0, 5.0, 0.0]}
