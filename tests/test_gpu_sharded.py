"""Row-sharded per-tensor cast: the shards together equal the single-device result
bit for bit.  On one GPU the ranks are emulated one after another through the same
C-ABI calls; with two or more GPUs a real NCCL group of child processes runs too."""

import os
import socket

import pytest
import torch

import oracle
import transformer_nuggets_b200 as tn
from conftest import as_u8
from transformer_nuggets_b200 import _lib
from transformer_nuggets_b200.dist.sharded import plan_row_shards, sharded_dynamic_scaled_quant
from transformer_nuggets_b200.workloads import make_input

pytestmark = pytest.mark.gpu
DEV = "cuda"


def emulate_ranks(x, world):
    """local amax per shard -> MAX on the host side of the test -> cast per shard."""
    plan = plan_row_shards(x.shape[0], world)
    ws = _lib.workspace(x.device)
    stream = _lib.stream_ptr(x.device)
    amaxes = []
    for s, e in plan:
        a = torch.zeros(1, dtype=torch.float32, device=DEV)
        sh = x[s:e]
        _lib.call("tnq_fp8_amax", sh.data_ptr(), sh.numel(), _lib.IN_BF16, _lib.FP8_E4M3, ws.data_ptr(), a.data_ptr(), stream)
        amaxes.append(a)
    g = torch.stack(amaxes).max().reshape(1).contiguous()
    outs = []
    for s, e in plan:
        sh = x[s:e]
        o = torch.empty_like(sh, dtype=torch.float8_e4m3fn)
        _lib.call("tnq_fp8_scaled_cast", sh.data_ptr(), o.data_ptr(), sh.numel(), _lib.IN_BF16, _lib.FP8_E4M3,
                  g.data_ptr(), _lib.SCALE_IS_AMAX, 1, 0, 0, stream)
        outs.append(o)
    return torch.cat(outs), g


@pytest.mark.parametrize("world", [1, 2, 4, 8])
def test_emulated_shards_equal_unsharded_small(world):
    x = make_input("fp8_sharded", "cpu", rows=2048, cols=1024)
    want, wscale = oracle.fp8_dynamic_quant(x, torch.float8_e4m3fn)
    got, amax = emulate_ranks(x.to(DEV), world)
    assert torch.equal(torch.tensor(448.0) / amax.cpu(), wscale)
    assert torch.equal(as_u8(got).cpu(), as_u8(want))


def test_config_sharded_full_size():
    """131072 x 8192 (2 GiB): 8 emulated shards == one device, bit for bit; the scale equals
    448 / amax; every byte of the result against the oracle (4096-row chunks, fed the scale)."""
    x = make_input("fp8_sharded", DEV)
    full, scale = tn.dynamic_scaled_quant_with_scale(x)
    got, amax = emulate_ranks(x, 8)
    assert torch.equal(as_u8(got), as_u8(full))
    del got
    assert amax.item() == x.abs().max().float().item()
    assert torch.equal(scale.cpu(), torch.tensor([448.0]) / amax.cpu())
    one, amax1 = sharded_dynamic_scaled_quant(x)  # world size 1 through the product entry point
    assert torch.equal(as_u8(one), as_u8(full)) and torch.equal(amax1, amax)
    del one
    sc = scale.cpu()
    for r0 in range(0, x.shape[0], 4096):
        want = oracle.fp8_scaled_quant(x[r0:r0 + 4096].cpu(), sc, torch.zeros(1), torch.float8_e4m3fn, True)
        assert torch.equal(as_u8(full[r0:r0 + 4096]).cpu(), as_u8(want)), r0


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _nccl_rank(rank, world, port, results):
    import torch.distributed as dist

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        x = make_input("fp8_sharded", "cpu", rows=4096, cols=1024)
        want, wscale = oracle.fp8_dynamic_quant(x, torch.float8_e4m3fn)
        s, e = plan_row_shards(x.shape[0], world)[rank]
        ok = True
        for exch in ("nccl", "peer"):
            exchange = None
            if exch == "peer":
                from transformer_nuggets_b200.dist.exchange import PeerAmaxExchange

                exchange = PeerAmaxExchange(None)
            for _ in range(3):  # repeated calls reuse the exchange slots
                q, amax = sharded_dynamic_scaled_quant(x[s:e].cuda(), None, exchange=exchange)
                torch.cuda.synchronize()
                ok = ok and torch.equal(torch.tensor(448.0) / amax.cpu(), wscale)
                ok = ok and torch.equal(as_u8(q).cpu(), as_u8(want[s:e]))
            # NVFP4 with the tensor-wide scale: each rank's rows equal the same rows of the unsharded result
            from transformer_nuggets_b200.dist.sharded import sharded_quantize_nvfp4

            wp, wsf, wg = oracle.nvfp4_quantize(x)
            got = sharded_quantize_nvfp4(x[s:e].cuda(), None, exchange=exchange, swizzle=False)
            torch.cuda.synchronize()
            ok = ok and torch.equal(got.global_scale.cpu(), wg)
            ok = ok and torch.equal(got.packed.view(torch.uint8).cpu(), wp[s:e])
            ok = ok and torch.equal(as_u8(got.block_scales).cpu(), as_u8(wsf[s:e]))
            if exchange is not None:
                ok = ok and exchange.status() == 0
                exchange.close()
        # delayed scaling, data parallel: every rank casts its rows with the shared scale, sync()
        # MAX-reduces the amax words over the group, so all ranks derive the same next scale
        from transformer_nuggets_b200.fp8 import DelayedScaling

        state = DelayedScaling(1, history_len=4, device=torch.device("cuda", rank))
        o_hist, o_scale = torch.zeros(1, 4), torch.ones(1)
        for step in range(3):
            xs = (x * (0.5 + step)).to(torch.bfloat16)
            q = state.cast(0, xs[s:e].cuda(), saturated=True)
            am = torch.zeros(1)
            want_q = oracle.fp8_scaled_quant(xs, o_scale.clone(), am, torch.float8_e4m3fn, True)
            ok = ok and torch.equal(as_u8(q).cpu(), as_u8(want_q[s:e]))
            state.sync(None)
            o_hist, o_scale = oracle.delayed_scale_update(o_hist, am, torch.float8_e4m3fn)
            ok = ok and torch.equal(state.scale.cpu(), o_scale) and torch.equal(state.amax_history.cpu(), o_hist)
        results[rank] = 1 if ok else 0
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_nccl_and_peer_exchange_ranks():
    import torch.multiprocessing as mp

    world = min(torch.cuda.device_count(), 8)
    results = mp.get_context("spawn").Manager().dict()
    mp.spawn(_nccl_rank, args=(world, _free_port(), results), nprocs=world, join=True)
    assert dict(results) == {r: 1 for r in range(world)}


def test_exchange_wait_runs_out_and_reports():
    """A peer that never publishes its amax: the cast kernel's bounded wait (about one
    second) expires, the status word reports it and the context stays usable.  The
    missing peer is a slot that nothing writes - no fault, no endless loop."""
    import ctypes

    local = ctypes.c_void_p()
    handle = (ctypes.c_ubyte * 64)()
    _lib.call("tnq_exchange_create", ctypes.byref(local), handle)
    try:
        ptrs = (ctypes.c_void_p * 2)(local.value, local.value)  # "rank 1" never stores anything
        x = make_input("fp8_sharded", DEV, rows=256, cols=1024)
        out = torch.empty_like(x, dtype=torch.float8_e4m3fn)
        amax = torch.zeros(1, dtype=torch.float32, device=DEV)
        ws = _lib.workspace(x.device)
        _lib.call("tnq_fp8_sharded_cast", x.data_ptr(), out.data_ptr(), x.numel(), _lib.IN_BF16, _lib.FP8_E4M3,
                  ws.data_ptr(), ptrs, 2, 0, 1, amax.data_ptr(), _lib.stream_ptr(x.device))
        torch.cuda.synchronize()
        status = ctypes.c_uint32(0)
        _lib.call("tnq_exchange_status", local, ctypes.byref(status))
        assert status.value == 6  # TNQ_ETIMEOUT
        # the device is fine afterwards
        q, s = tn.dynamic_scaled_quant_with_scale(x)
        want, ws_ = oracle.fp8_dynamic_quant(x.cpu(), torch.float8_e4m3fn)
        assert torch.equal(as_u8(q).cpu(), as_u8(want)) and torch.equal(s.cpu(), ws_)
    finally:
        torch.cuda.synchronize()
        _lib.call("tnq_exchange_destroy", local)


def test_single_rank_exchange_through_c_abi():
    """world_size 1 through the peer-exchange entry point equals the plain dynamic cast."""
    import ctypes

    local = ctypes.c_void_p()
    handle = (ctypes.c_ubyte * 64)()
    _lib.call("tnq_exchange_create", ctypes.byref(local), handle)
    try:
        ptrs = (ctypes.c_void_p * 1)(local.value)
        x = make_input("fp8_sharded", DEV, rows=1024, cols=2048)
        ref = tn.dynamic_scaled_quant(x)
        ws = _lib.workspace(x.device)
        for seq in (1, 2, 3, 4):
            out = torch.empty_like(x, dtype=torch.float8_e4m3fn)
            amax = torch.zeros(1, dtype=torch.float32, device=DEV)
            _lib.call("tnq_fp8_sharded_cast", x.data_ptr(), out.data_ptr(), x.numel(), _lib.IN_BF16, _lib.FP8_E4M3,
                      ws.data_ptr(), ptrs, 1, 0, seq, amax.data_ptr(), _lib.stream_ptr(x.device))
            torch.cuda.synchronize()
            assert torch.equal(as_u8(out), as_u8(ref)) and amax.item() == x.abs().max().float().item()
        amax = torch.zeros(1, dtype=torch.float32, device=DEV)
        _lib.call("tnq_sharded_amax", x.data_ptr(), x.numel(), _lib.IN_BF16, ws.data_ptr(), ptrs, 1, 0, 5,
                  amax.data_ptr(), _lib.stream_ptr(x.device))
        torch.cuda.synchronize()
        assert amax.item() == x.abs().max().float().item()
        status = ctypes.c_uint32(9)
        _lib.call("tnq_exchange_status", local, ctypes.byref(status))
        assert status.value == 0
    finally:
        _lib.call("tnq_exchange_destroy", local)


def test_host_pipeline_matches_device_path():
    from transformer_nuggets_b200.dist.host_pipeline import HostCastPipeline

    x = make_input("fp8_sharded", "cpu", rows=2048, cols=1024)
    want, _ = oracle.fp8_dynamic_quant(x, torch.float8_e4m3fn)
    hin = x.pin_memory()
    houts = [torch.empty(x.shape, dtype=torch.uint8).pin_memory() for _ in range(5)]
    pipe = HostCastPipeline(x.shape, x.dtype, torch.float8_e4m3fn, torch.device(DEV, 0))
    for h in houts:
        pipe.submit(hin, h)
    pipe.synchronize()
    for h in houts:
        assert torch.equal(h, as_u8(want))
