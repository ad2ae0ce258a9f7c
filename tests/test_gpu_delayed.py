"""Delayed-scaling state update on the GPU against the oracle restatement (bit-exact), and
a multi-step cast sequence through DelayedScaling against the oracle's loop."""

import pytest
import torch

import oracle
from conftest import as_u8
from transformer_nuggets_b200 import _lib
from transformer_nuggets_b200.fp8 import DelayedScaling

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _update(hist, amax, dtype):
    scale = torch.empty(hist.shape[0], dtype=torch.float32, device=DEV)
    _lib.call("tnq_delayed_scale_update", hist.data_ptr(), amax.data_ptr(), scale.data_ptr(), hist.shape[0],
              hist.shape[1], _lib.FP8_DTYPES[dtype], _lib.stream_ptr(hist.device))
    torch.cuda.synchronize()
    return scale


@pytest.mark.parametrize("tensors,length", [(1, 1), (5, 16), (257, 33), (3, 1024), (64, 2)])
@pytest.mark.parametrize("dtype", [torch.float8_e4m3fn, torch.float8_e5m2])
def test_update_matches_oracle(tensors, length, dtype):
    g = torch.Generator().manual_seed(tensors * 1000 + length)
    hist = (torch.rand(tensors, length, generator=g) * 2 ** (torch.rand(tensors, 1, generator=g) * 40 - 20)).float()
    amax = torch.rand(tensors, generator=g).float() * 3
    hist[0, -1] = 1e30  # the oldest entry must drop out of the maximum
    if tensors > 2:
        hist[1] = 0.0
        amax[1] = 0.0  # all-zero history: scale = max / 1e-12
        hist[2, 0] = float("nan")
    want_hist, want_scale = oracle.delayed_scale_update(hist, amax, dtype)
    d_hist, d_amax = hist.to(DEV), amax.to(DEV)
    scale = _update(d_hist, d_amax, dtype)
    assert torch.equal(d_hist.cpu().view(torch.int32), want_hist.view(torch.int32))
    got = scale.cpu()
    nan = torch.isnan(want_scale)  # a NaN's payload bits are not part of the contract
    assert torch.equal(torch.isnan(got), nan)
    assert torch.equal(got[~nan].view(torch.int32), want_scale[~nan].view(torch.int32))
    assert torch.count_nonzero(d_amax).item() == 0


def test_update_rejects_bad_arguments():
    hist = torch.zeros(2, 2048, device=DEV)
    amax = torch.zeros(2, device=DEV)
    with pytest.raises(_lib.TnqError):
        _update(hist, amax, torch.float8_e4m3fn)


@pytest.mark.parametrize("dtype", [torch.float8_e4m3fn, torch.float8_e5m2])
def test_multi_step_sequence_matches_oracle_loop(dtype):
    g = torch.Generator().manual_seed(5)
    state = DelayedScaling(2, history_len=3, fp8_dtype=dtype, device=DEV)
    o_hist = torch.zeros(2, 3)
    o_scale = torch.ones(2)
    for step in range(6):
        xs = [(torch.randn(256, 512, generator=g) * (4.0 ** ((step * 7 + t) % 5 - 2))).to(torch.bfloat16) for t in range(2)]
        o_amax = torch.zeros(2)
        for t, x in enumerate(xs):
            q = state.cast(t, x.to(DEV), saturated=True)
            am = torch.zeros(1)
            want = oracle.fp8_scaled_quant(x, o_scale[t:t + 1].clone(), am, dtype, saturated=True)
            o_amax[t] = am[0]
            assert torch.equal(as_u8(q).cpu(), as_u8(want)), f"step {step} tensor {t}"
        assert torch.equal(state.amax.cpu(), o_amax)
        state.sync()
        o_hist, o_scale = oracle.delayed_scale_update(o_hist, o_amax, dtype)
        assert torch.equal(state.amax_history.cpu(), o_hist)
        assert torch.equal(state.scale.cpu().view(torch.int32), o_scale.view(torch.int32))
