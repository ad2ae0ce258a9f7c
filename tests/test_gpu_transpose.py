"""Cast + transpose from one read: both outputs bit-exact against the oracle's cast (and its
transpose), including ragged shapes, NaN / inf / overflow corner cases and the abs_max side
output."""

import pytest
import torch

import oracle
from conftest import as_u8
from transformer_nuggets_b200.fp8 import dynamic_scaled_quant_transpose, scaled_quant, scaled_quant_transpose

pytestmark = pytest.mark.gpu
DEV = "cuda"
SHAPES = [(128, 128), (256, 384), (2048, 1024), (100, 72), (130, 136), (33, 8), (4096, 264), (96, 128), (1, 8), (31, 4096)]


def _data(rows, cols, seed, special=True):
    g = torch.Generator().manual_seed(seed)
    x = (torch.randn(rows, cols, generator=g) * 3.0).to(torch.bfloat16)
    if special and rows * cols >= 64:
        flat = x.view(-1)
        flat[5] = 1000.0      # overflows e4m3 at scale 2 without saturation
        flat[11] = -1e6
        flat[17] = float("inf")
        flat[23] = float("-inf")
        flat[29] = float("nan")
        flat[-1] = -float("nan")
    return x


@pytest.mark.parametrize("rows,cols", SHAPES)
@pytest.mark.parametrize("dtype", [torch.float8_e4m3fn, torch.float8_e5m2])
@pytest.mark.parametrize("saturated", [True, False])
def test_scaled_quant_transpose_matches_oracle(rows, cols, dtype, saturated):
    x = _data(rows, cols, rows * 131 + cols)
    scale = torch.tensor([2.0])
    want_am = torch.zeros(1)
    want = oracle.fp8_scaled_quant(x, scale, want_am, dtype, saturated)
    am = torch.tensor([0.5], device=DEV)
    q, q_t = scaled_quant_transpose(x.to(DEV), scale.to(DEV), am, dtype, saturated)
    assert q.shape == (rows, cols) and q_t.shape == (cols, rows)
    assert torch.equal(as_u8(q).cpu(), as_u8(want))
    assert torch.equal(as_u8(q_t).cpu(), as_u8(want).t().contiguous())
    got_am = am.cpu()
    if torch.isnan(want_am).any():
        assert torch.isnan(got_am).all()
    else:
        assert torch.equal(got_am, torch.maximum(want_am, torch.tensor([0.5])))


@pytest.mark.parametrize("rows,cols", [(256, 384), (130, 136), (2048, 1024)])
def test_transposing_cast_agrees_with_plain_cast(rows, cols):
    x = _data(rows, cols, 9, special=False).to(DEV)
    scale = torch.tensor([0.37], device=DEV)
    am1, am2 = torch.zeros(1, device=DEV), torch.zeros(1, device=DEV)
    plain = scaled_quant(x, scale, am1, torch.float8_e4m3fn, True)
    q, q_t = scaled_quant_transpose(x, scale, am2, torch.float8_e4m3fn, True)
    assert torch.equal(as_u8(q), as_u8(plain)) and torch.equal(as_u8(q_t), as_u8(plain).t().contiguous())
    assert torch.equal(am1, am2)


@pytest.mark.parametrize("rows,cols", [(128, 128), (1000, 520), (4096, 4096)])
@pytest.mark.parametrize("dtype", [torch.float8_e4m3fn, torch.float8_e5m2])
def test_dynamic_transpose_matches_oracle(rows, cols, dtype):
    x = _data(rows, cols, 77, special=False)
    x[rows // 2, cols // 3] = 250.0
    want, want_scale = oracle.fp8_dynamic_quant(x, dtype)
    q, q_t, scale = dynamic_scaled_quant_transpose(x.to(DEV), dtype)
    assert torch.equal(scale.cpu(), want_scale)
    assert torch.equal(as_u8(q).cpu(), as_u8(want))
    assert torch.equal(as_u8(q_t).cpu(), as_u8(want).t().contiguous())


def test_argument_checks():
    x = torch.zeros(4, 12, dtype=torch.bfloat16, device=DEV)
    s = torch.ones(1, device=DEV)
    with pytest.raises(ValueError):
        scaled_quant_transpose(x, s)  # 12 columns
    with pytest.raises(TypeError):
        scaled_quant_transpose(torch.zeros(4, 8, device=DEV), s)  # fp32 input
    with pytest.raises(ValueError):
        scaled_quant_transpose(torch.zeros(2, 4, 8, dtype=torch.bfloat16, device=DEV), s)
    q, q_t = scaled_quant_transpose(torch.zeros(0, 8, dtype=torch.bfloat16, device=DEV), s)
    assert q.shape == (0, 8) and q_t.shape == (8, 0)


@pytest.mark.parametrize("start", [float("nan"), -1.0, 0.0, 1.0e9])
def test_abs_max_history_word_same_rule_in_both_casts(start):
    """abs_max becomes max(abs_max, max|x|) on the bit patterns in the plain and in the transposing
    cast alike: a NaN already stored stays, a negative starting value (-1.0, as the reference's
    tests use) loses, a larger previous value is kept."""
    x = _data(256, 384, 11, special=False).to(DEV)
    scale = torch.tensor([0.5], device=DEV)
    am1 = torch.tensor([start], device=DEV)
    am2 = torch.tensor([start], device=DEV)
    scaled_quant(x, scale, am1, torch.float8_e4m3fn, True)
    scaled_quant_transpose(x, scale, am2, torch.float8_e4m3fn, True)
    true_amax = x.abs().max().float().item()
    if start != start:
        assert torch.isnan(am1).item() and torch.isnan(am2).item()
    else:
        assert am1.item() == am2.item() == max(start, true_amax)
    z = torch.zeros(128, 128, dtype=torch.bfloat16, device=DEV)  # all-zero tensor from -1.0: both report 0
    am1, am2 = torch.tensor([-1.0], device=DEV), torch.tensor([-1.0], device=DEV)
    scaled_quant(z, scale, am1, torch.float8_e4m3fn, True)
    scaled_quant_transpose(z, scale, am2, torch.float8_e4m3fn, True)
    assert am1.item() == 0.0 and am2.item() == 0.0
