"""Argument validation before any launch, and run-twice determinism of every op
(the only atomics anywhere are MAX reductions, which are order independent)."""

import pytest
import torch

import transformer_nuggets_b200 as tn
from conftest import as_u8
from transformer_nuggets_b200.cute.mxfp8_tma import mxfp8_tma_gemv
from transformer_nuggets_b200.cute.nvfp4_tma import nvfp4_tma_gemv
from transformer_nuggets_b200.cute.blockscaled_tma import BlockScaleLayout
from transformer_nuggets_b200.fp8 import (dynamic_scaled_quant, rowwise_scaled_quant, scaled_quant,
                                          scaled_quant_transpose)
from transformer_nuggets_b200.mx.to_blocked import to_blocked

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _x(rows=64, cols=256, dtype=torch.bfloat16):
    return torch.randn(rows, cols, device=DEV).to(dtype)


def test_fp8_casts_reject_bad_arguments():
    one = torch.ones(1, device=DEV)
    with pytest.raises(AssertionError):
        scaled_quant(_x().t(), one, one.clone())  # not contiguous
    with pytest.raises(AssertionError):
        dynamic_scaled_quant(_x().t())
    with pytest.raises(TypeError):
        scaled_quant(_x(dtype=torch.float16), one, one.clone())
    with pytest.raises(TypeError):
        scaled_quant(_x(), one, one.clone(), fp8_dtype=torch.int8)
    with pytest.raises(ValueError):
        dynamic_scaled_quant(_x().view(-1)[1:257])  # starts two bytes past a 32-byte boundary
    with pytest.raises(AssertionError):
        scaled_quant(_x(), torch.ones(2, device=DEV), one.clone())  # scale of two elements
    with pytest.raises(AssertionError):
        scaled_quant(_x(), one.double(), one.clone())
    with pytest.raises(AssertionError):
        scaled_quant(_x(), one, torch.ones(3, device=DEV))
    with pytest.raises(ValueError):
        rowwise_scaled_quant(_x().view(-1))  # 1-D
    with pytest.raises(ValueError):
        rowwise_scaled_quant(_x(), (torch.float8_e4m3fn, torch.float8_e4m3fn))


def test_block_scaled_quantizers_reject_bad_arguments():
    with pytest.raises(TypeError):
        tn.quantize_mxfp8(_x(dtype=torch.float32))
    with pytest.raises(ValueError):
        tn.quantize_mxfp8(_x(64, 48))  # 48 is not a multiple of 32
    with pytest.raises(ValueError):
        tn.quantize_mxfp8(_x(48, 64), columnwise=True)  # 48 rows for column-wise blocks
    with pytest.raises(ValueError):
        tn.quantize_mxfp8(_x(), scale_mode="nearest")
    with pytest.raises(ValueError):
        tn.quantize_mxfp8(_x().t())
    with pytest.raises(ValueError):
        tn.quantize_mxfp8_tensor(_x(64, 40))
    with pytest.raises(TypeError):
        tn.quantize_nvfp4(_x(dtype=torch.float32))
    with pytest.raises(ValueError):
        tn.quantize_nvfp4(_x(64, 40))  # 40 is not a multiple of 16
    with pytest.raises(ValueError):
        tn.quantize_nvfp4(_x().t())
    with pytest.raises(TypeError):
        to_blocked(torch.zeros(128, 4, dtype=torch.int32, device=DEV))
    with pytest.raises(ValueError):
        to_blocked(torch.zeros(128, dtype=torch.uint8, device=DEV))


def test_every_op_is_deterministic():
    g = torch.Generator(device=DEV).manual_seed(3)
    x = torch.randn(512, 1024, device=DEV, generator=g).to(torch.bfloat16)

    def snapshot():
        out = []
        out.append(as_u8(dynamic_scaled_quant(x)))
        (q43, s43), (q52, s52) = rowwise_scaled_quant(x)
        out += [as_u8(q43), as_u8(q52), s43, s52]
        r = tn.quantize_mxfp8(x, columnwise=True, swizzle=True)
        out += [as_u8(r.q_row), as_u8(r.q_col), as_u8(r.scale_row), as_u8(r.scale_col)]
        a = tn.quantize_nvfp4(x)
        out += [as_u8(a.packed), as_u8(a.block_scales), a.global_scale]
        q, q_t = scaled_quant_transpose(x, torch.full((1,), 1.5, device=DEV), None, torch.float8_e5m2, True)
        out += [as_u8(q), as_u8(q_t)]
        xr = tn.quantize_mxfp8(x[:1].contiguous(), swizzle=True)
        out.append(mxfp8_tma_gemv(xr.q_row, r.q_row, xr.scale_row, r.scale_row, block_scale_layout=BlockScaleLayout.SWIZZLE_32_4_4))
        ax = tn.quantize_nvfp4(x[:1].contiguous())
        out.append(nvfp4_tma_gemv(ax.packed, a.packed, ax.block_scales, a.block_scales,
                                  input_global_scale=ax.global_scale, weight_global_scale=a.global_scale,
                                  block_scale_layout=BlockScaleLayout.SWIZZLE_32_4_4))
        return [t.clone() for t in out]

    first, second = snapshot(), snapshot()
    assert len(first) == len(second)
    for a, b in zip(first, second):
        assert torch.equal(a.contiguous().view(torch.uint8), b.contiguous().view(torch.uint8))


def test_check_status_reports_and_repairs_the_workspace():
    """What a kernel leaves behind when a bounded wait expires (status word set, a grid-barrier
    counter not rewound) is written into the workspace from the host here - no wait is made to
    expire.  check_status turns it into TnqError(ETIMEOUT), zeroes the header, and the single-launch
    cast that uses those barrier words is bit-exact again afterwards."""
    import oracle
    from transformer_nuggets_b200 import _lib
    from transformer_nuggets_b200.workloads import make_input

    x = make_input("fp8_tensor", DEV, rows=512, cols=512)
    want, want_scale = oracle.fp8_dynamic_quant(x.cpu(), torch.float8_e4m3fn)
    q, s = tn.dynamic_scaled_quant_with_scale(x)
    _lib.check_status(x.device)  # clean
    ws = _lib.workspace(x.device)
    ws[_lib.WS_STATUS_WORD] = 6
    ws[6] = 3  # arrival counters of the grid-wide exchange as an abandoned call would leave them
    ws[8] = 3
    with pytest.raises(_lib.TnqError) as e:
        _lib.check_status(x.device, what="tnq_fp8_dynamic_cast")
    assert e.value.status == 6
    assert int(ws[:16].abs().sum().item()) == 0
    q, s = tn.dynamic_scaled_quant_with_scale(x)
    _lib.check_status(x.device)
    assert torch.equal(q.view(torch.uint8).cpu(), want.view(torch.uint8)) and torch.equal(s.cpu(), want_scale)
