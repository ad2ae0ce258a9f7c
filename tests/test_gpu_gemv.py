"""Block-scaled M = 1 GEMV (the consumer of the quantizers' outputs) against the
dequantised fp32 matmul, with the tolerances and cases of the reference's own GEMV tests
(test/test_mxfp8_tma.py:113-203, 351-417; test/test_nvfp4_tma.py:186-224, 376-397,
511-548).  Floating point: atol 1.0 / rtol 0.05 for MXFP8 and atol 2.0 / rtol 0.05 for
NVFP4, as there; raw-versus-swizzled scale storage must agree exactly."""

import pytest
import torch

import oracle
import transformer_nuggets_b200 as tn
from transformer_nuggets_b200.cute.blockscaled_tma import BlockScaleLayout
from transformer_nuggets_b200.cute.mxfp8_tma import mxfp8_tma_gemv, mxfp8_tma_scaled_mm
from transformer_nuggets_b200.cute.nvfp4_tma import nvfp4_tma_gemv, nvfp4_tma_scaled_mm

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _quant(shape, seed):
    torch.manual_seed(seed)
    x = torch.randn(shape, dtype=torch.bfloat16, device=DEV)
    q, s = tn.quantize_mxfp8_tensor(x)
    return x, q, s


@pytest.mark.parametrize("n,k", [(128, 2048), (128, 4096), (264, 2048), (8, 512), (1, 32), (130, 2080), (512, 8192)])
def test_mxfp8_gemv_matches_dequantised_matmul(n, k):
    _, qx, sx = _quant((1, k), k)
    _, qw, sw = _quant((n, k), k + n)
    expected = oracle.mxfp8_gemv(qx.cpu(), qw.cpu(), sx.cpu(), sw.cpu())
    out = torch.empty(1, n, dtype=torch.bfloat16, device=DEV)
    actual = mxfp8_tma_gemv(qx, qw, sx, sw, block_n=4, num_stages=2, output=out, num_compute_warps=2)
    assert actual is out
    torch.testing.assert_close(actual.cpu(), expected, atol=1.0, rtol=0.05)
    # blocked scale storage across 128-row atoms gives the same bits
    sw_x, sw_w = tn.to_blocked(sx), tn.to_blocked(sw)
    blocked = mxfp8_tma_gemv(qx, qw, sw_x, sw_w, block_scale_layout=BlockScaleLayout.SWIZZLE_32_4_4)
    assert torch.equal(blocked, actual)


def test_mxfp8_gemv_e8m0_extremes():
    """Scale bytes 254 and 0 cancel exactly; 0xFF poisons the output with NaN
    (test/test_mxfp8_tma.py:351-417)."""
    n, k = 128, 2048
    qx = torch.ones(1, k, device=DEV).to(torch.float8_e4m3fn)
    qw = torch.ones(n, k, device=DEV).to(torch.float8_e4m3fn)
    sx = torch.full((1, k // 32), 254, dtype=torch.uint8, device=DEV)
    sw = torch.zeros(n, k // 32, dtype=torch.uint8, device=DEV)
    out = mxfp8_tma_gemv(qx, qw, sx, sw)
    assert torch.equal(out.float(), torch.full((1, n), float(k), device=DEV))
    sw[5, 3] = 255
    out = mxfp8_tma_gemv(qx, qw, sx, sw)
    assert torch.isnan(out[0, 5]).item() and int(torch.isnan(out).sum()) == 1


def test_mxfp8_scaled_mm_adapter_matches_library_gemm():
    from torch.nn.functional import ScalingType, SwizzleType, scaled_mm

    n, k = 128, 2048
    _, qx, sx = _quant((1, k), 1)
    _, qw, sw = _quant((n, k), 2)
    bx, bw = tn.to_blocked(sx).view(torch.float8_e8m0fnu), tn.to_blocked(sw).view(torch.float8_e8m0fnu)
    actual = mxfp8_tma_scaled_mm(qx, qw.t(), bx, bw, block_n=8, num_compute_warps=4)
    expected = scaled_mm(qx, qw.t(), scale_a=[bx], scale_recipe_a=[ScalingType.BlockWise1x32],
                         swizzle_a=[SwizzleType.SWIZZLE_32_4_4], scale_b=[bw], scale_recipe_b=[ScalingType.BlockWise1x32],
                         swizzle_b=[SwizzleType.SWIZZLE_32_4_4], output_dtype=torch.bfloat16)
    torch.testing.assert_close(actual, expected, atol=1.0, rtol=0.05)


def _nvfp4_case(n, k, seed):
    """Random codes and block scales, as the reference's test inputs (cute/nvfp4_tma.py:967-993)."""
    g = torch.Generator(device=DEV).manual_seed(seed)
    cx = torch.randint(0, 16, (1, k), device=DEV, dtype=torch.uint8, generator=g)
    cw = torch.randint(0, 16, (n, k), device=DEV, dtype=torch.uint8, generator=g)
    choices = torch.tensor([0.5, 1.0, 2.0, 3.0], device=DEV)
    sx = choices[torch.randint(0, 4, (1, k // 16), device=DEV, generator=g)].to(torch.float8_e4m3fn)
    sw = choices[torch.randint(0, 4, (n, k // 16), device=DEV, generator=g)].to(torch.float8_e4m3fn)
    return tn.pack_nvfp4_codes(cx), tn.pack_nvfp4_codes(cw), sx, sw


@pytest.mark.parametrize("n,k", [(128, 2048), (264, 4096), (4, 32), (130, 2080), (256, 16384)])
@pytest.mark.parametrize("with_global", [False, True])
def test_nvfp4_gemv_matches_dequantised_matmul(n, k, with_global):
    px, pw, sx, sw = _nvfp4_case(n, k, n + k)
    gx = torch.tensor([1.5], device=DEV) if with_global else None
    gw = torch.tensor([0.75], device=DEV) if with_global else None
    expected = oracle.nvfp4_gemv(px.view(torch.uint8).cpu(), pw.view(torch.uint8).cpu(), sx.cpu(), sw.cpu(),
                                 None if gx is None else gx.cpu(), None if gw is None else gw.cpu())
    raw = nvfp4_tma_gemv(px, pw, sx.reshape(-1), sw.reshape(-1), input_global_scale=gx, weight_global_scale=gw,
                         block_scale_layout=BlockScaleLayout.RAW)
    torch.testing.assert_close(raw.cpu(), expected, atol=2.0, rtol=0.05)
    blocked = nvfp4_tma_gemv(px, pw, tn.swizzle_nvfp4_scales(sx), tn.swizzle_nvfp4_scales(sw), input_global_scale=gx,
                             weight_global_scale=gw)
    assert torch.equal(blocked, raw)


def test_nvfp4_scaled_mm_adapter_matches_library_gemm():
    from torch.nn.functional import ScalingType, SwizzleType, scaled_mm

    px, pw, sx, sw = _nvfp4_case(128, 2048, 7)
    bx, bw = tn.swizzle_nvfp4_scales(sx), tn.swizzle_nvfp4_scales(sw)
    gx, gw = torch.tensor([1.5], device=DEV), torch.tensor([0.75], device=DEV)
    actual = nvfp4_tma_scaled_mm(px, pw.t(), bx, bw, block_n=4, global_scale_a=gx, global_scale_b=gw)
    expected = scaled_mm(px, pw.t(), scale_a=[bx, gx], scale_recipe_a=[ScalingType.BlockWise1x16, ScalingType.TensorWise],
                         swizzle_a=[SwizzleType.SWIZZLE_32_4_4, SwizzleType.NO_SWIZZLE], scale_b=[bw, gw],
                         scale_recipe_b=[ScalingType.BlockWise1x16, ScalingType.TensorWise],
                         swizzle_b=[SwizzleType.SWIZZLE_32_4_4, SwizzleType.NO_SWIZZLE], output_dtype=torch.bfloat16)
    torch.testing.assert_close(actual, expected, atol=2.0, rtol=0.05)


def test_quantize_then_gemv_end_to_end():
    """bf16 -> our quantizers -> our GEMV stays close to the bf16 matmul."""
    torch.manual_seed(3)
    n, k = 512, 4096
    x = torch.randn(1, k, dtype=torch.bfloat16, device=DEV)
    w = torch.randn(n, k, dtype=torch.bfloat16, device=DEV)
    exact = x.float() @ w.float().T
    rx, rw = tn.quantize_mxfp8(x, swizzle=True), tn.quantize_mxfp8(w, swizzle=True)
    y8 = mxfp8_tma_gemv(rx.q_row, rw.q_row, rx.scale_row, rw.scale_row, block_scale_layout=BlockScaleLayout.SWIZZLE_32_4_4)
    assert float((y8.float() - exact).abs().mean() / exact.abs().mean()) < 0.08
    ax, aw = tn.quantize_nvfp4(x), tn.quantize_nvfp4(w)
    y4 = nvfp4_tma_gemv(ax.packed, aw.packed, ax.block_scales, aw.block_scales, input_global_scale=ax.global_scale,
                        weight_global_scale=aw.global_scale)
    assert float((y4.float() - exact).abs().mean() / exact.abs().mean()) < 0.2


def test_gemv_argument_checks():
    _, qx, sx = _quant((1, 2048), 1)
    _, qw, sw = _quant((128, 2048), 2)
    with pytest.raises(ValueError):
        mxfp8_tma_gemv(qx, qw[:, :1024].contiguous(), sx, sw)
    with pytest.raises(TypeError):
        mxfp8_tma_gemv(qx.view(torch.uint8), qw, sx, sw)
    with pytest.raises(ValueError):
        mxfp8_tma_gemv(qx, qw, sx, sw[:, :8].contiguous())
    with pytest.raises(ValueError):
        mxfp8_tma_gemv(qx, qw, sx, sw, output=torch.empty(1, 64, dtype=torch.bfloat16, device=DEV))
