"""The quantizers' outputs are accepted, as they are, by the block-scaled tensor-core
GEMM that consumes this storage format (`torch.nn.functional.scaled_mm`: E8M0 / E4M3 block
scales in the swizzled 128x4 layout, packed e2m1, fp32 global scale applied at decode) and
give the product of the dequantised operands within the tolerances the reference uses for
the same comparison (test/test_mxfp8_tma.py:174-203: atol 1.0, rtol 0.05;
test/test_nvfp4_tma.py:511-548: atol 2.0, rtol 0.05).  The library GEMM is only the
consumer under test here; nothing in the package calls it."""

import pytest
import torch

import oracle
import transformer_nuggets_b200 as tn

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _scaled_mm_api():
    try:
        from torch.nn.functional import ScalingType, SwizzleType, scaled_mm
    except ImportError:
        pytest.skip("torch.nn.functional.scaled_mm with block-wise recipes is not available in this torch")
    return ScalingType, SwizzleType, scaled_mm


def _dequant_mxfp8(q, s_raw):
    scale = torch.exp2(s_raw.float() - 127.0).repeat_interleave(32, dim=1)
    return q.float() * scale


@pytest.mark.parametrize("m,n,k", [(128, 256, 2048), (1, 128, 2048), (264, 128, 4096)])
def test_mxfp8_outputs_feed_scaled_mm(m, n, k):
    ScalingType, SwizzleType, scaled_mm = _scaled_mm_api()
    torch.manual_seed(k + m)
    x = torch.randn(m, k, dtype=torch.bfloat16, device=DEV)
    w = torch.randn(n, k, dtype=torch.bfloat16, device=DEV)
    ax, aw = tn.quantize_mxfp8(x, swizzle=True), tn.quantize_mxfp8(w, swizzle=True)
    rx, rw = tn.quantize_mxfp8(x, swizzle=False), tn.quantize_mxfp8(w, swizzle=False)
    expected = (_dequant_mxfp8(rx.q_row, rx.scale_row) @ _dequant_mxfp8(rw.q_row, rw.scale_row).T).bfloat16()
    actual = scaled_mm(
        ax.q_row, aw.q_row.t(),
        scale_a=[ax.scale_row.view(torch.float8_e8m0fnu)], scale_recipe_a=[ScalingType.BlockWise1x32],
        swizzle_a=[SwizzleType.SWIZZLE_32_4_4],
        scale_b=[aw.scale_row.view(torch.float8_e8m0fnu)], scale_recipe_b=[ScalingType.BlockWise1x32],
        swizzle_b=[SwizzleType.SWIZZLE_32_4_4],
        output_dtype=torch.bfloat16,
    )
    torch.cuda.synchronize()
    torch.testing.assert_close(actual, expected, atol=1.0, rtol=0.05)
    # and the quantisation itself is close to the unquantised product
    exact = (x.float() @ w.float().T)
    assert float((actual.float() - exact).abs().mean() / exact.abs().mean()) < 0.08


@pytest.mark.parametrize("m,n,k", [(128, 256, 2048), (1, 128, 2048)])
def test_nvfp4_outputs_feed_scaled_mm(m, n, k):
    ScalingType, SwizzleType, scaled_mm = _scaled_mm_api()
    torch.manual_seed(k + m + 1)
    x = torch.randn(m, k, dtype=torch.bfloat16, device=DEV)
    w = torch.randn(n, k, dtype=torch.bfloat16, device=DEV)
    a, b = tn.quantize_nvfp4(x, swizzle=True), tn.quantize_nvfp4(w, swizzle=True)
    ra, rb = tn.quantize_nvfp4(x, swizzle=False), tn.quantize_nvfp4(w, swizzle=False)
    da = oracle.nvfp4_dequantize(ra.packed.view(torch.uint8).cpu(), ra.block_scales.cpu(), ra.global_scale.cpu())
    db = oracle.nvfp4_dequantize(rb.packed.view(torch.uint8).cpu(), rb.block_scales.cpu(), rb.global_scale.cpu())
    expected = (da @ db.T).bfloat16()
    actual = scaled_mm(
        a.packed, b.packed.t(),
        scale_a=[a.block_scales, a.global_scale], scale_recipe_a=[ScalingType.BlockWise1x16, ScalingType.TensorWise],
        swizzle_a=[SwizzleType.SWIZZLE_32_4_4, SwizzleType.NO_SWIZZLE],
        scale_b=[b.block_scales, b.global_scale], scale_recipe_b=[ScalingType.BlockWise1x16, ScalingType.TensorWise],
        swizzle_b=[SwizzleType.SWIZZLE_32_4_4, SwizzleType.NO_SWIZZLE],
        output_dtype=torch.bfloat16,
    )
    torch.cuda.synchronize()
    torch.testing.assert_close(actual.cpu(), expected, atol=2.0, rtol=0.05)
    exact = (x.float() @ w.float().T).cpu()
    assert float((actual.float().cpu() - exact).abs().mean() / exact.abs().mean()) < 0.2
