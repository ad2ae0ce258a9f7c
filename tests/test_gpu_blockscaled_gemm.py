"""MXFP8 GEMM on the block-scaled tensor cores, fed by this library's quantizer (payload and
swizzled scales as written): against the oracle's dequantise-then-matmul in fp32 and against
torch's block-scaled scaled_mm on the same operands."""

import pytest
import torch

import oracle
import transformer_nuggets_b200 as tn
from transformer_nuggets_b200 import _lib
from transformer_nuggets_b200.mx.gemm import mxfp8_scaled_mm, nvfp4_scaled_mm

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _case(m, n, k, seed):
    g = torch.Generator().manual_seed(seed)
    x = (torch.randn(m, k, generator=g) * torch.exp2(torch.rand(m, 1, generator=g) * 6 - 3)).to(torch.bfloat16)
    w = (torch.randn(n, k, generator=g) * torch.exp2(torch.rand(n, 1, generator=g) * 6 - 3)).to(torch.bfloat16)
    return x, w


@pytest.mark.parametrize("m,n,k", [(128, 256, 128), (128, 256, 512), (256, 512, 1024), (100, 72, 256), (300, 520, 384),
                                   (1024, 2048, 2048)])
def test_matches_dequantised_matmul(m, n, k):
    x, w = _case(m, n, k, m + n + k)
    rx = tn.quantize_mxfp8(x.to(DEV), swizzle=True)
    rw = tn.quantize_mxfp8(w.to(DEV), swizzle=True)
    got = mxfp8_scaled_mm(rx.q_row, rw.q_row.t(), rx.scale_row, rw.scale_row)
    assert int(_lib.workspace(torch.device(DEV, 0))[_lib.WS_STATUS_WORD].item()) == 0
    qx, sx = oracle.mxfp8_quantize(x, "ceil")
    qw, sw = oracle.mxfp8_quantize(w, "ceil")
    want = (oracle.mxfp8_dequantize(qx, sx) @ oracle.mxfp8_dequantize(qw, sw).T).to(torch.bfloat16)
    scale = want.float().abs().max().item()
    torch.testing.assert_close(got.cpu().float(), want.float(), rtol=2 ** -6, atol=2 ** -8 * scale)


# (4096, 8192) gives 1024 tiles: every CTA of the persistent grid walks several tiles, so the stage
# ring, the single accumulator's hand-over and the scale-column sets wrap across tile boundaries;
# K = 640 / 768 makes the number of stages per tile odd or not a multiple of the ring depth
@pytest.mark.parametrize("m,n,k", [(512, 1024, 1024), (4096, 8192, 640), (2304, 4352, 1536)])
def test_against_library_block_scaled_mm(m, n, k):
    try:
        from torch.nn.functional import ScalingType, SwizzleType, scaled_mm
    except ImportError:
        pytest.skip("this torch has no block-scaled scaled_mm")

    x, w = _case(m, n, k, 9)
    rx = tn.quantize_mxfp8(x.to(DEV), swizzle=True)
    rw = tn.quantize_mxfp8(w.to(DEV), swizzle=True)
    got = mxfp8_scaled_mm(rx.q_row, rw.q_row.t(), rx.scale_row, rw.scale_row)
    ref = scaled_mm(
        rx.q_row, rw.q_row.t(),
        scale_a=[rx.scale_row.view(torch.float8_e8m0fnu)], scale_recipe_a=[ScalingType.BlockWise1x32],
        swizzle_a=[SwizzleType.SWIZZLE_32_4_4],
        scale_b=[rw.scale_row.view(torch.float8_e8m0fnu)], scale_recipe_b=[ScalingType.BlockWise1x32],
        swizzle_b=[SwizzleType.SWIZZLE_32_4_4],
        output_dtype=torch.bfloat16,
    )
    scale = ref.float().abs().max().item()
    torch.testing.assert_close(got.float(), ref.float(), rtol=2 ** -6, atol=2 ** -8 * scale)


@pytest.mark.parametrize("m,n,k", [(128, 256, 256), (128, 256, 1024), (256, 512, 2048), (100, 72, 256), (300, 520, 768),
                                   (1024, 2048, 2048)])
def test_nvfp4_matches_dequantised_matmul(m, n, k):
    x, w = _case(m, n, k, m + n + k + 1)
    a, b = tn.quantize_nvfp4(x.to(DEV), swizzle=True), tn.quantize_nvfp4(w.to(DEV), swizzle=True)
    got = nvfp4_scaled_mm(a.packed, b.packed.t(), a.block_scales, b.block_scales, a.global_scale, b.global_scale)
    assert int(_lib.workspace(torch.device(DEV, 0))[_lib.WS_STATUS_WORD].item()) == 0
    ra, rb = tn.quantize_nvfp4(x.to(DEV), swizzle=False), tn.quantize_nvfp4(w.to(DEV), swizzle=False)
    da = oracle.nvfp4_dequantize(ra.packed.view(torch.uint8).cpu(), ra.block_scales.cpu(), ra.global_scale.cpu())
    db = oracle.nvfp4_dequantize(rb.packed.view(torch.uint8).cpu(), rb.block_scales.cpu(), rb.global_scale.cpu())
    want = (da @ db.T).to(torch.bfloat16)
    scale = want.float().abs().max().item()
    torch.testing.assert_close(got.cpu().float(), want.float(), rtol=2 ** -6, atol=2 ** -8 * scale)


@pytest.mark.parametrize("m,n,k", [(512, 1024, 2048), (4096, 8192, 768), (2304, 4352, 1280)])
def test_nvfp4_against_library_block_scaled_mm(m, n, k):
    try:
        from torch.nn.functional import ScalingType, SwizzleType, scaled_mm
    except ImportError:
        pytest.skip("this torch has no block-scaled scaled_mm")
    x, w = _case(m, n, k, 10)
    a, b = tn.quantize_nvfp4(x.to(DEV), swizzle=True), tn.quantize_nvfp4(w.to(DEV), swizzle=True)
    got = nvfp4_scaled_mm(a.packed, b.packed.t(), a.block_scales, b.block_scales, a.global_scale, b.global_scale)
    ref = scaled_mm(
        a.packed, b.packed.t(),
        scale_a=[a.block_scales, a.global_scale], scale_recipe_a=[ScalingType.BlockWise1x16, ScalingType.TensorWise],
        swizzle_a=[SwizzleType.SWIZZLE_32_4_4, SwizzleType.NO_SWIZZLE],
        scale_b=[b.block_scales, b.global_scale], scale_recipe_b=[ScalingType.BlockWise1x16, ScalingType.TensorWise],
        swizzle_b=[SwizzleType.SWIZZLE_32_4_4, SwizzleType.NO_SWIZZLE],
        output_dtype=torch.bfloat16,
    )
    scale = ref.float().abs().max().item()
    torch.testing.assert_close(got.float(), ref.float(), rtol=2 ** -6, atol=2 ** -8 * scale)
