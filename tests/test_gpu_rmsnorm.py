"""RMSNorm fused into the row-wise FP8 cast.

Two-stage parity: (1) the normalised bf16 rows the kernel used (returned on request) agree
with the reference's eager RMSNorm up to an occasional last-place bf16 rounding - the one
step that is not bit-reproducible is the fp32 sum of squares, whose order differs between a
CPU and a GPU; (2) given those rows, the quantised bytes and the per-row scales are
bit-exact against the oracle's row-wise cast."""

import pytest
import torch

import oracle
from conftest import as_u8, bf16_from_bits
from transformer_nuggets_b200.fp8 import (rms_norm_quantize_mxfp8, rms_norm_rowwise_quant, swiglu_quantize_mxfp8,
                                          swiglu_rowwise_quant)

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _ulp_distance(a, b):
    """Distance in bf16 representable steps between two finite bf16 tensors."""
    ia = a.contiguous().view(torch.int16).to(torch.int32)
    ib = b.contiguous().view(torch.int16).to(torch.int32)
    ia = torch.where(ia < 0, -(ia & 0x7FFF), ia)
    ib = torch.where(ib < 0, -(ib & 0x7FFF), ib)
    return (ia - ib).abs()


def _check(x, w, eps, want_y=None):
    q, scale, y = rms_norm_rowwise_quant(x.to(DEV), w.to(DEV), eps, return_normed=True)
    y_cpu = y.cpu()
    ref_y = oracle.rms_norm(x, w, eps) if want_y is None else want_y
    finite = torch.isfinite(ref_y.float()) & torch.isfinite(y_cpu.float())
    assert torch.equal(torch.isnan(ref_y.float()), torch.isnan(y_cpu.float()))
    d = _ulp_distance(y_cpu[finite], ref_y[finite])
    assert d.max().item() <= 1 if d.numel() else True
    assert (d != 0).float().mean().item() <= 5e-3 if d.numel() else True
    # stage 2: exact cast of the rows actually used
    want_q, want_scale = oracle.fp8_rowwise_quant(y_cpu.reshape(-1, y_cpu.shape[-1]), torch.float8_e4m3fn)
    got_scale = scale.cpu().reshape(-1, 1)
    nan = torch.isnan(want_scale)
    assert torch.equal(torch.isnan(got_scale), nan)
    assert torch.equal(got_scale[~nan].view(torch.int32), want_scale[~nan].view(torch.int32))
    assert torch.equal(as_u8(q).cpu().reshape(want_q.shape), as_u8(want_q))
    q2, scale2 = rms_norm_rowwise_quant(x.to(DEV), w.to(DEV), eps)
    assert torch.equal(as_u8(q2), as_u8(q)) and torch.equal(scale2.view(torch.int32), scale.view(torch.int32))
    return y_cpu


@pytest.mark.parametrize("name", ["a", "b", "c"])
def test_against_reference_fixture(golden, name):
    z = golden("rms_norm.npz")
    x, w, y = (bf16_from_bits(z[f"{k}_{name}"]) for k in ("x", "w", "y"))
    _check(x, w, float(z["eps"]), want_y=y)


@pytest.mark.parametrize("shape", [(1, 16), (7, 32), (64, 512), (33, 1040), (256, 4096), (128, 8192), (16, 16384),
                                   (5, 5120), (2, 17, 1024), (300, 2048), (3, 12288)])
def test_shapes(shape):
    g = torch.Generator().manual_seed(sum(shape))
    x = (torch.randn(*shape, generator=g) * torch.exp2(torch.rand(*shape[:-1], 1, generator=g) * 10 - 5)).to(torch.bfloat16)
    w = (1.0 + 0.3 * torch.randn(shape[-1], generator=g)).to(torch.bfloat16)
    _check(x, w, 1e-5)


def test_special_rows():
    g = torch.Generator().manual_seed(11)
    x = torch.randn(8, 1024, generator=g).to(torch.bfloat16)
    w = torch.ones(1024, dtype=torch.bfloat16)
    x[1] = 0.0                    # zero row: y = 0, scale = 448 / 1e-12
    x[2, 7] = float("nan")        # NaN row: every y of the row is NaN
    x[3, 9] = float("inf")        # inf row: rstd = 0, inf * 0 = NaN at the inf, 0 elsewhere
    x[4] = 3.0e38                 # squares overflow fp32: var = inf, rstd = 0, y = 0
    x[5] = 1.0e-30                # squares underflow: var = 0, rstd = 1/sqrt(eps)
    _check(x, w, 1e-6)


def test_deterministic():
    g = torch.Generator().manual_seed(12)
    x = torch.randn(512, 4096, generator=g).to(torch.bfloat16).to(DEV)
    w = torch.randn(4096, generator=g).to(torch.bfloat16).to(DEV)
    a = rms_norm_rowwise_quant(x, w, 1e-6, return_normed=True)
    b = rms_norm_rowwise_quant(x, w, 1e-6, return_normed=True)
    for s, t in zip(a, b):
        assert torch.equal(s.view(torch.uint8), t.view(torch.uint8))


def test_argument_checks():
    x = torch.zeros(4, 64, dtype=torch.bfloat16, device=DEV)
    w = torch.ones(64, dtype=torch.bfloat16, device=DEV)
    with pytest.raises(TypeError):
        rms_norm_rowwise_quant(x.float(), w)
    with pytest.raises(ValueError):
        rms_norm_rowwise_quant(x, w[:48])
    with pytest.raises(ValueError):
        rms_norm_rowwise_quant(x[:, :40], w[:40])
    with pytest.raises(ValueError):
        rms_norm_rowwise_quant(torch.zeros(2, 32768, dtype=torch.bfloat16, device=DEV),
                               torch.ones(32768, dtype=torch.bfloat16, device=DEV))
    q, s = rms_norm_rowwise_quant(torch.zeros(0, 64, dtype=torch.bfloat16, device=DEV), w)
    assert q.shape == (0, 64) and s.shape == (0, 1)


@pytest.mark.parametrize("shape", [(1, 32), (7, 64), (130, 1056), (256, 4096), (128, 8192), (9, 16384), (2, 5, 2048)])
@pytest.mark.parametrize("mode", ["ceil", "floor"])
def test_fused_mxfp8(shape, mode):
    """Stage 1 as above; stage 2: payload and E8M0 bytes bit-exact against the oracle's MXFP8
    quantizer applied to the normalised rows the kernel used; swizzled == to_blocked(raw)."""
    g = torch.Generator().manual_seed(sum(shape) + len(mode))
    x = (torch.randn(*shape, generator=g) * torch.exp2(torch.rand(*shape[:-1], 1, generator=g) * 10 - 5)).to(torch.bfloat16)
    w = (1.0 + 0.3 * torch.randn(shape[-1], generator=g)).to(torch.bfloat16)
    q, sf, y = rms_norm_quantize_mxfp8(x.to(DEV), w.to(DEV), 1e-5, scale_mode=mode, return_normed=True)
    y_cpu = y.cpu()
    d = _ulp_distance(y_cpu, oracle.rms_norm(x, w, 1e-5))
    assert d.max().item() <= 1 and (d != 0).float().mean().item() <= 5e-3
    y2 = y_cpu.reshape(-1, shape[-1])
    want_q, want_sf = oracle.mxfp8_quantize(y2, mode)
    assert torch.equal(as_u8(q).cpu().reshape(want_q.shape), as_u8(want_q))
    assert torch.equal(sf.cpu(), want_sf)
    q2, sf2 = rms_norm_quantize_mxfp8(x.to(DEV), w.to(DEV), 1e-5, scale_mode=mode, swizzle=True)
    assert torch.equal(as_u8(q2), as_u8(q)) and torch.equal(sf2.cpu(), oracle.to_blocked(want_sf))


def test_fused_mxfp8_argument_checks():
    x = torch.zeros(4, 64, dtype=torch.bfloat16, device=DEV)
    w = torch.ones(64, dtype=torch.bfloat16, device=DEV)
    with pytest.raises(ValueError):
        rms_norm_quantize_mxfp8(x[:, :48].contiguous(), w[:48].contiguous())  # 48 is not a multiple of 32
    with pytest.raises(ValueError):
        rms_norm_quantize_mxfp8(x, w, scale_mode="nearest")
    with pytest.raises(TypeError):
        rms_norm_quantize_mxfp8(x.float(), w)


def _swiglu_inputs(shape, seed):
    g = torch.Generator().manual_seed(seed)
    a = (torch.randn(*shape, generator=g) * 3.0).to(torch.bfloat16)
    b = (torch.randn(*shape, generator=g) * torch.exp2(torch.rand(*shape[:-1], 1, generator=g) * 8 - 4)).to(torch.bfloat16)
    return a, b


@pytest.mark.parametrize("shape", [(1, 16), (9, 48), (130, 1040), (256, 4096), (64, 8192), (5, 14336), (2, 3, 2048)])
def test_swiglu_rowwise(shape):
    a, b = _swiglu_inputs(shape, sum(shape))
    q, scale, y = swiglu_rowwise_quant(a.to(DEV), b.to(DEV), return_activation=True)
    y_cpu = y.cpu()
    d = _ulp_distance(y_cpu, oracle.swiglu(a, b))
    assert d.max().item() <= 1 and (d != 0).float().mean().item() <= 2e-2
    want_q, want_scale = oracle.fp8_rowwise_quant(y_cpu.reshape(-1, shape[-1]), torch.float8_e4m3fn)
    assert torch.equal(as_u8(q).cpu().reshape(want_q.shape), as_u8(want_q))
    assert torch.equal(scale.cpu().reshape(-1, 1).view(torch.int32), want_scale.view(torch.int32))
    q2, scale2 = swiglu_rowwise_quant(a.to(DEV), b.to(DEV))
    assert torch.equal(as_u8(q2), as_u8(q)) and torch.equal(scale2, scale)


@pytest.mark.parametrize("shape", [(3, 32), (130, 1056), (256, 4096), (33, 8192), (4, 14336)])
@pytest.mark.parametrize("mode", ["ceil", "floor"])
def test_swiglu_mxfp8(shape, mode):
    a, b = _swiglu_inputs(shape, sum(shape) + 1)
    q, sf, y = swiglu_quantize_mxfp8(a.to(DEV), b.to(DEV), scale_mode=mode, return_activation=True)
    y_cpu = y.cpu()
    d = _ulp_distance(y_cpu, oracle.swiglu(a, b))
    assert d.max().item() <= 1 and (d != 0).float().mean().item() <= 2e-2
    want_q, want_sf = oracle.mxfp8_quantize(y_cpu.reshape(-1, shape[-1]), mode)
    assert torch.equal(as_u8(q).cpu().reshape(want_q.shape), as_u8(want_q)) and torch.equal(sf.cpu(), want_sf)
    q2, sf2 = swiglu_quantize_mxfp8(a.to(DEV), b.to(DEV), scale_mode=mode, swizzle=True)
    assert torch.equal(as_u8(q2), as_u8(q)) and torch.equal(sf2.cpu(), oracle.to_blocked(want_sf))


def test_swiglu_large_negative_gate():
    """Gate values in (-88.7, -87.3): 1 + exp(-a) lies in (2^126, 2^128), where an approximate division
    would return 0 although silu(a) is about -5e-37, still a normal bf16 value.  The activation must stay
    within one bf16 step of the eager result there too, and beyond -88.8 (exp overflows) it is -0."""
    vals = torch.tensor([-86.0, -87.0, -87.5, -88.0, -88.5, -88.7, -89.0, -100.0, -3.0, 0.0, 2.0, 88.0])
    a = vals.repeat(64 * 32 // vals.numel() + 1)[: 64 * 32].reshape(64, 32).to(torch.bfloat16)
    b = torch.full_like(a, 1.5)
    q, scale, y = swiglu_rowwise_quant(a.to(DEV), b.to(DEV), return_activation=True)
    want = oracle.swiglu(a, b)
    d = _ulp_distance(y.cpu(), want)
    assert d.max().item() <= 1
    nz = want.float() != 0
    assert bool(((y.cpu().float() != 0) == nz).all())  # nothing that should be non-zero was flushed to zero


def test_swiglu_argument_checks():
    a = torch.zeros(4, 64, dtype=torch.bfloat16, device=DEV)
    with pytest.raises(ValueError):
        swiglu_rowwise_quant(a, a[:, :32].contiguous())
    with pytest.raises(TypeError):
        swiglu_rowwise_quant(a.float(), a.float())
    with pytest.raises(ValueError):
        swiglu_quantize_mxfp8(a[:, :48].contiguous(), a[:, :48].contiguous())
