"""The CPU oracle against the fixtures written by the reference's own functions
(tests/golden/make_golden.py).  CPU only."""

import numpy as np
import pytest
import torch

import oracle
from conftest import as_u8, bf16_from_bits

DT = {"e4m3": torch.float8_e4m3fn, "e5m2": torch.float8_e5m2}


@pytest.mark.parametrize("dname", ["e4m3", "e5m2"])
@pytest.mark.parametrize("sat", [False, True])
@pytest.mark.parametrize("sname", ["s1", "s3p7", "s2e10", "s2em9"])
def test_delayed_cast_all_bf16_patterns(golden, dname, sat, sname):
    g = golden("fp8_all_bf16_patterns.npz")
    x = bf16_from_bits(g["x_bits"])
    scale = torch.from_numpy(g[f"scale_{sname}"])
    am = torch.tensor([-1.0])
    q = oracle.fp8_scaled_quant(x, scale, am, DT[dname], sat)
    want = g[f"q_{sname}_{dname}_{'sat' if sat else 'unsat'}"]
    assert np.array_equal(as_u8(q).numpy(), want)


@pytest.mark.parametrize("dname", ["e4m3", "e5m2"])
@pytest.mark.parametrize("iname", ["f32", "bf16"])
def test_seeded_delayed_and_dynamic(golden, dname, iname):
    g = golden("fp8_seeded.npz")
    x = torch.from_numpy(g["x_f32"]) if iname == "f32" else bf16_from_bits(g["x_bf16_bits"])
    scale = torch.tensor([4.0])
    for sat in (False, True):
        am = torch.tensor([-1.0])
        q = oracle.fp8_scaled_quant(x, scale, am, DT[dname], sat)
        assert np.array_equal(as_u8(q).numpy(), g[f"delayed_{iname}_{dname}_{'sat' if sat else 'unsat'}"])
        assert np.array_equal(am.numpy(), g[f"delayed_{iname}_amax"])
    q, s = oracle.fp8_dynamic_quant(x, DT[dname])
    assert np.array_equal(as_u8(q).numpy(), g[f"dynamic_{iname}_{dname}"])
    assert np.array_equal(s.numpy(), g[f"dynamic_{iname}_{dname}_scale"])


@pytest.mark.parametrize("dname", ["e4m3", "e5m2"])
def test_reference_saturation_case(golden, dname):
    g = golden("fp8_seeded.npz")
    a = torch.from_numpy(g[f"sattest_{dname}_x"])
    am = torch.tensor([-1.0])
    q = oracle.fp8_scaled_quant(a, torch.tensor([4.0]), am, DT[dname], True)
    assert np.array_equal(as_u8(q).numpy(), g[f"sattest_{dname}_q"])
    assert np.array_equal(am.numpy(), g[f"sattest_{dname}_amax"])
    assert am.item() == torch.finfo(DT[dname]).max + 100


@pytest.mark.parametrize("dname", ["e4m3", "e5m2"])
def test_rowwise_matches_reference_applied_per_row(golden, dname):
    """The row-wise oracle against bytes and scales produced by the reference's
    eager_scaled_quant called once per row (zero, outlier, NaN, -inf and subnormal rows)."""
    g = golden("fp8_rowwise.npz")
    x = bf16_from_bits(g["x_bits"])
    q, s = oracle.fp8_rowwise_quant(x, DT[dname])
    assert np.array_equal(as_u8(q).numpy(), g[f"q_{dname}"])
    assert np.array_equal(s.numpy().view(np.uint32), g[f"scale_{dname}"].view(np.uint32))


def test_mxfp8_ceil_matches_reference(golden):
    g = golden("mxfp8.npz")
    x = bf16_from_bits(g["x_bits"])
    q, s = oracle.mxfp8_quantize(x, "ceil")
    assert np.array_equal(as_u8(q).numpy(), g["q_row"])
    assert np.array_equal(s.numpy(), g["s_row"])
    qt, st = oracle.mxfp8_quantize(x.t().contiguous(), "ceil")
    assert np.array_equal(as_u8(qt).numpy(), g["q_col"])
    assert np.array_equal(st.numpy(), g["s_col"])
    assert np.array_equal(oracle.to_blocked(s).numpy(), g["s_row_blocked"])
    assert np.array_equal(oracle.to_blocked(st).numpy(), g["s_col_blocked"])


def test_e8m0_integer_rule_on_every_bf16_amax(golden):
    """The integer exponent rule the kernel evaluates equals the reference's
    ceil(log2(amax/448)) on all 32 640 finite non-negative bf16 values."""
    g = golden("mxfp8.npz")
    amax = bf16_from_bits(g["enum_amax_bits"]).float()
    e = oracle.e8m0_exponent_ceil_int(amax)
    assert np.array_equal((e + 127).to(torch.uint8).numpy(), g["enum_scale"])
    assert g["enum_scale"].min() >= 1 and g["enum_scale"].max() <= 247
    # and the log2 restatement agrees too
    blk = torch.zeros(amax.numel(), 32, dtype=torch.bfloat16)
    a16 = bf16_from_bits(g["enum_amax_bits"])
    blk[:, 0], blk[:, 1], blk[:, 2], blk[:, 3] = a16, -a16, a16 * 0.5, a16 * 0.013
    q, s = oracle.mxfp8_quantize(blk, "ceil")
    assert np.array_equal(s.reshape(-1).numpy(), g["enum_scale"])
    assert np.array_equal(as_u8(q[:, :4]).numpy(), g["enum_q4"])


def test_e8m0_floor_rule_integer_form():
    bits = torch.arange(0, 0x7F80, dtype=torch.int32).to(torch.uint16)
    amax = bits.view(torch.bfloat16).float()
    blk = torch.zeros(amax.numel(), 32, dtype=torch.bfloat16)
    blk[:, 0] = bits.view(torch.bfloat16)
    _, s = oracle.mxfp8_quantize(blk, "floor")
    e = oracle.e8m0_exponent_floor_int(amax)
    assert torch.equal((e + 127).to(torch.uint8), s.reshape(-1))
    # ceil and floor differ exactly where the mantissa is above 1.75
    ec = oracle.e8m0_exponent_ceil_int(amax)
    mant = amax.view(torch.int32) & 0x7FFFFF
    normal = (amax.view(torch.int32) >> 23) > 0
    inner = normal & (ec > -126) & (e > -126)
    assert torch.equal((ec != e)[inner], (mant > 0x600000)[inner])


@pytest.mark.parametrize("shape", [(128, 4), (256, 8), (300, 9), (264, 64), (1, 1), (129, 5)])
def test_to_blocked(golden, shape):
    g = golden("to_blocked.npz")
    m = torch.from_numpy(g[f"in_{shape[0]}x{shape[1]}"])
    want = g[f"out_{shape[0]}x{shape[1]}"]
    assert np.array_equal(oracle.to_blocked(m).numpy(), want)
    assert np.array_equal(oracle.to_blocked_closed_form(m).numpy(), want)


def test_nvfp4_storage_contract(golden):
    g = golden("nvfp4_format.npz")
    assert np.array_equal(oracle.pack_nvfp4_codes(torch.from_numpy(g["codes"])).numpy(), g["packed"])
    assert np.array_equal(oracle.to_blocked(torch.from_numpy(g["scales"])).numpy(), g["swizzled"])


def test_e2m1_rounding_table():
    v = torch.tensor([0.0, 0.25, 0.26, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 5.01, 6.0, 7.0, 1e9,
                      -0.0, -0.25, -0.75, -5.0, -100.0])
    want = torch.tensor([0.0, 0.0, 0.5, 1.0, 1.0, 2.0, 2.0, 4.0, 4.0, 6.0, 6.0, 6.0, 6.0,
                         -0.0, -0.0, -1.0, -4.0, -6.0])
    codes = oracle.e2m1_encode(v)
    dec = oracle.e2m1_decode(codes)
    assert torch.equal(dec, want)
    assert torch.equal(torch.signbit(dec), torch.signbit(want))
    assert codes[13].item() == 8  # -0.0 keeps its sign bit


def test_nvfp4_roundtrip_error_bound():
    g = torch.Generator().manual_seed(5)
    x = (torch.randn(64, 256, generator=g) * 3).to(torch.bfloat16)
    x[2, 16:32] = 0
    packed, s_q, g_dec = oracle.nvfp4_quantize(x)
    assert packed.shape == (64, 128) and s_q.shape == (64, 16) and g_dec.shape == (1,)
    y = oracle.nvfp4_dequantize(packed, s_q, g_dec)
    blocks = x.float().reshape(64, -1, 16)
    amax_b = blocks.abs().amax(-1, keepdim=True)
    # e2m1 step is at most 2 of 6 (between 4 and 6); the e4m3 block scale adds <= 1/16
    err = (y.reshape(64, -1, 16) - blocks).abs()
    assert bool((err <= amax_b * (1.0 / 6.0 + 1.0 / 8.0) + 1e-30).all())
    assert bool((y.reshape(64, -1, 16)[2, 1] == 0).all())


def test_sharded_equals_unsharded():
    g = torch.Generator().manual_seed(11)
    x = torch.randn(64, 128, generator=g).to(torch.bfloat16)
    x[50] *= 1000
    full, s = oracle.fp8_dynamic_quant(x, torch.float8_e4m3fn)
    for n in (1, 2, 4, 8):
        parts, s2 = oracle.sharded_fp8_dynamic_quant(list(x.chunk(n)), torch.float8_e4m3fn)
        assert torch.equal(s, s2)
        assert torch.equal(as_u8(torch.cat(parts)), as_u8(full))


@pytest.mark.parametrize("name", ["a", "b", "c"])
def test_rms_norm_matches_reference_fixture(golden, name):
    """oracle.rms_norm against the rows the reference's eager RMSNorm produced
    (examples/rms_norm_fusion_profile.py:26-31).  The same formula on the same CPU build is
    identical; another vector width may add the squares in another order, hence the
    last-place allowance."""
    z = golden("rms_norm.npz")
    x, w, y = (bf16_from_bits(z[f"{k}_{name}"]) for k in ("x", "w", "y"))
    got = oracle.rms_norm(x, w, float(z["eps"]))
    ia, ib = got.view(torch.int16).to(torch.int32), y.view(torch.int16).to(torch.int32)
    assert (ia - ib).abs().max().item() <= 1
    assert (ia != ib).float().mean().item() <= 5e-3
    q, scale, y2 = oracle.rms_norm_rowwise_quant(x, w, float(z["eps"]))
    assert torch.equal(y2.view(torch.int16), got.view(torch.int16)) and scale.shape == (x.shape[0], 1)
