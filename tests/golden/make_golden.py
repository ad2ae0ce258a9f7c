"""Write the golden fixtures of this directory by running the REFERENCE's own
Python functions on CPU.

Run once, in a container that has the reference checkout:

    PYTHONDONTWRITEBYTECODE=1 python tests/golden/make_golden.py /path/to/transformer_nuggets

The reference checkout does not exist where the GPU tests run, so the outputs
are committed as small ``.npz`` files (bf16 stored as its uint16 bit pattern,
fp8 as uint8).  Functions called, by reference path:

* fp8/scaled_quant.py:78   eager_scaled_quant
* cute/mxfp8_tma.py:497    quantize_mxfp8_tensor
* mx/to_blocked.py:10,75   to_blocked, to_blocked_manual
* cute/nvfp4_tma.py:941    pack_nvfp4_codes
* cute/nvfp4_tma.py:946    swizzle_nvfp4_scales
* examples/rms_norm_fusion_profile.py:26  handwritten_rms_norm  (``--only rmsnorm`` writes just this one)
* fp8/scaled_quant.py:78   eager_scaled_quant once per ROW with that row's scale as a ``[1]`` tensor: the
                           row-wise cast is the per-tensor cast at row granularity (``--only rowwise``)
"""

import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def bf16_bits(t):
    return t.contiguous().view(torch.uint16).numpy().copy()


def u8(t):
    return t.contiguous().view(torch.uint8).numpy().copy()


def all_bf16_patterns():
    return torch.arange(65536, dtype=torch.int32).to(torch.uint16).view(torch.bfloat16).reshape(256, 256)


def rms_norm_fixture(ref_root):
    """The eager RMSNorm of the reference's fusion example on seeded bf16 rows (CPU)."""
    import importlib.util

    spec = importlib.util.spec_from_file_location("ref_rms_norm_example",
                                                  os.path.join(ref_root, "examples", "rms_norm_fusion_profile.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    g = torch.Generator().manual_seed(20244)
    out = {"eps": np.float32(mod.EPS)}
    for name, (rows, cols) in (("a", (48, 1024)), ("b", (20, 4096)), ("c", (33, 80))):
        x = (torch.randn(rows, cols, generator=g) * torch.exp2(torch.rand(rows, 1, generator=g) * 12 - 6)).to(torch.bfloat16)
        w = (1.0 + 0.25 * torch.randn(cols, generator=g)).to(torch.bfloat16)
        if name == "c":
            x[5] = 0.0  # an all-zero row: y = 0 * rsqrt(eps) * w = 0
        y = mod.handwritten_rms_norm(x, w)
        out[f"x_{name}"], out[f"w_{name}"], out[f"y_{name}"] = bf16_bits(x), bf16_bits(w), bf16_bits(y)
    np.savez_compressed(os.path.join(HERE, "rms_norm.npz"), **out)


def rowwise_fixture():
    """Row-wise cast through the reference's ``eager_scaled_quant`` (fp8/scaled_quant.py:78-102), one call
    per row: ``scale_r = finfo.max / max(amax_r, 1e-12)`` as one fp32 division, handed over with shape
    ``[1]`` (a 0-dim scale would make the product bf16), ``saturated=True``.  Rows: seeded normal data
    with per-row sigma, an all-zero row, a row with one outlier, a row holding a NaN, a row holding an
    infinity, a row of bf16 subnormals."""
    from transformer_nuggets.fp8.scaled_quant import eager_scaled_quant

    g = torch.Generator().manual_seed(20245)
    rows, cols = 40, 384
    x = torch.randn(rows, cols, generator=g) * torch.exp2(torch.rand(rows, 1, generator=g) * 12 - 6)
    x[3] = 0.0
    x[5, 17] = 3.0e4
    x[7, 100] = float("nan")
    x[9, 0] = float("-inf")
    x[11] = x[11] * 1e-39
    xb = x.to(torch.bfloat16)
    out = {"x_bits": bf16_bits(xb)}
    for dname, dt in (("e4m3", torch.float8_e4m3fn), ("e5m2", torch.float8_e5m2)):
        fmax = torch.tensor(torch.finfo(dt).max, dtype=torch.float32)
        q = torch.empty(rows, cols, dtype=torch.uint8)
        scales = torch.empty(rows, 1, dtype=torch.float32)
        for r in range(rows):
            row = xb[r : r + 1]
            amax = row.abs().max().float()
            scale = (fmax / torch.clamp(amax, min=1e-12)).reshape(1)
            am = torch.tensor([-1.0])
            q[r] = eager_scaled_quant(row, scale, am, dt, True).view(torch.uint8)[0]
            scales[r, 0] = scale[0]
        out[f"q_{dname}"] = q.numpy()
        out[f"scale_{dname}"] = scales.numpy()
    np.savez_compressed(os.path.join(HERE, "fp8_rowwise.npz"), **out)


def main(ref_root, only=None):
    sys.path.insert(0, ref_root)
    if only == "rmsnorm":
        rms_norm_fixture(ref_root)
        print("rms_norm.npz written to", HERE)
        return
    if only == "rowwise":
        rowwise_fixture()
        print("fp8_rowwise.npz written to", HERE)
        return
    from transformer_nuggets.cute.mxfp8_tma import quantize_mxfp8_tensor
    from transformer_nuggets.cute.nvfp4_tma import pack_nvfp4_codes, swizzle_nvfp4_scales
    from transformer_nuggets.fp8.scaled_quant import eager_scaled_quant
    from transformer_nuggets.mx.to_blocked import to_blocked, to_blocked_manual

    dtypes = {"e4m3": torch.float8_e4m3fn, "e5m2": torch.float8_e5m2}

    # ---- 1. delayed-scale cast on every bf16 bit pattern -------------------
    pats = all_bf16_patterns()
    out = {"x_bits": bf16_bits(pats)}
    for sname, sval in (("s1", 1.0), ("s3p7", 3.7), ("s2e10", 1024.0), ("s2em9", 2.0**-9)):
        scale = torch.tensor([sval], dtype=torch.float32)
        out[f"scale_{sname}"] = scale.numpy()
        for dname, dt in dtypes.items():
            for sat in (False, True):
                am = torch.tensor([-1.0])
                q = eager_scaled_quant(pats, scale, am, dt, sat)
                out[f"q_{sname}_{dname}_{'sat' if sat else 'unsat'}"] = u8(q)
    np.savez_compressed(os.path.join(HERE, "fp8_all_bf16_patterns.npz"), **out)

    # ---- 2. seeded normal data, bf16 and fp32, plus the reference's own test inputs
    g = torch.Generator().manual_seed(20240)
    x = torch.randn(96, 320, generator=g) * 9.6
    x.view(-1)[torch.randint(0, x.numel(), (40,), generator=g)] *= 100.0
    xb = x.to(torch.bfloat16)
    out = {"x_f32": x.numpy(), "x_bf16_bits": bf16_bits(xb)}
    for dname, dt in dtypes.items():
        fmax = torch.finfo(dt).max
        for iname, inp in (("f32", x), ("bf16", xb)):
            # delayed scaling, the reference's test constants (test/test_fp8.py:19-21)
            scale = torch.tensor([4.0], dtype=torch.float32)
            for sat in (False, True):
                am = torch.tensor([-1.0])
                q = eager_scaled_quant(inp, scale, am, dt, sat)
                out[f"delayed_{iname}_{dname}_{'sat' if sat else 'unsat'}"] = u8(q)
                out[f"delayed_{iname}_amax"] = am.numpy().copy()
            # dynamic: scale = max/amax (fp32 division), saturated cast
            amax = inp.abs().max().float()
            dscale = (torch.tensor(fmax, dtype=torch.float32) / amax).reshape(1)
            am = torch.tensor([-1.0])
            q = eager_scaled_quant(inp, dscale, am, dt, True)
            out[f"dynamic_{iname}_{dname}"] = u8(q)
            out[f"dynamic_{iname}_{dname}_scale"] = dscale.numpy().copy()
    # the reference's saturation test: 100 outliers at finfo.max + 100 (test/test_fp8.py:31-33)
    for dname, dt in dtypes.items():
        g2 = torch.Generator().manual_seed(0)
        a = torch.rand(64, 256, generator=g2)
        a[0, :100] = torch.finfo(dt).max + 100
        scale = torch.tensor([4.0], dtype=torch.float32)
        am = torch.tensor([-1.0])
        q = eager_scaled_quant(a, scale, am, dt, True)
        out[f"sattest_{dname}_x"] = a.numpy().copy()
        out[f"sattest_{dname}_q"] = u8(q)
        out[f"sattest_{dname}_amax"] = am.numpy().copy()
    np.savez_compressed(os.path.join(HERE, "fp8_seeded.npz"), **out)

    # ---- 3. MXFP8 -----------------------------------------------------------
    g = torch.Generator().manual_seed(20241)
    x = torch.randn(160, 256, generator=g) * torch.exp2(torch.rand(160, 1, generator=g) * 16 - 8)
    x[3, 32:64] = 0.0  # an all-zero block
    x[5, 0] = 3.0e38  # near the top of the bf16 range
    x[7, 64:96] *= 1e-36  # subnormal-ish block
    xb = x.to(torch.bfloat16)
    q, s = quantize_mxfp8_tensor(xb)
    qt, st = quantize_mxfp8_tensor(xb.t().contiguous())
    out = {"x_bits": bf16_bits(xb), "q_row": u8(q), "s_row": s.numpy(), "q_col": u8(qt), "s_col": st.numpy(),
           "s_row_blocked": to_blocked(s).numpy(), "s_col_blocked": to_blocked(st).numpy()}
    # every positive finite bf16 value (and zero) as the amax of one block
    amax_bits = torch.arange(0, 0x7F80, dtype=torch.int32).to(torch.uint16)
    amax = amax_bits.view(torch.bfloat16)
    blk = torch.zeros(amax.numel(), 32, dtype=torch.bfloat16)
    blk[:, 0] = amax
    blk[:, 1] = -amax
    blk[:, 2] = amax * 0.5
    blk[:, 3] = amax * 0.013
    q, s = quantize_mxfp8_tensor(blk)
    out["enum_amax_bits"] = amax_bits.numpy()
    out["enum_scale"] = s.reshape(-1).numpy()
    out["enum_q4"] = u8(q[:, :4])
    np.savez_compressed(os.path.join(HERE, "mxfp8.npz"), **out)

    # ---- 4. to_blocked (shapes of test/test_mx.py:22 plus cross-atom cases) -
    out = {}
    g = torch.Generator().manual_seed(20242)
    for shape in ((128, 4), (256, 8), (300, 9), (264, 64), (1, 1), (129, 5)):
        m = torch.randint(256, size=shape, dtype=torch.uint8, generator=g)
        a, b = to_blocked(m), to_blocked_manual(m)
        assert torch.equal(a, b)
        out[f"in_{shape[0]}x{shape[1]}"] = m.numpy()
        out[f"out_{shape[0]}x{shape[1]}"] = a.numpy()
    np.savez_compressed(os.path.join(HERE, "to_blocked.npz"), **out)

    # ---- 5. NVFP4 storage contract -------------------------------------------
    g = torch.Generator().manual_seed(20243)
    codes = torch.randint(0, 16, (40, 64), dtype=torch.uint8, generator=g)
    packed = pack_nvfp4_codes(codes).view(torch.uint8)
    scales = torch.randint(0, 0x7F, (200, 6), dtype=torch.uint8, generator=g)
    sw = swizzle_nvfp4_scales(scales.view(torch.float8_e4m3fn)).view(torch.uint8)
    np.savez_compressed(
        os.path.join(HERE, "nvfp4_format.npz"),
        codes=codes.numpy(), packed=packed.numpy(), scales=scales.numpy(), swizzled=sw.numpy(),
    )
    rms_norm_fixture(ref_root)
    rowwise_fixture()
    print("golden fixtures written to", HERE)


if __name__ == "__main__":
    args = [a for a in sys.argv[1:] if not a.startswith("--")]
    only = next((a for a in ("rmsnorm", "rowwise") if "--only" in sys.argv and a in sys.argv), None)
    roots = [a for a in args if a not in ("rmsnorm", "rowwise")]
    root = roots[0] if roots else os.environ.get("TNQ_REFERENCE_ROOT")
    if not root:
        sys.exit("usage: make_golden.py /path/to/transformer_nuggets [--only rmsnorm|rowwise]  (or set TNQ_REFERENCE_ROOT)")
    main(root, only)
