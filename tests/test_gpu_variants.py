"""The selectable kernel variants behind one entry point produce the same bytes: direct-store and
TMA-store forms of the row + column MXFP8 quantizer and of the transposing cast, and the tuning switches
of the per-tensor cast.  Every variant is also compared with the oracle."""

import pytest
import torch

import oracle
import transformer_nuggets_b200 as tn
from conftest import as_u8
from transformer_nuggets_b200 import _lib
from transformer_nuggets_b200.fp8 import scaled_quant, scaled_quant_transpose
from transformer_nuggets_b200.workloads import make_input

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.fixture
def restore_defaults():
    yield
    _lib.call("tnq_mxfp8_set_store_variant", 1 + 4 * 1)
    _lib.call("tnq_cast_transpose_set_store_variant", 1)
    _lib.call("tnq_set_option", 5, 1)
    _lib.call("tnq_set_option", 6, 0)


@pytest.mark.parametrize("shape", [(128, 128), (160, 256), (1024, 1056), (264, 64), (4096, 7168)])
def test_mxfp8_store_variants_agree(shape, restore_defaults):
    rows, cols = shape
    rows -= rows % 32
    x = make_input("mxfp8", "cpu", rows=rows, cols=cols)
    wq, ws = oracle.mxfp8_quantize(x, "ceil")
    wqt, wst = oracle.mxfp8_quantize(x.t().contiguous(), "ceil")
    for code in (0, 1, 1 + 4 * 1, 1 + 4 * 2, 1 + 4 * 3):  # variant + 4 * (load / store eviction policy bits)
        _lib.call("tnq_mxfp8_set_store_variant", code)
        r = tn.quantize_mxfp8(x.to(DEV), columnwise=True, swizzle=True)
        assert torch.equal(as_u8(r.q_row).cpu(), as_u8(wq)) and torch.equal(as_u8(r.q_col).cpu(), as_u8(wqt)), code
        assert torch.equal(r.scale_row.cpu(), oracle.to_blocked(ws)) and torch.equal(r.scale_col.cpu(), oracle.to_blocked(wst)), code
    with pytest.raises(_lib.TnqError):
        _lib.call("tnq_mxfp8_set_store_variant", 2)


@pytest.mark.parametrize("shape", [(128, 128), (160, 264), (2048, 1024), (144, 200), (16, 8), (48, 4104), (130, 136)])
@pytest.mark.parametrize("dtype", [torch.float8_e4m3fn, torch.float8_e5m2])
def test_cast_transpose_variants_agree(shape, dtype, restore_defaults):
    """Variant 1 (convert once, byte transpose, TMA store) and variant 0 (convert twice, direct stores);
    (130, 136) has an out_t pitch that is not a multiple of 16 bytes and takes variant 0 either way."""
    rows, cols = shape
    g = torch.Generator().manual_seed(rows * 7 + cols)
    x = (torch.randn(rows, cols, generator=g) * 30).to(torch.bfloat16)
    x.view(-1)[3] = float("nan")
    x.view(-1)[5] = float("-inf")
    scale = torch.tensor([2.0])
    for sat in (True, False):
        want = as_u8(oracle.fp8_scaled_quant(x, scale, torch.zeros(1), dtype, sat))
        for variant in (0, 1):
            _lib.call("tnq_cast_transpose_set_store_variant", variant)
            am = torch.zeros(1, device=DEV)
            q, q_t = scaled_quant_transpose(x.to(DEV), scale.to(DEV), am, dtype, sat)
            assert torch.equal(as_u8(q).cpu(), want) and torch.equal(as_u8(q_t).cpu(), want.t().contiguous()), (variant, sat)
            assert torch.isnan(am).item()


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_cast_pair_switch_agrees(dtype, restore_defaults):
    """256-bit-store form of the forward per-tensor cast on and off, odd vector counts and a ragged tail included,
    with and without the abs_max side output, NaN / inf inputs included."""
    for n in (16 * 1000 + 7, 32 * 4096, 16 * 3 + 1, 5):
        g = torch.Generator().manual_seed(n)
        x = (torch.randn(n, generator=g) * 50).to(dtype)
        if n > 40:
            x[11] = float("nan")
            x[29] = float("inf")
        scale = torch.tensor([3.0])
        for sat in (True, False):
            want_am = torch.tensor([-1.0])
            want = as_u8(oracle.fp8_scaled_quant(x, scale, want_am, torch.float8_e4m3fn, sat))
            for on in (0, 1):
                _lib.call("tnq_set_option", 5, on)
                am = torch.tensor([-1.0], device=DEV)
                q = scaled_quant(x.to(DEV), scale.to(DEV), am, torch.float8_e4m3fn, sat)
                assert torch.equal(as_u8(q).cpu(), want), (n, sat, on)
                assert torch.isnan(am).item() if n > 40 else am.item() == want_am.item()


@pytest.fixture
def restore_launch_defaults():
    yield
    _lib.call("tnq_set_option", 7, 1)
    _lib.call("tnq_set_option", 8, 1)


def test_launch_modes_agree(restore_launch_defaults):
    """Single-launch dynamic cast launched plain or cooperatively, every kernel chained to the stream's previous
    kernel or in plain stream order: the same bytes, equal to the oracle's, and a clean status word."""
    x = make_input("fp8_tensor", "cpu", rows=1024, cols=4096)
    want = as_u8(oracle.fp8_dynamic_quant(x, torch.float8_e4m3fn)[0])
    xd = x.to(DEV)
    for coop, chain in ((0, 0), (0, 1), (1, 0), (1, 1)):
        _lib.call("tnq_set_option", 7, coop)
        _lib.call("tnq_set_option", 8, chain)
        outs = [tn.dynamic_scaled_quant(xd) for _ in range(6)]  # back to back: each call overlaps the previous one's tail
        r = tn.quantize_mxfp8(xd, columnwise=True, swizzle=True)
        tn.check_status(xd.device, "launch modes")
        for q in outs:
            assert torch.equal(as_u8(q).cpu(), want), (coop, chain)
        wq, _ = oracle.mxfp8_quantize(x, "ceil")
        assert torch.equal(as_u8(r.q_row).cpu(), as_u8(wq)), (coop, chain)
    with pytest.raises(_lib.TnqError):
        _lib.call("tnq_set_option", 7, 2)


def test_chained_launch_sees_the_previous_kernels_output():
    """A chained kernel starts while the stream's previous kernel drains and must not read its input early:
    the input buffer is rewritten by a torch kernel right before every cast (torch kernel -> cast), the cast's
    output feeds the next kernel of ours (amax -> cast, quantize -> swizzle), twenty times without a host sync."""
    g = torch.Generator().manual_seed(5)
    src = [(torch.randn(2048, 4096, generator=g) * (i + 1)).to(torch.bfloat16) for i in range(4)]
    src_d = [s.to(DEV) for s in src]
    x = torch.empty_like(src_d[0])
    big = torch.empty(8192, 4096, dtype=torch.bfloat16, device=DEV)  # 64 MiB: the two-launch path
    outs, outs_big, swz = [], [], []
    for i in range(20):
        x.copy_(src_d[i % 4])
        outs.append(tn.dynamic_scaled_quant(x))
        big.copy_(src_d[i % 4].repeat(4, 1))
        outs_big.append(tn.dynamic_scaled_quant(big))
        r = tn.quantize_mxfp8(x, swizzle=False)
        swz.append((r.scale_row, tn.to_blocked(r.scale_row)))
    tn.check_status(x.device, "chained launches")
    want = []
    for s in src:
        want.append(as_u8(oracle.fp8_dynamic_quant(s, torch.float8_e4m3fn)[0]))
    for i in range(20):
        assert torch.equal(as_u8(outs[i]).cpu(), want[i % 4]), i
        assert torch.equal(as_u8(outs_big[i]).cpu(), want[i % 4].repeat(4, 1)), i
        assert torch.equal(swz[i][1].cpu(), oracle.to_blocked(swz[i][0].cpu())), i


@pytest.mark.parametrize("n_streams", [2, 4])
def test_single_launch_casts_on_several_streams(n_streams):
    """Host threads cast on streams of their own at once, each with its own workspace, every call chained to its
    predecessor: each call's CTAs are placed together although the launches are not cooperative, so no call runs
    into the bounded wait of its exchange."""
    import threading

    x = make_input("fp8_tensor", "cpu")
    want = as_u8(oracle.fp8_dynamic_quant(x, torch.float8_e4m3fn)[0])
    dev = torch.device(DEV, torch.cuda.current_device())
    xd = x.to(dev)
    torch.cuda.synchronize()
    results, errors = {}, []

    def worker(k):
        try:
            s = torch.cuda.Stream(device=dev)
            ws = torch.zeros(_lib.WORKSPACE_BYTES // 4, dtype=torch.int32, device=dev)
            outs = [torch.empty_like(xd, dtype=torch.float8_e4m3fn) for _ in range(4)]
            s.wait_stream(torch.cuda.current_stream(dev))
            with torch.cuda.stream(s):
                for i in range(200):
                    _lib.call("tnq_fp8_dynamic_cast", xd.data_ptr(), outs[i % 4].data_ptr(), xd.numel(), _lib.IN_BF16,
                              _lib.FP8_E4M3, ws.data_ptr(), 0, s.cuda_stream)
            s.synchronize()
            results[k] = (outs, int(ws[_lib.WS_STATUS_WORD]))
        except Exception as e:  # pragma: no cover - reported below
            errors.append(e)

    threads = [threading.Thread(target=worker, args=(k,)) for k in range(n_streams)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    assert not errors, errors
    for k in range(n_streams):
        outs, status = results[k]
        assert status == 0, (k, status)
        for q in outs:
            assert torch.equal(as_u8(q).cpu(), want), k


@pytest.mark.parametrize("shape,stages,per_sm", [((128, 128), 2, 1), ((1024, 896), 2, 2), ((2048, 4096), 3, 2), ((512, 256), 6, 1)])
def test_tile_copy_diagnostic(shape, stages, per_sm):
    """The arithmetic-free twin of the tile pipeline copies every byte; shapes that are not whole tiles and
    stage counts that do not fit are refused before any launch."""
    g = torch.Generator().manual_seed(shape[0] + shape[1])
    x = torch.randn(*shape, generator=g).to(torch.bfloat16).to(DEV)
    y = torch.zeros_like(x)
    ws = _lib.workspace(x.device)
    status = ws.data_ptr() + 4 * _lib.WS_STATUS_WORD
    for _ in range(3):
        _lib.call("tnq_tile_copy", x.data_ptr(), y.data_ptr(), shape[0], shape[1], stages, per_sm, status, _lib.stream_ptr(x.device))
    tn.check_status(x.device, "tile copy")
    assert torch.equal(as_u8(x), as_u8(y))
    with pytest.raises(_lib.TnqError):
        _lib.call("tnq_tile_copy", x.data_ptr(), y.data_ptr(), shape[0] - 1, shape[1], stages, per_sm, status, _lib.stream_ptr(x.device))
    with pytest.raises(_lib.TnqError):
        _lib.call("tnq_tile_copy", x.data_ptr(), y.data_ptr(), shape[0], shape[1], 6, 4, status, _lib.stream_ptr(x.device))


def test_dynamic_entries_match_their_two_call_forms():
    """tnq_nvfp4_quantize_dynamic and tnq_fp8_dynamic_cast_transpose (amax pass + quantizer in one call) give the
    bytes of the amax call followed by the plain entry point, on a matrix larger than L2 and on ragged small ones."""
    dev = torch.device(DEV, torch.cuda.current_device())
    ws = _lib.workspace(dev)
    stream = _lib.stream_ptr(dev)
    status = ws.data_ptr() + 4 * _lib.WS_STATUS_WORD
    for rows, cols in ((8192, 8192), (160, 272), (128, 128), (32, 16)):
        g = torch.Generator().manual_seed(rows + cols)
        x = (torch.randn(rows, cols, generator=g) * 3).to(torch.bfloat16).to(dev)
        r = tn.quantize_nvfp4(x)  # dynamic entry
        packed = torch.empty(rows, cols // 2, dtype=torch.uint8, device=dev)
        sf = torch.empty_like(r.block_scales.view(torch.uint8))
        gs = torch.empty(1, dtype=torch.float32, device=dev)
        _lib.call("tnq_fp8_amax", x.data_ptr(), x.numel(), _lib.IN_BF16, _lib.FP8_E4M3, ws.data_ptr(), 0, stream)
        _lib.call("tnq_nvfp4_quantize", x.data_ptr(), rows, cols, _lib.IN_BF16, ws.data_ptr() + 4 * _lib.WS_AMAX_WORD,
                  packed.data_ptr(), sf.data_ptr(), _lib.SCALES_SWIZZLED, gs.data_ptr(), status, stream)
        assert torch.equal(r.packed.view(torch.uint8), packed) and torch.equal(r.block_scales.view(torch.uint8), sf)
        assert torch.equal(r.global_scale, gs)
        if cols % 8 == 0:
            q, q_t, scale = tn.fp8.dynamic_scaled_quant_transpose(x)
            want, want_scale = oracle.fp8_dynamic_quant(x.cpu(), torch.float8_e4m3fn)
            assert torch.equal(as_u8(q).cpu(), as_u8(want)) and torch.equal(as_u8(q_t).cpu(), as_u8(want).t().contiguous())
            assert torch.equal(scale.cpu(), want_scale)
    tn.check_status(dev, "dynamic entries")
    x = torch.zeros(128, 128, dtype=torch.bfloat16, device=dev)
    out = torch.empty(128 * 128, dtype=torch.uint8, device=dev)
    with pytest.raises(_lib.TnqError):  # no workspace
        _lib.call("tnq_nvfp4_quantize_dynamic", x.data_ptr(), 128, 128, _lib.IN_BF16, 0, out.data_ptr(), out.data_ptr(),
                  _lib.SCALES_SWIZZLED, 0, stream)
    with pytest.raises(_lib.TnqError):
        _lib.call("tnq_fp8_dynamic_cast_transpose", x.data_ptr(), 128, 128, _lib.IN_BF16, _lib.FP8_E4M3, 0, out.data_ptr(),
                  out.data_ptr(), 0, stream)


@pytest.mark.parametrize("n,k", [(128, 2048), (264, 4096), (130, 2080), (1024, 16384), (8, 65536)])
def test_gemv_cta_shapes_agree(n, k):
    """The two CTA shapes of the block-scaled GEMVs (128 threads x 4 ring slots, 512 threads x 3 slots) agree to a
    bf16 rounding (they cut the rows' sums at different steps), raw and swizzled scales, MXFP8 and NVFP4; at K = 65536
    the wide shape does not fit and the narrow one runs."""
    from transformer_nuggets_b200.cute.blockscaled_tma import BlockScaleLayout
    from transformer_nuggets_b200.cute.mxfp8_tma import mxfp8_tma_gemv
    from transformer_nuggets_b200.cute.nvfp4_tma import nvfp4_tma_gemv

    g = torch.Generator(device=DEV).manual_seed(n + k)
    w = torch.randn(n, k, dtype=torch.bfloat16, device=DEV, generator=g)
    x = torch.randn(1, k, dtype=torch.bfloat16, device=DEV, generator=g)
    try:
        outs = {}
        for shape in (1, 2, 0):
            _lib.call("tnq_gemv_set_shape", shape)
            if k % 32 == 0:
                rw, rx = tn.quantize_mxfp8(w, swizzle=True), tn.quantize_mxfp8(x, swizzle=True)
                y8 = mxfp8_tma_gemv(rx.q_row, rw.q_row, rx.scale_row, rw.scale_row, block_scale_layout=BlockScaleLayout.SWIZZLE_32_4_4)
                rw, rx = tn.quantize_mxfp8(w, swizzle=False), tn.quantize_mxfp8(x, swizzle=False)
                y8r = mxfp8_tma_gemv(rx.q_row, rw.q_row, rx.scale_row, rw.scale_row, block_scale_layout=BlockScaleLayout.RAW)
            aw, ax = tn.quantize_nvfp4(w), tn.quantize_nvfp4(x)
            y4 = nvfp4_tma_gemv(ax.packed, aw.packed, ax.block_scales, aw.block_scales, input_global_scale=ax.global_scale,
                                weight_global_scale=aw.global_scale)
            outs[shape] = (y8.clone(), y8r.clone(), y4.clone())
        for shape in (2, 0):
            for a, b in zip(outs[1], outs[shape]):
                torch.testing.assert_close(a, b, rtol=2.0 ** -7, atol=1e-2)
        assert torch.equal(outs[0][0], outs[0][1])  # swizzled and raw scales: the same kernel, the same cuts
        exact = (x.float() @ w.float().t())
        assert float((outs[0][0].float() - exact).abs().mean() / exact.abs().mean()) < 0.08
        assert float((outs[0][2].float() - exact).abs().mean() / exact.abs().mean()) < 0.2
    finally:
        _lib.call("tnq_gemv_set_shape", 0)
    with pytest.raises(_lib.TnqError):
        _lib.call("tnq_gemv_set_shape", 3)
