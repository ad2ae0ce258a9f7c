"""CUDA-graph capture of the cast entry points with caller-owned outputs: capture,
replay on changed input, compare with the oracle.  Mirrors the reference's capture test
for its CuTe ops (test/test_mxfp8_tma.py:249-285)."""

import pytest
import torch

import oracle
from conftest import as_u8
from transformer_nuggets_b200 import _lib
from transformer_nuggets_b200.workloads import make_input

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _capture(fn):
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        fn(s)  # warm-up outside capture: attribute queries, first-use set-up
    torch.cuda.current_stream().wait_stream(s)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g, stream=s):
        fn(s)
    return g


@pytest.mark.parametrize("rows", [512, 8192])  # single-launch kernel / two-launch path (128 MiB > shared memory)
def test_dynamic_cast_graph(rows):
    x = make_input("fp8_tensor", DEV, rows=rows, cols=8192)
    out = torch.empty_like(x, dtype=torch.float8_e4m3fn)
    scale = torch.zeros(1, dtype=torch.float32, device=DEV)
    ws = torch.zeros(_lib.WORKSPACE_BYTES // 4, dtype=torch.int32, device=DEV)

    def run(stream):
        _lib.call("tnq_fp8_dynamic_cast", x.data_ptr(), out.data_ptr(), x.numel(), _lib.IN_BF16, _lib.FP8_E4M3,
                  ws.data_ptr(), scale.data_ptr(), stream.cuda_stream)

    g = _capture(run)
    for k in (1.0, 0.25):
        x.mul_(k)
        g.replay()
        torch.cuda.synchronize()
        want, wscale = oracle.fp8_dynamic_quant(x.cpu(), torch.float8_e4m3fn)
        assert torch.equal(scale.cpu(), wscale) and torch.equal(as_u8(out).cpu(), as_u8(want))


def test_rowwise_and_blockscaled_graph():
    x = make_input("mxfp8", DEV, rows=512, cols=1024)
    rows, cols = x.shape
    q43 = torch.empty(rows, cols, dtype=torch.uint8, device=DEV)
    q52 = torch.empty_like(q43)
    s43 = torch.empty(rows, dtype=torch.float32, device=DEV)
    s52 = torch.empty_like(s43)
    qr = torch.empty_like(q43)
    qc = torch.empty(cols, rows, dtype=torch.uint8, device=DEV)
    sr = torch.empty(rows, cols // 32, dtype=torch.uint8, device=DEV)
    sc = torch.empty(cols, rows // 32, dtype=torch.uint8, device=DEV)
    packed = torch.empty(rows, cols // 2, dtype=torch.uint8, device=DEV)
    sf = torch.empty(rows, cols // 16, dtype=torch.uint8, device=DEV)
    gs = torch.empty(1, dtype=torch.float32, device=DEV)
    ws = torch.zeros(_lib.WORKSPACE_BYTES // 4, dtype=torch.int32, device=DEV)
    status = ws.data_ptr() + 4 * _lib.WS_STATUS_WORD
    amax = ws.data_ptr() + 4 * _lib.WS_AMAX_WORD

    def run(stream):
        st = stream.cuda_stream
        _lib.call("tnq_fp8_rowwise", x.data_ptr(), rows, cols, _lib.IN_BF16, q43.data_ptr(), s43.data_ptr(),
                  q52.data_ptr(), s52.data_ptr(), status, st)
        _lib.call("tnq_mxfp8_quantize", x.data_ptr(), rows, cols, _lib.IN_BF16, qr.data_ptr(), sr.data_ptr(),
                  qc.data_ptr(), sc.data_ptr(), _lib.E8M0_CEIL, _lib.SCALES_RAW, status, st)
        _lib.call("tnq_fp8_amax", x.data_ptr(), x.numel(), _lib.IN_BF16, _lib.FP8_E4M3, ws.data_ptr(), 0, st)
        _lib.call("tnq_nvfp4_quantize", x.data_ptr(), rows, cols, _lib.IN_BF16, amax, packed.data_ptr(), sf.data_ptr(),
                  _lib.SCALES_RAW, gs.data_ptr(), status, st)

    g = _capture(run)
    x.mul_(0.5)
    g.replay()
    torch.cuda.synchronize()
    xc = x.cpu()
    w43, ws43 = oracle.fp8_rowwise_quant(xc, torch.float8_e4m3fn)
    w52, _ = oracle.fp8_rowwise_quant(xc, torch.float8_e5m2)
    assert torch.equal(q43.cpu(), as_u8(w43)) and torch.equal(q52.cpu(), as_u8(w52))
    assert torch.equal(s43.cpu(), ws43.reshape(-1))
    wq, wsr = oracle.mxfp8_quantize(xc, "ceil")
    wqt, wsc = oracle.mxfp8_quantize(xc.t().contiguous(), "ceil")
    assert torch.equal(qr.cpu(), as_u8(wq)) and torch.equal(sr.cpu(), wsr)
    assert torch.equal(qc.cpu(), as_u8(wqt)) and torch.equal(sc.cpu(), wsc)
    wp, wsf, wg = oracle.nvfp4_quantize(xc)
    assert torch.equal(packed.cpu(), wp) and torch.equal(sf.cpu(), as_u8(wsf)) and torch.equal(gs.cpu(), wg)
    assert int(ws[_lib.WS_STATUS_WORD].item()) == 0


def test_dynamic_tile_entries_graph():
    """The one-call dynamic NVFP4 quantizer and the dynamic transposing cast captured in a graph and replayed
    on changed input (chained launches inside the graph: each node starts behind its predecessor)."""
    x = make_input("mxfp8", DEV, rows=1024, cols=2048)
    rows, cols = x.shape
    packed = torch.empty(rows, cols // 2, dtype=torch.uint8, device=DEV)
    sf = torch.empty(512 * (rows // 128) * (cols // 64), dtype=torch.uint8, device=DEV)
    gs = torch.empty(1, dtype=torch.float32, device=DEV)
    q = torch.empty(rows, cols, dtype=torch.uint8, device=DEV)
    q_t = torch.empty(cols, rows, dtype=torch.uint8, device=DEV)
    scale = torch.empty(1, dtype=torch.float32, device=DEV)
    ws = torch.zeros(_lib.WORKSPACE_BYTES // 4, dtype=torch.int32, device=DEV)

    def run(stream):
        st = stream.cuda_stream
        _lib.call("tnq_nvfp4_quantize_dynamic", x.data_ptr(), rows, cols, _lib.IN_BF16, ws.data_ptr(), packed.data_ptr(),
                  sf.data_ptr(), _lib.SCALES_SWIZZLED, gs.data_ptr(), st)
        _lib.call("tnq_fp8_dynamic_cast_transpose", x.data_ptr(), rows, cols, _lib.IN_BF16, _lib.FP8_E4M3, ws.data_ptr(),
                  q.data_ptr(), q_t.data_ptr(), scale.data_ptr(), st)

    g = _capture(run)
    for k in (1.0, 3.0):
        x.mul_(k)
        g.replay()
        torch.cuda.synchronize()
        xc = x.cpu()
        wp, wsf, wg = oracle.nvfp4_quantize(xc)
        assert torch.equal(packed.cpu(), wp) and torch.equal(sf.cpu(), oracle.to_blocked(as_u8(wsf))) and torch.equal(gs.cpu(), wg)
        want, wscale = oracle.fp8_dynamic_quant(xc, torch.float8_e4m3fn)
        assert torch.equal(q.cpu(), as_u8(want)) and torch.equal(q_t.cpu(), as_u8(want).t().contiguous())
        assert torch.equal(scale.cpu(), wscale)
    assert int(ws[_lib.WS_STATUS_WORD].item()) == 0
