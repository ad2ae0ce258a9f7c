"""FP8 GEMM with scale epilogue (tcgen05) against the oracle's fp32 matmul of the same fp8
operands and against the library GEMM (torch._scaled_mm).  Floating point: products are exact,
the accumulation order differs, the result is rounded to bf16 - compared within one bf16 step
of relative error."""

import pytest
import torch

import oracle
from transformer_nuggets_b200 import _lib
from transformer_nuggets_b200.fp8.fp8_matmul import matmul_persistent, matmul_tma_persistent

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _operands(m, n, k, dtype, seed):
    g = torch.Generator().manual_seed(seed)
    a = (torch.randn(m, k, generator=g) * 2.0).to(dtype)
    b_nk = (torch.randn(n, k, generator=g) * 2.0).to(dtype)  # weight stored [N, K]
    return a, b_nk


@pytest.mark.parametrize("m,n,k", [(128, 256, 128), (128, 256, 512), (256, 512, 1024), (100, 72, 80), (2, 8, 16),
                                   (300, 520, 272), (1024, 1024, 4096)])
@pytest.mark.parametrize("dtype", [torch.float8_e4m3fn, torch.float8_e5m2])
@pytest.mark.parametrize("row_wise", [False, True])
def test_matches_oracle(m, n, k, dtype, row_wise):
    a, b_nk = _operands(m, n, k, dtype, m + n + k)
    g = torch.Generator().manual_seed(7)
    if row_wise:
        a_scale = torch.rand(m, 1, generator=g) + 0.5
        b_scale = torch.rand(1, n, generator=g) + 0.5
    else:
        a_scale, b_scale = torch.tensor([0.75]), torch.tensor([1.5])
    want = oracle.fp8_matmul(a, a_scale, b_nk.t(), b_scale)
    got = matmul_persistent(a.to(DEV), a_scale.to(DEV), b_nk.to(DEV).t(), b_scale.to(DEV), torch.bfloat16)
    st = int(_lib.workspace(torch.device(DEV, 0))[_lib.WS_STATUS_WORD].item())
    assert st == 0
    assert got.shape == (m, n) and got.dtype == torch.bfloat16
    torch.testing.assert_close(got.cpu().float(), want.float(), rtol=2 ** -7, atol=2 ** -7 * float(k) ** 0.5)


def test_against_library_gemm():
    m, n, k = 2048, 4096, 4096
    a, b_nk = _operands(m, n, k, torch.float8_e4m3fn, 3)
    a, b_nk = a.to(DEV), b_nk.to(DEV)
    sa, sb = torch.tensor([0.5], device=DEV), torch.tensor([0.25], device=DEV)
    got = matmul_tma_persistent(a, sa, b_nk.t(), sb, torch.bfloat16)
    ref = torch._scaled_mm(a, b_nk.t(), scale_a=sa, scale_b=sb, out_dtype=torch.bfloat16)
    torch.testing.assert_close(got.float(), ref.float(), rtol=2 ** -7, atol=1.0)


def test_argument_checks():
    a = torch.zeros(16, 32, device=DEV).to(torch.float8_e4m3fn)
    b = torch.zeros(8, 32, device=DEV).to(torch.float8_e4m3fn)
    one = torch.ones(1, device=DEV)
    with pytest.raises(AssertionError):
        matmul_persistent(a, one, b, one)  # b is [N, K], not [K, N]
    with pytest.raises(ValueError):
        matmul_persistent(a, one, b.t().contiguous(), one)  # b row-major
    with pytest.raises(AssertionError):
        matmul_persistent(a, torch.ones(16, 1, device=DEV), b.t(), torch.ones(1, 5, device=DEV))
    with pytest.raises(TypeError):
        matmul_persistent(a, one, b.t(), one, torch.float16)


@pytest.mark.parametrize("row_wise", [False, True])
def test_casts_feed_the_gemm_end_to_end(row_wise):
    """bf16 activation and weight -> this library's casts -> this library's GEMM with the
    reciprocal scales: close to the bf16 matmul within fp8 quantisation error."""
    import transformer_nuggets_b200 as tn

    g = torch.Generator(device=DEV).manual_seed(17)
    x = torch.randn(512, 1024, device=DEV, generator=g).to(torch.bfloat16)
    w = (torch.randn(768, 1024, device=DEV, generator=g) * 0.05).to(torch.bfloat16)  # stored [N, K]
    if row_wise:
        qx, sx = tn.rowwise_scaled_quant(x, torch.float8_e4m3fn)
        qw, sw = tn.rowwise_scaled_quant(w, torch.float8_e4m3fn)
        a_scale, b_scale = 1.0 / sx, (1.0 / sw).t().contiguous()
    else:
        qx, sx = tn.dynamic_scaled_quant_with_scale(x)
        qw, sw = tn.dynamic_scaled_quant_with_scale(w)
        a_scale, b_scale = 1.0 / sx, 1.0 / sw
    got = matmul_persistent(qx, a_scale, qw.t(), b_scale, torch.bfloat16).float()
    ref = x.float() @ w.float().t()
    err = (got - ref).abs().max().item() / ref.abs().max().item()
    assert err < 0.06, err


def test_graph_capture_and_replay():
    m, n, k = 256, 512, 512
    a, b_nk = _operands(m, n, k, torch.float8_e4m3fn, 23)
    a, b_nk = a.to(DEV), b_nk.to(DEV)
    sa, sb = torch.tensor([1.0], device=DEV), torch.tensor([0.5], device=DEV)
    c = torch.zeros(m, n, dtype=torch.bfloat16, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    side = torch.cuda.Stream()

    def launch():
        _lib.call("tnq_fp8_gemm", a.data_ptr(), b_nk.data_ptr(), sa.data_ptr(), sb.data_ptr(), 0, _lib.FP8_E4M3, m, n, k,
                  c.data_ptr(), status.data_ptr(), side.cuda_stream)

    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        launch()
    torch.cuda.synchronize()
    first = c.clone()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=side):
        launch()
    c.zero_()
    a.copy_((a.float() * 0.5).to(torch.float8_e4m3fn))  # new operand values, same buffers
    graph.replay()
    torch.cuda.synchronize()
    want = oracle.fp8_matmul(a.cpu(), sa.cpu(), b_nk.cpu().t(), sb.cpu())
    torch.testing.assert_close(c.cpu().float(), want.float(), rtol=2 ** -7, atol=0.5)
    assert status.item() == 0 and not torch.equal(first, c)


def test_output_on_a_16_byte_boundary_only():
    """The epilogue writes 256 bits per lane when every output row starts on a 32-byte boundary
    and 128 bits otherwise; both paths give the same bits."""
    m, n, k = 256, 512, 256
    a, b_nk = _operands(m, n, k, torch.float8_e4m3fn, 11)
    a, b_nk = a.to(DEV), b_nk.to(DEV)
    one = torch.ones(1, device=DEV)
    want = matmul_persistent(a, one, b_nk.t(), one)
    dev = torch.device(DEV, 0)
    buf = torch.zeros(m * n + 16, dtype=torch.bfloat16, device=DEV)
    assert buf.data_ptr() % 32 == 0
    shifted = buf[8:8 + m * n]  # 16 bytes past a 32-byte boundary
    with torch.cuda.device(dev):
        _lib.call("tnq_fp8_gemm", a.data_ptr(), b_nk.data_ptr(), one.data_ptr(), one.data_ptr(), 0,
                  _lib.FP8_DTYPES[a.dtype], m, n, k, shifted.data_ptr(),
                  _lib.workspace(dev).data_ptr() + 4 * _lib.WS_STATUS_WORD, _lib.stream_ptr(dev))
    torch.cuda.synchronize()
    assert torch.equal(shifted.view(m, n).view(torch.int16), want.view(torch.int16))
    assert int(buf[:8].view(torch.int16).abs().sum()) == 0 and int(buf[8 + m * n:].view(torch.int16).abs().sum()) == 0
