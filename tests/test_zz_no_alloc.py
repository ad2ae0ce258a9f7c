"""The allocation-free entry point ``tnq_fp8_dynamic_cast_static`` against the
ordinary ``tnq_fp8_dynamic_cast``, both called through the C ABI.

Some users of the library cannot create device scratch at all - a plug-in that its
host framework hands tensors and a stream but no allocator, or a server whose memory
pool took the whole device at start-up.  For them the library keeps the reduction
scratch in a fixed array of its own, shared by every call on the device.  Because
that array keeps what the previous call left behind, the check runs two calls in a
row with different inputs (a large amax first, a small one second) and demands the
same bytes and the same scale as the caller-scratch entry point each time - bit for
bit, the tolerance every cast test here uses - and the same again against the CPU
oracle.  Further cases cover the branches the two small tensors do not reach: a
tensor above 96 MiB (the cast then walks the tensor backwards behind an amax pass
that asks L2 to keep the tail) and fp32 input with a ragged element count.

The file name sorts last so that a run stopping at the first failure has already
run every other test; the test also passes on its own in a fresh process.
"""

import ctypes

import pytest
import torch

import oracle
from transformer_nuggets_b200 import _lib
from transformer_nuggets_b200.workloads import make_input

pytestmark = pytest.mark.gpu


def _both(x, fp8, out_code):
    dev = x.device
    stream = _lib.stream_ptr(dev)
    n = x.numel()
    in_code = _lib.IN_DTYPES[x.dtype]
    ref_out = torch.empty_like(x, dtype=fp8)
    ref_scale = torch.zeros(1, dtype=torch.float32, device=dev)
    ws = torch.zeros(_lib.WORKSPACE_BYTES // 4, dtype=torch.int32, device=dev)
    _lib.call("tnq_fp8_dynamic_cast", x.data_ptr(), ref_out.data_ptr(), n, in_code, out_code, ws.data_ptr(),
              ref_scale.data_ptr(), stream)
    got_out = torch.empty_like(x, dtype=fp8)
    got_scale = torch.zeros(1, dtype=torch.float32, device=dev)
    _lib.call("tnq_fp8_dynamic_cast_static", x.data_ptr(), got_out.data_ptr(), n, in_code, out_code,
              got_scale.data_ptr(), stream)
    torch.cuda.synchronize()
    return ref_out, ref_scale, got_out, got_scale


@pytest.mark.parametrize("fp8,code", [(torch.float8_e4m3fn, _lib.FP8_E4M3), (torch.float8_e5m2, _lib.FP8_E5M2)])
def test_static_scratch_entry_point_matches_on_two_calls_in_a_row(fp8, code):
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    big = make_input("fp8_tensor", dev, rows=2048, cols=4096) * 64  # amax in the thousands
    small = make_input("fp8_sharded", dev, rows=1537, cols=999) * 0.01  # odd element count (ragged tail), small amax
    for x in (big, small):
        ref_out, ref_scale, got_out, got_scale = _both(x, fp8, code)
        assert torch.equal(got_scale, ref_scale)
        assert torch.equal(got_out.view(torch.uint8), ref_out.view(torch.uint8))
        want, want_scale = oracle.fp8_dynamic_quant(x.cpu(), fp8)
        assert torch.equal(got_scale.cpu(), want_scale)
        assert torch.equal(got_out.view(torch.uint8).cpu(), want.view(torch.uint8))
    assert float(ref_scale) > 1.0  # the second call really had a different scale from the first


def test_static_scratch_entry_point_large_and_fp32_inputs():
    """128 MiB of bf16 (above the size from which the cast walks backwards) and a ragged fp32
    tensor, each bit for bit against the caller-scratch entry point and the oracle."""
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    big = make_input("fp8_sharded", dev, rows=8192, cols=8192)
    ragged = (make_input("fp8_tensor", dev, rows=515, cols=1001).float() * 3.3).contiguous()
    for x in (big, ragged):
        ref_out, ref_scale, got_out, got_scale = _both(x, torch.float8_e4m3fn, _lib.FP8_E4M3)
        assert torch.equal(got_scale, ref_scale)
        assert torch.equal(got_out.view(torch.uint8), ref_out.view(torch.uint8))
        want, want_scale = oracle.fp8_dynamic_quant(x.cpu(), torch.float8_e4m3fn)
        assert torch.equal(got_scale.cpu(), want_scale)
        assert torch.equal(got_out.view(torch.uint8).cpu(), want.view(torch.uint8))


def test_static_scratch_entry_point_refuses_oversized_input():
    lib = _lib.load()
    limit = lib.tnq_fp8_dynamic_cast_static_max_elements()
    assert limit == 1 << 32
    rc = lib.tnq_fp8_dynamic_cast_static(ctypes.c_void_p(256), ctypes.c_void_p(256), limit + 16, _lib.IN_BF16,
                                         _lib.FP8_E4M3, None, None)
    assert rc == 4 and b"size" in lib.tnq_status_str(rc)
