"""FP8 matmul with per-tensor or row-wise scaling, entry points of
``transformer_nuggets/fp8/fp8_matmul.py``: ``c = (a @ b) * a_scale * b_scale``.

The reference ships three Triton kernels behind three launchers (``matmul_persistent``,
``matmul_tma_persistent``, ``matmul_device_tma_persistent``, fp8/fp8_matmul.py:241-288,
404-474, 604-651); here one tcgen05 kernel (``csrc/fp8_gemm.cu``) serves all three names.
"""

from __future__ import annotations

import torch

from .. import _lib


def validate_matmul_inputs(a: torch.Tensor, b: torch.Tensor, a_scale: torch.Tensor, b_scale: torch.Tensor) -> bool:
    """Same checks and messages as the reference (fp8/fp8_matmul.py:32-70); returns True for
    row-wise scaling (``a_scale [M, 1]``, ``b_scale [1, N]``), False for per-tensor scaling."""
    assert a.shape[1] == b.shape[0], "Incompatible dimensions"
    assert a.dtype == b.dtype, "Incompatible dtypes"
    row_wise = a_scale.numel() != 1
    if row_wise:
        assert a_scale.dim() == 2, f"a_scale must be a 2D tensor but got {a_scale.dim()}"
        assert b_scale.dim() == 2, f"b_scale must be a 2D tensor but got {b_scale.dim()}"
        assert a_scale.shape[0] == a.shape[0], (
            f"a_scale must have same number of rows as a, got {a_scale.shape[0]} vs {a.shape[0]}"
        )
        assert a_scale.shape[1] == 1, f"a_scale must have 1 column, got {a_scale.shape[1]}"
        assert b_scale.shape[1] == b.shape[1], (
            f"b_scale must have same number of columns as b, got {b_scale.shape[0]} vs {b.shape[1]}"
        )
        assert b_scale.shape[0] == 1, f"b_scale must have 1 column, got {b_scale.shape[1]}"
    else:
        assert a_scale.numel() == 1, f"a_scale must be a scalar for per-tensor scaling, got shape {a_scale.shape}"
        assert b_scale.numel() == 1, f"b_scale must be a scalar for per-tensor scaling, got shape {b_scale.shape}"
    return row_wise


def matmul_persistent(a: torch.Tensor, a_scale: torch.Tensor, b: torch.Tensor, b_scale: torch.Tensor,
                      output_dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    """``a [M, K]`` row-major fp8, ``b [K, N]`` column-major fp8 (``b.t()`` contiguous, the layout
    of a weight stored ``[N, K]``), fp32 scales in the dequantisation direction -> ``[M, N]`` bf16."""
    row_wise = validate_matmul_inputs(a, b, a_scale, b_scale)
    for name, t in (("a", a), ("b", b), ("a_scale", a_scale), ("b_scale", b_scale)):
        _lib.require_cuda(t, name)
    if a.dtype not in _lib.FP8_DTYPES:
        raise TypeError(f"a and b must be float8_e4m3fn or float8_e5m2, got {a.dtype}")
    if output_dtype != torch.bfloat16:
        raise TypeError("output_dtype must be torch.bfloat16")
    if a_scale.dtype != torch.float32 or b_scale.dtype != torch.float32:
        raise TypeError("scales must be float32")
    if not a.is_contiguous() or not b.t().is_contiguous():
        raise ValueError("a must be row-major and b column-major (b.t() contiguous)")
    m, k = a.shape
    n = b.shape[1]
    if k % 16 != 0:
        raise ValueError("K must be a multiple of 16")
    dev = a.device
    sa, sb = a_scale.contiguous(), b_scale.contiguous()
    c = torch.empty((m, n), device=dev, dtype=torch.bfloat16)
    with torch.cuda.device(dev):
        _lib.call("tnq_fp8_gemm", a.data_ptr(), b.data_ptr(), sa.data_ptr(), sb.data_ptr(), int(row_wise),
                  _lib.FP8_DTYPES[a.dtype], m, n, k, c.data_ptr(), _lib.workspace(dev).data_ptr() + 4 * _lib.WS_STATUS_WORD,
                  _lib.stream_ptr(dev))
    return c


matmul_tma_persistent = matmul_persistent
matmul_device_tma_persistent = matmul_persistent
