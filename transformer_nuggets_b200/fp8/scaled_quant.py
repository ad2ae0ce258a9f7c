"""FP8 casts with the entry points of ``transformer_nuggets/fp8/scaled_quant.py``.

``scaled_quant`` and ``dynamic_scaled_quant`` keep the reference's signatures
and return only the fp8 tensor (fp8/scaled_quant.py:35-41, 139-141).  The
``*_with_scale`` and row-wise functions are additions.
"""

from __future__ import annotations

import torch

from .. import _lib


def _check_input(inpt_tensor: torch.Tensor):
    _lib.require_cuda(inpt_tensor, "inpt_tensor")
    assert inpt_tensor.is_contiguous(), "Input tensor must be contiguous"
    if inpt_tensor.dtype not in _lib.IN_DTYPES:
        raise TypeError(f"input dtype must be bfloat16 or float32, got {inpt_tensor.dtype}")
    if inpt_tensor.data_ptr() % 32 != 0:
        raise ValueError("input tensor must start on a 32-byte boundary")


def _check_fp8(fp8_dtype):
    if fp8_dtype not in _lib.FP8_DTYPES:
        raise TypeError(f"fp8_dtype must be float8_e4m3fn or float8_e5m2, got {fp8_dtype}")


def scaled_quant(
    inpt_tensor: torch.Tensor,
    scale: torch.Tensor,
    abs_max: torch.Tensor,
    fp8_dtype: torch.dtype = torch.float8_e4m3fn,
    saturated: bool = False,
) -> torch.Tensor:
    """Quantize to fp8 with a delayed scale and update ``abs_max`` in place to
    ``max(abs_max, max|inpt_tensor|)`` for the next iteration.

    Same contract as the reference (fp8/scaled_quant.py:35-75): fp32 ``scale`` and
    ``abs_max`` of one element, contiguous input, returns the fp8 tensor.  With
    ``saturated=False`` an overflowing product becomes NaN (e4m3fn) or inf (e5m2),
    as in ``eager_scaled_quant`` (fp8/scaled_quant.py:95-102).
    """
    assert scale.dtype == torch.float32
    assert abs_max.dtype == torch.float32
    assert scale.numel() == 1
    assert abs_max.numel() == 1
    _check_input(inpt_tensor)
    _check_fp8(fp8_dtype)
    _lib.require_cuda(scale, "scale")
    _lib.require_cuda(abs_max, "abs_max")
    dev = inpt_tensor.device
    out = torch.empty_like(inpt_tensor, dtype=fp8_dtype)
    with torch.cuda.device(dev):
        _lib.call(
            "tnq_fp8_scaled_cast", inpt_tensor.data_ptr(), out.data_ptr(), inpt_tensor.numel(),
            _lib.IN_DTYPES[inpt_tensor.dtype], _lib.FP8_DTYPES[fp8_dtype], scale.data_ptr(),
            _lib.SCALE_IS_SCALE, int(bool(saturated)), abs_max.data_ptr(), _lib.workspace(dev).data_ptr(),
            _lib.stream_ptr(dev),
        )
    return out


def dynamic_scaled_quant_with_scale(
    inpt_tensor: torch.Tensor, fp8_dtype: torch.dtype = torch.float8_e4m3fn, out: torch.Tensor | None = None
):
    """Per-tensor dynamic cast returning ``(fp8 tensor, fp32 scale of shape [1])``
    with ``scale = finfo(fp8_dtype).max / max(amax, 1e-12)``."""
    _check_input(inpt_tensor)
    _check_fp8(fp8_dtype)
    dev = inpt_tensor.device
    if out is None:
        out = torch.empty_like(inpt_tensor, dtype=fp8_dtype)
    else:
        _lib.require_cuda(out, "out")
        if out.dtype != fp8_dtype or out.shape != inpt_tensor.shape or not out.is_contiguous():
            raise ValueError("out must be a contiguous fp8 tensor of the input's shape")
    scale = torch.empty(1, dtype=torch.float32, device=dev)
    with torch.cuda.device(dev):
        _lib.call(
            "tnq_fp8_dynamic_cast", inpt_tensor.data_ptr(), out.data_ptr(), inpt_tensor.numel(),
            _lib.IN_DTYPES[inpt_tensor.dtype], _lib.FP8_DTYPES[fp8_dtype], _lib.workspace(dev).data_ptr(),
            scale.data_ptr(), _lib.stream_ptr(dev),
        )
    return out, scale


def eager_scaled_quant(
    a: torch.Tensor,
    scale: torch.Tensor,
    abs_max: torch.Tensor,
    fp8_dtype: torch.dtype,
    saturated: bool = False,
) -> torch.Tensor:
    """The reference's ``eager_scaled_quant`` (fp8/scaled_quant.py:78-102) under its own name,
    served by the same CUDA kernel as ``scaled_quant``: identical bytes, and ``abs_max`` is
    OVERWRITTEN with ``max|a|`` (the eager twin fills, the fused kernel accumulates)."""
    abs_max.zero_()
    return scaled_quant(a, scale, abs_max, fp8_dtype, saturated)


def eager_dynamic_scaled_quant(a: torch.Tensor, fp8_dtype: torch.dtype) -> torch.Tensor:
    """The reference's ``eager_dynamic_scaled_quant`` (fp8/scaled_quant.py:172-186) under its own
    name: ``scale = finfo.max / max(amax, 1e-12)``, saturated cast, served by the CUDA path."""
    return dynamic_scaled_quant(a, fp8_dtype)


def _check_matrix(inpt_tensor: torch.Tensor):
    _check_input(inpt_tensor)
    if inpt_tensor.dim() != 2:
        raise ValueError("the transposing casts take a 2-D tensor")
    if inpt_tensor.dtype != torch.bfloat16:
        raise TypeError("the transposing casts take bfloat16 input")
    if inpt_tensor.shape[1] % 8 != 0:
        raise ValueError("the number of columns must be a multiple of 8")


def scaled_quant_transpose(
    inpt_tensor: torch.Tensor,
    scale: torch.Tensor,
    abs_max: torch.Tensor | None = None,
    fp8_dtype: torch.dtype = torch.float8_e4m3fn,
    saturated: bool = False,
):
    """``scaled_quant`` of a 2-D bf16 tensor that also returns the transposed copy:
    ``(q [R, C], q_t [C, R])`` with ``q_t == q.t().contiguous()`` byte for byte, from one
    read of the input.  ``abs_max`` (optional, one fp32 element) becomes
    ``max(abs_max, max|inpt_tensor|)`` as in ``scaled_quant``."""
    _check_matrix(inpt_tensor)
    _check_fp8(fp8_dtype)
    assert scale.dtype == torch.float32 and scale.numel() == 1
    _lib.require_cuda(scale, "scale")
    if abs_max is not None:
        assert abs_max.dtype == torch.float32 and abs_max.numel() == 1
        _lib.require_cuda(abs_max, "abs_max")
    dev = inpt_tensor.device
    rows, cols = inpt_tensor.shape
    out = torch.empty_like(inpt_tensor, dtype=fp8_dtype)
    out_t = torch.empty(cols, rows, dtype=fp8_dtype, device=dev)
    with torch.cuda.device(dev):
        _lib.call(
            "tnq_fp8_cast_transpose", inpt_tensor.data_ptr(), rows, cols, _lib.IN_BF16, _lib.FP8_DTYPES[fp8_dtype],
            scale.data_ptr(), _lib.SCALE_IS_SCALE, int(bool(saturated)), 0 if abs_max is None else abs_max.data_ptr(),
            out.data_ptr(), out_t.data_ptr(), _lib.workspace(dev).data_ptr() + 4 * _lib.WS_STATUS_WORD,
            _lib.stream_ptr(dev),
        )
    return out, out_t


def dynamic_scaled_quant_transpose(inpt_tensor: torch.Tensor, fp8_dtype: torch.dtype = torch.float8_e4m3fn):
    """Per-tensor dynamic saturated cast of a 2-D bf16 tensor in both layouts:
    ``(q [R, C], q_t [C, R], scale [1])``.  One amax pass, then one pass that reads the
    input once and writes both outputs."""
    _check_matrix(inpt_tensor)
    _check_fp8(fp8_dtype)
    dev = inpt_tensor.device
    rows, cols = inpt_tensor.shape
    out = torch.empty_like(inpt_tensor, dtype=fp8_dtype)
    out_t = torch.empty(cols, rows, dtype=fp8_dtype, device=dev)
    scale = torch.empty(1, dtype=torch.float32, device=dev)
    with torch.cuda.device(dev):
        _lib.call(
            "tnq_fp8_dynamic_cast_transpose", inpt_tensor.data_ptr(), rows, cols, _lib.IN_BF16, _lib.FP8_DTYPES[fp8_dtype],
            _lib.workspace(dev).data_ptr(), out.data_ptr(), out_t.data_ptr(), scale.data_ptr(), _lib.stream_ptr(dev),
        )
    return out, out_t, scale


def dynamic_scaled_quant(inpt_tensor: torch.Tensor, fp8_dtype: torch.dtype = torch.float8_e4m3fn) -> torch.Tensor:
    """Quantize to fp8 with the scale computed from the tensor's current amax;
    saturated cast.  Returns the fp8 tensor only, like the reference
    (fp8/scaled_quant.py:139-169)."""
    _check_input(inpt_tensor)
    _check_fp8(fp8_dtype)
    dev = inpt_tensor.device
    out = torch.empty_like(inpt_tensor, dtype=fp8_dtype)
    with torch.cuda.device(dev):
        _lib.call(
            "tnq_fp8_dynamic_cast", inpt_tensor.data_ptr(), out.data_ptr(), inpt_tensor.numel(),
            _lib.IN_DTYPES[inpt_tensor.dtype], _lib.FP8_DTYPES[fp8_dtype], _lib.workspace(dev).data_ptr(),
            0, _lib.stream_ptr(dev),
        )
    return out


def rowwise_scaled_quant(inpt_tensor: torch.Tensor, fp8_dtypes=(torch.float8_e4m3fn, torch.float8_e5m2)):
    """Row-wise dynamic cast of a 2-D tensor.  For each dtype in ``fp8_dtypes``
    returns ``(fp8 [M, K], fp32 scale [M, 1])`` with ``scale_r = max / max(amax_r,
    1e-12)``; all requested outputs come from one read of the input.  The scale
    shape is the per-row contract of the reference's fp8 matmul
    (fp8/fp8_matmul.py:50-61)."""
    _check_input(inpt_tensor)
    if inpt_tensor.dim() != 2:
        raise ValueError("rowwise_scaled_quant expects a 2-D tensor")
    if isinstance(fp8_dtypes, torch.dtype):
        fp8_dtypes = (fp8_dtypes,)
    for d in fp8_dtypes:
        _check_fp8(d)
    if len(set(fp8_dtypes)) != len(fp8_dtypes) or not fp8_dtypes:
        raise ValueError("fp8_dtypes must name each dtype at most once")
    rows, cols = inpt_tensor.shape
    per_vec = 16 if inpt_tensor.dtype == torch.bfloat16 else 8
    if cols % per_vec != 0:
        raise ValueError(f"the row length must be a multiple of {per_vec} elements")
    dev = inpt_tensor.device
    outs = {}
    for d in fp8_dtypes:
        outs[d] = (torch.empty_like(inpt_tensor, dtype=d), torch.empty(rows, 1, dtype=torch.float32, device=dev))
    q43, s43 = outs.get(torch.float8_e4m3fn, (None, None))
    q52, s52 = outs.get(torch.float8_e5m2, (None, None))
    with torch.cuda.device(dev):
        _lib.call(
            "tnq_fp8_rowwise", inpt_tensor.data_ptr(), rows, cols, _lib.IN_DTYPES[inpt_tensor.dtype],
            _lib.ptr(q43), _lib.ptr(s43), _lib.ptr(q52), _lib.ptr(s52),
            _lib.workspace(dev).data_ptr() + 4 * _lib.WS_STATUS_WORD, _lib.stream_ptr(dev),
        )
    res = tuple(outs[d] for d in fp8_dtypes)
    return res[0] if len(res) == 1 else res
