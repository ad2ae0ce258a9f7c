"""Producer epilogues: RMSNorm or SwiGLU fused into the row-wise FP8 cast or the MXFP8
row-wise quantizer (the bf16 activation the producer would write is never stored unless
asked for)."""

from __future__ import annotations

import torch

from .. import _lib


def _check(x: torch.Tensor, weight: torch.Tensor, multiple: int):
    _lib.require_cuda(x, "x")
    _lib.require_cuda(weight, "weight")
    if x.dtype != torch.bfloat16 or weight.dtype != torch.bfloat16:
        raise TypeError("x and weight must be bfloat16")
    if x.dim() < 1 or weight.dim() != 1 or weight.shape[0] != x.shape[-1]:
        raise ValueError("weight must be a vector of x's last dimension")
    if not x.is_contiguous() or not weight.is_contiguous():
        raise ValueError("x and weight must be contiguous")
    cols = x.shape[-1]
    if cols % multiple != 0 or cols > 16384:
        raise ValueError(f"the normalised dimension must be a multiple of {multiple} and at most 16384")
    if x.data_ptr() % 32 != 0 or weight.data_ptr() % 32 != 0:
        raise ValueError("x and weight must start on a 32-byte boundary")
    if weight.device != x.device:
        raise ValueError("x and weight must be on the same device")


def rms_norm_quantize_mxfp8(x: torch.Tensor, weight: torch.Tensor, eps: float = 1e-6, *, scale_mode: str = "ceil",
                            swizzle: bool = False, return_normed: bool = False):
    """``y = rms_norm(x, weight, eps)`` followed by the MXFP8 row-wise quantizer
    (``quantize_mxfp8_tensor``'s rule, or the floor rule) on ``y``, in one pass over ``x``.

    Returns ``(q e4m3 [..., C], scales uint8)`` - scales ``[rows, C/32]`` raw, or the flat
    swizzled 128x4 buffer when ``swizzle`` is set - plus ``y`` when ``return_normed`` is set.
    """
    _check(x, weight, 32)
    if scale_mode not in ("ceil", "floor"):
        raise ValueError("scale_mode must be 'ceil' or 'floor'")
    cols = x.shape[-1]
    rows = x.numel() // cols
    dev = x.device
    q = torch.empty_like(x, dtype=torch.float8_e4m3fn)
    w = cols // 32
    if swizzle:
        n = 512 * ((rows + 127) // 128) * ((w + 3) // 4)
        padded = rows % 128 != 0 or w % 4 != 0
        sf = (torch.zeros if padded else torch.empty)(n, dtype=torch.uint8, device=dev)
    else:
        sf = torch.empty(rows, w, dtype=torch.uint8, device=dev)
    y = torch.empty_like(x) if return_normed else None
    with torch.cuda.device(dev):
        _lib.call("tnq_rmsnorm_mxfp8", x.data_ptr(), weight.data_ptr(), float(eps), rows, cols, q.data_ptr(), sf.data_ptr(),
                  _lib.E8M0_CEIL if scale_mode == "ceil" else _lib.E8M0_FLOOR, _lib.SCALES_SWIZZLED if swizzle else _lib.SCALES_RAW,
                  0 if y is None else y.data_ptr(), _lib.stream_ptr(dev))
    return (q, sf, y) if return_normed else (q, sf)


def rms_norm_rowwise_quant(x: torch.Tensor, weight: torch.Tensor, eps: float = 1e-6, *, return_normed: bool = False):
    """``y = rms_norm(x, weight, eps)`` (the eager formula of the reference's fusion example,
    examples/rms_norm_fusion_profile.py:26-31) followed by the per-row dynamic saturated
    e4m3 cast of ``y``, in one pass over ``x``.

    ``x``: bf16 ``[..., C]`` contiguous, ``C`` a multiple of 16 and at most 16384;
    ``weight``: bf16 ``[C]``.  Returns ``(q e4m3 [..., C], scale fp32 [..., 1])`` with
    ``scale = 448 / max(max|y_row|, 1e-12)`` (quantisation direction, as
    ``rowwise_scaled_quant``), plus ``y`` (bf16) when ``return_normed`` is set.
    """
    _check(x, weight, 16)
    cols = x.shape[-1]
    rows = x.numel() // cols if cols else 0
    dev = x.device
    q = torch.empty_like(x, dtype=torch.float8_e4m3fn)
    scale = torch.empty(*x.shape[:-1], 1, dtype=torch.float32, device=dev)
    y = torch.empty_like(x) if return_normed else None
    with torch.cuda.device(dev):
        _lib.call("tnq_rmsnorm_fp8_rowwise", x.data_ptr(), weight.data_ptr(), float(eps), rows, cols, q.data_ptr(),
                  scale.data_ptr(), 0 if y is None else y.data_ptr(), _lib.stream_ptr(dev))
    return (q, scale, y) if return_normed else (q, scale)


def _check_pair(a: torch.Tensor, b: torch.Tensor, multiple: int):
    _lib.require_cuda(a, "a")
    _lib.require_cuda(b, "b")
    if a.dtype != torch.bfloat16 or b.dtype != torch.bfloat16:
        raise TypeError("a and b must be bfloat16")
    if a.dim() < 1 or a.shape != b.shape:
        raise ValueError("a and b must have the same shape")
    if not a.is_contiguous() or not b.is_contiguous():
        raise ValueError("a and b must be contiguous")
    cols = a.shape[-1]
    if cols % multiple != 0 or cols > 16384:
        raise ValueError(f"the last dimension must be a multiple of {multiple} and at most 16384")
    if a.data_ptr() % 32 != 0 or b.data_ptr() % 32 != 0:
        raise ValueError("a and b must start on a 32-byte boundary")
    if a.device != b.device:
        raise ValueError("a and b must be on the same device")


def swiglu_rowwise_quant(a: torch.Tensor, b: torch.Tensor, *, return_activation: bool = False):
    """``y = F.silu(a) * b`` as eager bf16 PyTorch evaluates it (the reference's
    ``FeedForward``, llama/model.py:228) followed by the per-row dynamic saturated e4m3 cast of
    ``y``, in one pass.  Returns ``(q e4m3, scale fp32 [..., 1])`` (+ ``y``)."""
    _check_pair(a, b, 16)
    cols = a.shape[-1]
    rows = a.numel() // cols if cols else 0
    dev = a.device
    q = torch.empty_like(a, dtype=torch.float8_e4m3fn)
    scale = torch.empty(*a.shape[:-1], 1, dtype=torch.float32, device=dev)
    y = torch.empty_like(a) if return_activation else None
    with torch.cuda.device(dev):
        _lib.call("tnq_swiglu_fp8_rowwise", a.data_ptr(), b.data_ptr(), rows, cols, q.data_ptr(), scale.data_ptr(),
                  0 if y is None else y.data_ptr(), _lib.stream_ptr(dev))
    return (q, scale, y) if return_activation else (q, scale)


def swiglu_quantize_mxfp8(a: torch.Tensor, b: torch.Tensor, *, scale_mode: str = "ceil", swizzle: bool = False,
                          return_activation: bool = False):
    """``y = F.silu(a) * b`` followed by the MXFP8 row-wise quantizer on ``y``, in one pass.
    Returns ``(q e4m3, scales uint8)`` as ``rms_norm_quantize_mxfp8`` (+ ``y``)."""
    _check_pair(a, b, 32)
    if scale_mode not in ("ceil", "floor"):
        raise ValueError("scale_mode must be 'ceil' or 'floor'")
    cols = a.shape[-1]
    rows = a.numel() // cols
    dev = a.device
    q = torch.empty_like(a, dtype=torch.float8_e4m3fn)
    w = cols // 32
    if swizzle:
        n = 512 * ((rows + 127) // 128) * ((w + 3) // 4)
        padded = rows % 128 != 0 or w % 4 != 0
        sf = (torch.zeros if padded else torch.empty)(n, dtype=torch.uint8, device=dev)
    else:
        sf = torch.empty(rows, w, dtype=torch.uint8, device=dev)
    y = torch.empty_like(a) if return_activation else None
    with torch.cuda.device(dev):
        _lib.call("tnq_swiglu_mxfp8", a.data_ptr(), b.data_ptr(), rows, cols, q.data_ptr(), sf.data_ptr(),
                  _lib.E8M0_CEIL if scale_mode == "ceil" else _lib.E8M0_FLOOR,
                  _lib.SCALES_SWIZZLED if swizzle else _lib.SCALES_RAW, 0 if y is None else y.data_ptr(),
                  _lib.stream_ptr(dev))
    return (q, sf, y) if return_activation else (q, sf)
