"""RMSNorm fused into the row-wise FP8 cast (a producer epilogue: the normalised bf16
activation is never written to memory unless asked for)."""

from __future__ import annotations

import torch

from .. import _lib


def rms_norm_rowwise_quant(x: torch.Tensor, weight: torch.Tensor, eps: float = 1e-6, *, return_normed: bool = False):
    """``y = rms_norm(x, weight, eps)`` (the eager formula of the reference's fusion example,
    examples/rms_norm_fusion_profile.py:26-31) followed by the per-row dynamic saturated
    e4m3 cast of ``y``, in one pass over ``x``.

    ``x``: bf16 ``[..., C]`` contiguous, ``C`` a multiple of 16 and at most 16384;
    ``weight``: bf16 ``[C]``.  Returns ``(q e4m3 [..., C], scale fp32 [..., 1])`` with
    ``scale = 448 / max(max|y_row|, 1e-12)`` (quantisation direction, as
    ``rowwise_scaled_quant``), plus ``y`` (bf16) when ``return_normed`` is set.
    """
    _lib.require_cuda(x, "x")
    _lib.require_cuda(weight, "weight")
    if x.dtype != torch.bfloat16 or weight.dtype != torch.bfloat16:
        raise TypeError("x and weight must be bfloat16")
    if x.dim() < 1 or weight.dim() != 1 or weight.shape[0] != x.shape[-1]:
        raise ValueError("weight must be a vector of x's last dimension")
    if not x.is_contiguous() or not weight.is_contiguous():
        raise ValueError("x and weight must be contiguous")
    cols = x.shape[-1]
    if cols % 16 != 0 or cols > 16384:
        raise ValueError("the normalised dimension must be a multiple of 16 and at most 16384")
    if x.data_ptr() % 32 != 0 or weight.data_ptr() % 32 != 0:
        raise ValueError("x and weight must start on a 32-byte boundary")
    if weight.device != x.device:
        raise ValueError("x and weight must be on the same device")
    rows = x.numel() // cols if cols else 0
    dev = x.device
    q = torch.empty_like(x, dtype=torch.float8_e4m3fn)
    scale = torch.empty(*x.shape[:-1], 1, dtype=torch.float32, device=dev)
    y = torch.empty_like(x) if return_normed else None
    with torch.cuda.device(dev):
        _lib.call("tnq_rmsnorm_fp8_rowwise", x.data_ptr(), weight.data_ptr(), float(eps), rows, cols, q.data_ptr(),
                  scale.data_ptr(), 0 if y is None else y.data_ptr(), _lib.stream_ptr(dev))
    return (q, scale, y) if return_normed else (q, scale)
