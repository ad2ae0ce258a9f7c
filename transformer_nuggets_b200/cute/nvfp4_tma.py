"""NVFP4 helpers under the module path the reference uses (cute/nvfp4_tma.py:941-964)
plus the quantizer the reference lacks."""

from __future__ import annotations

from typing import NamedTuple

import torch

from .. import _lib
from ..mx.to_blocked import ceil_div, to_blocked


def pack_nvfp4_codes(codes: torch.Tensor) -> torch.Tensor:
    """Pack low-nibble-first E2M1 codes (uint8 ``[M, K]``, values 0..15) into
    ``torch.float4_e2m1fn_x2`` ``[M, K/2]`` (cute/nvfp4_tma.py:941-943)."""
    _lib.require_cuda(codes, "codes")
    if codes.dim() != 2 or codes.dtype != torch.uint8:
        raise TypeError("codes must be a 2-D uint8 tensor")
    rows, cols = codes.shape
    if cols % 16 != 0:
        raise ValueError("the number of codes per row must be a multiple of 16")
    src = codes.contiguous()
    out = torch.empty(rows, cols // 2, dtype=torch.uint8, device=codes.device)
    with torch.cuda.device(codes.device):
        _lib.call("tnq_pack_fp4_codes", src.data_ptr(), rows, cols, out.data_ptr(), _lib.stream_ptr(codes.device))
    return out.view(torch.float4_e2m1fn_x2)


def swizzle_nvfp4_scales(scales: torch.Tensor) -> torch.Tensor:
    """Convert natural row-major block scales to SWIZZLE_32_4_4 storage (flat),
    as cute/nvfp4_tma.py:946-964."""
    return to_blocked(scales)


class NVFP4Result(NamedTuple):
    """``packed``: ``float4_e2m1fn_x2 [M, K/2]``; ``block_scales``: e4m3, flat
    swizzled (or ``[M, K/16]`` when ``swizzle=False``); ``global_scale``: fp32
    ``[1]``, decode direction (value = e2m1 * block_scale * global_scale)."""

    packed: torch.Tensor
    block_scales: torch.Tensor
    global_scale: torch.Tensor


def quantize_nvfp4(x: torch.Tensor, global_amax: torch.Tensor | None = None, *, swizzle: bool = True) -> NVFP4Result:
    """Quantize a 2-D bf16 tensor to NVFP4 (16-element blocks along the last
    dimension).  ``global_amax`` (fp32, one element, on the device) skips the
    tensor-wide amax pass; it must be ``max|x|`` of the tensor the scales should
    be relative to.  The storage follows the reference's contract
    (cute/nvfp4_tma.py:941-964, :527-547)."""
    _lib.require_cuda(x, "x")
    if x.dim() != 2:
        raise ValueError("quantize_nvfp4 expects a 2-D tensor")
    if x.dtype != torch.bfloat16:
        raise TypeError(f"quantize_nvfp4 expects bfloat16, got {x.dtype}")
    if not x.is_contiguous():
        raise ValueError("x must be contiguous")
    rows, cols = x.shape
    if cols % 16 != 0:
        raise ValueError("the last dimension must be a multiple of 16")
    if x.data_ptr() % 32 != 0:
        raise ValueError("x must start on a 32-byte boundary")
    dev = x.device
    ws = _lib.workspace(dev)
    packed = torch.empty(rows, cols // 2, dtype=torch.uint8, device=dev)
    if swizzle:
        sf = torch.empty(512 * ceil_div(rows, 128) * ceil_div(cols // 16, 4), dtype=torch.float8_e4m3fn, device=dev)
    else:
        sf = torch.empty(rows, cols // 16, dtype=torch.float8_e4m3fn, device=dev)
    gscale = torch.empty(1, dtype=torch.float32, device=dev)
    with torch.cuda.device(dev):
        stream = _lib.stream_ptr(dev)
        if global_amax is None:
            _lib.call("tnq_fp8_amax", x.data_ptr(), x.numel(), _lib.IN_BF16, _lib.FP8_E4M3, ws.data_ptr(), 0, stream)
            amax_ptr = ws.data_ptr() + 4 * _lib.WS_AMAX_WORD
        else:
            _lib.require_cuda(global_amax, "global_amax")
            if global_amax.dtype != torch.float32 or global_amax.numel() != 1:
                raise TypeError("global_amax must be one fp32 element")
            amax_ptr = global_amax.data_ptr()
        if rows and cols:
            _lib.call(
                "tnq_nvfp4_quantize", x.data_ptr(), rows, cols, _lib.IN_BF16, amax_ptr, packed.data_ptr(),
                sf.data_ptr(), _lib.SCALES_SWIZZLED if swizzle else _lib.SCALES_RAW, gscale.data_ptr(),
                ws.data_ptr() + 4 * _lib.WS_STATUS_WORD, stream,
            )
    return NVFP4Result(packed.view(torch.float4_e2m1fn_x2), sf, gscale)
