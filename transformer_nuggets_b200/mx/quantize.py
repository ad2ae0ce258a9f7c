"""MXFP8 quantizer (32-element blocks, E8M0 scales, e4m3 payload)."""

from __future__ import annotations

from typing import NamedTuple

import torch

from .. import _lib
from .to_blocked import ceil_div


class MXFP8Result(NamedTuple):
    """Row-wise pair: ``q_row [M, K]`` e4m3 and its scales; column-wise pair:
    ``q_col [K, M]`` e4m3 (the row-wise quantisation of ``x.t()``) and its scales.
    Scales are uint8 E8M0 bytes: raw ``[rows, K/32]`` matrices, or flat swizzled
    buffers when ``swizzle=True``.  Unrequested members are ``None``."""

    q_row: torch.Tensor | None
    scale_row: torch.Tensor | None
    q_col: torch.Tensor | None
    scale_col: torch.Tensor | None


def quantize_mxfp8(
    value: torch.Tensor,
    *,
    scale_mode: str = "ceil",
    rowwise: bool = True,
    columnwise: bool = False,
    swizzle: bool = False,
) -> MXFP8Result:
    """Quantize a 2-D bf16 tensor to MXFP8 in one pass over the input.

    ``scale_mode="ceil"`` is the rule of the reference's ``quantize_mxfp8_tensor``
    (``ceil(log2(amax/448))``, cute/mxfp8_tma.py:497-504); ``"floor"`` is the OCP
    rule ``floor(log2(amax)) - 8``.  ``swizzle=True`` emits the scales directly in
    the layout ``to_blocked`` produces (mx/to_blocked.py:10-42).
    """
    _lib.require_cuda(value, "value")
    if value.dim() != 2:
        raise ValueError("quantize_mxfp8 expects a 2-D tensor")
    if value.dtype != torch.bfloat16:
        raise TypeError(f"quantize_mxfp8 expects bfloat16, got {value.dtype}")
    if not value.is_contiguous():
        raise ValueError("value must be contiguous")
    if scale_mode not in ("ceil", "floor"):
        raise ValueError("scale_mode must be 'ceil' or 'floor'")
    if not (rowwise or columnwise):
        raise ValueError("request at least one of rowwise / columnwise")
    rows, cols = value.shape
    if cols % 8 != 0:
        raise ValueError("the row length must be a multiple of 8")
    if rowwise and cols % 32 != 0:
        raise ValueError("row-wise MXFP8 needs the last dimension to be a multiple of 32")
    if columnwise and rows % 32 != 0:
        raise ValueError("column-wise MXFP8 needs the first dimension to be a multiple of 32")
    if value.data_ptr() % 16 != 0:
        raise ValueError("value must start on a 16-byte boundary")
    dev = value.device
    u8 = torch.uint8

    def scale_buf(h, w):
        if swizzle:
            return torch.empty(512 * ceil_div(h, 128) * ceil_div(w, 4), dtype=u8, device=dev)
        return torch.empty(h, w, dtype=u8, device=dev)

    q_row = s_row = q_col = s_col = None
    if rowwise:
        q_row = torch.empty(rows, cols, dtype=torch.float8_e4m3fn, device=dev)
        s_row = scale_buf(rows, cols // 32)
    if columnwise:
        q_col = torch.empty(cols, rows, dtype=torch.float8_e4m3fn, device=dev)
        s_col = scale_buf(cols, rows // 32)
    ws = _lib.workspace(dev)
    status_ptr = ws.data_ptr() + 4 * _lib.WS_STATUS_WORD
    if rows and cols:
        with torch.cuda.device(dev):
            _lib.call(
                "tnq_mxfp8_quantize", value.data_ptr(), rows, cols, _lib.IN_BF16, _lib.ptr(q_row), _lib.ptr(s_row),
                _lib.ptr(q_col), _lib.ptr(s_col), _lib.E8M0_CEIL if scale_mode == "ceil" else _lib.E8M0_FLOOR,
                _lib.SCALES_SWIZZLED if swizzle else _lib.SCALES_RAW, status_ptr, _lib.stream_ptr(dev),
            )
    return MXFP8Result(q_row, s_row, q_col, s_col)
