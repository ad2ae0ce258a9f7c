"""``quantize_mxfp8_tensor`` under the module path the reference uses
(cute/mxfp8_tma.py:497)."""

from __future__ import annotations

import torch

from ..mx.quantize import quantize_mxfp8


def quantize_mxfp8_tensor(value: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """Create E4M3 values and raw E8M0 block scales: returns ``(e4m3 tensor of
    value's shape, uint8 [rows, K/32])`` exactly like the reference helper
    (cute/mxfp8_tma.py:497-504)."""
    r = quantize_mxfp8(value, scale_mode="ceil", rowwise=True, columnwise=False, swizzle=False)
    return r.q_row, r.scale_row
