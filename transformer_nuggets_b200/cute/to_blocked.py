"""``to_blocked_mx`` under the module path the reference uses (cute/to_blocked.py:127)."""

from __future__ import annotations

import torch

from ..mx.to_blocked import to_blocked


def to_blocked_mx(scales: torch.Tensor) -> torch.Tensor:
    """Swizzle ``[H, W]`` block scales; returns the buffer viewed ``(-1, 32, 16)``
    as the reference's kernel wrapper does (cute/to_blocked.py:127-153).  Unlike
    the reference kernel, H and W need not be multiples of 128."""
    return to_blocked(scales).view(-1, 32, 16)
