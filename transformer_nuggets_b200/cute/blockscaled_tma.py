"""Enums shared by the block-scaled GEMV entry points, with the reference's names
(cute/blockscaled_tma.py:23-36)."""

from __future__ import annotations

from enum import Enum


class BlockScaleLayout(str, Enum):
    """Describe caller-owned block-scale storage."""

    RAW = "raw"
    SWIZZLE_32_4_4 = "swizzle_32_4_4"


class GridScheduler(str, Enum):
    """Map logical output tiles onto the launched CTA grid.  Accepted for signature
    compatibility; the kernels always run a persistent grid sized by occupancy."""

    STATIC = "static"
    PERSISTENT = "persistent"
