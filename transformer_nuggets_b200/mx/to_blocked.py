"""Scale swizzle with the entry point of ``transformer_nuggets/mx/to_blocked.py``."""

from __future__ import annotations

import torch

from .. import _lib

Tensor = torch.Tensor


def ceil_div(a, b):
    return (a + b - 1) // b


def to_blocked(input_matrix: Tensor) -> Tensor:
    """Rearrange an ``(H, W)`` matrix of one-byte block scales into the 128x4
    block-scaling-factor layout of cuBLAS / tcgen05 block-scaled MMA.

    Same contract as the reference (mx/to_blocked.py:10-42): the input is padded
    with zeros to multiples of (128, 4) and the result is the flat tensor of
    ``32*ceil_div(H,128) * 16*ceil_div(W,4)`` elements, in the input's dtype.
    """
    _lib.require_cuda(input_matrix, "input_matrix")
    if input_matrix.dim() != 2:
        raise ValueError("to_blocked expects a 2-D tensor")
    if input_matrix.element_size() != 1:
        raise TypeError("to_blocked handles one-byte scale types (uint8, float8_e8m0fnu, float8_e4m3fn)")
    src = input_matrix.contiguous()
    rows, cols = src.shape
    out = torch.empty(512 * ceil_div(rows, 128) * ceil_div(cols, 4), dtype=src.dtype, device=src.device)
    with torch.cuda.device(src.device):
        _lib.call("tnq_to_blocked", src.data_ptr(), rows, cols, out.data_ptr(), _lib.stream_ptr(src.device))
    return out


def to_blocked_manual(input_matrix: Tensor) -> Tensor:
    """The reference's second implementation of the same rearrangement
    (mx/to_blocked.py:67-105) under its own name; one kernel serves both."""
    return to_blocked(input_matrix)


def _to_blocked_single(scales: Tensor) -> Tensor:
    """One 128 x 4 block of scales -> its ``(32, 16)`` atom (mx/to_blocked.py:56-65 of the
    reference): a single-atom call of the same kernel."""
    assert scales.shape == (128, 4)
    return to_blocked(scales).view(32, 16)


def _to_blocked_single_manual(scales: Tensor) -> Tensor:
    """The reference's slow twin of ``_to_blocked_single`` (mx/to_blocked.py:45-53) under its
    own name; one kernel serves both."""
    return _to_blocked_single(scales.reshape(128, 4))
