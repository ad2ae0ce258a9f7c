"""Delayed-scaling state around ``scaled_quant``: amax history -> next step's scale.

``scaled_quant(x, scale, abs_max)`` (fp8/scaled_quant.py:35-75 in the reference) casts with
a scale "calculated from previous abs_max" and leaves this step's ``abs_max`` behind; the
reference hands the step in between to float8_experimental's
``sync_float8_amax_and_scale_history`` (llama/train.py:251-263), a dependency outside its
tree.  :class:`DelayedScaling` is that step for any number of tensors: one fp32 amax word,
one amax history row and one scale per tensor, all updated by ONE kernel launch
(``tnq_delayed_scale_update``), with the amax words MAX-reduced over the data-parallel
group first when there is one.
"""

from __future__ import annotations

import torch
import torch.distributed as dist

from .. import _lib
from .scaled_quant import scaled_quant


def combine_amaxes(amax: torch.Tensor, group=None) -> torch.Tensor:
    """In-place MAX all-reduce of the per-tensor amax words over ``group`` (a no-op
    without an initialised multi-rank group).  MAX of non-negative floats is exact and
    order independent, so every rank derives the same scales."""
    if amax.dtype != torch.float32:
        raise TypeError("amax must be fp32")
    if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(amax, op=dist.ReduceOp.MAX, group=group)
    return amax


class DelayedScaling:
    """State of ``num_tensors`` delayed-scaled tensors on one device.

    ``scale`` starts at 1 and ``amax_history`` at 0, so the first step casts unscaled and
    the first :meth:`sync` sets every scale from the first step's amax.
    """

    def __init__(self, num_tensors: int, history_len: int = 16, fp8_dtype: torch.dtype = torch.float8_e4m3fn,
                 device="cuda"):
        if fp8_dtype not in _lib.FP8_DTYPES:
            raise TypeError(f"fp8_dtype must be float8_e4m3fn or float8_e5m2, got {fp8_dtype}")
        if num_tensors < 1:
            raise ValueError("num_tensors must be positive")
        if not 1 <= history_len <= 1024:
            raise ValueError("history_len must be in [1, 1024]")
        device = torch.device(device)
        if device.type != "cuda":
            raise ValueError("DelayedScaling lives on a CUDA device; there is no CPU path")
        self.fp8_dtype = fp8_dtype
        self.amax_history = torch.zeros(num_tensors, history_len, dtype=torch.float32, device=device)
        self.amax = torch.zeros(num_tensors, dtype=torch.float32, device=device)
        self.scale = torch.ones(num_tensors, dtype=torch.float32, device=device)

    @property
    def num_tensors(self) -> int:
        return self.amax.numel()

    def cast(self, index: int, inpt_tensor: torch.Tensor, saturated: bool = True) -> torch.Tensor:
        """``scaled_quant`` of tensor ``index`` with its current scale; the tensor's amax
        word accumulates ``max|inpt_tensor|`` (several casts per step are folded by MAX)."""
        return scaled_quant(inpt_tensor, self.scale[index:index + 1], self.amax[index:index + 1], self.fp8_dtype,
                            saturated)

    def sync(self, group=None) -> None:
        """End of a step: MAX-reduce the amax words over ``group``, push them into the
        histories, recompute every scale, clear the amax words.  One launch, no host sync."""
        combine_amaxes(self.amax, group)
        dev = self.amax.device
        with torch.cuda.device(dev):
            _lib.call("tnq_delayed_scale_update", self.amax_history.data_ptr(), self.amax.data_ptr(),
                      self.scale.data_ptr(), self.num_tensors, self.amax_history.shape[1],
                      _lib.FP8_DTYPES[self.fp8_dtype], _lib.stream_ptr(dev))
