"""Scaled-quantization casts (bf16/fp32 -> fp8 / MXFP8 / NVFP4) for NVIDIA B200.

The Python entry points keep the names, argument order and return layouts of
drisspg/transformer_nuggets and dispatch to hand-written sm_100a CUDA kernels
in ``csrc/libtnq.so`` through its C ABI (``include/tnq.h``).  CUDA tensors only.
"""

from .fp8.scaled_quant import (  # noqa: F401
    dynamic_scaled_quant,
    dynamic_scaled_quant_with_scale,
    rowwise_scaled_quant,
    scaled_quant,
)
from .mx.to_blocked import to_blocked  # noqa: F401
from .mx.quantize import quantize_mxfp8  # noqa: F401
from .cute.mxfp8_tma import quantize_mxfp8_tensor  # noqa: F401
from .cute.nvfp4_tma import pack_nvfp4_codes, quantize_nvfp4, swizzle_nvfp4_scales  # noqa: F401
from .cute.to_blocked import to_blocked_mx  # noqa: F401
from ._lib import TnqError, check_status  # noqa: F401

__all__ = [
    "scaled_quant",
    "dynamic_scaled_quant",
    "dynamic_scaled_quant_with_scale",
    "rowwise_scaled_quant",
    "to_blocked",
    "to_blocked_mx",
    "quantize_mxfp8",
    "quantize_mxfp8_tensor",
    "quantize_nvfp4",
    "pack_nvfp4_codes",
    "swizzle_nvfp4_scales",
    "check_status",
    "TnqError",
]
