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


# --------------------------------------------------------------------------- consumer
from .. import _lib  # noqa: E402
from .blockscaled_tma import BlockScaleLayout, GridScheduler  # noqa: E402,F401


def mxfp8_tma_gemv(
    q_input: torch.Tensor,
    weight: torch.Tensor,
    input_scale: torch.Tensor,
    weight_scale: torch.Tensor,
    *,
    block_n: int | None = None,
    num_stages: int = 2,
    output: torch.Tensor | None = None,
    num_compute_warps: int | None = None,
    grid_scheduler: GridScheduler = GridScheduler.STATIC,
    num_persistent_ctas: int | None = None,
    block_scale_layout: BlockScaleLayout = BlockScaleLayout.RAW,
) -> torch.Tensor:
    """Compute MXFP8 GEMV (M = 1) on prequantized inputs and caller-owned scales:
    ``[1, K]`` e4m3 input, ``[N, K]`` e4m3 weight, E8M0 scales raw (``[1, K/32]`` /
    ``[N, K/32]``) or ``SWIZZLE_32_4_4`` -> ``[1, N]`` bf16.  Same contract and checks as
    the reference (cute/mxfp8_tma.py:392-460, 219-302); ``block_n``, ``num_stages``,
    ``num_compute_warps``, ``grid_scheduler`` and ``num_persistent_ctas`` are the
    reference's tuning knobs and are accepted but not needed here."""
    if q_input.ndim != 2 or weight.ndim != 2:
        raise ValueError("q_input and weight must be rank-2 tensors")
    layout = BlockScaleLayout(block_scale_layout)
    k = q_input.shape[1]
    n = weight.shape[0]
    sf_k = k // 32
    for name, tensor, expected_shape in (("q_input", q_input, (1, k)), ("weight", weight, (n, k))):
        if tuple(tensor.shape) != expected_shape:
            raise ValueError(f"{name} must have shape {expected_shape}, got {tuple(tensor.shape)}")
        if not tensor.is_cuda or not tensor.is_contiguous():
            raise ValueError(f"{name} must be a contiguous CUDA tensor")
    if k % 32 != 0 or k == 0:
        raise ValueError("K must be a positive multiple of 32")
    if layout is BlockScaleLayout.RAW:
        for name, tensor, shape in (("input_scale", input_scale, (1, sf_k)), ("weight_scale", weight_scale, (n, sf_k))):
            if tuple(tensor.shape) != shape:
                raise ValueError(f"{name} must have shape {shape}, got {tuple(tensor.shape)}")
    else:
        padded_sf_k = ((sf_k + 3) // 4) * 4
        for name, tensor, numel in (("input_scale", input_scale, 128 * padded_sf_k),
                                    ("weight_scale", weight_scale, ((n + 127) // 128) * 128 * padded_sf_k)):
            if tensor.numel() != numel:
                raise ValueError(f"{name} must contain {numel} swizzled elements")
    for name, tensor in (("input_scale", input_scale), ("weight_scale", weight_scale)):
        if not tensor.is_cuda or not tensor.is_contiguous():
            raise ValueError(f"{name} must be a contiguous CUDA tensor")
    if q_input.dtype != torch.float8_e4m3fn or weight.dtype != torch.float8_e4m3fn:
        raise TypeError("q_input and weight must use torch.float8_e4m3fn")
    if input_scale.element_size() != 1 or weight_scale.element_size() != 1:
        raise TypeError("input_scale and weight_scale must use one-byte E8M0 storage")
    if any(t.device != q_input.device for t in (weight, input_scale, weight_scale)):
        raise ValueError("all inputs must be on the same CUDA device")
    if output is None:
        output = torch.empty((1, n), dtype=torch.bfloat16, device=q_input.device)
    elif (tuple(output.shape) != (1, n) or output.dtype != torch.bfloat16 or output.device != q_input.device
          or not output.is_contiguous()):
        raise ValueError("output must be a contiguous [1, N] BF16 tensor on the input device")
    with torch.cuda.device(q_input.device):
        _lib.call(
            "tnq_mxfp8_gemv", q_input.data_ptr(), weight.data_ptr(), input_scale.data_ptr(), weight_scale.data_ptr(),
            n, k, _lib.SCALES_RAW if layout is BlockScaleLayout.RAW else _lib.SCALES_SWIZZLED, output.data_ptr(),
            _lib.stream_ptr(q_input.device),
        )
    return output


def mxfp8_tma_scaled_mm(
    mat_a: torch.Tensor,
    mat_b: torch.Tensor,
    scale_a: torch.Tensor,
    scale_b: torch.Tensor,
    *,
    block_n: int | None = None,
    output: torch.Tensor | None = None,
    num_stages: int = 2,
    num_compute_warps: int | None = None,
    grid_scheduler: GridScheduler = GridScheduler.STATIC,
    num_persistent_ctas: int | None = None,
) -> torch.Tensor:
    """Run the M=1 subset using scaled_mm's blocked-scale and transposed-B convention
    (cute/mxfp8_tma.py:463-494)."""
    if mat_b.ndim != 2:
        raise ValueError("mat_b must be rank-2")
    weight = mat_b.t()
    if not weight.is_contiguous():
        raise ValueError("mat_b must be a metadata transpose of contiguous [N, K] storage")
    return mxfp8_tma_gemv(mat_a, weight, scale_a, scale_b, block_n=block_n, num_stages=num_stages, output=output,
                          num_compute_warps=num_compute_warps, grid_scheduler=grid_scheduler,
                          num_persistent_ctas=num_persistent_ctas, block_scale_layout=BlockScaleLayout.SWIZZLE_32_4_4)
