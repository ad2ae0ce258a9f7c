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
        layout = _lib.SCALES_SWIZZLED if swizzle else _lib.SCALES_RAW
        if global_amax is None:
            if rows and cols:  # amax pass + quantizer in one call (the quantizer re-reads the end of x from L2)
                _lib.call("tnq_nvfp4_quantize_dynamic", x.data_ptr(), rows, cols, _lib.IN_BF16, ws.data_ptr(),
                          packed.data_ptr(), sf.data_ptr(), layout, gscale.data_ptr(), stream)
        else:
            _lib.require_cuda(global_amax, "global_amax")
            if global_amax.dtype != torch.float32 or global_amax.numel() != 1:
                raise TypeError("global_amax must be one fp32 element")
            if rows and cols:
                _lib.call(
                    "tnq_nvfp4_quantize", x.data_ptr(), rows, cols, _lib.IN_BF16, global_amax.data_ptr(), packed.data_ptr(),
                    sf.data_ptr(), layout, gscale.data_ptr(), ws.data_ptr() + 4 * _lib.WS_STATUS_WORD, stream,
                )
    return NVFP4Result(packed.view(torch.float4_e2m1fn_x2), sf, gscale)


# --------------------------------------------------------------------------- consumer
from .blockscaled_tma import BlockScaleLayout, GridScheduler  # noqa: E402,F401


def _check_global_scale(name, t, device):
    if t is None:
        return
    if not isinstance(t, torch.Tensor) or t.dtype != torch.float32 or t.numel() != 1 or t.device != device:
        raise ValueError(f"{name} must be a one-element float32 tensor on the input device")


def nvfp4_tma_gemv(
    q_input: torch.Tensor,
    weight: torch.Tensor,
    input_scale: torch.Tensor,
    weight_scale: torch.Tensor,
    *,
    block_n: int | None = None,
    num_stages: int = 2,
    input_global_scale: torch.Tensor | None = None,
    weight_global_scale: torch.Tensor | None = None,
    output: torch.Tensor | None = None,
    num_compute_warps: int | None = None,
    grid_scheduler: GridScheduler = GridScheduler.STATIC,
    num_persistent_ctas: int | None = None,
    block_scale_layout: BlockScaleLayout = BlockScaleLayout.SWIZZLE_32_4_4,
) -> torch.Tensor:
    """Compute M=1 NVFP4 GEMV: packed FP4 input ``[1, K/2]`` and weight ``[N, K/2]``
    (``float4_e2m1fn_x2`` or uint8), E4M3 block scales (canonically swizzled as in the
    reference, or raw with ``block_scale_layout=RAW``), optional tensorwise fp32 scales
    multiplied in at the end -> ``[1, N]`` bf16.  Contract of cute/nvfp4_tma.py:833-938;
    the reference's tuning arguments are accepted and not needed."""
    if q_input.ndim != 2 or weight.ndim != 2:
        raise ValueError("q_input and weight must be rank-2 tensors")
    for name, t in (("q_input", q_input), ("weight", weight), ("input_scale", input_scale), ("weight_scale", weight_scale)):
        if not t.is_cuda or not t.is_contiguous():
            raise ValueError(f"{name} must be a contiguous CUDA tensor")
    for name, t in (("q_input", q_input), ("weight", weight)):
        if t.dtype not in (torch.float4_e2m1fn_x2, torch.uint8):
            raise TypeError(f"{name} must use torch.float4_e2m1fn_x2 (or uint8) packed storage")
    layout = BlockScaleLayout(block_scale_layout)
    k = q_input.shape[1] * 2
    n = weight.shape[0]
    if q_input.shape[0] != 1 or weight.shape[1] * 2 != k:
        raise ValueError("q_input must be [1, K/2] and weight [N, K/2] packed bytes")
    if k % 32 != 0 or k == 0:
        raise ValueError("K must be a positive multiple of 32")
    sf_k = k // 16
    if input_scale.element_size() != 1 or weight_scale.element_size() != 1:
        raise TypeError("block scales must use one-byte E4M3 storage")
    if layout is BlockScaleLayout.RAW:
        want = (sf_k, n * sf_k)
    else:
        padded = ((sf_k + 3) // 4) * 4
        want = (128 * padded, ((n + 127) // 128) * 128 * padded)
    if input_scale.numel() != want[0] or weight_scale.numel() != want[1]:
        raise ValueError(f"block scales must contain {want[0]} (input) and {want[1]} (weight) elements")
    dev = q_input.device
    _check_global_scale("input_global_scale", input_global_scale, dev)
    _check_global_scale("weight_global_scale", weight_global_scale, dev)
    if output is None:
        output = torch.empty((1, n), dtype=torch.bfloat16, device=dev)
    elif (tuple(output.shape) != (1, n) or output.dtype != torch.bfloat16 or output.device != dev
          or not output.is_contiguous()):
        raise ValueError("output must be a contiguous [1, N] BF16 tensor on the input device")
    with torch.cuda.device(dev):
        _lib.call(
            "tnq_nvfp4_gemv", q_input.data_ptr(), weight.data_ptr(), input_scale.data_ptr(), weight_scale.data_ptr(),
            _lib.ptr(input_global_scale), _lib.ptr(weight_global_scale), n, k,
            _lib.SCALES_RAW if layout is BlockScaleLayout.RAW else _lib.SCALES_SWIZZLED, output.data_ptr(),
            _lib.stream_ptr(dev),
        )
    return output


def nvfp4_tma_scaled_mm(
    mat_a: torch.Tensor,
    mat_b: torch.Tensor,
    scale_a: torch.Tensor,
    scale_b: torch.Tensor,
    *,
    block_n: int | None = None,
    global_scale_a: torch.Tensor | None = None,
    global_scale_b: torch.Tensor | None = None,
    output: torch.Tensor | None = None,
    **tuning,
) -> torch.Tensor:
    """M=1 subset with scaled_mm's blocked-scale and transposed-B convention: ``mat_b`` is
    the metadata transpose of contiguous ``[N, K/2]`` packed storage."""
    if mat_b.ndim != 2:
        raise ValueError("mat_b must be rank-2")
    weight = mat_b.t()
    if not weight.is_contiguous():
        raise ValueError("mat_b must be a metadata transpose of contiguous [N, K] storage")
    return nvfp4_tma_gemv(mat_a, weight, scale_a, scale_b, block_n=block_n, input_global_scale=global_scale_a,
                          weight_global_scale=global_scale_b, output=output)
