"""MXFP8 and NVFP4 GEMMs on the block-scaled tensor cores: they consume the quantizers' payloads
and swizzled block scales as they are written."""

from __future__ import annotations

import torch

from .. import _lib


def mxfp8_scaled_mm(mat_a: torch.Tensor, mat_b: torch.Tensor, scale_a: torch.Tensor, scale_b: torch.Tensor) -> torch.Tensor:
    """``mat_a [M, K]`` e4m3 row-major, ``mat_b [K, N]`` e4m3 column-major (the ``.t()`` of a
    weight stored ``[N, K]``), ``scale_a`` / ``scale_b`` the flat swizzled E8M0 buffers of
    ``[M, K/32]`` / ``[N, K/32]`` (``quantize_mxfp8(..., swizzle=True)`` or ``to_blocked``)
    -> ``[M, N]`` bf16.  The operand convention of ``F.scaled_mm`` with ``BlockWise1x32`` scaling
    and ``SWIZZLE_32_4_4``, which is how the reference's tests consume these tensors
    (test/test_mxfp8_tma.py:174-203).  K must be a multiple of 128."""
    for name, t in (("mat_a", mat_a), ("mat_b", mat_b), ("scale_a", scale_a), ("scale_b", scale_b)):
        _lib.require_cuda(t, name)
    if mat_a.dim() != 2 or mat_b.dim() != 2 or mat_a.shape[1] != mat_b.shape[0]:
        raise ValueError("mat_a must be [M, K] and mat_b [K, N]")
    if mat_a.dtype != torch.float8_e4m3fn or mat_b.dtype != torch.float8_e4m3fn:
        raise TypeError("mat_a and mat_b must be float8_e4m3fn")
    if not mat_a.is_contiguous() or not mat_b.t().is_contiguous():
        raise ValueError("mat_a must be row-major and mat_b column-major (mat_b.t() contiguous)")
    m, k = mat_a.shape
    n = mat_b.shape[1]
    if k % 128 != 0:
        raise ValueError("K must be a multiple of 128")
    for name, t, rows in (("scale_a", scale_a, m), ("scale_b", scale_b, n)):
        if t.element_size() != 1 or not t.is_contiguous():
            raise TypeError(f"{name} must be a contiguous one-byte (E8M0) tensor")
        want = 512 * ((rows + 127) // 128) * (k // 128)
        if t.numel() != want:
            raise ValueError(f"{name} must hold {want} swizzled bytes, got {t.numel()}")
    dev = mat_a.device
    out = torch.empty((m, n), dtype=torch.bfloat16, device=dev)
    with torch.cuda.device(dev):
        _lib.call("tnq_mxfp8_gemm", mat_a.data_ptr(), mat_b.data_ptr(), scale_a.data_ptr(), scale_b.data_ptr(), m, n, k,
                  out.data_ptr(), _lib.workspace(dev).data_ptr() + 4 * _lib.WS_STATUS_WORD, _lib.stream_ptr(dev))
    return out


def nvfp4_scaled_mm(mat_a: torch.Tensor, mat_b: torch.Tensor, scale_a: torch.Tensor, scale_b: torch.Tensor,
                    global_scale_a: torch.Tensor | None = None, global_scale_b: torch.Tensor | None = None) -> torch.Tensor:
    """``mat_a [M, K/2]`` packed e2m1 (``float4_e2m1fn_x2`` or uint8), ``mat_b [K/2, N]`` the ``.t()``
    of a packed weight ``[N, K/2]``, ``scale_a`` / ``scale_b`` the flat swizzled E4M3 block scales of
    ``[M, K/16]`` / ``[N, K/16]``, optional fp32 tensor-wide scales (decode direction) -> ``[M, N]``
    bf16.  The operand convention of ``F.scaled_mm`` with ``BlockWise1x16`` + ``TensorWise``
    scaling, which is how the reference's tests consume these tensors
    (test/test_nvfp4_tma.py:511-548).  K must be a multiple of 256."""
    for name, t in (("mat_a", mat_a), ("mat_b", mat_b), ("scale_a", scale_a), ("scale_b", scale_b)):
        _lib.require_cuda(t, name)
    if mat_a.dim() != 2 or mat_b.dim() != 2 or mat_a.shape[1] != mat_b.shape[0]:
        raise ValueError("mat_a must be [M, K/2] and mat_b [K/2, N] packed bytes")
    if mat_a.element_size() != 1 or mat_b.element_size() != 1:
        raise TypeError("mat_a and mat_b must use packed one-byte storage (float4_e2m1fn_x2 or uint8)")
    if not mat_a.is_contiguous() or not mat_b.t().is_contiguous():
        raise ValueError("mat_a must be row-major and mat_b column-major (mat_b.t() contiguous)")
    m, kh = mat_a.shape
    n = mat_b.shape[1]
    k = 2 * kh
    if k % 256 != 0:
        raise ValueError("K must be a multiple of 256")
    for name, t, rows in (("scale_a", scale_a, m), ("scale_b", scale_b, n)):
        if t.element_size() != 1 or not t.is_contiguous():
            raise TypeError(f"{name} must be a contiguous one-byte (E4M3) tensor")
        want = 512 * ((rows + 127) // 128) * (k // 64)
        if t.numel() != want:
            raise ValueError(f"{name} must hold {want} swizzled bytes, got {t.numel()}")
    for name, t in (("global_scale_a", global_scale_a), ("global_scale_b", global_scale_b)):
        if t is not None and (t.dtype != torch.float32 or t.numel() != 1 or t.device != mat_a.device):
            raise ValueError(f"{name} must be a one-element float32 tensor on the operands' device")
    dev = mat_a.device
    out = torch.empty((m, n), dtype=torch.bfloat16, device=dev)
    with torch.cuda.device(dev):
        _lib.call("tnq_nvfp4_gemm", mat_a.data_ptr(), mat_b.data_ptr(), scale_a.data_ptr(), scale_b.data_ptr(),
                  0 if global_scale_a is None else global_scale_a.data_ptr(),
                  0 if global_scale_b is None else global_scale_b.data_ptr(), m, n, k, out.data_ptr(),
                  _lib.workspace(dev).data_ptr() + 4 * _lib.WS_STATUS_WORD, _lib.stream_ptr(dev))
    return out
