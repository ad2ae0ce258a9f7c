"""Row-sharded per-tensor dynamic FP8 cast: one process per GPU, each rank owns a
contiguous block of rows; the only data that crosses GPUs is one fp32 - the
tensor-wide amax, combined with MAX.  MAX over non-negative floats is exact and
order independent, so the shards together are bit-identical to the single-device
result.  The reference has no multi-device cast; its only collective code is a
peer-load sum over symmetric memory (cute/symmetric_memory.py:20-79).
"""

from __future__ import annotations

import torch
import torch.distributed as dist

from .. import _lib


def plan_row_shards(rows: int, world_size: int, multiple: int = 128):
    """Contiguous row ranges ``[(start, stop), ...]``, one per rank.  Every range
    but possibly the last is a multiple of ``multiple`` rows (128 keeps swizzled
    scale atoms from straddling ranks); trailing ranks may be empty."""
    if rows < 0 or world_size < 1 or multiple < 1:
        raise ValueError("rows >= 0, world_size >= 1 and multiple >= 1 are required")
    units = -(-rows // multiple)
    base, extra = divmod(units, world_size)
    out, start = [], 0
    for r in range(world_size):
        n_units = base + (1 if r < extra else 0)
        stop = min(rows, start + n_units * multiple)
        out.append((start, stop))
        start = stop
    return out


def combine_amax(local_amax: torch.Tensor, group=None) -> torch.Tensor:
    """In-place MAX all-reduce of a one-element fp32 amax over ``group`` (NCCL for
    CUDA tensors; any backend that implements MAX works, e.g. gloo on CPU)."""
    if local_amax.dtype != torch.float32 or local_amax.numel() != 1:
        raise TypeError("local_amax must be one fp32 element")
    if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(local_amax, op=dist.ReduceOp.MAX, group=group)
    return local_amax


def combine_amax_bounded(local_amax: torch.Tensor, group=None, timeout_s: float = 10.0) -> bool:
    """``combine_amax`` that gives up: the MAX all-reduce is issued asynchronously and waited
    for at most ``timeout_s`` seconds.  Returns True when every rank contributed, False when
    the wait ran out (a rank is late or gone); ``local_amax`` is then not to be trusted and
    the caller should skip the step or tear the group down.  The host-side counterpart of the
    bounded device-side wait of the peer exchange."""
    import datetime

    if local_amax.dtype != torch.float32 or local_amax.numel() != 1:
        raise TypeError("local_amax must be one fp32 element")
    if not (dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1):
        return True
    work = dist.all_reduce(local_amax, op=dist.ReduceOp.MAX, group=group, async_op=True)
    try:
        return bool(work.wait(datetime.timedelta(seconds=timeout_s)))
    except RuntimeError:
        return False


def sharded_dynamic_scaled_quant(
    local_rows: torch.Tensor,
    group=None,
    fp8_dtype: torch.dtype = torch.float8_e4m3fn,
    *,
    exchange=None,
    out: torch.Tensor | None = None,
):
    """Cast this rank's row block with the scale of the WHOLE tensor.

    local amax kernel -> MAX over ranks -> saturated cast with
    ``scale = max / max(global amax, 1e-12)``.  ``exchange`` is an
    :class:`~transformer_nuggets_b200.dist.exchange.PeerAmaxExchange` for the
    NVLink peer-store exchange; ``None`` uses an NCCL all-reduce.
    Returns ``(fp8 rows, global amax fp32 [1])``; the scale is
    ``finfo.max / max(amax, 1e-12)`` on every rank.
    """
    _lib.require_cuda(local_rows, "local_rows")
    if not local_rows.is_contiguous():
        raise ValueError("local_rows must be contiguous")
    if local_rows.dtype not in _lib.IN_DTYPES or fp8_dtype not in _lib.FP8_DTYPES:
        raise TypeError("unsupported dtype")
    if local_rows.numel() and local_rows.data_ptr() % 32 != 0:
        raise ValueError("local_rows must start on a 32-byte boundary")
    dev = local_rows.device
    if out is None:
        out = torch.empty_like(local_rows, dtype=fp8_dtype)
    in_dt, out_dt = _lib.IN_DTYPES[local_rows.dtype], _lib.FP8_DTYPES[fp8_dtype]
    n = local_rows.numel()
    with torch.cuda.device(dev):
        ws = _lib.workspace(dev)
        stream = _lib.stream_ptr(dev)
        if exchange is not None:
            amax = exchange.run(local_rows, n, in_dt, out_dt, ws, stream, out)
        else:
            amax = torch.empty(1, dtype=torch.float32, device=dev)
            _lib.call("tnq_fp8_amax", local_rows.data_ptr(), n, in_dt, out_dt, ws.data_ptr(), amax.data_ptr(), stream)
            combine_amax(amax, group)
            _lib.call(
                "tnq_fp8_scaled_cast", local_rows.data_ptr(), out.data_ptr(), n, in_dt, out_dt, amax.data_ptr(),
                _lib.SCALE_IS_AMAX, 1, 0, 0, stream,
            )
    return out, amax


def sharded_global_amax(local_rows: torch.Tensor, group=None, *, exchange=None) -> torch.Tensor:
    """Tensor-wide ``max|x|`` of a row-sharded tensor as a one-element fp32 device tensor
    (identical on every rank): peer-store exchange when ``exchange`` is given, else local
    amax kernel + NCCL all-reduce(MAX)."""
    _lib.require_cuda(local_rows, "local_rows")
    if exchange is not None:
        return exchange.global_amax(local_rows)
    if local_rows.dtype not in _lib.IN_DTYPES or not local_rows.is_contiguous():
        raise TypeError("local_rows must be a contiguous bfloat16 / float32 tensor")
    dev = local_rows.device
    amax = torch.empty(1, dtype=torch.float32, device=dev)
    with torch.cuda.device(dev):
        _lib.call("tnq_fp8_amax", local_rows.data_ptr(), local_rows.numel(), _lib.IN_DTYPES[local_rows.dtype],
                  _lib.FP8_E4M3, _lib.workspace(dev).data_ptr(), amax.data_ptr(), _lib.stream_ptr(dev))
    return combine_amax(amax, group)


def sharded_quantize_nvfp4(local_rows: torch.Tensor, group=None, *, exchange=None, swizzle: bool = True):
    """NVFP4-quantize this rank's row block of a row-sharded tensor with the global scale
    of the WHOLE tensor.  Block scales and payload are row-local; only the tensor-wide amax
    is exchanged.  With row blocks that are multiples of 128 rows (``plan_row_shards``) the
    per-rank swizzled scale buffers concatenate to the unsharded one."""
    from ..cute.nvfp4_tma import quantize_nvfp4

    amax = sharded_global_amax(local_rows, group, exchange=exchange)
    return quantize_nvfp4(local_rows, amax, swizzle=swizzle)
