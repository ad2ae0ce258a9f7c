"""ctypes binding of ``libtnq.so`` - the only route from Python to the kernels.

There is no CPU path behind these functions: if the library is missing or an
argument is not a CUDA tensor the call raises.
"""

from __future__ import annotations

import collections
import ctypes
import os
import threading

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "csrc", "libtnq.so")

TNQ_OK = 0
STATUS_NAMES = {1: "EINVAL", 2: "EALIGN", 3: "ESHAPE", 4: "EUNSUPPORTED", 5: "ECUDA", 6: "ETIMEOUT"}
IN_BF16, IN_F32 = 0, 1
FP8_E4M3, FP8_E5M2 = 0, 1
E8M0_CEIL, E8M0_FLOOR = 0, 1
SCALES_RAW, SCALES_SWIZZLED = 0, 1
SCALE_IS_SCALE, SCALE_IS_AMAX = 0, 1
WORKSPACE_BYTES = 16384
WS_AMAX_WORD, WS_SCALE_WORD, WS_STATUS_WORD = 1, 2, 3
OPT_CAST_REVERSE = 1

IN_DTYPES = {torch.bfloat16: IN_BF16, torch.float32: IN_F32}
FP8_DTYPES = {torch.float8_e4m3fn: FP8_E4M3, torch.float8_e5m2: FP8_E5M2}

_p, _i64, _i = ctypes.c_void_p, ctypes.c_int64, ctypes.c_int

# name -> argument types (all return int unless noted)
SIGNATURES = {
    "tnq_fp8_amax": [_p, _i64, _i, _i, _p, _p, _p],
    "tnq_fp8_scaled_cast": [_p, _p, _i64, _i, _i, _p, _i, _i, _p, _p, _p],
    "tnq_fp8_dynamic_cast": [_p, _p, _i64, _i, _i, _p, _p, _p],
    "tnq_fp8_dynamic_cast_profile": [_p, _p, _i64, _p, _p, _p, _p, _p],
    "tnq_tile_copy": [_p, _p, _i64, _i64, _i, _i, _p, _p],
    "tnq_fp8_dynamic_cast_static": [_p, _p, _i64, _i, _i, _p, _p],
    "tnq_fp8_dynamic_cast_static_max_elements": [],
    "tnq_fp8_rowwise": [_p, _i64, _i64, _i, _p, _p, _p, _p, _p, _p],
    "tnq_rowwise_set_tma": [_i],
    "tnq_rowwise_set_group": [_i],
    "tnq_gemv_set_shape": [_i],
    "tnq_mxfp8_quantize": [_p, _i64, _i64, _i, _p, _p, _p, _p, _i, _i, _p, _p],
    "tnq_mxfp8_set_store_variant": [_i],
    "tnq_nvfp4_quantize": [_p, _i64, _i64, _i, _p, _p, _p, _i, _p, _p, _p],
    "tnq_nvfp4_quantize_dynamic": [_p, _i64, _i64, _i, _p, _p, _p, _i, _p, _p],
    "tnq_pack_fp4_codes": [_p, _i64, _i64, _p, _p],
    "tnq_to_blocked": [_p, _i64, _i64, _p, _p],
    "tnq_exchange_create": [_p, _p],
    "tnq_exchange_open": [_p, _p],
    "tnq_exchange_close": [_p],
    "tnq_exchange_destroy": [_p],
    "tnq_exchange_status": [_p, _p],
    "tnq_fp8_sharded_cast": [_p, _p, _i64, _i, _i, _p, _p, _i, _i, ctypes.c_uint32, _p, _p],
    "tnq_sharded_amax": [_p, _i64, _i, _p, _p, _i, _i, ctypes.c_uint32, _p, _p],
    "tnq_fp8_cast_transpose": [_p, _i64, _i64, _i, _i, _p, _i, _i, _p, _p, _p, _p, _p],
    "tnq_fp8_dynamic_cast_transpose": [_p, _i64, _i64, _i, _i, _p, _p, _p, _p, _p],
    "tnq_cast_transpose_set_store_variant": [_i],
    "tnq_rmsnorm_fp8_rowwise": [_p, _p, ctypes.c_float, _i64, _i64, _p, _p, _p, _p],
    "tnq_rmsnorm_mxfp8": [_p, _p, ctypes.c_float, _i64, _i64, _p, _p, _i, _i, _p, _p],
    "tnq_swiglu_fp8_rowwise": [_p, _p, _i64, _i64, _p, _p, _p, _p],
    "tnq_swiglu_mxfp8": [_p, _p, _i64, _i64, _p, _p, _i, _i, _p, _p],
    "tnq_fp8_gemm": [_p, _p, _p, _p, _i, _i, _i64, _i64, _i64, _p, _p, _p],
    "tnq_mxfp8_gemm": [_p, _p, _p, _p, _i64, _i64, _i64, _p, _p, _p],
    "tnq_nvfp4_gemm": [_p, _p, _p, _p, _p, _p, _i64, _i64, _i64, _p, _p, _p],
    "tnq_delayed_scale_update": [_p, _p, _p, _i64, _i, _i, _p],
    "tnq_mxfp8_gemv": [_p, _p, _p, _p, _i64, _i64, _i, _p, _p],
    "tnq_nvfp4_gemv": [_p, _p, _p, _p, _p, _p, _i64, _i64, _i, _p, _p],
    "tnq_set_option": [_i, _i],
    "tnq_last_cuda_error": [],
    "tnq_abi_version": [],
}

_lib = None
_lock = threading.Lock()


class TnqError(RuntimeError):
    def __init__(self, fn, status, detail=""):
        self.status = status
        super().__init__(f"{fn} failed: {STATUS_NAMES.get(status, status)} {detail}".strip())


def load():
    """Load (once) and return the ctypes handle.  Raises if the library is absent:
    build it with ``python -m transformer_nuggets_b200.build``."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is None:
            if not os.path.exists(LIB_PATH):
                raise ImportError(
                    f"{LIB_PATH} not found. The cast kernels are CUDA only and have no fallback; "
                    "build them with `python -m transformer_nuggets_b200.build`."
                )
            lib = ctypes.CDLL(LIB_PATH)
            for name, argtypes in SIGNATURES.items():
                fn = getattr(lib, name)
                fn.argtypes = argtypes
                fn.restype = _i
            lib.tnq_fp8_dynamic_cast_static_max_elements.restype = ctypes.c_int64
            lib.tnq_status_str.argtypes = [_i]
            lib.tnq_status_str.restype = ctypes.c_char_p
            _lib = lib
    return _lib


#: ``TNQ_CHECK_STATUS=1`` in the environment makes every entry point synchronise and read the
#: device status word after its launch (debugging aid; costs a device synchronisation per call).
CHECK_EVERY_CALL = os.environ.get("TNQ_CHECK_STATUS", "0") not in ("", "0")


def call(name, *args):
    lib = load()
    rc = getattr(lib, name)(*args)
    if rc != TNQ_OK:
        detail = lib.tnq_status_str(rc).decode()
        if rc == 5:
            detail += f" (cudaError {lib.tnq_last_cuda_error()})"
        raise TnqError(name, rc, detail)
    if CHECK_EVERY_CALL and name not in _NO_LAUNCH:
        check_status(torch.cuda.current_device(), what=name)


def stream_ptr(device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def ptr(t) -> int:
    return 0 if t is None else t.data_ptr()


#: compute capabilities the library image holds code for (built for sm_100a only)
SUPPORTED_CAPABILITIES = {(10, 0)}
_capability_ok: dict = {}


def require_capability(index: int):
    """Raise ``ValueError`` unless device ``index`` is a B200-class GPU.  The reference's CuTe
    entry points refuse other parts the same way before any launch (cute/mxfp8_tma.py:275); here
    the check also keeps a launch on another architecture from surfacing as a bare CUDA error."""
    if _capability_ok.get(index):
        return
    cap = tuple(torch.cuda.get_device_capability(index))
    if cap not in SUPPORTED_CAPABILITIES:
        raise ValueError(
            f"device {index} has compute capability {cap[0]}.{cap[1]}; these kernels are built for "
            "sm_100a (compute capability 10.0) only"
        )
    _capability_ok[index] = True


def require_cuda(t: torch.Tensor, what: str):
    if not isinstance(t, torch.Tensor):
        raise TypeError(f"{what} must be a torch.Tensor")
    if not t.is_cuda:
        raise ValueError(f"{what} must be a CUDA tensor: the cast kernels have no CPU path")
    require_capability(t.device.index if t.device.index is not None else torch.cuda.current_device())


#: entry points that launch nothing (no status to look at afterwards)
_NO_LAUNCH = {"tnq_set_option", "tnq_gemv_set_shape", "tnq_mxfp8_set_store_variant", "tnq_cast_transpose_set_store_variant", "tnq_rowwise_set_tma", "tnq_rowwise_set_group", "tnq_exchange_create",
              "tnq_exchange_open", "tnq_exchange_close", "tnq_exchange_destroy", "tnq_exchange_status"}

#: most recently used (device, stream) -> workspace; bounded so that a program that keeps creating
#: streams does not accumulate scratch tensors for streams that no longer exist
MAX_WORKSPACES = 64
_workspaces: "collections.OrderedDict" = collections.OrderedDict()


def workspace(device) -> torch.Tensor:
    """Zero-initialised per-(device, stream) scratch for the tensor-wide reductions."""
    device = torch.device(device)
    idx = device.index if device.index is not None else torch.cuda.current_device()
    key = (idx, torch.cuda.current_stream(idx).cuda_stream)
    ws = _workspaces.get(key)
    if ws is None:
        ws = torch.zeros(WORKSPACE_BYTES // 4, dtype=torch.int32, device=torch.device("cuda", idx))
        _workspaces[key] = ws
        while len(_workspaces) > MAX_WORKSPACES:  # the evicted tensor returns to the allocator of its own stream
            _workspaces.popitem(last=False)
    else:
        _workspaces.move_to_end(key)
    return ws


def check_status(device=None, what: str = "a kernel"):
    """Synchronise ``device`` and read the status word of every workspace this module handed out on
    it.  The kernels never wait without a bound: a wait that gives up (a TMA copy, the grid barrier
    of the single-launch cast, a peer's amax word) records ``TNQ_ETIMEOUT`` there and the kernel
    returns, leaving its outputs incomplete.  This is the call that turns that record into an
    exception.  It also puts the workspace header (the first 64 bytes: ticket, barrier counters,
    status) back to zero, because a kernel that left early may not have rewound them.  Raises
    ``TnqError`` with ``status == 6`` if any word was set."""
    if device is None:
        idx = torch.cuda.current_device()
    else:
        device = torch.device(device) if not isinstance(device, int) else torch.device("cuda", device)
        idx = device.index if device.index is not None else torch.cuda.current_device()
    bad = None
    for (dev_idx, _stream), ws in list(_workspaces.items()):
        if dev_idx != idx:
            continue
        if ws.is_cuda:
            torch.cuda.synchronize(idx)
        st = int(ws[WS_STATUS_WORD].item())
        if st != 0:
            bad = st
            ws[:16].zero_()
    if bad is not None:
        raise TnqError(what, bad, "(device status word: a bounded device-side wait expired; outputs of the "
                                  "calls since the last check are incomplete)")
