"""The C-ABI library loads on a machine without a GPU, exports every function that
include/tnq.h declares, and rejects bad arguments before touching CUDA."""

import ctypes
import os
import re

import pytest
import torch

from conftest import ROOT
from transformer_nuggets_b200 import _lib


def declared_functions():
    text = open(os.path.join(ROOT, "include", "tnq.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(tnq_[a-z0-9_]+)\s*\(", text)))


def test_header_functions_are_exported():
    lib = _lib.load()
    names = declared_functions()
    assert len(names) >= 10
    for n in names:
        assert hasattr(lib, n), f"{n} declared in include/tnq.h but not exported by libtnq.so"


def test_binding_covers_header():
    bound = set(_lib.SIGNATURES) | {"tnq_status_str"}
    assert set(declared_functions()) <= bound


def test_status_strings():
    lib = _lib.load()
    assert lib.tnq_status_str(0) == b"ok"
    for code in range(1, 7):
        assert lib.tnq_status_str(code) not in (b"ok", b"unknown status")
    assert lib.tnq_abi_version() >= 1


def test_bad_arguments_are_rejected_without_cuda():
    lib = _lib.load()
    # null input with n > 0, unknown dtypes, misaligned pointers: all refused up front
    assert lib.tnq_fp8_amax(None, 16, 0, 0, None, None, None) == 1
    assert lib.tnq_fp8_amax(ctypes.c_void_p(64), 16, 7, 0, ctypes.c_void_p(64), None, None) == 4
    assert lib.tnq_fp8_amax(ctypes.c_void_p(72), 16, 0, 0, ctypes.c_void_p(64), None, None) == 2
    assert lib.tnq_fp8_scaled_cast(ctypes.c_void_p(64), None, 16, 0, 0, ctypes.c_void_p(64), 0, 1, None, None, None) == 1
    assert lib.tnq_fp8_rowwise(ctypes.c_void_p(64), 4, 24, 0, ctypes.c_void_p(64), ctypes.c_void_p(64), None, None, None, None) == 3
    assert lib.tnq_mxfp8_quantize(ctypes.c_void_p(64), 32, 48, 0, ctypes.c_void_p(64), ctypes.c_void_p(64), None, None, 0, 0, None, None) == 3
    assert lib.tnq_mxfp8_quantize(ctypes.c_void_p(64), 32, 64, 1, ctypes.c_void_p(64), ctypes.c_void_p(64), None, None, 0, 0, None, None) == 4
    assert lib.tnq_nvfp4_quantize(ctypes.c_void_p(64), 32, 24, 0, ctypes.c_void_p(64), ctypes.c_void_p(64), ctypes.c_void_p(64), 0, None, None, None) == 3
    assert lib.tnq_to_blocked(None, 4, 4, ctypes.c_void_p(64), None) == 1
    assert lib.tnq_pack_fp4_codes(ctypes.c_void_p(64), 4, 8, ctypes.c_void_p(64), None) == 3


def test_python_entry_points_refuse_cpu_tensors():
    import transformer_nuggets_b200 as tn

    x = torch.zeros(32, 64, dtype=torch.bfloat16)
    with pytest.raises(ValueError, match="no CPU path"):
        tn.dynamic_scaled_quant(x)
    with pytest.raises(ValueError, match="no CPU path"):
        tn.rowwise_scaled_quant(x)
    with pytest.raises(ValueError, match="no CPU path"):
        tn.quantize_mxfp8_tensor(x)
    with pytest.raises(ValueError, match="no CPU path"):
        tn.quantize_nvfp4(x)
    with pytest.raises(ValueError, match="no CPU path"):
        tn.to_blocked(torch.zeros(4, 4, dtype=torch.uint8))
    # the reference's own argument checks (fp8/scaled_quant.py:53-57) come first
    with pytest.raises(AssertionError):
        tn.scaled_quant(x, torch.ones(1, dtype=torch.float64), torch.zeros(1))
    with pytest.raises(AssertionError):
        tn.scaled_quant(x, torch.ones(2), torch.zeros(1))


def test_missing_library_fails_loudly(monkeypatch):
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", "/nonexistent/libtnq.so")
    with pytest.raises(ImportError, match="no fallback"):
        _lib.load()
