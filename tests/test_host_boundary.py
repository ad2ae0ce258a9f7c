"""Host-side boundary behaviour that needs no GPU: the names the reference's own tests import,
the capability gate, and the status-word check."""

import pytest
import torch

from transformer_nuggets_b200 import _lib


def test_reference_test_imports_resolve():
    """test/test_mx.py of the reference imports these four names from mx.to_blocked."""
    from transformer_nuggets_b200.mx.to_blocked import (  # noqa: F401
        _to_blocked_single,
        _to_blocked_single_manual,
        to_blocked,
        to_blocked_manual,
    )
    from transformer_nuggets_b200.fp8.scaled_quant import (  # noqa: F401  (test/test_fp8.py)
        dynamic_scaled_quant,
        eager_dynamic_scaled_quant,
        eager_scaled_quant,
        scaled_quant,
    )


@pytest.mark.parametrize("cap,ok", [((10, 0), True), ((9, 0), False), ((10, 3), False), ((12, 0), False)])
def test_capability_gate(monkeypatch, cap, ok):
    """Only compute capability 10.0 passes (the library image holds sm_100a code only); anything
    else is a ValueError before any launch, as in the reference's CuTe entry points."""
    monkeypatch.setattr(torch.cuda, "get_device_capability", lambda index=None: cap)
    monkeypatch.setattr(_lib, "_capability_ok", {})
    if ok:
        _lib.require_capability(0)
        _lib.require_capability(0)  # cached
    else:
        with pytest.raises(ValueError, match="sm_100a"):
            _lib.require_capability(0)


def test_cpu_tensor_is_refused():
    with pytest.raises(ValueError, match="CUDA tensor"):
        _lib.require_cuda(torch.zeros(4), "x")
    with pytest.raises(TypeError):
        _lib.require_cuda([1, 2], "x")


def test_check_status_raises_and_rezeroes(monkeypatch):
    """A status word left by a kernel whose bounded wait expired becomes a TnqError(ETIMEOUT) and
    the workspace header is put back to zero (stand-in workspace on the host: no GPU involved)."""
    ws = torch.zeros(_lib.WORKSPACE_BYTES // 4, dtype=torch.int32)
    fake = {(0, 0): ws}
    monkeypatch.setattr(_lib, "_workspaces", fake)
    _lib.check_status(0)  # clean: nothing raised
    ws[_lib.WS_STATUS_WORD] = 6
    ws[6] = 17  # an arrival counter the kernel did not rewind
    ws[100] = 5  # beyond the header: untouched
    with pytest.raises(_lib.TnqError) as e:
        _lib.check_status(0, what="tnq_mxfp8_quantize")
    assert e.value.status == 6 and "ETIMEOUT" in str(e.value)
    assert int(ws[:16].abs().sum()) == 0 and int(ws[100]) == 5
    _lib.check_status(0)  # the next check is clean again
    ws[_lib.WS_STATUS_WORD] = 6
    _lib.check_status(1)  # another device's check does not look at this workspace
    assert int(ws[_lib.WS_STATUS_WORD]) == 6
