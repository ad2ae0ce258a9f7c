"""CPU oracle for the scaled-quantization cast path.

TEST INFRASTRUCTURE ONLY.  Nothing in the shipped package imports this
directory: it is the checker that the parity tests, the smoke check and the
benchmark's CPU-baseline leg compare against or time.  The product path is the
CUDA library under ``transformer_nuggets_b200/csrc`` and has no CPU fallback.

Parity status of each function is stated in its docstring:

* pinned      - checked bit-for-bit against the reference's own Python
                function imported in the build container (fixtures under
                ``tests/golden`` were written by that import).
* restatement - the reference has no such function; the oracle applies the
                reference's per-tensor formula at another granularity.
* unpinned    - the reference has no quantizer for the format at all
                (NVFP4); only the storage contract is pinned.
"""

from .cast_oracle import (  # noqa: F401
    FP8_MAX,
    delayed_scale_update,
    e2m1_decode,
    e2m1_encode,
    e8m0_exponent_ceil_int,
    e8m0_exponent_floor_int,
    fp8_dynamic_quant,
    fp8_matmul,
    fp8_rowwise_quant,
    fp8_scaled_quant,
    mxfp8_dequantize,
    mxfp8_gemv,
    nvfp4_gemv,
    mxfp8_quantize,
    nvfp4_dequantize,
    nvfp4_quantize,
    pack_nvfp4_codes,
    rms_norm,
    rms_norm_rowwise_quant,
    sharded_fp8_dynamic_quant,
    swiglu,
    swizzle_offset,
    to_blocked,
    to_blocked_closed_form,
)
