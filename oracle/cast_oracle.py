"""CPU restatement (PyTorch CPU ops, fp32 arithmetic) of the reference's cast path.

TEST INFRASTRUCTURE ONLY - see the package docstring.  Every function cites
the reference file:line it follows (paths are relative to the root of
drisspg/transformer_nuggets).

Numerics rules shared by all functions
--------------------------------------
* All arithmetic is IEEE fp32 with round-to-nearest-even; bf16 -> fp32
  widening is exact.
* The fp32 -> fp8 conversion is PyTorch's CPU cast: RNE, *non*-saturating
  (e4m3fn: |y| that rounds above 448 becomes NaN 0x7F|sign; e5m2: |y| >= 61440
  becomes inf 0x7C|sign; NaN becomes 0x7F|sign).  Saturation is the explicit
  pair of ``torch.where`` clamps in front of the cast, which let NaN through.
* A ``scale`` tensor is always used with shape ``[1]`` (or ``[M, 1]``): a 0-dim
  fp32 scale would make ``bf16 * scale`` a bf16 product (type promotion) and
  round twice.
"""

from __future__ import annotations

import torch

FP8_MAX = {torch.float8_e4m3fn: 448.0, torch.float8_e5m2: 57344.0}

# Guard that keeps 448/amax finite for an all-zero tensor.  The reference's
# Triton kernel has `tl.clamp(amax, -1e12, inf)` (fp8/scaled_quant.py:132),
# evidently meant as a lower bound of 1e-12; torchao's tensor_to_scale (the
# eager twin's dependency, fp8/scaled_quant.py:182-185) clamps amax the same
# way.  It never binds for a tensor with any nonzero finite element >= 1e-12.
AMAX_EPS = 1e-12


# --------------------------------------------------------------------------- #
# per-tensor FP8                                                               #
# --------------------------------------------------------------------------- #
def fp8_scaled_quant(
    a: torch.Tensor,
    scale: torch.Tensor,
    abs_max: torch.Tensor,
    fp8_dtype: torch.dtype,
    saturated: bool = False,
) -> torch.Tensor:
    """Delayed-scale cast.  Parity: pinned.

    Follows ``eager_scaled_quant`` (fp8/scaled_quant.py:78-102): product in
    fp32, optional clamp by two ``where`` (:96-100), amax side output (:101),
    non-saturating cast (:102).  ``abs_max`` is updated as
    ``max(abs_max, max|a|)``, which is what the Triton twin's ``atomic_max``
    does (fp8/scaled_quant.py:24) and equals the eager ``fill_`` whenever the
    caller starts below the true amax, as the reference's tests do with -1.0
    (test/test_fp8.py:21).
    """
    assert scale.dtype == torch.float32 and scale.dim() >= 1
    fmax = FP8_MAX[fp8_dtype]
    out = a * scale
    assert out.dtype == torch.float32
    if saturated:
        out = torch.where(out > fmax, fmax, out)
        out = torch.where(out < -fmax, -fmax, out)
    amax = torch.max(torch.abs(a)).to(torch.float32)
    old = abs_max.reshape(())
    new = amax if (not bool(old >= amax)) else old  # NaN amax wins, like torch.max
    abs_max.fill_(new)
    return out.to(fp8_dtype)


def _scale_from_amax(amax: torch.Tensor, fp8_dtype: torch.dtype) -> torch.Tensor:
    """scale = finfo.max / max(amax, 1e-12), one fp32 division.

    This is `max_val / clamp(amax)` of the Triton kernel
    (fp8/scaled_quant.py:132).
    """
    amax = amax.to(torch.float32)
    return torch.tensor(FP8_MAX[fp8_dtype], dtype=torch.float32) / torch.clamp(amax, min=AMAX_EPS)


def fp8_dynamic_quant(a: torch.Tensor, fp8_dtype: torch.dtype):
    """Per-tensor dynamic cast -> (fp8 tensor, fp32 scale of shape [1]).

    Parity: pinned through ``eager_scaled_quant`` fed ``scale = max/amax`` with
    ``saturated=True``; that is the arithmetic of ``dynamic_scaled_cast``
    (fp8/scaled_quant.py:108-136: amax, ``scale = max_val/amax``, clamp, cast).
    The reference's ``eager_dynamic_scaled_quant`` (:172-186) delegates the
    same three steps to torchao, which is not installed here (unpinned there).
    """
    amax = torch.max(torch.abs(a)).to(torch.float32)
    scale = _scale_from_amax(amax, fp8_dtype).reshape(1)
    dummy = torch.zeros(1, dtype=torch.float32)
    q = fp8_scaled_quant(a, scale, dummy, fp8_dtype, saturated=True)
    return q, scale


def fp8_rowwise_quant(a: torch.Tensor, fp8_dtype: torch.dtype):
    """Row-wise dynamic cast -> (fp8 [M, K], fp32 scale [M, 1]).

    Parity: pinned through ``eager_scaled_quant`` (fp8/scaled_quant.py:78-102)
    called once per row with that row's ``[1]``-shaped scale and
    ``saturated=True`` (fixture ``tests/golden/fp8_rowwise.npz``).  The
    reference has no rowwise cast of its own, only the consumer contract - a
    per-row fp32 scale of shape [M, 1] (fp8/fp8_matmul.py:50-61); the scale
    rule ``max / clamp(amax_r, 1e-12)`` is the per-tensor one of :132-135 at
    row granularity.  The returned scale is the quantisation-direction one
    (``max/amax_r``), like the per-tensor scale.
    """
    assert a.dim() == 2
    fmax = FP8_MAX[fp8_dtype]
    amax = a.abs().amax(dim=-1, keepdim=True).to(torch.float32)
    scale = torch.tensor(fmax, dtype=torch.float32) / torch.clamp(amax, min=AMAX_EPS)
    out = a.to(torch.float32) * scale
    out = torch.where(out > fmax, fmax, out)
    out = torch.where(out < -fmax, -fmax, out)
    return out.to(fp8_dtype), scale


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """Eager RMSNorm: ``(x.float() * rsqrt(mean(x.float()^2, -1) + eps) * weight.float()).to(x.dtype)``.

    Parity: pinned up to summation order - a line-for-line restatement of
    ``handwritten_rms_norm`` (examples/rms_norm_fusion_profile.py:26-31), checked against
    the fixture that function wrote.  Every step but ``mean`` is one correctly rounded fp32
    operation; ``mean`` depends on the order in which the squares are added, so a GPU
    kernel agrees with this function up to an occasional last-place bf16 rounding."""
    x32 = x.float()
    variance = x32.square().mean(dim=-1, keepdim=True)
    normalized = x32 * torch.rsqrt(variance + eps)
    return (normalized * weight.float()).to(x.dtype)


def rms_norm_rowwise_quant(x: torch.Tensor, weight: torch.Tensor, eps: float, fp8_dtype: torch.dtype = torch.float8_e4m3fn):
    """RMSNorm followed by the row-wise dynamic cast of its bf16 result:
    ``(fp8 [M, C], scale [M, 1], y bf16)``.  Restatement (composition of ``rms_norm`` and
    ``fp8_rowwise_quant``; the reference has no fused op)."""
    y = rms_norm(x, weight, eps)
    q, scale = fp8_rowwise_quant(y, fp8_dtype)
    return q, scale, y


def swiglu(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """``F.silu(a) * b`` on bf16 tensors, evaluated eagerly: the operand of ``w2`` in the
    reference's ``FeedForward`` (llama/model.py:228).  Parity: restatement of that expression
    (the same two torch ops); ``exp`` is not correctly rounded, so a GPU evaluation agrees up
    to an occasional last-place bf16 rounding."""
    return torch.nn.functional.silu(a) * b


def fp8_matmul(a: torch.Tensor, a_scale: torch.Tensor, b: torch.Tensor, b_scale: torch.Tensor) -> torch.Tensor:
    """``bf16((a.float() @ b.float()) * (a_scale * b_scale))`` with ``a [M, K]``, ``b [K, N]`` fp8 and
    per-tensor (one element) or row-wise (``[M, 1]``, ``[1, N]``) fp32 scales: the arithmetic of
    ``apply_scaling`` behind the reference's matmul kernels (fp8/fp8_matmul.py:109-138, 215-238).
    Floating point: products of two fp8 values are exact in fp32, the order of the fp32
    accumulation is not fixed, so comparisons use a tolerance."""
    acc = a.float() @ b.float()
    return (acc * (a_scale.float() * b_scale.float())).to(torch.bfloat16)


def delayed_scale_update(amax_history: torch.Tensor, amax: torch.Tensor, fp8_dtype: torch.dtype):
    """Delayed-scaling state update for a stack of tensors: returns (new history
    [T, L], new scale [T]).  ``history <- roll(history, 1, dim=1); history[:, 0] = amax;
    scale = finfo.max / clamp(max(history, dim=1), 1e-12)`` in fp32.

    Parity: UNPINNED restatement.  The reference calls float8_experimental's
    ``sync_float8_amax_and_scale_history`` (llama/train.py:251-263); that package is not in
    the reference tree and its version is not pinned by pyproject.toml.  This follows its
    published "max" recipe (``_update_history_stack`` + ``amax_history_to_scale_stack``)
    with the single fp32 division the other casts use.
    """
    hist = torch.roll(amax_history.to(torch.float32), 1, dims=1)
    hist[:, 0] = amax.to(torch.float32).reshape(-1)
    return hist, _scale_from_amax(hist.max(dim=1).values, fp8_dtype)


def sharded_fp8_dynamic_quant(shards, fp8_dtype: torch.dtype):
    """Row-sharded per-tensor cast: local amax -> MAX over shards -> same scale
    on every shard -> cast.  Returns (list of fp8 shards, scale [1]).

    Parity: restatement (the reference has no multi-device cast).  MAX over
    non-negative floats is exact and order independent, so the concatenated
    result equals ``fp8_dynamic_quant`` of the concatenated input bit for bit.
    """
    amax = torch.stack([s.abs().max().to(torch.float32) for s in shards]).max()
    scale = _scale_from_amax(amax, fp8_dtype).reshape(1)
    dummy = torch.zeros(1, dtype=torch.float32)
    return [fp8_scaled_quant(s, scale, dummy, fp8_dtype, saturated=True) for s in shards], scale


# --------------------------------------------------------------------------- #
# MXFP8                                                                        #
# --------------------------------------------------------------------------- #
def mxfp8_quantize(value: torch.Tensor, scale_mode: str = "ceil"):
    """32-element blocks along the last dim -> (e4m3 same shape, uint8 E8M0
    raw scales [rows, K/32], row-major).  Stored byte = exponent + 127.

    ``scale_mode="ceil"``: parity pinned - a line-for-line restatement of
    ``quantize_mxfp8_tensor`` (cute/mxfp8_tma.py:497-504):
    ``e = clamp(ceil(log2(amax/448)), -126, 127)``.
    ``scale_mode="floor"``: the OCP rule ``e = clamp(floor(log2(amax)) - 8,
    -126, 127)`` with the same divide / clamp / cast; restatement.
    Column-wise quantisation is this function applied to ``value.t().contiguous()``.
    """
    assert value.dim() == 2 and value.shape[1] % 32 == 0
    blocks = value.float().reshape(value.shape[0], -1, 32)
    max_abs = blocks.abs().amax(dim=-1).clamp_min(torch.finfo(torch.float32).tiny)
    if scale_mode == "ceil":
        exponent = torch.ceil(torch.log2(max_abs / 448.0)).clamp(-126, 127)
    elif scale_mode == "floor":
        exponent = (torch.floor(torch.log2(max_abs)) - 8.0).clamp(-126, 127)
    else:
        raise ValueError(scale_mode)
    scale = torch.exp2(exponent).unsqueeze(-1)
    quantized = (blocks / scale).clamp(-448, 448).to(torch.float8_e4m3fn)
    return quantized.reshape_as(value), (exponent + 127).to(torch.uint8)


def _f32_fields(amax_f32: torch.Tensor):
    bits = amax_f32.contiguous().view(torch.int32)
    return ((bits >> 23) & 0xFF) - 127, bits & 0x7FFFFF, ((bits >> 23) & 0xFF)


def e8m0_exponent_ceil_int(amax_f32: torch.Tensor) -> torch.Tensor:
    """Integer form of the ceil rule, the one the CUDA kernel evaluates:
    with E the unbiased exponent and M the 23-bit mantissa of amax,
    ``e = clamp(E - 8 + (M > 0x600000), -126, 127)``; zero / subnormal amax
    gives -126.  (448 = 1.75 * 2^8, and 0x600000 is the mantissa of 1.75.)
    Equal to the log2 form for every bf16-valued amax - checked exhaustively in
    the tests against the reference function itself.
    """
    E, M, biased = _f32_fields(amax_f32.to(torch.float32))
    e = E - 8 + (M > 0x600000).to(torch.int32)
    e = torch.where(biased == 0, torch.full_like(e, -126), e)
    return e.clamp(-126, 127)


def e8m0_exponent_floor_int(amax_f32: torch.Tensor) -> torch.Tensor:
    """Integer form of the floor rule: ``e = clamp(E - 8, -126, 127)``."""
    E, _, biased = _f32_fields(amax_f32.to(torch.float32))
    e = torch.where(biased == 0, torch.full_like(E, -126), E - 8)
    return e.clamp(-126, 127)


# --------------------------------------------------------------------------- #
# scale swizzle (SWIZZLE_32_4_4, the "128x4" layout of block-scaled MMA)       #
# --------------------------------------------------------------------------- #
def to_blocked(input_matrix: torch.Tensor) -> torch.Tensor:
    """[H, W] one-byte scales -> flat swizzled buffer of
    512*ceil(H/128)*ceil(W/4) elements, zero padded.  Parity: pinned.

    Follows ``to_blocked`` (mx/to_blocked.py:10-42): pad to (128, 4) multiples
    (:22-34), split into 128x4 blocks (:37), interleave the four 32-row groups
    of each block (:38), flatten (:40).
    """
    rows, cols = input_matrix.shape
    nrb, ncb = -(-rows // 128), -(-cols // 4)
    padded = torch.zeros((nrb * 128, ncb * 4), dtype=input_matrix.dtype)
    padded[:rows, :cols] = input_matrix
    blocks = padded.view(nrb, 128, ncb, 4).permute(0, 2, 1, 3)
    return blocks.reshape(-1, 4, 32, 4).transpose(1, 2).reshape(-1, 32, 16).flatten()


def swizzle_offset(r, c, n_col_blocks):
    """Closed form of the same layout: byte offset of scale element (r, c)."""
    return (
        ((r // 128) * n_col_blocks + (c // 4)) * 512
        + (r % 32) * 16
        + ((r % 128) // 32) * 4
        + (c % 4)
    )


def to_blocked_closed_form(input_matrix: torch.Tensor) -> torch.Tensor:
    """``to_blocked`` through :func:`swizzle_offset` (the form the kernels use)."""
    rows, cols = input_matrix.shape
    nrb, ncb = -(-rows // 128), -(-cols // 4)
    out = torch.zeros(512 * nrb * ncb, dtype=input_matrix.dtype)
    r = torch.arange(rows).unsqueeze(1).expand(rows, cols)
    c = torch.arange(cols).unsqueeze(0).expand(rows, cols)
    out[swizzle_offset(r, c, ncb).reshape(-1)] = input_matrix.reshape(-1)
    return out


# --------------------------------------------------------------------------- #
# NVFP4                                                                        #
# --------------------------------------------------------------------------- #
_E2M1_VALUES = torch.tensor(
    [0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0, -0.0, -0.5, -1.0, -1.5, -2.0, -3.0, -4.0, -6.0],
    dtype=torch.float32,
)  # code -> value table pinned by test/test_nvfp4_tma.py:32-35


def e2m1_encode(v: torch.Tensor) -> torch.Tensor:
    """fp32 -> 4-bit e2m1 code (uint8 0..15): round to nearest on the grid
    {0, .5, 1, 1.5, 2, 3, 4, 6}, ties to the even code, saturating at +-6;
    bit 3 is the sign (-0.0 -> 8).  NaN is outside the domain."""
    mag = v.abs()
    code = (
        (mag > 0.25).to(torch.uint8)
        + (mag >= 0.75).to(torch.uint8)
        + (mag > 1.25).to(torch.uint8)
        + (mag >= 1.75).to(torch.uint8)
        + (mag > 2.5).to(torch.uint8)
        + (mag >= 3.5).to(torch.uint8)
        + (mag > 5.0).to(torch.uint8)
    )
    return code | (torch.signbit(v).to(torch.uint8) << 3)


def e2m1_decode(codes: torch.Tensor) -> torch.Tensor:
    return _E2M1_VALUES[codes.long()]


def pack_nvfp4_codes(codes: torch.Tensor) -> torch.Tensor:
    """Low nibble first: byte = code[2i] | code[2i+1] << 4 (uint8 [M, K/2]).
    Parity: pinned - cute/nvfp4_tma.py:941-943 (returned here as uint8, the
    reference views the same bytes as ``torch.float4_e2m1fn_x2``)."""
    return (codes[:, 0::2] | (codes[:, 1::2] << 4)).contiguous()


def nvfp4_quantize(x: torch.Tensor, global_amax: torch.Tensor | None = None):
    """16-element blocks along the last dim -> (packed uint8 [M, K/2], e4m3
    block scales [M, K/16] raw row-major, fp32 global scale [1] in the decode
    direction: value = e2m1 * block_scale * global_scale).

    Parity: UNPINNED.  The reference contains no NVFP4 quantizer; it fixes only
    the storage contract (nibble order cute/nvfp4_tma.py:941-943, swizzled e4m3
    block scales :946-964, fp32 [1] global scale multiplied in at decode
    :527-547 and cute/blockscaled_tma.py:807-818).  The arithmetic below is
    this build's specification:

      amax_t = max(max|x|, 1e-12)      g_dec = amax_t / 2688    g_enc = 2688 / amax_t
      per block: s = (amax_b / 6) * g_enc ; s_q = e4m3_rne(min(s, 448))
                 d = f32(s_q) * g_dec ;  r = 0 if d == 0 else 1 / d
                 code_i = e2m1_rne_sat(x_i * r)
    with every operation a single correctly rounded fp32 operation.
    """
    assert x.dim() == 2 and x.shape[1] % 16 == 0
    f = torch.float32
    xf = x.to(f)
    if global_amax is None:
        global_amax = xf.abs().max()
    amax_t = torch.clamp(global_amax.to(f).reshape(()), min=AMAX_EPS)
    k2688 = torch.tensor(2688.0, dtype=f)
    g_dec = amax_t / k2688
    g_enc = k2688 / amax_t
    blocks = xf.reshape(x.shape[0], -1, 16)
    amax_b = blocks.abs().amax(dim=-1)
    s = (amax_b / torch.tensor(6.0, dtype=f)) * g_enc
    s_q = torch.clamp(s, max=448.0).to(torch.float8_e4m3fn)
    d = s_q.to(f) * g_dec
    r = torch.where(d == 0, torch.zeros_like(d), torch.tensor(1.0, dtype=f) / d)
    v = blocks * r.unsqueeze(-1)
    codes = e2m1_encode(v).reshape(x.shape)
    return pack_nvfp4_codes(codes), s_q, g_dec.reshape(1)


def nvfp4_dequantize(packed: torch.Tensor, s_q: torch.Tensor, g_dec: torch.Tensor) -> torch.Tensor:
    """Decode with the reference's convention (cute/nvfp4_tma.py:37-65,
    cute/blockscaled_tma.py:807-818): value = table[code] * f32(block scale) *
    global scale."""
    lo = packed & 0xF
    hi = packed >> 4
    codes = torch.stack([lo, hi], dim=-1).reshape(packed.shape[0], -1)
    vals = e2m1_decode(codes).reshape(packed.shape[0], -1, 16)
    return (vals * s_q.to(torch.float32).unsqueeze(-1) * g_dec).reshape(packed.shape[0], -1)


# --------------------------------------------------------------------------- #
# block-scaled M = 1 GEMV (the consumer of the quantizers' outputs)            #
# --------------------------------------------------------------------------- #
def mxfp8_dequantize(q: torch.Tensor, scale_u8: torch.Tensor) -> torch.Tensor:
    """e4m3 payload * 2^(byte-127) per 32-element block -> fp32.  Follows
    ``dequantize_mxfp8`` of the reference's tests (test/test_mxfp8_tma.py:89-93) and the
    byte semantics of ``combined_e8m0_to_f32`` (cute/mxfp8_tma.py:28-42): 0xFF is NaN."""
    s = torch.exp2(scale_u8.to(torch.float64) - 127.0).to(torch.float32)
    s = torch.where(scale_u8 == 255, torch.full_like(s, float("nan")), s)
    return q.to(torch.float32) * s.repeat_interleave(32, dim=1)


def mxfp8_gemv(q_input, weight, input_scale, weight_scale) -> torch.Tensor:
    """[1, K] x [N, K]^T with raw E8M0 scales -> [1, N] bf16: the dequantised fp32 matmul
    the reference checks its GEMV against (test/test_mxfp8_tma.py:113-140, atol 1.0,
    rtol 0.05).  Floating point: compared with a tolerance, not bit for bit."""
    return (mxfp8_dequantize(q_input, input_scale) @ mxfp8_dequantize(weight, weight_scale).T).to(torch.bfloat16)


def nvfp4_gemv(q_input_packed, weight_packed, input_scale, weight_scale, input_global=None, weight_global=None):
    """Packed e2m1 [1, K/2] x [N, K/2]^T with raw e4m3 block scales and optional fp32
    tensorwise scales -> [1, N] bf16 (test/test_nvfp4_tma.py:186-224, 376-397: decode,
    accumulate, then multiply by the global scales; atol 2.0, rtol 0.05)."""
    one = torch.ones(1)
    a = nvfp4_dequantize(q_input_packed, input_scale, one)
    b = nvfp4_dequantize(weight_packed, weight_scale, one)
    g = (one if input_global is None else input_global.float().cpu()) * (one if weight_global is None else weight_global.float().cpu())
    return ((a @ b.T) * g).to(torch.bfloat16)
