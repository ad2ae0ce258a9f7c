/*
 * tnq - scaled-quantization casts for NVIDIA B200 (sm_100a).
 *
 * C ABI of libtnq.so.  Plain pointers and sizes only; every pointer is a CUDA
 * device pointer unless a comment says "host".  Except for the tnq_exchange_*
 * set-up functions, no function allocates, frees or synchronises; all work is
 * enqueued on `stream`.  Each function returns a tnq_status; on anything but
 * TNQ_OK nothing was launched.
 *
 * Each entry point names the function of drisspg/transformer_nuggets whose
 * device work it replaces (path:line within that project).
 */
#ifndef TNQ_H_
#define TNQ_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct CUstream_st* tnq_stream_t;

typedef enum {
  TNQ_OK = 0,
  TNQ_EINVAL = 1,       /* null pointer, negative size, unknown enum          */
  TNQ_EALIGN = 2,       /* pointer or row pitch not 16-byte aligned            */
  TNQ_ESHAPE = 3,       /* shape not a multiple of the block size              */
  TNQ_EUNSUPPORTED = 4, /* dtype / size combination not built                  */
  TNQ_ECUDA = 5,        /* a CUDA runtime call failed (see tnq_last_cuda_error)*/
  TNQ_ETIMEOUT = 6      /* a bounded device-side wait gave up (status word)    */
} tnq_status;

typedef enum { TNQ_IN_BF16 = 0, TNQ_IN_F32 = 1 } tnq_in_dtype;
typedef enum { TNQ_FP8_E4M3 = 0, TNQ_FP8_E5M2 = 1 } tnq_fp8_dtype;
typedef enum { TNQ_E8M0_CEIL = 0, TNQ_E8M0_FLOOR = 1 } tnq_e8m0_mode;
typedef enum { TNQ_SCALES_RAW = 0, TNQ_SCALES_SWIZZLED = 1 } tnq_scale_layout;
typedef enum { TNQ_SCALE_IS_SCALE = 0, TNQ_SCALE_IS_AMAX = 1 } tnq_scale_source;

/* Caller-owned scratch for the per-tensor reductions: TNQ_WORKSPACE_BYTES
 * bytes, 256-byte aligned, zero-filled ONCE after allocation.  The kernels
 * leave it ready for the next call.  Two calls that share a workspace must be
 * ordered (same stream); use one workspace per concurrent stream.
 * Layout (uint32 words): [0] ticket  [1] amax as fp32 bits  [2] scale (fp32)
 * [3] device status  [5..9] call counter and grid-exchange words of the single-launch cast
 * [16..] per-CTA partial maxima.
 * Device status: every wait inside a kernel is bounded (about one second); a wait
 * that gives up stores TNQ_ETIMEOUT in word [3] (or in the `status` word an entry
 * point takes) and the kernel returns with its outputs incomplete.  Nothing reads
 * the word for the caller: read it after synchronising the stream.  A kernel that
 * left early may not have rewound words [0] and [6..9], so after a TNQ_ETIMEOUT zero the
 * first 64 bytes of the workspace before using it again. */
#define TNQ_WORKSPACE_BYTES 16384
#define TNQ_WS_AMAX_WORD 1
#define TNQ_WS_SCALE_WORD 2
#define TNQ_WS_STATUS_WORD 3

const char* tnq_status_str(int status);
/* cudaError_t of the most recent failing runtime call on this thread (0 if none). */
int tnq_last_cuda_error(void);
/* Library ABI version; bumped when a signature changes. */
int tnq_abi_version(void);

/* Process-wide tuning switches (not part of any result: outputs are identical).
 * TNQ_OPT_CAST_REVERSE (default 1): for tensors between 96 MiB and 1.5 GiB the cast pass of
 * the dynamic and sharded casts walks the tensor from its end, so that the tail the amax pass
 * left in L2 is re-read from L2 instead of HBM (larger tensors: the tail is too small a part). */
#define TNQ_OPT_CAST_REVERSE 1
/* TNQ_OPT_FUSED_SMALL (default 1): tnq_fp8_dynamic_cast uses the single-launch kernel
 * that keeps the whole tensor in shared memory when it fits (up to ~33.5 MB). */
#define TNQ_OPT_FUSED_SMALL 2
/* TNQ_OPT_L2_KEEP_MB (default 64; 0 = off): the amax pass of the dynamic / sharded cast
 * loads the last that-many MiB of the tensor with an L2 evict_last policy and the rest
 * with evict_first, so more of the tail survives until the reversed cast pass.
 * TNQ_OPT_CAST_L2_MODE (default 0): bit 0 = that cast pass loads with evict_first,
 * bit 1 = it stores with evict_first. */
#define TNQ_OPT_L2_KEEP_MB 3
#define TNQ_OPT_CAST_L2_MODE 4
/* TNQ_OPT_CAST_PAIR (default 1): a per-tensor cast of bf16 input that walks the tensor forwards
 * (delayed scale, plain cast) takes 64 contiguous input bytes per thread and step and writes their
 * 32 fp8 bytes with one 256-bit store. */
#define TNQ_OPT_CAST_PAIR 5
/* TNQ_OPT_TILE_EVICT_FIRST (default 0): the NVFP4 quantizer and the one-direction MXFP8 quantizer load
 * their input tiles with an L2 evict-first policy.  (The row + column MXFP8 quantizer and the
 * transposing cast always do: it pays there, here it measured 2 % slower for NVFP4.) */
#define TNQ_OPT_TILE_EVICT_FIRST 6
/* TNQ_OPT_FUSED_LAUNCH (default 1): how the single-launch dynamic cast (tensors up to ~33.5 MB) is
 * launched.  1 = plain launch of at most one CTA per SM, chained like the other kernels (see
 * TNQ_OPT_PDL_CHAIN); if other streams keep SMs busy for longer than the kernel's bounded wait (about a
 * second) the call reports TNQ_ETIMEOUT in the workspace's status word.  0 = cooperative launch: the
 * driver guarantees that all CTAs are resident together whatever else runs, and the chained launch is
 * honoured only inside CUDA graphs (about 2 us more per eager call). */
#define TNQ_OPT_FUSED_LAUNCH 7
/* TNQ_OPT_PDL_CHAIN (default 1): the quantizer kernels are launched with programmatic stream
 * serialization: a kernel's CTAs are placed and set up while the stream's previous kernel drains
 * (they wait for it before they touch memory), which hides the launch latency between
 * back-to-back calls.  0 = plain stream order. */
#define TNQ_OPT_PDL_CHAIN 8
/* TNQ_OPT_EXCHANGE_CAST_WAITS (default 0): 1 = the cast pass of tnq_fp8_sharded_cast waits for the amax
 * launch to complete before it polls for the ranks' amax words.  By default it does not: it needs
 * nothing of that launch but the words it polls, and so does not sit behind the acknowledgement of the
 * amax kernel's stores into the peers' memory (4 GPUs: 210.0-211.3 -> 209.1-210.3 us per step). */
#define TNQ_OPT_EXCHANGE_CAST_WAITS 10
int tnq_set_option(int option, int value);

/* amax = max|x| over n elements, written as fp32 to ws word TNQ_WS_AMAX_WORD and,
 * if non-null, to *amax_out; ws word TNQ_WS_SCALE_WORD receives
 * fp8_max(out_dtype) / max(amax, 1e-12).
 * Replaces pass one of `dynamic_scaled_cast` (fp8/scaled_quant.py:115-119). */
int tnq_fp8_amax(const void* x, int64_t n, int in_dtype, int out_dtype, void* workspace,
                 float* amax_out, tnq_stream_t stream);

/* out[i] = fp8(x[i] * s), s = *scale (TNQ_SCALE_IS_SCALE) or
 * fp8_max / max(*scale, 1e-12) (TNQ_SCALE_IS_AMAX).  saturated != 0 clamps to
 * +-fp8_max first; saturated == 0 overflows to NaN (e4m3) / inf (e5m2) exactly as
 * a non-saturating RNE cast does.  If abs_max_inout is non-null it becomes
 * max(*abs_max_inout, max|x|) - an atomic max on the bit patterns compared as signed integers,
 * so a NaN already stored stays and a negative starting value (-1.0, say) loses; `workspace`
 * must then be given (reserved: the current kernel does not touch it).
 * Replaces `scaled_cast` / `scaled_quant` (fp8/scaled_quant.py:6-32, 35-75) with
 * the overflow semantics of `eager_scaled_quant` (:78-102). */
int tnq_fp8_scaled_cast(const void* x, void* out, int64_t n, int in_dtype, int out_dtype,
                        const float* scale, int scale_source, int saturated,
                        float* abs_max_inout, void* workspace, tnq_stream_t stream);

/* Delayed-scaling state update between two steps, for `tensors` tensors in one launch.
 * amax_history is fp32 [tensors, history_len], newest first; amax and scale are fp32
 * [tensors].  For every t: the history is shifted by one (oldest dropped),
 * history[t][0] = amax[t], scale[t] = fp8_max / max(max over history[t], 1e-12) (a NaN in
 * the history gives a NaN scale), amax[t] = 0.  history_len <= 1024.
 * amax[t] is what `tnq_fp8_scaled_cast` accumulates through abs_max_inout during the step;
 * scale[t] is what the next step passes as its scale.
 * The reference leaves this step to float8_experimental's
 * `sync_float8_amax_and_scale_history` (called from llama/train.py:251-263; the package is
 * not part of the reference tree and is not version-pinned by it); this follows that
 * function's published "max" recipe: roll the history, take its maximum, scale =
 * fp8_max / clamp(amax, 1e-12). */
int tnq_delayed_scale_update(float* amax_history, float* amax, float* scale, int64_t tensors,
                             int history_len, int out_dtype, tnq_stream_t stream);

/* Per-tensor scaled cast of a bf16 [rows, cols] matrix that also writes the transposed
 * copy, from one read: out [rows, cols] = fp8(x * s), out_t [cols, rows] = out^T.  Scale
 * argument, saturation and overflow semantics and the abs_max side output exactly as in
 * tnq_fp8_scaled_cast (abs_max_inout is updated with an atomic max and needs no workspace;
 * it must hold a non-negative value or NaN on entry).  cols % 8 == 0; out_t is written with
 * 32-byte stores when rows % 32 == 0 and out_t is 32-byte aligned, else byte by byte.
 * `status` (nullable) receives TNQ_ETIMEOUT if a bounded wait on a tile load gives up.
 * No counterpart in the reference: its casts (fp8/scaled_quant.py:35-75, 139-169) produce one
 * layout; the transposed operand of the backward GEMM is left to the caller. */
int tnq_fp8_cast_transpose(const void* x, int64_t rows, int64_t cols, int in_dtype, int out_dtype,
                           const float* scale, int scale_kind, int saturated, float* abs_max_inout,
                           void* out, void* out_t, uint32_t* status, tnq_stream_t stream);

/* Dynamic-scale form of tnq_fp8_cast_transpose: amax pass into the workspace, then the saturated cast in
 * both layouts with scale = fp8_max / max(amax, 1e-12).  *scale_out (nullable) receives the scale; status =
 * word 3 of the workspace. */
int tnq_fp8_dynamic_cast_transpose(const void* x, int64_t rows, int64_t cols, int in_dtype, int out_dtype,
                                   void* workspace, void* out, void* out_t, float* scale_out,
                                   tnq_stream_t stream);
/* Tuning switch for the transposing cast, same results either way.  1 (default): every element is
 * converted once, the fp8 bytes are transposed in shared memory and out_t is written by TMA stores
 * (rows % 16 == 0, else variant 0 runs); 0: both outputs converted separately and stored straight to
 * global memory. */
int tnq_cast_transpose_set_store_variant(int variant);

/* RMSNorm fused into the row-wise dynamic e4m3 cast, bf16 [rows, cols] in, one read:
 *   y = bf16((f32(x) * rstd) * f32(weight)),  rstd = 1 / sqrt(mean(f32(x)^2) + eps)   per row
 *   q = e4m3_sat(f32(y) * s),  scale[r] = s = 448 / max(max|y|, 1e-12)                per row
 * weight is bf16 [cols]; y_bf16 (nullable) also returns the normalised rows.  cols % 16 == 0,
 * cols <= 16384; x, weight and y_bf16 32-byte aligned, q 16-byte aligned.
 * The norm is the eager formula the reference profiles for fusion
 * (`handwritten_rms_norm`, examples/rms_norm_fusion_profile.py:26-31); the cast is
 * tnq_fp8_rowwise applied to its result.  The mean of squares is summed in a fixed order
 * (per thread in index order, lanes by butterfly, warps in order): results are run-to-run
 * identical, and equal to a CPU evaluation except where the other summation order moves a
 * value across a bf16 rounding boundary. */
int tnq_rmsnorm_fp8_rowwise(const void* x, const void* weight, float eps, int64_t rows, int64_t cols,
                            void* q_e4m3, float* scale, void* y_bf16, tnq_stream_t stream);

/* The same fused RMSNorm with the MXFP8 row-wise quantizer behind it: q = e4m3(y * 2^-e) per
 * 32-element block along the row, E8M0 byte e + 127 into sf (raw [rows, cols / 32] or swizzled
 * 128x4; a swizzled buffer must be zero-filled by the caller where rows % 128 or
 * (cols / 32) % 4 leave padding), exponent rule as tnq_mxfp8_quantize.  cols % 32 == 0,
 * cols <= 16384.  Norm: examples/rms_norm_fusion_profile.py:26-31; quantizer:
 * `quantize_mxfp8_tensor`, cute/mxfp8_tma.py:497-504. */
int tnq_rmsnorm_mxfp8(const void* x, const void* weight, float eps, int64_t rows, int64_t cols, void* q_e4m3,
                      void* sf, int scale_mode, int scale_layout, void* y_bf16, tnq_stream_t stream);

/* SwiGLU fused into the same two quantizers: y = bf16(f32(bf16(silu(f32(a)))) * f32(b)) with
 * silu(a) = a / (1 + exp(-a)), a and b bf16 [rows, cols] - the eager bf16 evaluation of
 * `F.silu(self.w1(x)) * self.w3(x)` (llama/model.py:228), the operand of the next GEMM - then
 * the row-wise dynamic e4m3 cast / the MXFP8 row-wise quantizer on y.  Shapes, alignment and
 * the optional y_bf16 as for the RMSNorm entry points. */
int tnq_swiglu_fp8_rowwise(const void* a, const void* b, int64_t rows, int64_t cols, void* q_e4m3, float* scale,
                           void* y_bf16, tnq_stream_t stream);
int tnq_swiglu_mxfp8(const void* a, const void* b, int64_t rows, int64_t cols, void* q_e4m3, void* sf,
                     int scale_mode, int scale_layout, void* y_bf16, tnq_stream_t stream);

/* FP8 GEMM with a scale epilogue on the tensor cores (tcgen05, accumulator in tensor memory):
 *   out[m, n] = bf16( (sum_k a[m, k] * b[n, k]) * a_scale[rowwise ? m : 0] * b_scale[rowwise ? n : 0] )
 * a [M, K] and b [N, K] hold fp8 bytes of `fp8_dtype` with K contiguous (row-major activation,
 * "column-major" weight); scales are fp32 in the DEQUANTISATION direction (the reciprocal of what
 * the casts return), one element each or a_scale [M], b_scale [N].  K % 16 == 0; a, b, out
 * 16-byte aligned.  `status` (nullable) receives TNQ_ETIMEOUT if a bounded wait gives up.
 * Replaces `matmul_kernel_persistent` / `matmul_kernel_tma_persistent` and their launchers with
 * `apply_scaling` (fp8/fp8_matmul.py:97-138, 142-288, 290-474). */
int tnq_fp8_gemm(const void* a, const void* b, const float* a_scale, const float* b_scale, int rowwise,
                 int fp8_dtype, int64_t m, int64_t n, int64_t k, void* out_bf16, uint32_t* status,
                 tnq_stream_t stream);

/* MXFP8 GEMM on the block-scaled tensor-core path (tcgen05.mma kind::mxf8f6f4.block_scale):
 *   out[m, n] = bf16( sum over 32-element blocks b of 2^(sa[m,b]-127) * 2^(sb[n,b]-127) * dot(a[m, b], b[n, b]) )
 * a [M, K], b [N, K] e4m3 with K contiguous; sf_a, sf_b the E8M0 scales of [M, K/32] and
 * [N, K/32] in the swizzled 128x4 layout (flat, padded to whole atoms), i.e. exactly what
 * tnq_mxfp8_quantize / tnq_to_blocked write.  K % 128 == 0; all five buffers 16-byte aligned.
 * The reference has no kernel for this shape class: its tests hand the same operands to
 * `F.scaled_mm` with BlockWise1x32 + SWIZZLE_32_4_4 (test/test_mxfp8_tma.py:174-203). */
int tnq_mxfp8_gemm(const void* a, const void* b, const void* sf_a, const void* sf_b, int64_t m, int64_t n,
                   int64_t k, void* out_bf16, uint32_t* status, tnq_stream_t stream);

/* NVFP4 GEMM on the block-scaled tensor-core path (tcgen05.mma kind::mxf4nvf4.block_scale.block16):
 *   out[m, n] = bf16( ga * gb * sum over 16-element blocks b of sa[m,b] * sb[n,b] * dot(a[m, b], b[n, b]) )
 * a_packed [M, K/2], b_packed [N, K/2]: two e2m1 codes per byte, low nibble first, K contiguous;
 * sf_a, sf_b: E4M3 block scales of [M, K/16] and [N, K/16] in the swizzled 128x4 layout; a_global,
 * b_global: fp32 tensor-wide scales in the decode direction (nullable = 1), i.e. exactly what
 * tnq_nvfp4_quantize writes.  K % 256 == 0; buffers 16-byte aligned.
 * The reference has no kernel for this shape class: its tests hand the same operands to
 * `F.scaled_mm` with BlockWise1x16 + TensorWise scaling (test/test_nvfp4_tma.py:511-548). */
int tnq_nvfp4_gemm(const void* a_packed, const void* b_packed, const void* sf_a, const void* sf_b,
                   const float* a_global, const float* b_global, int64_t m, int64_t n, int64_t k, void* out_bf16,
                   uint32_t* status, tnq_stream_t stream);

/* amax -> scale = fp8_max / max(amax, 1e-12) -> saturated cast.  A tensor that fits in
 * the shared memory of all SMs together (and is a multiple of 16 bytes) takes one
 * cooperative launch that reads x from HBM once; larger tensors take two dependent
 * launches (the second re-reads x).  *scale_out (nullable) receives the scale.
 * Replaces `dynamic_scaled_cast` / `dynamic_scaled_quant` (fp8/scaled_quant.py:108-169). */
int tnq_fp8_dynamic_cast(const void* x, void* out, int64_t n, int in_dtype, int out_dtype,
                         void* workspace, float* scale_out, tnq_stream_t stream);

/* Diagnostic twin of tnq_fp8_dynamic_cast (bf16 -> e4m3, single-launch path only, else
 * TNQ_EUNSUPPORTED): the same kernel built with time stamps, for splitting its duration into
 * phases.  stamps: device buffer of 8 uint64 per CTA (256 CTAs at most); words 0..3 are SM
 * clock readings when the CTA is past its wait for the stream's previous kernel / slab loaded and CTA maximum known / grid-wide exchange
 * done / last store issued, words 4..7 the global nanosecond timer at the same four points.
 * *grid_out (host, nullable) receives the number of CTAs.
 * No counterpart in the reference. */
int tnq_fp8_dynamic_cast_profile(const void* x, void* out, int64_t n, void* workspace, float* scale_out,
                                 unsigned long long* stamps, int* grid_out, tnq_stream_t stream);

/* Diagnostic: copies a row-major [rows, cols] bf16 matrix (rows, cols multiples of 128) through the
 * block-scaled quantizers' tile pipeline with the arithmetic taken out: 2-D TMA load of a 128 x 128
 * tile into a ring of `stages` (2..6) shared-memory stages, 2-D TMA store of the same bytes,
 * `ctas_per_sm` (1..4) persistent CTAs per SM.  Its time is the practical floor of a kernel that reads
 * and writes that many bytes tile by tile; bench.py reports the quantizers against it.
 * TNQ_EUNSUPPORTED if the stages do not fit that many CTAs.  No counterpart in the reference. */
int tnq_tile_copy(const void* x, void* y, int64_t rows, int64_t cols, int stages, int ctas_per_sm,
                  uint32_t* status, tnq_stream_t stream);

/* The same cast as tnq_fp8_dynamic_cast for callers that cannot provide (or create)
 * device scratch: plug-ins that receive only tensors and a stream from their host
 * framework, processes whose device memory is entirely owned by a pool reserved at
 * start-up, loops that must never hit cudaMalloc's device-wide synchronisation.
 * This entry point has no counterpart in the reference.
 * It allocates nothing and frees nothing: the reduction scratch is a fixed 4 KiB
 * array inside the library (every GPU that loads libtnq.so holds it until the
 * process ends).  Limits, refused with TNQ_EUNSUPPORTED: n above
 * TNQ_STATIC_MAX_ELEMENTS, and devices on which the amax launch would need more
 * than the 1008 per-CTA slots the array has.
 * The first call on each device looks up the array's device address
 * (cudaGetSymbolAddress); make that first call outside any stream capture.
 * All calls on a device share the one array: the entry point re-zeroes the words
 * that must start at zero on every call, but two calls whose kernels can overlap on
 * the GPU (different streams without an ordering between them) race on it and give
 * wrong results - order them, or use tnq_fp8_dynamic_cast with separate workspaces. */
#define TNQ_STATIC_MAX_ELEMENTS (1LL << 32)
int tnq_fp8_dynamic_cast_static(const void* x, void* out, int64_t n, int in_dtype, int out_dtype,
                                float* scale_out, tnq_stream_t stream);
int64_t tnq_fp8_dynamic_cast_static_max_elements(void);

/* Row-wise dynamic cast of x[rows, cols] (row-major, contiguous).  For each
 * requested output (a null q pointer skips it) q[r, :] = sat_fp8(x[r, :] * s_r),
 * s_r = fp8_max / max(amax_r, 1e-12) written to scale[r] (fp32, [rows]).
 * cols must be a multiple of 16 (bf16) / 8 (fp32).  `status` (nullable): device word
 * that receives TNQ_ETIMEOUT if a bounded wait inside the kernel gives up.
 * The reference has no row-wise cast; the scale shape is the [M, 1] fp32 contract
 * of fp8/fp8_matmul.py:50-61 and the arithmetic is fp8/scaled_quant.py:132-135 per row. */
int tnq_fp8_rowwise(const void* x, int64_t rows, int64_t cols, int in_dtype, void* q_e4m3,
                    float* scale_e4m3, void* q_e5m2, float* scale_e5m2, uint32_t* status,
                    tnq_stream_t stream);
/* Tuning switches, same results either way.  set_tma: 1 = rows staged in shared memory
 * by bulk async copies, 0 (default) = direct 256-bit global loads into registers.
 * set_group: threads that share one row in the direct kernel (32/64/128/256), 0 = automatic. */
int tnq_rowwise_set_tma(int on);
int tnq_rowwise_set_group(int threads_per_row);

/* MXFP8: 32-element blocks, E8M0 scale byte = exponent + 127, e4m3 payload.
 * Row-wise outputs (blocks along cols): q_row[rows, cols], sf_row for the
 * [rows, cols/32] scale matrix.  Column-wise outputs (blocks along rows, i.e. the
 * row-wise quantisation of x^T): q_col[cols, rows], sf_col for [cols, rows/32].
 * Either pair may be null.  scale_layout RAW = row-major scale matrix;
 * SWIZZLED = the 128x4 layout of `to_blocked`, whose buffers hold
 * 512*ceil(H/128)*ceil(W/4) bytes; the kernel writes every byte of them (padding
 * positions become 0).  Requires cols % 32 == 0 for the row-wise pair, rows % 32 == 0
 * for the column-wise pair, bf16 input.  `status` (nullable) is a device word that
 * receives TNQ_ETIMEOUT if a bounded wait inside the kernel gives up.
 * Replaces `quantize_mxfp8_tensor` (cute/mxfp8_tma.py:497-504) and, when
 * swizzled, the following `to_blocked` (mx/to_blocked.py:10-42). */
int tnq_mxfp8_quantize(const void* x, int64_t rows, int64_t cols, int in_dtype, void* q_row,
                       void* sf_row, void* q_col, void* sf_col, int e8m0_mode, int scale_layout,
                       uint32_t* status, tnq_stream_t stream);
/* Tuning switch for the row + column quantizer, same results either way.  variant + 4 * policy:
 * variant 0 = both passes store straight to global memory, 1 (default) = the transposed payload is
 * staged in shared memory and written by TMA stores; policy bit 0 (default on) = input tiles are
 * loaded with an L2 evict-first policy, bit 1 = so are the stored lines. */
int tnq_mxfp8_set_store_variant(int variant);

/* NVFP4: 16-element blocks along cols, e4m3 block scales, two e2m1 codes per byte
 * (low nibble first), fp32 global scale.  *global_amax is max|x| of the whole
 * tensor (device fp32, e.g. ws word TNQ_WS_AMAX_WORD after tnq_fp8_amax).
 * packed[rows, cols/2]; sf for the [rows, cols/16] scale matrix in scale_layout;
 * *global_scale_out (nullable) = max(amax, 1e-12) / 2688, the decode-direction scale.
 * Requires cols % 16 == 0, bf16 input.  `status` as for tnq_mxfp8_quantize.
 * The reference has no NVFP4 quantizer; the outputs follow its storage contract
 * (cute/nvfp4_tma.py:941-964, :527-547). */
int tnq_nvfp4_quantize(const void* x, int64_t rows, int64_t cols, int in_dtype,
                       const float* global_amax, void* packed, void* sf, int scale_layout,
                       float* global_scale_out, uint32_t* status, tnq_stream_t stream);

/* The same with the tensor-wide amax taken first (dynamic global scale): an amax pass into the workspace
 * (word 1), then the quantizer, in one call.  x additionally 32-byte aligned; the status word is word 3 of
 * the workspace. */
int tnq_nvfp4_quantize_dynamic(const void* x, int64_t rows, int64_t cols, int in_dtype, void* workspace,
                               void* packed, void* sf, int scale_layout, float* global_scale_out,
                               tnq_stream_t stream);

/* codes[rows, cols] (one e2m1 code 0..15 per byte) -> packed[rows, cols/2] with
 * byte = code[2i] | code[2i+1] << 4.  Requires cols % 16 == 0.
 * Replaces `pack_nvfp4_codes` (cute/nvfp4_tma.py:941-943). */
int tnq_pack_fp4_codes(const void* codes, int64_t rows, int64_t cols, void* packed,
                       tnq_stream_t stream);

/* One-byte scale matrix in[rows, cols] (row-major) -> 128x4-swizzled flat buffer of
 * 512*ceil(rows/128)*ceil(cols/4) bytes, padding zero-filled by the kernel.
 * Replaces `to_blocked` (mx/to_blocked.py:10-42) and `ToBlocked.kernel`
 * (cute/to_blocked.py:26-73). */
int tnq_to_blocked(const void* in, int64_t rows, int64_t cols, void* out, tnq_stream_t stream);

/* ---- row-sharded per-tensor cast: one process per GPU, amax exchanged by peer stores.
 * The reference has no multi-device cast; its collective precedent is the peer-load
 * all-reduce over symmetric memory of cute/symmetric_memory.py:20-79. ---- */

/* Set-up, once per process group (these allocate / synchronise).  create: a 4 KiB
 * zeroed slot buffer on the current device and its 64-byte CUDA IPC handle (host
 * memory).  open: map a peer process's buffer from its handle (enables peer access).
 * close / destroy: undo open / create.  status: synchronising read of the buffer's
 * status word into *host_status (host memory); non-zero = a bounded wait expired. */
int tnq_exchange_create(void** local_slots, unsigned char ipc_handle[64]);
int tnq_exchange_open(const unsigned char ipc_handle[64], void** peer_slots);
int tnq_exchange_close(void* peer_slots);
int tnq_exchange_destroy(void* local_slots);
int tnq_exchange_status(const void* local_slots, uint32_t* host_status);

/* Cast this rank's n elements with the scale of the whole sharded tensor:
 * local amax -> one 8-byte store (sequence number, amax) into every rank's slot
 * buffer -> the cast kernel waits (bounded, about 1 s) until its OWN buffer holds all
 * world_size words of sequence `seq`, takes their MAX and casts saturated.
 * slot_buffers is a HOST array of world_size device pointers (slot_buffers[rank] is
 * this rank's own buffer, the others come from tnq_exchange_open).  seq must be
 * non-zero, identical on all ranks for the same call and different from the previous
 * two calls' (increment it).  *amax_out (nullable) receives the global amax.
 * world_size <= 16. */
int tnq_fp8_sharded_cast(const void* x, void* out, int64_t n, int in_dtype, int out_dtype,
                         void* workspace, void* const* slot_buffers, int world_size, int rank,
                         uint32_t seq, float* amax_out, tnq_stream_t stream);

/* ---- block-scaled M = 1 GEMV: the consumer directly downstream of the quantizers ---- */

/* y[n] = sum over 32-element blocks b of 2^(x_sf[b]-127) * 2^(w_sf[n,b]-127) *
 * sum_{k in b} x[k] * w[n,k]; x [K] and w [N, K] e4m3, scales E8M0 bytes for the
 * [1, K/32] and [N, K/32] scale matrices in scale_layout (RAW or SWIZZLED), fp32
 * accumulation, y bf16 [N].  A scale byte 0xFF gives NaN.  K % 32 == 0, K <= 65536.
 * Replaces Mxfp8TmaGemv / mxfp8_tma_gemv (cute/blockscaled_tma.py:820-1355,
 * cute/mxfp8_tma.py:392-494). */
int tnq_mxfp8_gemv(const void* x, const void* w, const void* x_sf, const void* w_sf, int64_t n, int64_t k,
                   int scale_layout, void* y_bf16, tnq_stream_t stream);

/* y[n] = gx * gw * sum over 16-element blocks b of x_sf[b] * w_sf[n,b] * sum_{k in b}
 * x[k] * w[n,k]; x [K/2] and w [N, K/2] packed e2m1 (low nibble first), block scales
 * e4m3 bytes, *x_global / *w_global optional fp32 tensorwise scales (null = 1).
 * K % 32 == 0, K <= 65536.  Replaces Nvfp4TmaGemv / nvfp4_tma_gemv
 * (cute/nvfp4_tma.py:833-938, decode convention cute/blockscaled_tma.py:807-818). */
int tnq_nvfp4_gemv(const void* x_packed, const void* w_packed, const void* x_sf, const void* w_sf,
                   const float* x_global, const float* w_global, int64_t n, int64_t k, int scale_layout,
                   void* y_bf16, tnq_stream_t stream);

/* CTA shape of the two GEMVs: 0 (default) and 2 = 512 threads and three ring slots per lane sharing one fp16 copy
 * of x (128 threads where that does not fit: K = 65536), 1 = 128 threads and four slots.  The shapes cut the rows'
 * sums at different steps: results agree to an fp32 rounding of the sums. */
int tnq_gemv_set_shape(int shape);

/* Tensor-wide amax of a row-sharded tensor, for quantizers that take the amax as an
 * input (tnq_nvfp4_quantize): local amax -> 8-byte store into every rank's slot buffer ->
 * a one-CTA kernel waits (bounded) for all ranks' words and writes their MAX to
 * *amax_out on this rank.  Arguments as for tnq_fp8_sharded_cast; shares its sequence
 * numbering (every collective call of a process group uses the next number). */
int tnq_sharded_amax(const void* x, int64_t n, int in_dtype, void* workspace, void* const* slot_buffers,
                     int world_size, int rank, uint32_t seq, float* amax_out, tnq_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* TNQ_H_ */
