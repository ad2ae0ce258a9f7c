"""Benchmark of the scaled-quantization cast path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--workload NAME] [--exchange peer|nccl] [--no-extras]

Headline workload: the row-sharded per-tensor dynamic FP8 cast of a bf16
131072 x 8192 tensor (2 GiB), split by rows over N GPUs (strong scaling: the total
is fixed).  One step = local amax kernel -> amax exchange -> saturated e4m3 cast.
`value` is algorithmic GB/s (5 bytes per element: the shard does not fit in L2, so
the input is read twice and the output written once) summed over all ranks, timed
with CUDA events, max over ranks.  `e2e` is the same metric through the public
Python entry point with pinned HOST input and output buffers, the copies inside the
timed region.  One JSON line on stdout from rank 0.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "quant_cast_hbm_bandwidth"
UNIT = "GB/s"
HEADLINE = "fp8_sharded"
# the arithmetic type of the path: one fp32 product per element between the bf16 load and the fp8 cvt
DTYPE = "f32 (bf16 in, e4m3 out)"


def measured_peak_gbs():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


def measured_traffic(kernel, elements, input_bytes=None):
    """DRAM bytes one launch of `kernel` moves, from the counters of an ncu capture of a smaller launch
    of the same kernel (the full-size launch holds too much memory for a multi-pass capture), scaled by
    the element count: traffic of these streaming kernels is proportional to it.  The capture's figures
    live in a small data file beside its summary.  Tensors above 1.5 GiB are cast with the plain forward
    walk (nothing of the amax pass is found in L2): the capture with cold caches stands for them."""
    path = os.path.join(ROOT, "profiles", "dram_traffic.json")
    try:
        with open(path) as f:
            rec = json.load(f)[kernel]
        which = "the pass behind an amax pass that left the tensor's tail in L2"
        if input_bytes is not None and input_bytes > (1536 << 20) and "cold_cache_capture" in rec:
            rec = dict(rec, **rec["cold_cache_capture"])
            which = "cold caches: the plain forward walk used above 1.5 GiB"
        per_elem = (rec["dram_bytes_read"] + rec["dram_bytes_write"]) / rec["elements"]
        return {"traffic": per_elem * elements, "traffic_bytes_per_element": per_elem,
                "traffic_source": "ncu dram__bytes_read.sum + dram__bytes_write.sum of one 16384 x 8192 launch "
                                  f"(profiles/dram_traffic.json; {which}), scaled by elements"}
    except Exception:
        return {"traffic": None, "traffic_source": "no capture on file"}


# --------------------------------------------------------------------------- clocks
class ClockSampler:
    """nvidia-smi samples of one GPU while the timed kernels run."""

    QUERY = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.rows = []
        self.proc = None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(index)],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append((time.perf_counter(), line.strip()))

    def stop(self, t0, t1):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except Exception:
            self.proc.kill()
        sm, smax, power, reasons = [], [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for t, line in self.rows:
            if t < t0 or t > t1 + 0.1:
                continue
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0]))
                smax.append(float(parts[1]))
                power.append(float(parts[2]))
            except ValueError:
                continue
            for name, v in zip(names, parts[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {
            "sm_mhz": statistics.median(sm) if sm else None,
            "sm_max_mhz": max(smax) if smax else None,
            "power_w_max": max(power) if power else None,
            "samples": len(sm),
            "reasons": sorted(reasons),
        }


# --------------------------------------------------------------------------- CPU reference arm
CHUNK_ROWS = 4096  # the CPU passes walk the tensor in row chunks so that fp32 temporaries stay small


def reference_functions():
    """The reference's own Python functions from the unmodified copy under oracle/_ref, or
    (None, reason) when that copy cannot be imported here."""
    try:
        from oracle import reference

        sq = reference.load("fp8.scaled_quant")
        mx = reference.load("cute.mxfp8_tma")
        tb = reference.load("mx.to_blocked")
        return {"eager_scaled_quant": sq.eager_scaled_quant, "quantize_mxfp8_tensor": mx.quantize_mxfp8_tensor,
                "to_blocked": tb.to_blocked}, None
    except Exception as e:  # noqa: BLE001 - any import problem means "fall back to the port and say why"
        return None, f"{type(e).__name__}: {e}"[:200]


def cpu_reference_pass(name, x, ref):
    """One pass of the reference's CPU (eager PyTorch) path for workload `name` over all of `x`.
    With `ref` (see reference_functions) the reference's own functions run; otherwise, and for the
    two configurations the reference has no function for (row-wise, NVFP4), the oracle port.
    Returns "reference" or "port"."""
    import torch

    import oracle

    if name in ("fp8_sharded", "fp8_tensor"):
        # dynamic per-tensor cast = amax pass, then fp8/scaled_quant.py:78-102 with scale = 448 / amax, saturated
        amax = torch.zeros((), dtype=torch.float32)
        for r0 in range(0, x.shape[0], CHUNK_ROWS):
            amax = torch.maximum(amax, x[r0:r0 + CHUNK_ROWS].abs().max().float())
        scale = (torch.tensor(448.0) / amax.clamp(min=1e-12)).reshape(1)
        am = torch.zeros(1)
        fn = ref["eager_scaled_quant"] if ref else oracle.fp8_scaled_quant
        for r0 in range(0, x.shape[0], CHUNK_ROWS):
            fn(x[r0:r0 + CHUNK_ROWS], scale, am, torch.float8_e4m3fn, True)
        return "reference" if ref else "port"
    if name == "fp8_rowwise":
        for r0 in range(0, x.shape[0], CHUNK_ROWS):
            oracle.fp8_rowwise_quant(x[r0:r0 + CHUNK_ROWS], torch.float8_e4m3fn)
            oracle.fp8_rowwise_quant(x[r0:r0 + CHUNK_ROWS], torch.float8_e5m2)
        return "port"
    if name == "mxfp8":
        quant = ref["quantize_mxfp8_tensor"] if ref else (lambda v: oracle.mxfp8_quantize(v, "ceil"))
        blocked = ref["to_blocked"] if ref else oracle.to_blocked
        _, s = quant(x)
        blocked(s)
        _, s = quant(x.t().contiguous())
        blocked(s)
        return "reference" if ref else "port"
    if name == "nvfp4":
        amax = x.abs().max().float()
        for r0 in range(0, x.shape[0], CHUNK_ROWS):
            _, s, _ = oracle.nvfp4_quantize(x[r0:r0 + CHUNK_ROWS], amax)
            oracle.to_blocked(s.view(torch.uint8))
        return "port"
    raise KeyError(name)


def cpu_baseline(name, steps, warmup, sample_rows, budget_s=None):
    """Time the CPU path on the first `sample_rows` rows of workload `name` with every host thread.
    `budget_s`: shrink the sample (and say so) if warm-up shows that steps + warmup passes would
    take longer than that."""
    import torch

    from transformer_nuggets_b200.workloads import CONFIGS, make_input

    cfg = CONFIGS[name]
    try:
        torch.set_num_threads(len(os.sched_getaffinity(0)))  # torchrun exports OMP_NUM_THREADS=1
    except Exception:
        pass
    ref, why = reference_functions()
    x = make_input(name, "cpu", rows=sample_rows)
    t = time.perf_counter()
    kind = cpu_reference_pass(name, x, ref)
    first = time.perf_counter() - t
    if budget_s is not None and first * (steps + warmup) > budget_s and sample_rows > 1024:
        keep = max(1024, int(sample_rows * budget_s / (first * (steps + warmup))) // 1024 * 1024)
        x = x[:keep].contiguous()
        sample_rows = keep
    for _ in range(max(warmup - 1, 0)):
        cpu_reference_pass(name, x, ref)
    times = []
    for _ in range(steps):
        t = time.perf_counter()
        cpu_reference_pass(name, x, ref)
        times.append(time.perf_counter() - t)
    sec = sum(times) / len(times)
    nbytes = cfg.algo_bytes_per_elem * x.numel()
    what = {"reference": "the reference's own functions (unmodified copy under oracle/_ref)",
            "port": "the oracle port of the reference path" + (f" (reference copy not importable: {why})" if why else
                                                                " (the reference has no function for this configuration)")}[kind]
    return {
        "value": nbytes / sec / 1e9,
        "unit": UNIT,
        "cores": torch.get_num_threads(),
        "kind": kind,
        "sample": f"{sample_rows} of {cfg.rows} rows x {cfg.cols} cols ({name}), {steps} timed passes, "
                  f"{sec * 1e3:.1f} ms per pass, PyTorch CPU eager ops: {what}",
    }, sec


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    if args.workload == "comparators":
        emit(run_comparators())
        return
    from transformer_nuggets_b200.workloads import CONFIGS

    cfg = CONFIGS[args.workload]
    # the whole configuration when the host gets through steps + warmup passes of it in ~2.5 minutes
    base, sec = cpu_baseline(args.workload, args.steps, args.warmup, cfg.rows, budget_s=150.0)
    line = {
        "impl": "reference",
        "metric": METRIC, "value": base["value"], "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": sec * 1e3, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": DTYPE, "data": "synthetic",
        "config": workload_config(args.workload, args.gpus, "none (CPU)"),
        "cpu_baseline": base,
        "e2e": {"value": base["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    emit(line)


def run_comparators():
    """`--impl reference --workload comparators`: the reference's own GPU code on this machine, from the
    unmodified copy under oracle/_ref, timed with CUDA events on cuda:0 like this library's kernels
    (none of this library's kernels run in this process).  Each entry is {"us": ...} or
    {"unavailable": reason}.  The reference's Triton `dynamic_scaled_quant` is never run: its grid-wide
    spin lock is on record as hanging above 2^22 elements (benchmarks/fp8_dynamic_cast.py:43-45 there)."""
    import torch

    out = {"impl": "reference", "what": "reference GPU code on the same machine (oracle/_ref), CUDA events, cuda:0"}
    try:
        from oracle import reference

        sq = reference.load("fp8.scaled_quant")
    except Exception as e:  # noqa: BLE001
        out["unavailable"] = f"{type(e).__name__}: {e}"[:300]
        return out
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)

    def timed(fn, iters=20, warm=3):
        # fn(i): two inputs in turn, as in this library's own workloads (no call finds its own input in L2)
        for i in range(warm):
            fn(i & 1)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(iters):
            fn(i & 1)
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / iters * 1e3

    def attempt(name, build):
        """build() -> (callable taking 0 / 1 to pick one of two inputs, algorithmic bytes, note); guarded: a comparator
        that does not import, compile or launch here is reported, not fatal."""
        try:
            fn, nbytes, note = build()
            us = timed(fn)
            out[name] = {"us": us, "GBps": nbytes / (us * 1e-6) / 1e9, "note": note}
        except Exception as e:  # noqa: BLE001
            out[name] = {"unavailable": f"{type(e).__name__}: {e}"[:300]}
        torch.cuda.empty_cache()

    g = torch.Generator(device=dev).manual_seed(77)

    def eager_dynamic(rows, cols):
        def build():
            xs = [torch.randn(rows, cols, device=dev, generator=g).to(torch.bfloat16) for _ in range(2)]
            am = torch.zeros(1, device=dev)

            def fn(i):  # amax -> scale -> the reference's eager cast, as the dynamic cast's eager twin does
                scale = (448.0 / xs[i].abs().max().float().clamp(min=1e-12)).reshape(1)
                sq.eager_scaled_quant(xs[i], scale, am, torch.float8_e4m3fn, True)

            bpe = 3.0 if rows * cols * 2 <= (64 << 20) else 5.0
            return fn, bpe * rows * cols, f"eager_scaled_quant on CUDA tensors behind an eager amax, bf16 {rows}x{cols}"
        return build

    attempt("eager_dynamic_cast_4096x4096", eager_dynamic(4096, 4096))
    attempt("eager_dynamic_cast_16384x8192", eager_dynamic(16384, 8192))

    def triton_delayed(dtype):
        def build():
            rows, cols = 16384, 8192
            xs = [torch.randn(rows, cols, device=dev, generator=g).to(dtype) for _ in range(2)]
            scale = torch.full((1,), 0.5, device=dev)
            am = torch.zeros(1, device=dev)

            def fn(i):
                sq.scaled_quant(xs[i], scale, am, torch.float8_e4m3fn, True)

            return fn, (xs[0].element_size() + 1.0) * rows * cols, f"Triton scaled_quant (delayed scale + abs_max), {dtype} {rows}x{cols}"
        return build

    attempt("triton_delayed_cast_bf16_16384x8192", triton_delayed(torch.bfloat16))
    attempt("triton_delayed_cast_f32_16384x8192", triton_delayed(torch.float32))

    def eager_mxfp8():
        mx = reference.load("cute.mxfp8_tma")
        tb = reference.load("mx.to_blocked")
        rows, cols = 8192, 7168
        xs = [torch.randn(rows, cols, device=dev, generator=g).to(torch.bfloat16) for _ in range(2)]

        def fn(i):
            _, s = mx.quantize_mxfp8_tensor(xs[i])
            tb.to_blocked(s)
            _, s = mx.quantize_mxfp8_tensor(xs[i].t().contiguous())
            tb.to_blocked(s)

        return fn, 4.0625 * rows * cols, "quantize_mxfp8_tensor + to_blocked on x and x^T (eager CUDA ops), bf16 8192x7168"

    attempt("eager_mxfp8_row_col_8192x7168", eager_mxfp8)

    def gemv_mxfp8():
        mx = reference.load("cute.mxfp8_tma")
        tb = reference.load("mx.to_blocked")
        bs = reference.load("cute.blockscaled_tma")
        n, k = 32768, 8192
        w = [torch.randint(0, 0x7E, (n, k), device=dev, dtype=torch.uint8, generator=g).view(torch.float8_e4m3fn) for _ in range(2)]
        xq = torch.randint(0, 0x7E, (1, k), device=dev, dtype=torch.uint8, generator=g).view(torch.float8_e4m3fn)
        ws = [tb.to_blocked(torch.randint(120, 134, (n, k // 32), device=dev, dtype=torch.uint8, generator=g)) for _ in range(2)]
        xs = tb.to_blocked(torch.randint(120, 134, (1, k // 32), device=dev, dtype=torch.uint8, generator=g))
        y = torch.empty(1, n, dtype=torch.bfloat16, device=dev)

        def fn(i):  # block_n / stages / warps: the reference benchmark's B200 choice for K = 8192
            mx.mxfp8_tma_gemv(xq, w[i], xs, ws[i], block_n=4, num_stages=2, output=y, num_compute_warps=4,
                              grid_scheduler=bs.GridScheduler.STATIC, block_scale_layout=bs.BlockScaleLayout.SWIZZLE_32_4_4)

        return fn, n * k * (1 + 1 / 32) + k * (1 + 1 / 32) + 2 * n, f"mxfp8_tma_gemv (CuTe DSL), N={n} K={k}, swizzled scales"

    attempt("gemv_mxfp8_32768x8192", gemv_mxfp8)

    def gemv_nvfp4():
        nv = reference.load("cute.nvfp4_tma")
        n, k = 32768, 16384
        w = [torch.randint(0, 256, (n, k // 2), device=dev, dtype=torch.uint8, generator=g).view(torch.float4_e2m1fn_x2) for _ in range(2)]
        xq = torch.randint(0, 256, (1, k // 2), device=dev, dtype=torch.uint8, generator=g).view(torch.float4_e2m1fn_x2)
        ws = [nv.swizzle_nvfp4_scales(torch.randint(0x30, 0x40, (n, k // 16), device=dev, dtype=torch.uint8, generator=g).view(torch.float8_e4m3fn))
              for _ in range(2)]
        xs = nv.swizzle_nvfp4_scales(torch.randint(0x30, 0x40, (1, k // 16), device=dev, dtype=torch.uint8, generator=g).view(torch.float8_e4m3fn))
        gs = torch.full((1,), 0.5, device=dev)
        y = torch.empty(1, n, dtype=torch.bfloat16, device=dev)

        def fn(i):  # block_n=None: the reference's own B200 selector
            nv.nvfp4_tma_gemv(xq, w[i], xs, ws[i], input_global_scale=gs, weight_global_scale=gs, output=y)

        return fn, n * k * (0.5 + 1 / 16) + k * (0.5 + 1 / 16) + 2 * n, f"nvfp4_tma_gemv (CuTe DSL), N={n} K={k}, global scales"

    attempt("gemv_nvfp4_32768x16384", gemv_nvfp4)
    return out


def apply_env_options():
    """TNQ_SET_OPTIONS="option=value,..." -> tnq_set_option, for A/B runs of the tuning switches (include/tnq.h)."""
    from transformer_nuggets_b200 import _lib

    for item in filter(None, os.environ.get("TNQ_SET_OPTIONS", "").split(",")):
        opt, val = item.split("=")
        _lib.call("tnq_set_option", int(opt), int(val))


def workload_config(name, n_gpus, exchange, rows=None):
    import dataclasses

    from transformer_nuggets_b200.workloads import CONFIGS

    cfg = CONFIGS[name]
    if rows:
        cfg = dataclasses.replace(cfg, rows=rows)
    return {
        "workload": f"{name}: {cfg.description}; bf16 {cfg.rows}x{cfg.cols}",
        "rows": cfg.rows, "cols": cfg.cols, "shards": n_gpus, "exchange": exchange,
        "algorithmic_bytes_per_element": cfg.algo_bytes_per_elem,
        "l2": "inputs larger than L2 (each rank's shard is >= 256 MiB against 126 MB of L2), two input tensors cast in turn",
    }


def bind_near_gpu(index):
    """Restrict this process to the CPUs the driver reports as local to GPU `index`
    (intersected with the CPUs it may use), so that pinned host buffers allocated
    afterwards land on that NUMA node.  Returns a short description."""
    try:
        import pynvml

        pynvml.nvmlInit()
        h = pynvml.nvmlDeviceGetHandleByIndex(index)
        n_cpu = os.cpu_count() or 1
        words = pynvml.nvmlDeviceGetCpuAffinity(h, (n_cpu + 63) // 64)
        near = {64 * i + b for i, w in enumerate(words) for b in range(64) if (w >> b) & 1}
        allowed = os.sched_getaffinity(0)
        use = near & allowed
        if not use:
            return f"GPU-local CPUs not in this process's cpuset ({len(allowed)} CPUs allowed); unchanged"
        os.sched_setaffinity(0, use)
        return f"bound to {len(use)} GPU-local CPUs"
    except Exception as e:  # NVML missing or affinity not permitted
        return f"unchanged ({type(e).__name__})"


def headline_parity(x, got, amax_dev, rank, world, dist, dev):
    """Every rank checks 2048 of its rows (a seeded contiguous block) of the sharded cast against
    oracle.fp8_scaled_quant fed the scale of the whole tensor, and the exchanged amax against a plain
    torch reduction of its own rows MAX-reduced over the ranks.  Returns the record for the JSON line
    (ok = every rank agreed on every byte)."""
    import torch

    import oracle

    local = x.abs().max().float().reshape(1)
    if dist is not None:
        dist.all_reduce(local, op=dist.ReduceOp.MAX)
    amax_ok = bool(torch.equal(local, amax_dev.reshape(1)))
    scale = (torch.tensor([448.0]) / local.cpu().clamp(min=1e-12)).reshape(1)
    n = min(2048, x.shape[0])
    g = torch.Generator().manual_seed(4242 + rank)
    r0 = int(torch.randint(0, x.shape[0] - n + 1, (1,), generator=g))
    want = oracle.fp8_scaled_quant(x[r0:r0 + n].cpu(), scale, torch.zeros(1), torch.float8_e4m3fn, True)
    rows_ok = bool(torch.equal(got[r0:r0 + n].view(torch.uint8).cpu(), want.view(torch.uint8)))
    flag = torch.tensor([1 if (amax_ok and rows_ok) else 0], dtype=torch.int32, device=dev)
    if dist is not None:
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    return {"ok": bool(flag.item()), "rows_checked": n * world, "ranks": world,
            "against": "oracle.fp8_scaled_quant, 2048 seeded rows per rank, scale from the tensor-wide amax"}


# --------------------------------------------------------------------------- GPU arm
def run_ours(args):
    import torch
    import torch.distributed as dist

    import transformer_nuggets_b200 as tn
    from transformer_nuggets_b200 import _lib
    from transformer_nuggets_b200.dist.sharded import plan_row_shards, sharded_dynamic_scaled_quant
    from transformer_nuggets_b200.workloads import CONFIGS, make_input

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if args.workload != HEADLINE:  # a single-GPU configuration on its own (profiler captures, sweeps)
        if world != 1:
            raise SystemExit("the single-GPU configurations run with --gpus 1")
        peak, _ = measured_peak_gbs()
        r = other_workloads(dev, peak, only=args.workload, iters=args.steps, warm=args.warmup)
        emit({"workload_run": args.workload, "results": r})
        return
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(v):
        if world == 1:
            return v
        t = torch.tensor([v], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    apply_env_options()
    cfg = CONFIGS[HEADLINE]
    if args.rows:  # smaller same-shape case for profiler captures
        import dataclasses

        cfg = dataclasses.replace(cfg, rows=args.rows)
    s, e = plan_row_shards(cfg.rows, world)[rank]
    x = make_input(HEADLINE, dev, rows=e - s, row_offset=rank)
    out = torch.empty_like(x, dtype=torch.float8_e4m3fn)
    # Consecutive steps cast two different tensors in turn (the shard and its rows in reverse order: same amax).  Cast
    # over and over, ONE tensor flatters the step: the cast pass walks it from the end, so it finishes on the rows
    # the next step's amax pass starts with and leaves them in L2 (measured: 820.6 vs 827.0-828.5 us at 131072 rows,
    # 102.0 vs 106.5 us at 16384 rows).
    xs = [x.flip(0).contiguous(), x]
    n_local = x.numel()
    total_elems = cfg.rows * cfg.cols
    exchange = None
    exchange_name = "single GPU"
    if world > 1:
        if args.exchange == "peer":
            from transformer_nuggets_b200.dist.exchange import PeerAmaxExchange

            exchange = PeerAmaxExchange(None)
            exchange_name = "NVLink peer stores (8-byte word per rank), fused into the amax and cast kernels"
        else:
            exchange_name = "NCCL all-reduce(MAX) of one fp32"

    step_no = [0]

    def step():
        step_no[0] += 1
        sharded_dynamic_scaled_quant(xs[step_no[0] & 1], None, exchange=exchange, out=out)

    sampler = ClockSampler(local_rank) if rank == 0 else None
    t_load0 = time.perf_counter()
    for _ in range(args.warmup):
        step()
    barrier()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    for _ in range(args.steps):
        step()
    ev1.record()
    barrier()
    ms_total = max_over_ranks(ev0.elapsed_time(ev1))
    ms_step = ms_total / args.steps
    value = cfg.algo_bytes_per_elem * total_elems / (ms_step * 1e-3) / 1e9
    launches = 2 * args.steps
    if exchange is not None and exchange.status() != 0:
        raise SystemExit("a bounded wait of the amax exchange expired during the timed steps")

    if args.profile:  # profiler capture run: the timed steps only
        if rank == 0:
            if sampler:
                sampler.stop(t_load0, time.perf_counter())
            emit({"profile_run": True, "rows": cfg.rows, "ms_per_step": ms_step, "value": value})
        if exchange is not None:
            exchange.close()
        if world > 1:
            dist.destroy_process_group()
        return

    # ---- per-kernel durations of the same two kernels (CUDA events around each launch) ----
    ws = _lib.workspace(dev)
    stream = _lib.stream_ptr(dev)
    amax = torch.empty(1, dtype=torch.float32, device=dev)
    k_iters = max(args.steps, 20)
    evs = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(k_iters)]
    t_k0 = time.perf_counter()
    reps = 0
    while True:
        for it in range(k_iters):
            xi = xs[(it + k_iters) & 1]  # in turn, the last launch on x itself (its output is checked below)
            evs[it][0].record()
            _lib.call("tnq_fp8_amax", xi.data_ptr(), n_local, _lib.IN_BF16, _lib.FP8_E4M3, ws.data_ptr(), amax.data_ptr(), stream)
            evs[it][1].record()
            _lib.call("tnq_fp8_scaled_cast", xi.data_ptr(), out.data_ptr(), n_local, _lib.IN_BF16, _lib.FP8_E4M3,
                      amax.data_ptr(), _lib.SCALE_IS_AMAX, 1, 0, 0, stream)
            evs[it][2].record()
        torch.cuda.synchronize()
        reps += 1
        if time.perf_counter() - t_k0 > 1.2 or reps >= 50:
            break
    t_load1 = time.perf_counter()
    clocks = sampler.stop(t_load0, t_load1) if sampler else None
    amax_ms = statistics.mean(ev[0].elapsed_time(ev[1]) for ev in evs)
    cast_ms = statistics.mean(ev[1].elapsed_time(ev[2]) for ev in evs)
    peak, peak_kind = measured_peak_gbs()
    cast_bytes = 3.0 * n_local
    amax_bytes = 2.0 * n_local
    cast_gbs = cast_bytes / (cast_ms * 1e-3) / 1e9
    amax_gbs = amax_bytes / (amax_ms * 1e-3) / 1e9
    roofline = {
        "bound": "hbm", "kernel": "k_cast (bf16 -> e4m3 saturated cast, 2 B read + 1 B written per element)",
        "achieved": cast_gbs, "peak": peak, "peak_kind": f"{peak_kind} copy bandwidth", "unit": "GB/s", "frac": cast_gbs / peak,
        "traffic": None, "launch_ms": cast_ms, "algorithmic_bytes_per_launch": cast_bytes,
        "other_kernels": {"k_amax": {"achieved": amax_gbs, "frac": amax_gbs / peak, "launch_ms": amax_ms,
                                     "algorithmic_bytes_per_launch": amax_bytes}},
    }
    roofline.update(measured_traffic("k_cast", n_local, n_local * x.element_size()))

    # ---- end to end: pinned host buffers in, pinned host buffers out, every step ----
    from transformer_nuggets_b200.dist.host_pipeline import HostCastPipeline

    ref_out, amax_of_run = sharded_dynamic_scaled_quant(x, None, exchange=exchange)  # device-resident result to compare with
    amax_of_run = amax_of_run.clone()
    all_cpus = os.sched_getaffinity(0)
    numa = bind_near_gpu(local_rank)  # pinned buffers are first touched from the GPU's own NUMA node
    host_in = torch.empty(x.shape, dtype=x.dtype, pin_memory=True)
    host_in.copy_(x)
    host_out = [torch.empty(out.shape, dtype=torch.uint8, pin_memory=True) for _ in range(2)]
    for h in host_out:
        h.zero_()
    os.sched_setaffinity(0, all_cpus)  # the CPU baseline leg later uses every CPU again
    pipe = HostCastPipeline(x.shape, x.dtype, torch.float8_e4m3fn, dev, exchange=exchange)
    for i in range(max(min(args.warmup, 3), 2)):
        pipe.submit(host_in, host_out[i % 2])
    pipe.synchronize()
    barrier()
    ev0.record()
    pipe.s_h2d.wait_event(ev0)
    for i in range(args.steps):
        pipe.submit(host_in, host_out[i % 2])
    torch.cuda.current_stream().wait_stream(pipe.s_d2h)
    ev1.record()
    pipe.synchronize()
    barrier()
    e2e_ms = max_over_ranks(ev0.elapsed_time(ev1)) / args.steps
    ok_e2e = torch.equal(host_out[(args.steps - 1) % 2].view(torch.uint8), ref_out.view(torch.uint8).cpu())

    # ---- the same copies alone: what the host link gives this many ranks at once (no kernels) ----
    for i in range(2):
        pipe.copy_only(host_in, host_out[i % 2])
    pipe.synchronize()
    barrier()
    ev0.record()
    pipe.s_h2d.wait_event(ev0)
    for i in range(args.steps):
        pipe.copy_only(host_in, host_out[i % 2])
    torch.cuda.current_stream().wait_stream(pipe.s_d2h)
    torch.cuda.current_stream().wait_stream(pipe.s_h2d)
    ev1.record()
    pipe.synchronize()
    barrier()
    copy_ms = max_over_ranks(ev0.elapsed_time(ev1)) / args.steps

    # ---- parity of this rank's rows against the CPU oracle fed the tensor-wide amax ----
    parity = headline_parity(x, ref_out, amax_of_run, rank, world, dist if world > 1 else None, dev)
    e2e = {
        "value": cfg.algo_bytes_per_elem * total_elems / (e2e_ms * 1e-3) / 1e9, "unit": UNIT,
        "ms_per_step": e2e_ms, "h2d_bytes_per_step": x.numel() * x.element_size(), "d2h_bytes_per_step": out.numel(),
        "api": "HostCastPipeline.submit(pinned host rows -> pinned host fp8), copies of consecutive steps overlapped",
        "result_matches_device_path": bool(ok_e2e), "host_numa_binding": numa,
        "copy_only_ms_per_step": copy_ms,
        "copy_ceiling_gbs": cfg.algo_bytes_per_elem * total_elems / (copy_ms * 1e-3) / 1e9,
        "frac_of_copy_ceiling": copy_ms / e2e_ms,
        "h2d_gbs_per_gpu_in_copy_only": x.numel() * x.element_size() / (copy_ms * 1e-3) / 1e9,
    }
    extras = None
    if world == 1 and not args.no_extras:
        extras = other_workloads(dev, peak)

    base = None
    if rank == 0 and world == 1 and not args.no_cpu:
        base, _ = cpu_baseline(HEADLINE, 3, 1, cfg.rows // 8)
        if extras is not None:  # the CPU path beside every other configuration, on a bounded row sample
            for name, rows in (("fp8_tensor", 4096), ("fp8_rowwise", 2048), ("mxfp8", 1024), ("nvfp4", 512)):
                if name in extras:
                    b, _ = cpu_baseline(name, 2, 1, rows)
                    extras[name]["cpu"] = {"GBps": b["value"], "cores": b["cores"], "kind": b["kind"], "sample": b["sample"]}

    comparators = None
    if rank == 0 and world == 1 and not args.no_comparators:
        comparators = run_comparators_in_child()

    if exchange is not None:
        exchange.close()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    if not parity["ok"]:
        if rank == 0:
            print(f"PARITY FAILURE: {parity}", file=sys.stderr)
        raise SystemExit(3)
    if rank != 0:
        return

    def compact(r):  # one configuration -> the four numbers of the grading contract
        c = {"us": round(r["us"], 2), "GBps": round(r["GBps"], 1), "frac": round(r["frac_of_measured_peak"], 4),
             "frac_nominal": round(r["frac_of_nominal_8000"], 4)}
        if "parity" in r:
            c["parity"] = r["parity"]
        if "cpu" in r:
            c["cpu_GBps"] = round(r["cpu"]["GBps"], 2)
            c["cpu_kind"] = r["cpu"]["kind"]
        return c

    configs = {}
    if extras is not None:
        for key, name in (("cfg1_fp8_tensor_4096x4096", "fp8_tensor"), ("cfg2_fp8_rowwise_16384x8192", "fp8_rowwise"),
                          ("cfg3_mxfp8_row_col_8192x7168", "mxfp8"), ("cfg4_nvfp4_16384x16384", "nvfp4")):
            if name in extras:
                configs[key] = compact(extras[name])
    configs[f"cfg5_fp8_sharded_131072x8192_x{world}gpu"] = {
        "us": round(ms_step * 1e3, 2), "GBps": round(value, 1), "frac": round(value / world / peak, 4),
        "frac_nominal": round(value / world / 8000.0, 4), "parity": parity["ok"]}
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": DTYPE, "data": "synthetic", "config": workload_config(HEADLINE, world, exchange_name, cfg.rows),
        "configs": configs, "parity": parity,
        "roofline": roofline, "e2e": e2e, "gpu_launches": launches, "clocks": clocks,
    }
    if base is not None:
        line["cpu_baseline"] = base
    if extras is not None:
        line["next_rows"] = {k: ({kk: (round(vv, 4) if isinstance(vv, float) else vv) for kk, vv in v.items()
                                  if kk not in ("note", "per_launch_us", "cpu", "parity_note")} if isinstance(v, dict) else v)
                             for k, v in extras.items() if k not in ("fp8_tensor", "fp8_rowwise", "mxfp8", "nvfp4")}
    if comparators is not None:
        line["reference_same_box"] = comparators
    line["frac_of_measured_peak_by_config"] = {k.split("_")[0]: v["frac"] for k, v in configs.items()}
    if args.details:
        with open(args.details, "w") as f:
            json.dump({"line": line, "single_gpu_workloads": extras}, f, indent=1)
    emit(line)


def run_comparators_in_child():
    """The reference's GPU code, timed in a process of its own (`--impl reference --workload
    comparators`): this process never imports it, and a comparator that misbehaves cannot take the
    benchmark down with it.  Returns the child's record, or why there is none."""
    try:
        r = subprocess.run([sys.executable, os.path.abspath(__file__), "--impl", "reference", "--workload", "comparators"],
                           capture_output=True, text=True, timeout=420,
                           env={k: v for k, v in os.environ.items() if k not in ("RANK", "WORLD_SIZE", "LOCAL_RANK")})
        for ln in reversed(r.stdout.strip().splitlines()):
            if ln.startswith("{"):
                rec = json.loads(ln)
                rec.pop("impl", None)
                for v in rec.values():
                    if isinstance(v, dict):
                        v.pop("note", None)
                        if "unavailable" in v:
                            v["unavailable"] = " ".join(v["unavailable"].encode("ascii", "ignore").decode().split())[:160]
                        for k in ("us", "GBps"):
                            if k in v:
                                v[k] = round(v[k], 2)
                return rec
        return {"unavailable": f"no record from the child process (exit {r.returncode}): {r.stderr.strip()[-200:]}"}
    except Exception as e:  # noqa: BLE001
        return {"unavailable": f"{type(e).__name__}: {e}"[:200]}


def other_workloads(dev, peak, only=None, iters=None, warm=None):
    """Single-GPU configurations, timed the same way (CUDA events, cold L2 by rotating
    buffer sets larger than L2 together).  Reported beside the headline.  `only`
    restricts the run to one configuration (profiler captures)."""
    import torch

    import transformer_nuggets_b200 as tn
    from transformer_nuggets_b200 import _lib
    from transformer_nuggets_b200.workloads import CONFIGS, make_input

    res = {}

    def timed(fn, sets, n_it=30, n_warm=5):
        n_it = iters if iters is not None else n_it
        n_warm = warm if warm is not None else n_warm
        ms = _timed(fn, sets, n_it, n_warm)
        timed.last_distribution = _per_launch(fn, sets, 100) if iters is None else None
        return ms

    def _per_launch(fn, sets, n):
        """One CUDA-event pair around every launch (includes the idle-queue launch latency,
        a few microseconds): median, 5th and 95th percentile in microseconds."""
        ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(n)]
        for i, (a, b) in enumerate(ev):
            a.record()
            fn(sets[i % len(sets)])
            b.record()
        torch.cuda.synchronize()
        t = sorted(a.elapsed_time(b) * 1e3 for a, b in ev)
        return {"median": t[n // 2], "p05": t[n // 20], "p95": t[(19 * n) // 20], "launches": n}

    def _timed(fn, sets, iters, warm):
        for i in range(warm):
            fn(sets[i % len(sets)])
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(iters):
            fn(sets[i % len(sets)])
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / iters

    ws = _lib.workspace(dev)
    stream = _lib.stream_ptr(dev)
    # A/B switches of the row + column kernels (same bytes either way; see include/tnq.h)
    if os.environ.get("TNQ_MX_STORE_VARIANT"):
        _lib.call("tnq_mxfp8_set_store_variant", int(os.environ["TNQ_MX_STORE_VARIANT"]))
    if os.environ.get("TNQ_CT_STORE_VARIANT"):
        _lib.call("tnq_cast_transpose_set_store_variant", int(os.environ["TNQ_CT_STORE_VARIANT"]))
    apply_env_options()

    def report(name, ms, note, bytes_per_elem=None):
        cfg = CONFIGS[name]
        bpe = cfg.algo_bytes_per_elem if bytes_per_elem is None else bytes_per_elem
        gbs = bpe * cfg.rows * cfg.cols / (ms * 1e-3) / 1e9
        r = {"us": ms * 1e3, "GBps": gbs, "frac_of_measured_peak": gbs / peak, "frac_of_nominal_8000": gbs / 8000.0,
             "algorithmic_bytes_per_element": bpe, "note": note}
        if getattr(timed, "last_distribution", None):
            r["per_launch_us"] = timed.last_distribution
        return r

    def want(name):
        return only is None or only == name

    if want("fp8_tensor"):
        _bench_fp8_tensor(dev, res, timed, report, ws, stream)
    if want("fp8_rowwise"):
        _bench_rowwise(dev, res, timed, report, stream)
    if want("mxfp8"):
        _bench_mxfp8(dev, res, timed, report, ws, stream)
    if want("nvfp4"):
        _bench_nvfp4(dev, res, timed, report, ws, stream)
    if want("fp8_transpose"):
        _bench_transpose(dev, res, timed, peak, ws, stream)
    if want("rmsnorm_fp8"):
        _bench_rmsnorm(dev, res, timed, peak, stream)
    if want("fp8_delayed"):
        _bench_delayed(dev, res, timed, peak, ws, stream)
    if only == "mxfp8_gemm":
        _bench_mxfp8_gemm(dev, res, timed, stream)
    if only == "nvfp4_gemm":
        _bench_nvfp4_gemm(dev, res, timed, stream)
    if want("gemv") or only in ("gemv_mxfp8", "gemv_nvfp4"):
        _bench_gemv(dev, res, timed, peak, stream, None if only in (None, "gemv") else only)
    if want("fp8_gemm"):  # tensor-core row, last: a dense GEMM loop runs the board into its power cap, and whatever
        _bench_fp8_gemm(dev, res, timed, stream)  # is timed right behind it inherits the lowered clocks
    st = int(ws[_lib.WS_STATUS_WORD].item())
    if st != 0:
        raise SystemExit(f"device status word {st}: a bounded wait expired in a tile kernel")
    return res


def _in_turn(x):
    """Two inputs for a timed loop: the tensor and its rows in reverse order, cast alternately, so that no call
    finds parts of its own input left in L2 by the call before it (the last call of every loop is on x itself)."""
    return [x.flip(0).contiguous(), x]


def _bench_transpose(dev, res, timed, peak, ws, stream):
    """Per-tensor e4m3 cast that also writes the transposed copy (bf16 16384 x 8192, 256 MiB in):
    delayed scale with the abs_max side output (2 + 1 + 1 B/elem) and dynamic scale (amax pass
    first: 2 more B/elem, the tensor is larger than L2)."""
    import torch

    from transformer_nuggets_b200 import _lib
    from transformer_nuggets_b200.workloads import make_input

    x = make_input("fp8_rowwise", dev)
    rows, cols = x.shape
    q = torch.empty_like(x, dtype=torch.float8_e4m3fn)
    q_t = torch.empty(cols, rows, dtype=torch.float8_e4m3fn, device=dev)
    scale = torch.full((1,), 0.5, dtype=torch.float32, device=dev)
    am = torch.zeros(1, dtype=torch.float32, device=dev)
    status = ws.data_ptr() + 4 * _lib.WS_STATUS_WORD

    def report(ms, bpe, note):
        gbs = bpe * rows * cols / (ms * 1e-3) / 1e9
        r = {"us": ms * 1e3, "GBps": gbs, "frac_of_measured_peak": gbs / peak, "frac_of_nominal_8000": gbs / 8000.0,
             "algorithmic_bytes_per_element": bpe, "note": note}
        if getattr(timed, "last_distribution", None):
            r["per_launch_us"] = timed.last_distribution
        return r

    def delayed(xin):
        _lib.call("tnq_fp8_cast_transpose", xin.data_ptr(), rows, cols, _lib.IN_BF16, _lib.FP8_E4M3, scale.data_ptr(),
                  _lib.SCALE_IS_SCALE, 1, am.data_ptr(), q.data_ptr(), q_t.data_ptr(), status, stream)

    x_other = _in_turn(x)[0]

    def dynamic(xin):
        _lib.call("tnq_fp8_dynamic_cast_transpose", xin.data_ptr(), rows, cols, _lib.IN_BF16, _lib.FP8_E4M3, ws.data_ptr(),
                  q.data_ptr(), q_t.data_ptr(), 0, stream)

    res["fp8_cast_transpose"] = report(timed(delayed, [x_other, x]), 4.0,
                                       f"{rows}x{cols}, delayed scale + abs_max side output, both layouts from one read")
    res["fp8_dynamic_cast_transpose"] = report(timed(dynamic, [x_other, x]), 6.0,
                                               f"{rows}x{cols}, amax pass + transposing cast, two 256 MiB inputs in turn")
    del x, x_other, q, q_t


def _bench_delayed(dev, res, timed, peak, ws, stream):
    """Delayed-scale saturated e4m3 cast with the abs_max side output (`scaled_quant`), 16384 x 8192, bf16 and
    fp32 input: one read, one write (3 and 5 bytes per element).  The reference's Triton kernel for the same
    call is timed on the same machine by the comparator run."""
    import torch

    from transformer_nuggets_b200 import _lib
    from transformer_nuggets_b200.workloads import make_input

    xb = make_input("fp8_rowwise", dev)
    rows, cols = xb.shape
    q = torch.empty_like(xb, dtype=torch.float8_e4m3fn)
    scale = torch.full((1,), 0.5, dtype=torch.float32, device=dev)
    am = torch.zeros(1, dtype=torch.float32, device=dev)
    for name, x, code, bpe in (("fp8_delayed_cast_bf16", xb, _lib.IN_BF16, 3.0), ("fp8_delayed_cast_f32", None, _lib.IN_F32, 5.0)):
        if x is None:
            x = xb.float()

        def f(xin):
            _lib.call("tnq_fp8_scaled_cast", xin.data_ptr(), q.data_ptr(), xin.numel(), code, _lib.FP8_E4M3, scale.data_ptr(),
                      _lib.SCALE_IS_SCALE, 1, am.data_ptr(), ws.data_ptr(), stream)

        ms = timed(f, _in_turn(x))
        gbs = bpe * rows * cols / (ms * 1e-3) / 1e9
        res[name] = {"us": ms * 1e3, "GBps": gbs, "frac_of_measured_peak": gbs / peak, "frac_of_nominal_8000": gbs / 8000.0,
                     "algorithmic_bytes_per_element": bpe, "note": f"{rows}x{cols}, delayed scale, saturated, abs_max side output"}
    del xb, q

    # the state update between two steps (amax history -> next scale) for a model's worth of tensors in one launch
    tensors, hist = 1024, 16
    history = torch.rand(tensors, hist, dtype=torch.float32, device=dev)
    amaxes = torch.rand(tensors, dtype=torch.float32, device=dev)
    scales = torch.ones(tensors, dtype=torch.float32, device=dev)

    def upd(_):
        _lib.call("tnq_delayed_scale_update", history.data_ptr(), amaxes.data_ptr(), scales.data_ptr(), tensors, hist,
                  _lib.FP8_E4M3, stream)

    ms = timed(upd, [None])
    nbytes = 4.0 * tensors * (2 * hist + 2)  # history read and written back, amax read and cleared, scale written
    res["delayed_scale_update"] = {"us": ms * 1e3, "GBps": nbytes / (ms * 1e-3) / 1e9, "tensors": tensors, "history_len": hist,
                                   "note": "one launch for all tensors; launch-latency bound (146 KB moved)"}


def _bench_rmsnorm(dev, res, timed, peak, stream):
    """RMSNorm fused into the row-wise e4m3 cast (bf16 16384 x 8192): 2 B read + 1 B written per
    element; the unfused sequence (norm writes bf16, cast reads it back) moves 7 B per element."""
    import torch

    from transformer_nuggets_b200 import _lib
    from transformer_nuggets_b200.workloads import make_input

    x = make_input("fp8_rowwise", dev)
    rows, cols = x.shape
    w = torch.ones(cols, dtype=torch.bfloat16, device=dev)
    q = torch.empty_like(x, dtype=torch.float8_e4m3fn)
    scale = torch.empty(rows, 1, dtype=torch.float32, device=dev)

    xs = _in_turn(x)

    def fused(xin):
        _lib.call("tnq_rmsnorm_fp8_rowwise", xin.data_ptr(), w.data_ptr(), 1e-6, rows, cols, q.data_ptr(), scale.data_ptr(), 0,
                  stream)

    ms = timed(fused, xs)
    gbs = 3.0 * rows * cols / (ms * 1e-3) / 1e9
    r = {"us": ms * 1e3, "GBps": gbs, "frac_of_measured_peak": gbs / peak, "frac_of_nominal_8000": gbs / 8000.0,
         "algorithmic_bytes_per_element": 3.0, "note": f"{rows}x{cols}, norm + per-row scale + cast in one pass, input 256 MiB > L2"}
    if getattr(timed, "last_distribution", None):
        r["per_launch_us"] = timed.last_distribution
    res["rmsnorm_fp8_rowwise"] = r

    sf = torch.empty(512 * (rows // 128) * (cols // 128), dtype=torch.uint8, device=dev)  # swizzled, no padding here

    def fused_mx(xin):
        _lib.call("tnq_rmsnorm_mxfp8", xin.data_ptr(), w.data_ptr(), 1e-6, rows, cols, q.data_ptr(), sf.data_ptr(),
                  _lib.E8M0_CEIL, _lib.SCALES_SWIZZLED, 0, stream)

    ms = timed(fused_mx, xs)
    bpe = 3.0 + 1.0 / 32
    gbs = bpe * rows * cols / (ms * 1e-3) / 1e9
    r = {"us": ms * 1e3, "GBps": gbs, "frac_of_measured_peak": gbs / peak, "frac_of_nominal_8000": gbs / 8000.0,
         "algorithmic_bytes_per_element": bpe, "note": f"{rows}x{cols}, norm + MXFP8 row-wise quantize, swizzled scales"}
    if getattr(timed, "last_distribution", None):
        r["per_launch_us"] = timed.last_distribution
    res["rmsnorm_mxfp8"] = r

    # SwiGLU producer: two bf16 inputs (4 B read), one fp8 output (1 B written) per element
    b = make_input("fp8_rowwise", dev)
    pairs = list(zip(xs, _in_turn(b)))

    def fused_swiglu(ab):
        _lib.call("tnq_swiglu_fp8_rowwise", ab[0].data_ptr(), ab[1].data_ptr(), rows, cols, q.data_ptr(), scale.data_ptr(), 0, stream)

    ms = timed(fused_swiglu, pairs)
    gbs = 5.0 * rows * cols / (ms * 1e-3) / 1e9
    r = {"us": ms * 1e3, "GBps": gbs, "frac_of_measured_peak": gbs / peak, "frac_of_nominal_8000": gbs / 8000.0,
         "algorithmic_bytes_per_element": 5.0,
         "note": f"{rows}x{cols}, silu(a) * b + per-row scale + cast in one pass (unfused: 11 B/elem)"}
    if getattr(timed, "last_distribution", None):
        r["per_launch_us"] = timed.last_distribution
    res["swiglu_fp8_rowwise"] = r
    del x, xs, pairs, q, b


def _bench_fp8_gemm(dev, res, timed, stream):
    """e4m3 GEMM with per-tensor scale epilogue, M = N = K = 8192 (tensor-core bound: 2*M*N*K flops),
    with the library GEMM (torch._scaled_mm, cuBLASLt) timed beside it on the same operands."""
    import json

    import torch

    from transformer_nuggets_b200 import _lib

    m = n = k = int(os.environ.get("TNQ_BENCH_GEMM_SIZE", "8192"))  # a smaller cube for profiler captures
    g = torch.Generator(device=dev).manual_seed(4001)
    a = torch.randn(m, k, device=dev, generator=g).to(torch.float8_e4m3fn)
    b_nk = torch.randn(n, k, device=dev, generator=g).to(torch.float8_e4m3fn)
    sa = torch.full((1,), 0.5, dtype=torch.float32, device=dev)
    sb = torch.full((1,), 0.25, dtype=torch.float32, device=dev)
    c = torch.empty(m, n, dtype=torch.bfloat16, device=dev)
    status = _lib.workspace(dev).data_ptr() + 4 * _lib.WS_STATUS_WORD

    def ours(_):
        _lib.call("tnq_fp8_gemm", a.data_ptr(), b_nk.data_ptr(), sa.data_ptr(), sb.data_ptr(), 0, _lib.FP8_E4M3, m, n, k,
                  c.data_ptr(), status, stream)

    def library(_):
        torch._scaled_mm(a, b_nk.t(), scale_a=sa, scale_b=sb, out_dtype=torch.bfloat16)

    flops = 2.0 * m * n * k
    peaks = {}
    try:
        with open(os.path.join(os.path.dirname(os.path.abspath(__file__)), "MEASURED_PEAKS.json")) as f:
            peaks = json.load(f)
    except OSError:
        pass
    bf16_peak = float(peaks.get("bf16_tflops", 1590.0))
    ms = timed(ours, [None], 20, 5)
    ms_lib = timed(library, [None], 20, 5)
    res["fp8_gemm"] = {
        "us": ms * 1e3, "TFLOPs": flops / (ms * 1e-3) / 1e12, "library_us": ms_lib * 1e3,
        "library_TFLOPs": flops / (ms_lib * 1e-3) / 1e12, "frac_of_library": ms_lib / ms,
        "frac_of_measured_bf16_peak": flops / (ms * 1e-3) / 1e12 / bf16_peak,
        "note": f"e4m3 {m}x{n}x{k}, per-tensor scales, bf16 out; measured dense bf16 peak {bf16_peak} TF/s "
                "(fp8 nominal is twice the bf16 figure)",
    }


def _bench_mxfp8_gemm(dev, res, timed, stream):
    """MXFP8 block-scaled GEMM, M = N = K = 8192, operands and swizzled scales from this library's
    quantizer, with the library's block-scaled GEMM (F.scaled_mm, cuBLASLt) beside it."""
    import torch

    import transformer_nuggets_b200 as tn
    from transformer_nuggets_b200 import _lib

    m = n = k = int(os.environ.get("TNQ_BENCH_GEMM_SIZE", "8192"))
    g = torch.Generator(device=dev).manual_seed(4002)
    rx = tn.quantize_mxfp8(torch.randn(m, k, device=dev, generator=g).to(torch.bfloat16), swizzle=True)
    rw = tn.quantize_mxfp8(torch.randn(n, k, device=dev, generator=g).to(torch.bfloat16), swizzle=True)
    c = torch.empty(m, n, dtype=torch.bfloat16, device=dev)
    status = _lib.workspace(dev).data_ptr() + 4 * _lib.WS_STATUS_WORD

    def ours(_):
        _lib.call("tnq_mxfp8_gemm", rx.q_row.data_ptr(), rw.q_row.data_ptr(), rx.scale_row.data_ptr(),
                  rw.scale_row.data_ptr(), m, n, k, c.data_ptr(), status, stream)

    flops = 2.0 * m * n * k
    ms = timed(ours, [None])
    r = {"us": ms * 1e3, "TFLOPs": flops / (ms * 1e-3) / 1e12,
         "note": f"e4m3 + E8M0 1x32 blocks, {m}x{n}x{k}, swizzled scales straight from the quantizer, bf16 out"}
    try:
        from torch.nn.functional import ScalingType, SwizzleType, scaled_mm

        def library(_):
            scaled_mm(rx.q_row, rw.q_row.t(), scale_a=[rx.scale_row.view(torch.float8_e8m0fnu)],
                      scale_recipe_a=[ScalingType.BlockWise1x32], swizzle_a=[SwizzleType.SWIZZLE_32_4_4],
                      scale_b=[rw.scale_row.view(torch.float8_e8m0fnu)], scale_recipe_b=[ScalingType.BlockWise1x32],
                      swizzle_b=[SwizzleType.SWIZZLE_32_4_4], output_dtype=torch.bfloat16)

        ms_lib = timed(library, [None])
        r.update({"library_us": ms_lib * 1e3, "library_TFLOPs": flops / (ms_lib * 1e-3) / 1e12, "frac_of_library": ms_lib / ms})
    except ImportError:
        r["library_us"] = None
    res["mxfp8_gemm"] = r


def _bench_nvfp4_gemm(dev, res, timed, stream):
    """NVFP4 block-scaled GEMM, M = N = K = 8192, operands, swizzled E4M3 scales and global scales from
    this library's quantizer, with the library's block-scaled GEMM (F.scaled_mm) beside it."""
    import torch

    import transformer_nuggets_b200 as tn
    from transformer_nuggets_b200 import _lib

    m = n = k = int(os.environ.get("TNQ_BENCH_GEMM_SIZE", "8192"))
    g = torch.Generator(device=dev).manual_seed(4003)
    a = tn.quantize_nvfp4(torch.randn(m, k, device=dev, generator=g).to(torch.bfloat16), swizzle=True)
    b = tn.quantize_nvfp4(torch.randn(n, k, device=dev, generator=g).to(torch.bfloat16), swizzle=True)
    c = torch.empty(m, n, dtype=torch.bfloat16, device=dev)
    status = _lib.workspace(dev).data_ptr() + 4 * _lib.WS_STATUS_WORD

    def ours(_):
        _lib.call("tnq_nvfp4_gemm", a.packed.data_ptr(), b.packed.data_ptr(), a.block_scales.data_ptr(),
                  b.block_scales.data_ptr(), a.global_scale.data_ptr(), b.global_scale.data_ptr(), m, n, k, c.data_ptr(),
                  status, stream)

    flops = 2.0 * m * n * k
    ms = timed(ours, [None])
    r = {"us": ms * 1e3, "TFLOPs": flops / (ms * 1e-3) / 1e12,
         "note": f"packed e2m1 + E4M3 1x16 blocks + global scales, {m}x{n}x{k}, operands straight from the quantizer, bf16 out"}
    try:
        from torch.nn.functional import ScalingType, SwizzleType, scaled_mm

        def library(_):
            scaled_mm(a.packed, b.packed.t(), scale_a=[a.block_scales, a.global_scale],
                      scale_recipe_a=[ScalingType.BlockWise1x16, ScalingType.TensorWise],
                      swizzle_a=[SwizzleType.SWIZZLE_32_4_4, SwizzleType.NO_SWIZZLE],
                      scale_b=[b.block_scales, b.global_scale],
                      scale_recipe_b=[ScalingType.BlockWise1x16, ScalingType.TensorWise],
                      swizzle_b=[SwizzleType.SWIZZLE_32_4_4, SwizzleType.NO_SWIZZLE], output_dtype=torch.bfloat16)

        ms_lib = timed(library, [None])
        r.update({"library_us": ms_lib * 1e3, "library_TFLOPs": flops / (ms_lib * 1e-3) / 1e12, "frac_of_library": ms_lib / ms})
    except ImportError:
        r["library_us"] = None
    res["nvfp4_gemm"] = r


def _bench_gemv(dev, res, timed, peak, stream, which=None):
    """Block-scaled M = 1 GEMV on weights larger than L2 (the consumer of the quantizers'
    outputs).  Algorithmic bytes: the weight payload and block scales once, x, y.
    ``which`` restricts the run to "gemv_mxfp8" or "gemv_nvfp4" (one kernel per profile)."""
    import torch

    import transformer_nuggets_b200 as tn
    from transformer_nuggets_b200 import _lib

    g = torch.Generator(device=dev).manual_seed(2001)

    def report(us, nbytes, note):
        gbs = nbytes / (us * 1e-6) / 1e9
        r = {"us": us, "GBps": gbs, "frac_of_measured_peak": gbs / peak, "frac_of_nominal_8000": gbs / 8000.0,
             "algorithmic_bytes": nbytes, "note": note}
        if getattr(timed, "last_distribution", None):
            r["per_launch_us"] = timed.last_distribution
        return r

    if which in (None, "gemv_mxfp8"):
        n, k = 32768, 8192
        w = torch.randn(n, k, dtype=torch.bfloat16, device=dev, generator=g)
        x = torch.randn(1, k, dtype=torch.bfloat16, device=dev, generator=g)
        rw, rx = tn.quantize_mxfp8(w, swizzle=True), tn.quantize_mxfp8(x, swizzle=True)
        rw2 = tn.quantize_mxfp8(w.flip(0).contiguous(), swizzle=True)  # a second weight matrix: two in turn
        del w
        y = torch.empty(1, n, dtype=torch.bfloat16, device=dev)

        def f8(wq):
            _lib.call("tnq_mxfp8_gemv", rx.q_row.data_ptr(), wq.q_row.data_ptr(), rx.scale_row.data_ptr(),
                      wq.scale_row.data_ptr(), n, k, _lib.SCALES_SWIZZLED, y.data_ptr(), stream)

        nbytes = n * k * (1 + 1 / 32) + k * (1 + 1 / 32) + 2 * n
        res["gemv_mxfp8"] = report(timed(f8, [rw2, rw]) * 1e3, nbytes,
                                   f"N={n} K={k}, swizzled E8M0 scales, two 256 MiB weight matrices in turn")
        del rw, rw2
    if which not in (None, "gemv_nvfp4"):
        return

    n, k = 32768, 16384
    w = torch.randn(n, k, dtype=torch.bfloat16, device=dev, generator=g)
    x = torch.randn(1, k, dtype=torch.bfloat16, device=dev, generator=g)
    aw, ax = tn.quantize_nvfp4(w), tn.quantize_nvfp4(x)
    aw2 = tn.quantize_nvfp4(w.flip(0).contiguous())  # a second weight matrix: two in turn
    del w
    y = torch.empty(1, n, dtype=torch.bfloat16, device=dev)

    def f4(wq):
        _lib.call("tnq_nvfp4_gemv", ax.packed.data_ptr(), wq.packed.data_ptr(), ax.block_scales.data_ptr(),
                  wq.block_scales.data_ptr(), ax.global_scale.data_ptr(), wq.global_scale.data_ptr(), n, k,
                  _lib.SCALES_SWIZZLED, y.data_ptr(), stream)

    nbytes = n * k * (0.5 + 1 / 16) + k * (0.5 + 1 / 16) + 2 * n
    res["gemv_nvfp4"] = report(timed(f4, [aw2, aw]) * 1e3, nbytes,
                               f"N={n} K={k}, swizzled E4M3 scales + global scales, two 256 MiB weight matrices in turn")
    # the same product with row-major scales, the layout the reference's GEMV entry points take by default
    from transformer_nuggets_b200.cute.nvfp4_tma import quantize_nvfp4

    x_raw = quantize_nvfp4(x, swizzle=False)
    raws = []
    for wq in (aw2, aw):  # swizzled -> raw on the device: undo the 128x4 atoms of the [n, k / 16] scale matrix
        sc = wq.block_scales.view(torch.uint8).view(n // 128, k // 64, 32, 4, 4).permute(0, 3, 2, 1, 4).reshape(n, k // 16)
        raws.append((wq, sc.contiguous()))

    def f4r(pair):
        _lib.call("tnq_nvfp4_gemv", x_raw.packed.data_ptr(), pair[0].packed.data_ptr(), x_raw.block_scales.data_ptr(),
                  pair[1].data_ptr(), x_raw.global_scale.data_ptr(), pair[0].global_scale.data_ptr(), n, k, _lib.SCALES_RAW,
                  y.data_ptr(), stream)

    y_swz = y.clone()
    f4(aw)
    torch.cuda.synchronize()
    y_swz.copy_(y)
    res["gemv_nvfp4_raw_scales"] = report(timed(f4r, raws) * 1e3, nbytes,
                                          f"N={n} K={k}, row-major E4M3 scales, two weight matrices in turn")
    res["gemv_nvfp4_raw_scales"]["same_bits_as_swizzled"] = bool(torch.equal(y, y_swz))


def _bench_fp8_tensor(dev, res, timed, report, ws, stream):
    import torch

    from transformer_nuggets_b200 import _lib
    from transformer_nuggets_b200.workloads import make_input

    # per-tensor dynamic e4m3, 4096 x 4096: 8 rotating buffer sets (8 x 48 MiB > L2)
    base = make_input("fp8_tensor", dev)
    sets = [(base.clone(), torch.empty_like(base, dtype=torch.float8_e4m3fn)) for _ in range(8)]

    def f1(s):
        _lib.call("tnq_fp8_dynamic_cast", s[0].data_ptr(), s[1].data_ptr(), s[0].numel(), _lib.IN_BF16, _lib.FP8_E4M3,
                  ws.data_ptr(), 0, stream)

    res["fp8_tensor"] = report("fp8_tensor", timed(f1, sets, 64, 16), "cold L2: 8 rotating buffer sets")
    import oracle

    want, _ = oracle.fp8_dynamic_quant(base.cpu(), torch.float8_e4m3fn)
    res["fp8_tensor"]["parity"] = bool(torch.equal(sets[0][1].view(torch.uint8).cpu(), want.view(torch.uint8)))
    res["fp8_tensor_hot_l2"] = report("fp8_tensor", timed(f1, sets[:1], 64, 16), "hot L2: one buffer set")

    res["fp8_tensor_phases"] = _fused_phases(dev, sets, ws, stream, res["fp8_tensor"]["us"])

    # the same eight calls replayed from one CUDA graph (launch overhead out of the picture)
    side = torch.cuda.Stream()
    gws = torch.zeros(_lib.WORKSPACE_BYTES // 4, dtype=torch.int32, device=dev)

    def all_sets():
        for s in sets:
            _lib.call("tnq_fp8_dynamic_cast", s[0].data_ptr(), s[1].data_ptr(), s[0].numel(), _lib.IN_BF16,
                      _lib.FP8_E4M3, gws.data_ptr(), 0, side.cuda_stream)

    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        all_sets()
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=side):
        all_sets()
    for _ in range(3):
        graph.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(8):
        graph.replay()
    e1.record()
    torch.cuda.synchronize()
    res["fp8_tensor_graph_replay"] = report("fp8_tensor", e0.elapsed_time(e1) / 64,
                                            "cold L2, eight calls per CUDA graph, eight replays")
    res["fp8_tensor_graph_replay"].pop("per_launch_us", None)
    del sets, graph


def _fused_phases(dev, sets, ws, stream, event_us):
    """Where the single-launch cast's time goes: the kernel built with time stamps (at entry / slab loaded
    and CTA maximum known / grid-wide exchange done / last store issued), cold L2 by the same rotating
    buffer sets.  Per-CTA phase lengths from the SM clock (averaged over CTAs and launches, converted with
    the SM clock NVML reports during the run) and, from the global timer, the launch's timeline measured
    from the first CTA's start."""
    import ctypes

    import torch

    from transformer_nuggets_b200 import _lib

    stamps = torch.zeros(256 * 8, dtype=torch.int64, device=dev)
    grid = ctypes.c_int(0)
    try:
        import pynvml

        pynvml.nvmlInit()
        h = pynvml.nvmlDeviceGetHandleByIndex(dev.index or 0)
    except Exception:
        h = None

    def run(s):
        _lib.call("tnq_fp8_dynamic_cast_profile", s[0].data_ptr(), s[1].data_ptr(), s[0].numel(), ws.data_ptr(), 0,
                  stamps.data_ptr(), ctypes.byref(grid), stream)

    for it in range(16):
        run(sets[it % len(sets)])
    torch.cuda.synchronize()
    mhz = float(pynvml.nvmlDeviceGetClockInfo(h, pynvml.NVML_CLOCK_SM)) if h is not None else None
    acc, n = [0.0] * 7, 0
    for it in range(16):
        run(sets[it % len(sets)])
        torch.cuda.synchronize()
        t = stamps[: grid.value * 8].view(grid.value, 8).cpu().double()
        first = t[:, 4].min()
        acc[0] += float((t[:, 1] - t[:, 0]).mean())
        acc[1] += float((t[:, 2] - t[:, 1]).mean())
        acc[2] += float((t[:, 3] - t[:, 2]).mean())
        acc[3] += float(t[:, 4].max() - first)
        acc[4] += float((t[:, 5] - first).max())
        acc[5] += float((t[:, 6] - first).max())
        acc[6] += float((t[:, 7] - first).max())
        n += 1
    r = {"ctas": grid.value, "launches": n, "sm_mhz": mhz, "event_us_per_call": event_us,
         "timeline_us_from_first_cta_start": {"last_cta_start": acc[3] / n / 1e3, "last_load_done": acc[4] / n / 1e3,
                                              "exchange_done": acc[5] / n / 1e3, "last_exit": acc[6] / n / 1e3}}
    r["between_kernels_us"] = event_us - r["timeline_us_from_first_cta_start"]["last_exit"]
    if mhz:
        r["mean_per_cta_us"] = {"load_and_cta_amax": acc[0] / n / mhz, "grid_exchange": acc[1] / n / mhz,
                                "convert_and_store": acc[2] / n / mhz}
    return r


def _bench_rowwise(dev, res, timed, report, stream):
    import torch

    from transformer_nuggets_b200 import _lib
    from transformer_nuggets_b200.workloads import make_input

    x = make_input("fp8_rowwise", dev)
    q43, q52 = torch.empty_like(x, dtype=torch.float8_e4m3fn), torch.empty_like(x, dtype=torch.float8_e5m2)
    s43 = torch.empty(x.shape[0], 1, dtype=torch.float32, device=dev)
    s52 = torch.empty_like(s43)

    def f2(xin):
        _lib.call("tnq_fp8_rowwise", xin.data_ptr(), x.shape[0], x.shape[1], _lib.IN_BF16, q43.data_ptr(), s43.data_ptr(),
                  q52.data_ptr(), s52.data_ptr(), 0, stream)

    res["fp8_rowwise"] = report("fp8_rowwise", timed(f2, _in_turn(x)), "input 256 MiB > L2, two inputs in turn")
    import oracle

    xs = x[4096:5120].cpu()
    w43, ws43 = oracle.fp8_rowwise_quant(xs, torch.float8_e4m3fn)
    w52, ws52 = oracle.fp8_rowwise_quant(xs, torch.float8_e5m2)
    res["fp8_rowwise"]["parity"] = bool(
        torch.equal(q43[4096:5120].view(torch.uint8).cpu(), w43.view(torch.uint8))
        and torch.equal(q52[4096:5120].view(torch.uint8).cpu(), w52.view(torch.uint8))
        and torch.equal(s43[4096:5120].cpu(), ws43) and torch.equal(s52[4096:5120].cpu(), ws52))
    del x, q43, q52


def _bench_mxfp8(dev, res, timed, report, ws, stream):
    import torch

    from transformer_nuggets_b200 import _lib
    from transformer_nuggets_b200.workloads import make_input

    x = make_input("mxfp8", dev)
    rows, cols = x.shape
    qr = torch.empty(rows, cols, dtype=torch.uint8, device=dev)
    qc = torch.empty(cols, rows, dtype=torch.uint8, device=dev)
    sr = torch.empty(512 * (rows // 128) * ((cols // 32 + 3) // 4), dtype=torch.uint8, device=dev)
    sc = torch.empty(512 * ((cols + 127) // 128) * ((rows // 32 + 3) // 4), dtype=torch.uint8, device=dev)
    status = ws.data_ptr() + 4 * _lib.WS_STATUS_WORD

    xs = _in_turn(x)

    def f3(xin):
        _lib.call("tnq_mxfp8_quantize", xin.data_ptr(), rows, cols, _lib.IN_BF16, qr.data_ptr(), sr.data_ptr(), qc.data_ptr(),
                  sc.data_ptr(), _lib.E8M0_CEIL, _lib.SCALES_SWIZZLED, status, stream)

    def f3r(xin):
        _lib.call("tnq_mxfp8_quantize", xin.data_ptr(), rows, cols, _lib.IN_BF16, qr.data_ptr(), sr.data_ptr(), 0,
                  0, _lib.E8M0_CEIL, _lib.SCALES_SWIZZLED, status, stream)

    # input 112 MiB + outputs 114 MiB per call: rotate nothing, the footprint alone exceeds L2
    res["mxfp8"] = report("mxfp8", timed(f3, xs), "row + column outputs, swizzled scales; two inputs in turn, footprint 338 MiB > L2")
    import oracle

    xc = x.cpu()
    wq, wsr = oracle.mxfp8_quantize(xc[:1024], "ceil")  # 1024 rows of x, 1024 rows of x^T, and the scale atoms they own
    wqt, wsc = oracle.mxfp8_quantize(xc[:, :1024].t().contiguous(), "ceil")
    n_row, n_col = oracle.to_blocked(wsr).numel(), oracle.to_blocked(wsc).numel()
    res["mxfp8"]["parity"] = bool(
        torch.equal(qr[:1024].cpu(), wq.view(torch.uint8)) and torch.equal(qc[:1024].cpu(), wqt.view(torch.uint8))
        and torch.equal(sr[:n_row].cpu(), oracle.to_blocked(wsr)) and torch.equal(sc[:n_col].cpu(), oracle.to_blocked(wsc)))
    res["mxfp8_rowwise_only"] = report("mxfp8", timed(f3r, xs), "row-wise output only", 2.0 + 1.0 + 1.0 / 32)
    del qr, qc
    # the same tile pipeline with the arithmetic taken out: TMA load of a 128 x 128 tile, TMA store of the same bytes
    y = torch.empty_like(x)
    best = None
    for stages, per_sm in ((2, 2), (3, 1), (3, 2), (2, 3)):
        def fc(xin, stages=stages, per_sm=per_sm):
            _lib.call("tnq_tile_copy", xin.data_ptr(), y.data_ptr(), rows, cols, stages, per_sm, status, stream)
        try:
            ms = timed(fc, xs)
        except _lib.TnqError:
            continue
        if best is None or ms < best[0]:
            best = (ms, stages, per_sm)
    if best is not None:
        ok = bool(torch.equal(y[-256:], x[-256:]))
        res["tile_copy_ceiling"] = {
            "us": best[0] * 1e3, "GBps": 4.0 * rows * cols / (best[0] * 1e-3) / 1e9, "stages": best[1], "ctas_per_sm": best[2],
            "copied_correctly": ok,
            "note": "TMA tile load -> TMA tile store of the same 8192 x 7168 bf16 matrix, no arithmetic (4 B/elem): what a "
                    "tile pipeline reaches on this shape; best of four stage / occupancy settings"}
        per_byte = best[0] / (4.0 * rows * cols)
        res["mxfp8"]["frac_of_tile_copy"] = per_byte * 4.0625 * rows * cols / (res["mxfp8"]["us"] * 1e-3)
    del x, xs, y


def _bench_nvfp4(dev, res, timed, report, ws, stream):
    import torch

    from transformer_nuggets_b200 import _lib
    from transformer_nuggets_b200.workloads import make_input

    status = ws.data_ptr() + 4 * _lib.WS_STATUS_WORD
    x = make_input("nvfp4", dev)
    rows, cols = x.shape
    packed = torch.empty(rows, cols // 2, dtype=torch.uint8, device=dev)
    sf = torch.empty(512 * (rows // 128) * (cols // 64), dtype=torch.uint8, device=dev)
    gs = torch.empty(1, dtype=torch.float32, device=dev)
    amax_ptr = ws.data_ptr() + 4 * _lib.WS_AMAX_WORD

    # two inputs in turn: a call never finds parts of its own input left in L2 by the previous call
    x_other = _in_turn(x)[0]

    def f4(xin):
        _lib.call("tnq_nvfp4_quantize_dynamic", xin.data_ptr(), rows, cols, _lib.IN_BF16, ws.data_ptr(), packed.data_ptr(),
                  sf.data_ptr(), _lib.SCALES_SWIZZLED, gs.data_ptr(), stream)

    def f4s(xin):
        _lib.call("tnq_nvfp4_quantize", xin.data_ptr(), rows, cols, _lib.IN_BF16, amax_ptr, packed.data_ptr(), sf.data_ptr(),
                  _lib.SCALES_SWIZZLED, gs.data_ptr(), status, stream)

    res["nvfp4"] = report("nvfp4", timed(f4, [x_other, x], 20, 4),
                          "dynamic global scale (amax pass + quantize pass), two 512 MiB inputs in turn")
    import oracle

    wp, wsf, wg = oracle.nvfp4_quantize(x[:512].cpu(), x.abs().max().float().cpu())
    n_sf = oracle.to_blocked(wsf.view(torch.uint8)).numel()
    res["nvfp4"]["parity"] = bool(
        torch.equal(packed[:512].cpu(), wp.view(torch.uint8)) and torch.equal(gs.cpu(), wg.reshape(1))
        and torch.equal(sf[:n_sf].cpu(), oracle.to_blocked(wsf.view(torch.uint8))))
    res["nvfp4"]["parity_note"] = "against this build's own NVFP4 specification: the reference has no NVFP4 quantizer (unpinned)"
    res["nvfp4_given_global_amax"] = report("nvfp4", timed(f4s, [x_other, x], 20, 4), "global amax supplied", 2.5625)
    del x_other


def emit(line: dict):
    """The one JSON line, on the real stdout (see main: fd 1 is pointed at stderr while the
    benchmark runs so that library banners cannot land on stdout)."""
    os.write(_REAL_STDOUT, (json.dumps(line) + "\n").encode())


_REAL_STDOUT = 1


def main():
    global _REAL_STDOUT
    sys.stdout.flush()
    _REAL_STDOUT = os.dup(1)
    os.dup2(2, 1)
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default=HEADLINE)
    ap.add_argument("--exchange", default="peer", choices=["peer", "nccl"])
    ap.add_argument("--no-extras", action="store_true", help="skip the other single-GPU configurations")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-comparators", action="store_true", help="skip the reference's GPU code on the same machine")
    ap.add_argument("--details", default="", help="also write the full record (notes, per-launch distributions) to this file")
    ap.add_argument("--rows", type=int, default=0, help="override the headline workload's row count (profiling)")
    ap.add_argument("--profile", action="store_true", help="run only warm-up and timed steps (for ncu captures)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
