"""Seeded synthetic inputs for the five cast configurations.

The reference measures its casts on ``torch.randn`` tensors only
(benchmarks/fp8_dynamic_cast.py:94-96); no dataset is involved.  These
generators produce the value distributions the benchmark configurations name.
CPU and CUDA random streams differ, so a tensor that must be compared between
a kernel and a CPU checker is generated once and copied, never generated twice.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch


@dataclass(frozen=True)
class CastConfig:
    name: str
    rows: int
    cols: int
    seed: int
    #: bytes the op must move per input element (minimal reads + visible writes)
    algo_bytes_per_elem: float
    description: str


CONFIGS = {
    "fp8_tensor": CastConfig(
        "fp8_tensor", 4096, 4096, 1001, 3.0,
        "per-tensor dynamic e4m3 cast, N(0,1) with 0.1% entries x100",
    ),
    "fp8_rowwise": CastConfig(
        "fp8_rowwise", 16384, 8192, 1002, 4.0,
        "rowwise e4m3 + e5m2 cast, row sigma log-uniform in [2^-6, 2^6]",
    ),
    "mxfp8": CastConfig(
        "mxfp8", 8192, 7168, 1003, 4.0625,
        "MXFP8 row + column quantize, rows scaled by log-uniform 2^-8..2^8",
    ),
    "nvfp4": CastConfig(
        "nvfp4", 16384, 16384, 1004, 4.5625,
        "NVFP4 quantize with dynamic global scale, N(0,1) with 1% Student-t(3)",
    ),
    "fp8_sharded": CastConfig(
        "fp8_sharded", 131072, 8192, 1005, 5.0,
        "row-sharded per-tensor e4m3 cast, N(0,1) with 128 outlier rows x1000",
    ),
}


def _gen(device, seed):
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    return g


def make_input(name: str, device="cpu", rows: int | None = None, cols: int | None = None,
               row_offset: int = 0) -> torch.Tensor:
    """bf16 ``[rows, cols]`` tensor for configuration ``name``.

    ``rows``/``cols`` default to the configuration's full size; smaller values
    give a same-distribution test case.  ``row_offset`` is mixed into the seed
    so that each rank of a sharded run can generate its own row block.
    """
    cfg = CONFIGS[name]
    rows = cfg.rows if rows is None else rows
    cols = cfg.cols if cols is None else cols
    device = torch.device(device)
    g = _gen(device, cfg.seed + 7919 * row_offset)
    f32 = torch.float32
    # generate in row chunks so that the fp32 temporaries stay small
    out = torch.empty(rows, cols, dtype=torch.bfloat16, device=device)
    chunk = max(1, min(rows, (1 << 26) // max(cols, 1)))
    for r0 in range(0, rows, chunk):
        r1 = min(rows, r0 + chunk)
        n = r1 - r0
        x = torch.randn(n, cols, dtype=f32, device=device, generator=g)
        if name == "fp8_tensor":
            k = max(1, (n * cols) // 1000)
            idx = torch.randint(0, n * cols, (k,), device=device, generator=g)
            x.view(-1)[idx] *= 100.0
        elif name == "fp8_rowwise":
            sigma = torch.exp2(torch.rand(n, 1, dtype=f32, device=device, generator=g) * 12.0 - 6.0)
            x *= sigma
        elif name == "mxfp8":
            s = torch.exp2(torch.rand(n, 1, dtype=f32, device=device, generator=g) * 16.0 - 8.0)
            x *= s
        elif name == "nvfp4":
            mask = torch.rand(n, cols, dtype=f32, device=device, generator=g) < 0.01
            chi = torch.randn(3, n, cols, dtype=f32, device=device, generator=g).square_().sum(0)
            t = torch.randn(n, cols, dtype=f32, device=device, generator=g) / torch.sqrt(chi / 3.0)
            x = torch.where(mask, t, x)
            del mask, chi, t
        elif name == "fp8_sharded":
            k = max(1, n // 1024)  # 128 outlier rows at the full 131072 rows
            idx = torch.randint(0, n, (k,), device=device, generator=g)
            x[idx] *= 1000.0
        else:
            raise KeyError(name)
        out[r0:r1] = x.to(torch.bfloat16)
    return out
