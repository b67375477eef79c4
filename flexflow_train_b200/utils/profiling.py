"""Timing, NVTX ranges and roofline arithmetic.

``profiling_wrapper`` is the reference's helper (lib/kernels/include/kernels/profiling.h:13-107): warm-up
iterations, then CUDA-event timing on the GPU or a monotonic clock on the CPU, returning the mean in ms.
"""
from __future__ import annotations

import contextlib
import json
import os
import time
from dataclasses import dataclass
from typing import Callable, Optional

import torch


@dataclass
class ProfilingSettings:
    warmup_iters: int = 3
    measure_iters: int = 10


def profiling_wrapper(fn: Callable[[], None], settings: ProfilingSettings = ProfilingSettings(), device: str = "cuda") -> float:
    for _ in range(settings.warmup_iters):
        fn()
    if device.startswith("cuda") and torch.cuda.is_available():
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(settings.measure_iters):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / settings.measure_iters
    t0 = time.perf_counter()
    for _ in range(settings.measure_iters):
        fn()
    return (time.perf_counter() - t0) * 1e3 / settings.measure_iters


@contextlib.contextmanager
def nvtx_range(name: str):
    """NVTX range around a PCG layer (no-op without CUDA)."""
    on = torch.cuda.is_available()
    if on:
        torch.cuda.nvtx.range_push(name)
    try:
        yield
    finally:
        if on:
            torch.cuda.nvtx.range_pop()


def measured_peaks(path: Optional[str] = None) -> dict:
    """Roofline denominators: measured copy bandwidth and GEMM throughput when the measurement file exists,
    otherwise the documented fallback."""
    path = path or os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"], "bf16_tflops_sustained": d.get("bf16_tflops_sustained", d["bf16_tflops"]),
                "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


NVLINK_PEER_GBS = 770.0       # measured peer copy, per direction per GPU
NVLINK_ALLREDUCE_BUS_GBS = 725.0


def roofline(ms: float, *, flops: float = 0.0, hbm_bytes: float = 0.0, nvlink_bytes: float = 0.0, sustained: bool = False,
             peaks: Optional[dict] = None) -> dict:
    """Achieved time against the slower of compute-at-peak, HBM bytes at copy bandwidth and NVLink bytes at the
    measured peer bandwidth."""
    pk = peaks or measured_peaks()
    tf = pk["bf16_tflops_sustained" if sustained else "bf16_tflops"]
    t_compute = flops / (tf * 1e12) * 1e3
    t_hbm = hbm_bytes / (pk["hbm_gbs"] * 1e9) * 1e3
    t_link = nvlink_bytes / (NVLINK_PEER_GBS * 1e9) * 1e3
    bound = max(t_compute, t_hbm, t_link)
    which = "compute" if bound == t_compute else ("hbm" if bound == t_hbm else "nvlink")
    return {"ms": ms, "roofline_ms": bound, "fraction": bound / ms if ms > 0 else 0.0, "bound": which,
            "tflops": flops / ms / 1e9 if ms > 0 else 0.0, "hbm_gbs": hbm_bytes / ms / 1e6 if ms > 0 else 0.0,
            "nvlink_gbs": nvlink_bytes / ms / 1e6 if ms > 0 else 0.0, "peaks": pk["source"]}
