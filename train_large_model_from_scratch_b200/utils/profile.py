"""Peak-FLOPs table and MFU meter (reference: `utils/profile.py:1-45`).

The reference's table stops at Hopper, so on a B200 it prints a warning and
reports 0 % MFU. This table adds the Blackwell parts (dense, no 2:4 sparsity)
and can also report MFU against a measured cuBLAS peak.
"""
from __future__ import annotations

import json
import os

import torch

GPU_PEAK_FLOPS = {
    "T4":   {"fp32": 8.1e12, "fp16": 65e12, "bf16": 0},
    "V100": {"fp32": 15.7e12, "fp16": 125e12, "bf16": 0},
    "A100": {"fp32": 19.5e12, "fp16": 312e12, "bf16": 312e12},
    "A40":  {"fp32": 37.4e12, "fp16": 149e12, "bf16": 149e12},
    "A30":  {"fp32": 10.3e12, "fp16": 165e12, "bf16": 165e12},
    "RTX 6000 Ada": {"fp32": 91e12, "fp16": 181e12, "bf16": 181e12},
    "L40S": {"fp32": 91e12, "fp16": 181e12, "bf16": 181e12},
    "L40":  {"fp32": 91e12, "fp16": 181e12, "bf16": 181e12},
    "L4":   {"fp32": 30e12, "fp16": 120e12, "bf16": 120e12},
    "3090": {"fp32": 35.6e12, "fp16": 142e12, "bf16": 142e12},
    "4090": {"fp32": 82.6e12, "fp16": 330e12, "bf16": 330e12},
    "H100": {"fp32": 60e12, "fp16": 989e12, "bf16": 989e12, "fp8": 1979e12},
    "H800": {"fp32": 34e12, "fp16": 734e12, "bf16": 734e12, "fp8": 1468e12},
    "H200": {"fp32": 67e12, "fp16": 989e12, "bf16": 989e12, "fp8": 1979e12},
    "H20":  {"fp32": 21e12, "fp16": 494e12, "bf16": 494e12, "fp8": 988e12},
    # Blackwell, dense
    "GB200": {"fp32": 80e12, "fp16": 2.5e15, "bf16": 2.5e15, "fp8": 5e15},
    "B200": {"fp32": 80e12, "fp16": 2.25e15, "bf16": 2.25e15, "fp8": 4.5e15},
    "B100": {"fp32": 60e12, "fp16": 1.8e15, "bf16": 1.8e15, "fp8": 3.5e15},
}


def get_gpu_peak_flops(dtype: str = "bf16", per_device: bool = True, gpu_name: str | None = None) -> float:
    """Nominal peak FLOP/s of the visible GPU type (0 when unknown)."""
    if gpu_name is None:
        gpu_name = torch.cuda.get_device_name(0) if torch.cuda.is_available() else "cpu"
    peak = 0
    for key, row in GPU_PEAK_FLOPS.items():
        if key in gpu_name:
            peak = row.get(dtype.lower(), 0) or 0
            break
    if peak == 0:
        print(f"Warning: unknown or unsupported FLOPs for GPU {gpu_name} with dtype {dtype}")
    n = torch.cuda.device_count() if (torch.cuda.is_available() and not per_device) else 1
    return peak * n


def get_measured_peak_flops(path: str | None = None, sustained: bool = True) -> float | None:
    """bf16 GEMM throughput measured on this machine's GPUs, if a peaks file (JSON with
    `bf16_tflops[_sustained]`) is named by `path` or by the `TLM_MEASURED_PEAKS` environment variable; else None."""
    path = path or os.environ.get("TLM_MEASURED_PEAKS")
    if not path:
        return None
    try:
        with open(path) as f:
            d = json.load(f)
        return float(d["bf16_tflops_sustained" if sustained else "bf16_tflops"]) * 1e12
    except (OSError, KeyError, ValueError):
        return None


def compute_mfu(model, batch_size: int, seq_len: int, time: float, ga: int = 1, dtype: str = "bf16",
                peak_flops: float | None = None):
    """(mfu, achieved FLOP/s, peak FLOP/s) per device for one optimizer step of
    `ga` micro-steps that took `time` seconds."""
    flops = model.get_flops_per_fwd_bwd(batch_size, seq_len) * ga
    achieved = flops / time if time > 0 else 0.0
    peak = get_gpu_peak_flops(dtype=dtype) if peak_flops is None else peak_flops
    return (achieved / peak if peak else 0.0), achieved, peak
