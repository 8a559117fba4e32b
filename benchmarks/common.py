"""Helpers shared by the per-op benchmark scripts: CUDA-event timing with an L2 flush between
repetitions, the measured roofline denominators, and one-JSON-line reporting."""

from __future__ import annotations

import json
import os
import statistics
import sys
import time
from typing import Any, Callable, Dict, Optional

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def peaks() -> Dict[str, Any]:
    """Measured copy bandwidth / cuBLAS bf16 throughput of this machine when recorded, else the fallback pair."""
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            p = json.load(f)
        return {"hbm_gbs": float(p["hbm_gbs"]), "bf16_tflops": float(p["bf16_tflops"]), "source": "measured"}
    except Exception:
        return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


_FLUSH: Dict[str, torch.Tensor] = {}


def time_ms(fn: Callable[[], Any], warmup: int = 3, repeat: int = 10, device: Optional[torch.device] = None) -> Dict[str, float]:
    device = torch.device(device) if device is not None else torch.device("cuda" if torch.cuda.is_available() else "cpu")
    for _ in range(warmup):
        fn()
    samples = []
    for _ in range(max(repeat, 1)):
        if device.type == "cuda":
            key = str(device)
            if key not in _FLUSH:
                _FLUSH[key] = torch.empty(256 << 20, dtype=torch.uint8, device=device)
            _FLUSH[key].zero_()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize(device)
            a.record()
            fn()
            b.record()
            torch.cuda.synchronize(device)
            samples.append(a.elapsed_time(b))
        else:
            t0 = time.perf_counter()
            fn()
            samples.append((time.perf_counter() - t0) * 1e3)
    return {"ms": statistics.median(samples), "min_ms": min(samples), "max_ms": max(samples)}


def peak_gb(fn: Callable[[], Any], device: Optional[torch.device] = None) -> float:
    if not torch.cuda.is_available():
        return 0.0
    torch.cuda.synchronize(device)
    torch.cuda.reset_peak_memory_stats(device)
    base = torch.cuda.memory_allocated(device)
    fn()
    torch.cuda.synchronize(device)
    return (torch.cuda.max_memory_allocated(device) - base) / 2**30


def report(name: str, shape: Dict[str, Any], timing: Dict[str, float], flops: float = 0.0, nbytes: float = 0.0, **extra) -> Dict[str, Any]:
    pk = peaks()
    line: Dict[str, Any] = {"benchmark": name, **shape, "ms": round(timing["ms"], 4), "min_ms": round(timing["min_ms"], 4)}
    if flops:
        line["tflops"] = round(flops / timing["ms"] / 1e9, 2)
        line[f"frac_of_{pk['source']}_bf16_peak"] = round(line["tflops"] / pk["bf16_tflops"], 3)
    if nbytes:
        line["gbs"] = round(nbytes / timing["ms"] / 1e6, 1)
        line[f"frac_of_{pk['source']}_hbm_peak"] = round(line["gbs"] / pk["hbm_gbs"], 3)
    line.update(extra)
    print(json.dumps(line), flush=True)
    return line


def randn(shape, dtype=torch.bfloat16, scale: float = 1.0, seed: int = 0, device=None) -> torch.Tensor:
    device = device or ("cuda" if torch.cuda.is_available() else "cpu")
    g = torch.Generator(device=device).manual_seed(seed)
    return (torch.randn(shape, device=device, generator=g) * scale).to(dtype)
