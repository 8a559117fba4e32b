"""Time the tcgen05 GEMM against torch.matmul (cuBLAS) on Llama-3-8B shaped problems.

    python benchmarks/bench_gemm.py [--tokens 8192]

CUDA-event timing, L2 flushed between iterations, median of 10 after 3 warm-ups.
"""

import argparse
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from rl_engine.kernels.ops.sm100.gemm import gemm  # noqa: E402


def timed(fn, flush, iters=10, warmup=3):
    for _ in range(warmup):
        fn()
    times = []
    for _ in range(iters):
        flush.zero_()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        s.record()
        fn()
        e.record()
        torch.cuda.synchronize()
        times.append(s.elapsed_time(e))
    times.sort()
    return times[len(times) // 2]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=8192)
    args = ap.parse_args()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    m = args.tokens
    rows = []
    for name, n, k in [("qkv", 6144, 4096), ("o", 4096, 4096), ("gate_up", 28672, 4096), ("down", 4096, 14336)]:
        x = torch.randn(m, k, device="cuda").to(torch.bfloat16)
        w = (torch.randn(n, k, device="cuda") * 0.02).to(torch.bfloat16)
        dy = torch.randn(m, n, device="cuda").to(torch.bfloat16)
        flops = 2.0 * m * n * k
        for tag, ours, lib in [
            ("fwd NT", lambda: gemm(x, w), lambda: x @ w.t()),
            ("dgrad NN", lambda: gemm(dy, w, b_mn=True), lambda: dy @ w),
            ("wgrad TN", lambda: gemm(dy, x, a_mn=True, b_mn=True), lambda: dy.t() @ x),
        ]:
            t_ours, t_lib = timed(ours, flush), timed(lib, flush)
            rows.append(dict(op=name, kind=tag, m=m, n=n, k=k, ours_ms=round(t_ours, 4), cublas_ms=round(t_lib, 4),
                             ours_tflops=round(flops / t_ours / 1e9, 1), cublas_tflops=round(flops / t_lib / 1e9, 1)))
            print(json.dumps(rows[-1]), flush=True)


if __name__ == "__main__":
    main()
