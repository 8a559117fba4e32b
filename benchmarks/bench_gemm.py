"""Time the tcgen05 GEMM against torch.matmul (cuBLAS) on Llama-3-8B shaped problems.

    python benchmarks/bench_gemm.py [--tokens 8192]
    python benchmarks/bench_gemm.py --tokens 16384 --sustained 2.0      # seconds-long loops under the power cap

Default: CUDA-event timing, L2 flushed between iterations, median of 10 after 3 warm-ups (isolated launches, boost
clocks).  ``--sustained S`` instead runs every product back to back for about ``S`` seconds per arm (one CUDA-event pair
around the whole loop, no flush: every operand set is larger than L2 at the default sizes) and reports the median SM
clock sampled through NVML during the loop: this is the regime of a training step on a 1 kW part.
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


class _Clock:
    """Median SM clock over a loop, sampled every 50 ms through NVML (None if NVML is not there)."""

    def __init__(self):
        self.samples, self._stop, self._thread, self._h = [], None, None, None
        try:
            import pynvml

            pynvml.nvmlInit()
            self._nv = pynvml
            self._h = pynvml.nvmlDeviceGetHandleByIndex(torch.cuda.current_device())
        except Exception:  # noqa: BLE001
            self._h = None

    def __enter__(self):
        import threading

        self.samples = []
        self._stop = threading.Event()
        if self._h is not None:
            def run():
                while not self._stop.is_set():
                    try:
                        self.samples.append(self._nv.nvmlDeviceGetClockInfo(self._h, self._nv.NVML_CLOCK_SM))
                    except Exception:  # noqa: BLE001
                        pass
                    self._stop.wait(0.05)

            self._thread = threading.Thread(target=run, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread is not None:
            self._thread.join()

    def median(self):
        s = sorted(self.samples)
        return s[len(s) // 2] if s else None


def sustained(fn, seconds, clock):
    """(ms per call, median SM MHz) of ``fn`` called back to back for about ``seconds``."""
    for _ in range(3):
        fn()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    s.record()
    for _ in range(10):
        fn()
    e.record()
    torch.cuda.synchronize()
    calls = max(10, int(seconds * 1e3 / (s.elapsed_time(e) / 10)))
    with clock:
        torch.cuda.synchronize()
        s.record()
        for _ in range(calls):
            fn()
        e.record()
        torch.cuda.synchronize()
    return s.elapsed_time(e) / calls, clock.median()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=8192)
    ap.add_argument("--sustained", type=float, default=0.0, help="seconds per arm of back-to-back calls (0: isolated launches)")
    ap.add_argument("--pair", choices=["auto", "0", "1"], default="auto",
                    help="tile engine of our arm: library default per shape, single-CTA 128x256, or CTA-pair 256x256")
    ap.add_argument("--only", default="", help="comma-separated filter on 'op kind' names, e.g. 'down fwd,gate_up dgrad'")
    ap.add_argument("--no-lib", action="store_true", help="skip the torch.matmul arm (parameter sweeps of our kernel)")
    args = ap.parse_args()
    clock = _Clock()
    pair = {"auto": None, "0": False, "1": True}[args.pair]
    only = [f.strip() for f in args.only.split(",") if f.strip()]
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    m = args.tokens
    rows = []
    for name, n, k in [("qkv", 6144, 4096), ("o", 4096, 4096), ("gate_up", 28672, 4096), ("down", 4096, 14336)]:
        x = torch.randn(m, k, device="cuda").to(torch.bfloat16)
        w = (torch.randn(n, k, device="cuda") * 0.02).to(torch.bfloat16)
        dy = torch.randn(m, n, device="cuda").to(torch.bfloat16)
        flops = 2.0 * m * n * k
        for tag, ours, lib in [
            ("fwd NT", lambda: gemm(x, w, pair=pair), lambda: x @ w.t()),
            ("dgrad NN", lambda: gemm(dy, w, b_mn=True, pair=pair), lambda: dy @ w),
            ("wgrad TN", lambda: gemm(dy, x, a_mn=True, b_mn=True, pair=pair), lambda: dy.t() @ x),
        ]:
            if only and not any(f in f"{name} {tag}" for f in only):
                continue
            if args.no_lib:
                lib = ours
            extra = {"pair": args.pair}
            if args.sustained > 0:
                (t_ours, mhz_ours), (t_lib, mhz_lib) = sustained(ours, args.sustained, clock), sustained(lib, args.sustained, clock)
                extra.update(mode=f"sustained {args.sustained:g} s", ours_sm_mhz=mhz_ours, cublas_sm_mhz=mhz_lib)
            else:
                t_ours, t_lib = timed(ours, flush), timed(lib, flush)
            if args.no_lib:
                extra["cublas"] = "skipped (second arm repeats ours)"
            rows.append(dict(op=name, kind=tag, m=m, n=n, k=k, ours_ms=round(t_ours, 4), cublas_ms=round(t_lib, 4),
                             ours_tflops=round(flops / t_ours / 1e9, 1), cublas_tflops=round(flops / t_lib / 1e9, 1),
                             ratio=round(t_lib / t_ours, 3), **extra))
            print(json.dumps(rows[-1]), flush=True)


if __name__ == "__main__":
    main()
