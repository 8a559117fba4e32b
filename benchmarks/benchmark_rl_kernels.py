"""Kernel-level roofline table for every hand-written hot kernel at RL shapes (one JSON line each, with
the achieved fraction of the measured copy bandwidth / bf16 GEMM throughput of this machine).

Counterpart of the reference's ``benchmarks/benchmark_rl_kernels.py``; the workloads are the ones defined
in ``benchmarks/profile_kernels.py`` so that a timing here and an ``ncu`` capture there see the same launch.

    python benchmarks/benchmark_rl_kernels.py                 # all kernels
    python benchmarks/benchmark_rl_kernels.py --kernel gemm,attention_fwd --csv kernels.csv
"""

import argparse
import csv
import json

import profile_kernels as pk


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--kernel", default="all", help=f"comma-separated subset of: {', '.join(sorted(pk.CASES))}")
    ap.add_argument("--csv", default=None)
    args = ap.parse_args()
    names = sorted(pk.CASES) if args.kernel == "all" else [k.strip() for k in args.kernel.split(",") if k.strip()]
    unknown = sorted(set(names) - set(pk.CASES))
    if unknown:
        raise SystemExit(f"unknown kernels: {unknown}; choose from {sorted(pk.CASES)}")
    peaks = pk.peaks()
    rows = []
    for name in names:
        try:
            r = pk.CASES[name]()
            line = {"kernel": name, "ms": round(r["ms"], 4), "shape": str(r["shape"]), "peaks": peaks["source"], "status": "pass"}
            if r["flops"]:
                line["tflops"] = round(r["flops"] / r["ms"] / 1e9, 1)
                line["frac_of_bf16_peak"] = round(line["tflops"] / peaks["bf16_tflops"], 3)
            if r["bytes"]:
                line["gbs"] = round(r["bytes"] / r["ms"] / 1e6, 1)
                line["frac_of_hbm_peak"] = round(line["gbs"] / peaks["hbm_gbs"], 3)
        except Exception as exc:
            line = {"kernel": name, "status": "blocked", "notes": (str(exc).splitlines() or [type(exc).__name__])[0]}
        rows.append(line)
        print(json.dumps(line), flush=True)
    if args.csv:
        fields = sorted({k for r in rows for k in r})
        with open(args.csv, "w", newline="") as f:
            w = csv.DictWriter(f, fieldnames=fields)
            w.writeheader()
            w.writerows(rows)


if __name__ == "__main__":
    main()
