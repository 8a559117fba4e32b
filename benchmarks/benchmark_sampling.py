"""Temperature / top-k / top-p sampling: the radix-select kernel vs the sort-based PyTorch path.
Counterpart of the reference's ``benchmarks/benchmark_sampling.py`` (FlashInfer vs torch there).

    python benchmarks/benchmark_sampling.py --rows 256 --vocab 151936 --top-k 50 --top-p 0.9
"""

import argparse

import torch

from common import report, time_ms


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--rows", type=int, default=256)
    ap.add_argument("--vocab", type=int, default=151936)
    ap.add_argument("--top-k", type=int, default=50)
    ap.add_argument("--top-p", type=float, default=0.9)
    ap.add_argument("--temperature", type=float, default=0.7)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--repeat", type=int, default=20)
    args = ap.parse_args()
    from rl_engine.kernels.sampling import SamplerBackend

    dev = "cuda" if torch.cuda.is_available() else "cpu"
    logits = torch.randn(args.rows, args.vocab, device=dev) * 3
    shape = {"rows": args.rows, "vocab": args.vocab, "top_k": args.top_k, "top_p": args.top_p}
    results = {}
    for name in ("fused", "native"):
        sampler = SamplerBackend(seed=0)
        if name == "native":
            sampler.backend = "torch"
        run = lambda: sampler.sample(logits, top_k=args.top_k, top_p=args.top_p, temperature=args.temperature)
        results[name] = report(f"sampling_{name}", shape, time_ms(run, args.warmup, args.repeat), nbytes=logits.numel() * 4.0,
                               backend=sampler.backend)
        results[name]["rows_per_sec"] = args.rows / results[name]["ms"] * 1e3
    print({"speedup_fused_over_native": round(results["native"]["ms"] / results["fused"]["ms"], 2),
           "fused_rows_per_sec": round(results["fused"]["rows_per_sec"])})


if __name__ == "__main__":
    main()
