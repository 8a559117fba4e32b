"""Fused linear -> selected log-prob vs the materialise-logits PyTorch path.

Counterpart of the reference's ``benchmarks/benchmark_linear_logp.py`` (shapes ``--tokens/--hidden/--vocab``,
forward and forward+backward, peak memory of each path).

    python benchmarks/benchmark_linear_logp.py --tokens 8192 --hidden 4096 --vocab 128256 --backward
"""

import argparse

import torch

from common import peak_gb, randn, report, time_ms


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=8192)
    ap.add_argument("--hidden", type=int, default=4096)
    ap.add_argument("--vocab", type=int, default=128256)
    ap.add_argument("--backward", action="store_true")
    ap.add_argument("--skip-native", action="store_true")
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--repeat", type=int, default=10)
    args = ap.parse_args()
    from rl_engine.kernels.ops.pytorch.loss.linear_logp import NativeLinearLogpOp
    from rl_engine.kernels.registry import kernel_registry

    n, d, v = args.tokens, args.hidden, args.vocab
    h = randn((n, d)).requires_grad_(args.backward)
    w = randn((v, d), scale=0.02, seed=1).requires_grad_(args.backward)
    t = torch.randint(0, v, (n,), device=h.device)
    shape = {"tokens": n, "hidden": d, "vocab": v, "backward": args.backward}
    flops = (8.0 if args.backward else 2.0) * n * d * v  # backward = recompute + two gradient GEMMs
    paths = [("fused", kernel_registry.get_op("linear_logp"))] + ([] if args.skip_native else [("native", NativeLinearLogpOp())])
    results = {}
    for name, op in paths:
        def run():
            if args.backward:
                h.grad = w.grad = None
                op(h, w, t).sum().backward()
            else:
                with torch.no_grad():
                    op(h, w, t)
        try:
            timing = time_ms(run, args.warmup, args.repeat)
            results[name] = report(f"linear_logp_{name}", shape, timing, flops=flops, peak_gb=round(peak_gb(run), 3),
                                   backend=type(op).__name__)
        except Exception as exc:  # e.g. the native path running out of memory on [tokens, vocab] logits
            print({"benchmark": f"linear_logp_{name}", "status": "blocked", "notes": str(exc).splitlines()[0]})
            torch.cuda.empty_cache() if torch.cuda.is_available() else None
    if len(results) == 2:
        print({"speedup_fused_over_native": round(results["native"]["ms"] / results["fused"]["ms"], 2)})


if __name__ == "__main__":
    main()
