"""Fused policy/reference ratio + k3-KL streaming kernel vs the PyTorch oracle, forward and backward.

Counterpart of the reference's ``benchmarks/benchmark_ratio_kl.py``.

    python benchmarks/benchmark_ratio_kl.py --batch 8 --seq 512 --vocab 128256 --backward
"""

import argparse

import torch

from common import peak_gb, randn, report, time_ms


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--seq", type=int, default=512)
    ap.add_argument("--vocab", type=int, default=128256)
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float16", "float32"])
    ap.add_argument("--backward", action="store_true")
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--repeat", type=int, default=10)
    args = ap.parse_args()
    from rl_engine.kernels.ops.pytorch.loss.ratio_kl import NativeRatioKLOp
    from rl_engine.kernels.registry import kernel_registry

    dtype = getattr(torch, args.dtype)
    b, s, v = args.batch, args.seq, args.vocab
    pol = randn((b, s, v), dtype).requires_grad_(args.backward)
    ref = randn((b, s, v), dtype, seed=1)
    ids = torch.randint(0, v, (b, s), device=pol.device)
    mask = torch.ones(b, s, dtype=torch.bool, device=pol.device)
    old = torch.full((b, s), -5.0, device=pol.device)
    nbytes = pol.numel() * pol.element_size() * (3 if args.backward else 2)  # read both (+ write dlogits)
    shape = {"batch": b, "seq": s, "vocab": v, "dtype": args.dtype, "backward": args.backward}
    results = {}
    for name, op in (("fused", kernel_registry.get_op("ratio_kl")), ("native", NativeRatioKLOp())):
        def run():
            if args.backward:
                pol.grad = None
                ratio, kl = op(pol, ref, ids, mask, old)
                (ratio.sum() + kl.sum()).backward()
            else:
                with torch.no_grad():
                    op(pol, ref, ids, mask, old)
        try:
            results[name] = report(f"ratio_kl_{name}", shape, time_ms(run, args.warmup, args.repeat), nbytes=nbytes,
                                   peak_gb=round(peak_gb(run), 3), backend=type(op).__name__)
        except Exception as exc:
            print({"benchmark": f"ratio_kl_{name}", "status": "blocked", "notes": str(exc).splitlines()[0]})
    if len(results) == 2:
        print({"speedup_fused_over_native": round(results["native"]["ms"] / results["fused"]["ms"], 2)})


if __name__ == "__main__":
    main()
