"""GRPO loss from logits (streaming log-prob kernels + fused surrogate tail) vs the PyTorch oracle,
forward + backward.  Counterpart of the reference's ``benchmarks/benchmark_grpo_loss.py``.

    python benchmarks/benchmark_grpo_loss.py --groups 2 --samples 8 --seq 512 --vocab 128256
"""

import argparse

import torch

from common import peak_gb, randn, report, time_ms


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--groups", type=int, default=2)
    ap.add_argument("--samples", type=int, default=8, help="completions per prompt")
    ap.add_argument("--seq", type=int, default=512)
    ap.add_argument("--vocab", type=int, default=128256)
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float16", "float32"])
    ap.add_argument("--beta", type=float, default=0.04)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--repeat", type=int, default=10)
    args = ap.parse_args()
    from rl_engine.kernels.ops.pytorch.loss.grpo_loss import NativeGRPOLossOp
    from rl_engine.kernels.registry import kernel_registry

    dtype = getattr(torch, args.dtype)
    b, s, v = args.groups * args.samples, args.seq, args.vocab
    pol = randn((b, s, v), dtype).requires_grad_(True)
    ref = randn((b, s, v), dtype, seed=1)
    ids = torch.randint(0, v, (b, s), device=pol.device)
    mask = torch.ones(b, s, dtype=torch.bool, device=pol.device)
    mask[:, s // 2 :] &= torch.rand(b, s - s // 2, device=pol.device) > 0.2
    old = torch.full((b, s), -5.0, device=pol.device)
    rewards = torch.randn(b, device=pol.device)
    shape = {"sequences": b, "seq": s, "vocab": v, "dtype": args.dtype, "beta": args.beta}
    nbytes = pol.numel() * pol.element_size() * 4  # policy read twice (fwd, bwd), reference once, dlogits written
    results = {}
    for name, op in (("fused", kernel_registry.get_op("grpo_loss")), ("native", NativeGRPOLossOp())):
        def run():
            pol.grad = None
            loss, _, _ = op(pol, ref, ids, old, rewards, mask, samples_per_prompt=args.samples, beta=args.beta)
            loss.backward()
            return loss
        try:
            results[name] = report(f"grpo_loss_{name}", shape, time_ms(run, args.warmup, args.repeat), nbytes=nbytes,
                                   peak_gb=round(peak_gb(run), 3), loss=round(float(run()), 6), backend=type(op).__name__)
        except Exception as exc:
            print({"benchmark": f"grpo_loss_{name}", "status": "blocked", "notes": str(exc).splitlines()[0]})
    if len(results) == 2:
        print({"speedup_fused_over_native": round(results["native"]["ms"] / results["fused"]["ms"], 2),
               "loss_abs_diff": round(abs(results["native"]["loss"] - results["fused"]["loss"]), 6)})


if __name__ == "__main__":
    main()
