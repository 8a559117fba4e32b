"""The logp-space GRPO / PPO-clip tail alone (group advantages + clipped surrogate + k3 KL, forward and
backward) on ``[sequences, seq]`` log-probs.  Counterpart of the reference's ``benchmarks/benchmark_grpo_op.py``.

    python benchmarks/benchmark_grpo_op.py --sequences 4096 --seq 512
"""

import argparse

import torch

from common import report, time_ms


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--sequences", type=int, default=4096)
    ap.add_argument("--samples", type=int, default=16)
    ap.add_argument("--seq", type=int, default=512)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--repeat", type=int, default=20)
    args = ap.parse_args()
    from rl_engine.kernels.ops.pytorch.loss.grpo_loss import NativeGRPOLossOp
    from rl_engine.kernels.registry import kernel_registry

    dev = "cuda" if torch.cuda.is_available() else "cpu"
    b, s = args.sequences, args.seq
    lp = (-torch.rand(b, s, device=dev) * 3).requires_grad_(True)
    ref = -torch.rand(b, s, device=dev) * 3
    old = lp.detach() + 0.1 * torch.randn(b, s, device=dev)
    mask = torch.rand(b, s, device=dev) > 0.1
    rewards = torch.randn(b, device=dev)
    shape = {"sequences": b, "seq": s, "samples_per_prompt": args.samples}
    for name, op in (("fused", kernel_registry.get_op("grpo_loss")), ("native", NativeGRPOLossOp())):
        def run():
            lp.grad = None
            adv = op.group_advantages(rewards, samples_per_prompt=args.samples)
            loss, _, _ = op.apply_from_logps(lp, ref, old, adv, mask, clip_eps=0.2, beta=0.04)
            loss.backward()
        report(f"grpo_op_{name}", shape, time_ms(run, args.warmup, args.repeat), nbytes=b * s * 4.0 * 5, backend=type(op).__name__)


if __name__ == "__main__":
    main()
