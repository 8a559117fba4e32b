"""Single-device GRPO training loop on a tiny policy, exercising the registry's operators end to end.

Each step: policy logits -> selected log-probs (registry ``logp`` op, differentiable on the sm_100a path)
-> group-relative advantages -> clipped surrogate + k3 KL (registry ``grpo_loss`` op, logp-space entry
point) -> backward -> AdamW.  The kernel log-probs are compared with the fp32 PyTorch oracle every step
and the drift is printed.

Counterpart of the reference's ``examples/grpo_single_gpu.py:1-296`` (same flags).  The reference has to
train on its oracle log-probs because its fused op has no autograd; here the fused path carries gradients,
so ``train_logp_source`` is the kernel whenever a GPU is present.

    python examples/grpo_single_gpu.py --device cpu --steps 4
    python examples/grpo_single_gpu.py --device cuda --vocab-size 32768 --hidden-dim 512 --require-fused-logp
"""

from __future__ import annotations

import argparse
import os
import sys
from dataclasses import dataclass
from typing import List

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from rl_engine.kernels.registry import kernel_registry  # noqa: E402
from rl_engine.testing import (  # noqa: E402
    active_token_count,
    make_synthetic_rl_kernel_batch,
    selected_logprobs_reference,
    summarize_kernel_drift,
)


class TinyPolicy(torch.nn.Module):
    def __init__(self, vocab_size: int, hidden_dim: int) -> None:
        super().__init__()
        self.embedding = torch.nn.Embedding(vocab_size, hidden_dim)
        self.proj = torch.nn.Linear(hidden_dim, vocab_size)

    def forward(self, token_ids: torch.Tensor) -> torch.Tensor:
        return self.proj(self.embedding(token_ids))


@dataclass
class StepMetrics:
    step: int
    loss: float
    policy_loss: float
    kl: float
    active_tokens: int
    logp_backend: str
    train_logp_source: str
    kernel_max_abs_error: float


def parse_args(argv=None) -> argparse.Namespace:
    p = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    p.add_argument("--device", choices=("auto", "cuda", "cpu"), default="auto")
    p.add_argument("--steps", type=int, default=4)
    p.add_argument("--num-prompts", type=int, default=2)
    p.add_argument("--samples-per-prompt", type=int, default=4)
    p.add_argument("--prompt-len", type=int, default=8)
    p.add_argument("--completion-len", type=int, default=16)
    p.add_argument("--vocab-size", type=int, default=128)
    p.add_argument("--hidden-dim", type=int, default=64)
    p.add_argument("--valid-density", type=float, default=0.9)
    p.add_argument("--lr", type=float, default=1e-2)
    p.add_argument("--clip-eps", type=float, default=0.2)
    p.add_argument("--beta", type=float, default=0.01)
    p.add_argument("--seed", type=int, default=1234)
    p.add_argument("--require-fused-logp", action="store_true",
                   help="fail unless the registry dispatches the log-prob op to the fused sm_100a backend")
    return p.parse_args(argv)


def select_device(requested: str) -> torch.device:
    if requested == "cuda" and not torch.cuda.is_available():
        raise RuntimeError("--device cuda was requested but no CUDA device is available")
    if requested == "auto":
        requested = "cuda" if torch.cuda.is_available() else "cpu"
    return torch.device(requested)


def selected_logps_with_op(logp_op, logits, token_ids, mask):
    """Differentiable selected log-probs through the registry op where it supports autograd."""
    if logits.is_cuda and type(logp_op).__name__.endswith("SM100Op"):
        from rl_engine.kernels.ops.sm100.logp_autograd import selected_logprobs

        return selected_logprobs(logits, token_ids, mask)
    out = logp_op.apply_fp32(logits, token_ids)
    return torch.where(mask, out.reshape(mask.shape), torch.zeros_like(out.reshape(mask.shape)))


def run_training(args: argparse.Namespace) -> List[StepMetrics]:
    device = select_device(args.device)
    torch.manual_seed(args.seed)
    logp_op = kernel_registry.get_op("logp")
    loss_op = kernel_registry.get_op("grpo_loss")
    backend_name = type(logp_op).__name__
    fused = backend_name.endswith("SM100Op") and device.type == "cuda"
    if args.require_fused_logp and not fused:
        raise RuntimeError(f"--require-fused-logp: the registry dispatched {backend_name} on {device.type}, not the fused backend")

    policy = TinyPolicy(args.vocab_size, args.hidden_dim).to(device)
    optimizer = torch.optim.AdamW(policy.parameters(), lr=args.lr)
    batch = make_synthetic_rl_kernel_batch(
        num_prompts=args.num_prompts, samples_per_prompt=args.samples_per_prompt, prompt_len=args.prompt_len,
        completion_len=args.completion_len, vocab_size=args.vocab_size, valid_density=args.valid_density,
        device=device, seed=args.seed,
    )
    with torch.no_grad():
        start_logits = policy(batch.token_ids)
        old_logps = selected_logprobs_reference(start_logits, batch.token_ids, mask=batch.completion_mask, output_dtype=torch.float32)
        ref_logps = old_logps.clone()
    advantages = loss_op.group_advantages(batch.rewards, samples_per_prompt=args.samples_per_prompt)

    metrics: List[StepMetrics] = []
    for step in range(args.steps):
        optimizer.zero_grad(set_to_none=True)
        logits = policy(batch.token_ids)
        reference_logps = selected_logprobs_reference(logits, batch.token_ids, mask=batch.completion_mask, output_dtype=torch.float32)
        kernel_logps = selected_logps_with_op(logp_op, logits, batch.token_ids, batch.completion_mask)
        drift = summarize_kernel_drift(kernel_logps.detach(), reference_logps.detach(), batch.completion_mask)
        if kernel_logps.requires_grad:
            train_logps, source = kernel_logps, backend_name
        else:
            train_logps, source = reference_logps, "autograd_reference"
        loss, policy_loss, kl = loss_op.apply_from_logps(
            train_logps, ref_logps, old_logps, advantages, batch.completion_mask, clip_eps=args.clip_eps, beta=args.beta
        )
        if not torch.isfinite(loss):
            raise RuntimeError(f"non-finite loss at step {step}: {loss.item()}")
        loss.backward()
        optimizer.step()
        m = StepMetrics(step, float(loss.detach()), float(policy_loss.detach()), float(kl.detach()),
                        int(active_token_count(batch.completion_mask).item()), backend_name, source,
                        float(drift["max_abs_error"]))
        metrics.append(m)
        print(f"step={m.step} loss={m.loss:.6f} policy_loss={m.policy_loss:.6f} kl={m.kl:.6f} "
              f"train_logp_source={m.train_logp_source} kernel_max_abs_error={m.kernel_max_abs_error:.6e}")
    print(f"completed grpo_single_gpu steps={args.steps} device={device.type} backend={backend_name}")
    return metrics


def main() -> None:
    run_training(parse_args())


if __name__ == "__main__":
    main()
