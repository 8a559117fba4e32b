"""The whole RL loop on this library's own stack, in one file.

    python examples/rl_loop.py                         # CPU, tiny model: the mean reward goes from 0.5 to 1.0 in 30 iterations

Every iteration: the rollout executor samples G completions of a prompt with the native engine (and reports their
log-probs), a frozen copy of the initial policy scores them without a key/value cache (the KL reference), a toy reward
prefers even token ids, the GRPO training worker takes one optimiser step on the real model, publishes the new
weights through the weight bridge, and the rollout executor installs them before the next iteration.  The mean reward
climbs, which is the point of the demonstration: all pieces are wired to each other and the policy that generates is
the policy that was just trained.  ``--device cuda`` runs the same code with bf16 parameters and head_dim 128 (the
shape the fused attention kernels are written for); the CPU run is the one the test suite covers.

The reference has the worker contracts and a single-GPU loss example (``examples/grpo_single_gpu.py``) but no loop
that joins rollout, scoring, training and weight sync.
"""

from __future__ import annotations

import argparse
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from rl_engine.executors.bridge import make_weight_bridge  # noqa: E402
from rl_engine.executors.rollout import RolloutExecutor  # noqa: E402
from rl_engine.executors.stateless_executor import (  # noqa: E402
    StatelessForwardConfig, StatelessForwardExecutor, StatelessForwardInputs,
)
from rl_engine.executors.trainer import GRPOTrainingConfig, GRPOTrainingWorker  # noqa: E402
from rl_engine.executors.training_contract import make_rollout_result  # noqa: E402
from rl_engine.models.causal_lm import PackedCausalLM  # noqa: E402
from rl_engine.models.config import ModelConfig  # noqa: E402
from rl_engine.models.llama import LlamaModel  # noqa: E402


def parse_args(argv=None):
    p = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    p.add_argument("--device", default="cpu", choices=["cpu", "cuda"])
    p.add_argument("--iterations", type=int, default=30)
    p.add_argument("--generations", type=int, default=16, help="completions per prompt (G)")
    p.add_argument("--max-new-tokens", type=int, default=12)
    p.add_argument("--prompt-len", type=int, default=8)
    p.add_argument("--vocab", type=int, default=128)
    p.add_argument("--hidden", type=int, default=32)
    p.add_argument("--layers", type=int, default=2)
    p.add_argument("--heads", type=int, default=2)
    p.add_argument("--lr", type=float, default=3e-2)
    p.add_argument("--beta", type=float, default=0.01, help="weight of the KL term against the frozen reference")
    p.add_argument("--transport", default="local-clone", help="weight bridge transport (see make_weight_bridge)")
    p.add_argument("--seed", type=int, default=0)
    return p.parse_args(argv)


def build_model(args, seed: int) -> LlamaModel:
    on_gpu = args.device == "cuda"
    head_dim = 128 if on_gpu else 16            # the fused attention kernels are written for head_dim 128
    cfg = ModelConfig("loop-demo", args.vocab, args.hidden, args.layers, args.heads, max(1, args.heads // 2), head_dim,
                      args.hidden * 3 // 2 // 16 * 16)
    dtype = torch.bfloat16 if on_gpu else torch.float32
    return LlamaModel(cfg, dtype=dtype, device=args.device, seed=seed, max_positions=args.prompt_len + args.max_new_tokens + 8)


def reward_even_tokens(completions: torch.Tensor) -> torch.Tensor:
    """Fraction of even token ids per completion: easy to improve, impossible to satisfy by accident."""
    return (completions % 2 == 0).float().mean(dim=1)


def main(argv=None) -> dict:
    args = parse_args(argv)
    torch.manual_seed(args.seed)
    policy, rollout_copy, reference = build_model(args, 1), build_model(args, 2), build_model(args, 1)
    bridge = make_weight_bridge(args.transport, source_worker="trainer")
    worker = GRPOTrainingWorker(
        GRPOTrainingConfig(lr=args.lr, beta=args.beta, device=args.device, dtype=policy.flat.dtype, vocab_size=args.vocab),
        model=policy, weight_bridge=bridge)
    rollout = RolloutExecutor({"num_generations": args.generations}, weight_bridge=bridge, policy_model=rollout_copy)
    scorer = StatelessForwardExecutor(PackedCausalLM(reference),
                                      StatelessForwardConfig(mode="reference", attention_backend="model_default"))
    rollout.update_weights(worker.publish_weights(0))          # version 0: the rollout side starts from the trainer's weights

    prompt = torch.arange(3, 3 + args.prompt_len, device=args.device) % args.vocab
    g, p_len = args.generations, args.prompt_len
    history = []
    for iteration in range(args.iterations):
        out = rollout.execute_rollout(prompt, num_generations=g, max_new_tokens=args.max_new_tokens, temperature=1.0,
                                      top_k=0, top_p=1.0)
        completions = out["completion_ids"]
        rows = torch.cat([prompt.expand(g, -1), completions], dim=1)
        on_completion = torch.zeros_like(rows, dtype=torch.bool)
        on_completion[:, p_len:] = True
        scored = scorer.score(StatelessForwardInputs(rows, torch.ones_like(rows, dtype=torch.bool), on_completion))
        rewards = reward_even_tokens(completions)
        payload = {"prompt_ids": prompt, "completion_ids": completions, "rollout_logps": out["rollout_logps"],
                   "reference_logps": scored.reference_logps[:, p_len:], "rewards": rewards}
        result = worker.train(make_rollout_result(iteration=iteration, weight_version=out["weight_version"], payload=payload))
        rollout.update_weights(worker.publish_weights(result.published_weight_version))
        history.append({"iteration": iteration, "weight_version": rollout.active_weight_version,
                        "mean_reward": round(float(rewards.mean()), 4), "loss": round(float(result.metrics["loss"]), 6)})
        print(json.dumps(history[-1]), flush=True)
    first = sum(h["mean_reward"] for h in history[:3]) / max(1, len(history[:3]))
    last = sum(h["mean_reward"] for h in history[-3:]) / max(1, len(history[-3:]))
    summary = {"mean_reward_first3": round(first, 4), "mean_reward_last3": round(last, 4),
               "final_weight_version": rollout.active_weight_version, "training_backend": result.metrics["training_backend"]}
    print(json.dumps(summary), flush=True)
    rollout.release_weights()                                  # give the last update's segments back to the transport
    return summary


if __name__ == "__main__":
    main()
