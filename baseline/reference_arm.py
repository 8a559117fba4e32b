"""Reference arm of the headline benchmark: the UNMODIFIED reference package, nothing of this repo.

The reference (installed under ``baseline/_ref``) ships operators and loop contracts but no model,
so the step is assembled the way a user of the reference would: a Hugging Face ``LlamaForCausalLM``
(random-init bf16 from the Llama-3-8B config) provides hidden states, and everything RL-specific
goes through the reference's public API and stock dispatch:

* ``kernel_registry.get_op("linear_logp")`` for the selected-token log-probs (its Triton kernel
  where Triton is importable, else its PyTorch op -- whatever its registry picks on this GPU),
* ``kernel_registry.get_op("grpo_loss").group_advantages`` for the group normalisation,
* ``rl_engine.testing`` helpers for ratio / clip / KL / masked mean, exactly as the reference's own
  trainer composes them (``rl_engine/executors/deepspeed_trainer.py:152-169``),
* ``torch.optim.AdamW`` for the update (the reference delegates optimisation to DeepSpeed, which is
  not installed here) and, for N > 1, an NCCL all-reduce (average) of the gradients (its data
  parallelism is DeepSpeed's).

The reference has no prefix sharing in training, so every completion is a full ``prompt +
completion`` sequence (G x 1536 tokens per step), processed in micro-batches with gradient
checkpointing.  Same metric, same counting (completion tokens per second), same JSON line as
``bench.py`` with ``"impl": "reference"``.
"""

from __future__ import annotations

import argparse
import json
import os
import sys
import time

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path = [p for p in sys.path if os.path.abspath(p or ".") != os.path.dirname(HERE)]
sys.path.insert(0, os.path.join(HERE, "_ref"))

PROMPT_LEN, GROUP, COMPLETION_LEN = 1024, 256, 512
MICRO_BATCH = 8


def unavailable(reason: str) -> None:
    if int(os.environ.get("RANK", "0")) == 0:
        print(json.dumps({"impl": "reference", "unavailable": reason.replace("\n", " ")[:300]}), flush=True)
    sys.exit(0)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--dev-layers", type=int, default=0)
    ap.add_argument("--dev-group", type=int, default=0)
    args = ap.parse_args()

    try:
        import torch
        import torch.distributed as dist
        from transformers import LlamaConfig, LlamaForCausalLM

        import rl_engine  # the reference's package

        if "baseline" not in os.path.abspath(rl_engine.__file__):
            unavailable("import of rl_engine did not resolve to baseline/_ref")
        from rl_engine.kernels.registry import kernel_registry
        from rl_engine.testing import compute_policy_ratio, compute_reference_kl, masked_mean
    except Exception as exc:  # noqa: BLE001
        unavailable(f"reference import failed: {type(exc).__name__}: {exc}")

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)

    group = args.dev_group or GROUP
    local_group = group // world
    layers = args.dev_layers or 32
    try:
        import flash_attn  # noqa: F401

        attn_impl = "flash_attention_2"
    except Exception:  # noqa: BLE001
        attn_impl = "sdpa"
    config = LlamaConfig(
        vocab_size=128256, hidden_size=4096, intermediate_size=14336, num_hidden_layers=layers, num_attention_heads=32,
        num_key_value_heads=8, max_position_embeddings=8192, rms_norm_eps=1e-5, rope_theta=500000.0,
        tie_word_embeddings=False, attn_implementation=attn_impl, use_cache=False,
    )
    torch.manual_seed(0)
    with torch.device(device):
        model = LlamaForCausalLM(config).to(torch.bfloat16)
    model.gradient_checkpointing_enable()
    model.config.use_cache = False
    model.train()
    optimizer = torch.optim.AdamW(model.parameters(), lr=1e-6, betas=(0.9, 0.95), weight_decay=0.0, fused=True)
    linear_logp = kernel_registry.get_op("linear_logp")
    grpo = kernel_registry.get_op("grpo_loss")

    gen = torch.Generator().manual_seed(1234)
    prompt = torch.randint(0, 128256, (PROMPT_LEN,), generator=gen)
    completions = torch.randint(0, 128256, (group, COMPLETION_LEN), generator=gen)
    rewards = torch.randn(group, generator=gen)
    sl = slice(rank * local_group, (rank + 1) * local_group)
    host_ids = torch.cat([prompt.expand(local_group, -1), completions[sl]], dim=1).contiguous().pin_memory()
    host_rewards = rewards.pin_memory()
    mask_host = torch.ones(local_group, COMPLETION_LEN, dtype=torch.bool).pin_memory()

    def completion_logps(ids):
        # hidden state at position t predicts token t + 1
        base = model.model(input_ids=ids, use_cache=False).last_hidden_state
        hidden = base[:, PROMPT_LEN - 1 : PROMPT_LEN + COMPLETION_LEN - 1]
        targets = ids[:, PROMPT_LEN:]
        return linear_logp(hidden, model.lm_head.weight, targets, None)

    def step(ids_host, rewards_host, mask_h, old, ref):
        ids = ids_host.to(device, non_blocking=True)
        rew = rewards_host.to(device, non_blocking=True)
        mask = mask_h.to(device, non_blocking=True)
        optimizer.zero_grad(set_to_none=True)
        adv = grpo.group_advantages(rew.float(), samples_per_prompt=group)[sl]
        total = torch.zeros((), device=device)
        n_micro = (local_group + MICRO_BATCH - 1) // MICRO_BATCH
        for i in range(n_micro):
            rows = slice(i * MICRO_BATCH, min((i + 1) * MICRO_BATCH, local_group))
            cur = completion_logps(ids[rows])
            ratio = compute_policy_ratio(cur, old[rows], mask[rows])
            a = adv[rows].float()[:, None]
            policy = -torch.minimum(ratio * a, torch.clamp(ratio, 0.8, 1.2) * a)
            kl = compute_reference_kl(cur, ref[rows], mask[rows])
            loss = masked_mean(policy + 0.04 * kl, mask[rows]) / n_micro
            loss.backward()
            total += loss.detach()
        if world > 1:
            for p in model.parameters():
                if p.grad is not None:
                    dist.all_reduce(p.grad, op=dist.ReduceOp.AVG)
        optimizer.step()
        return total

    try:
        with torch.no_grad():
            cur0 = torch.cat([
                completion_logps(host_ids[i : i + MICRO_BATCH].to(device)).float()
                for i in range(0, local_group, MICRO_BATCH)
            ])
        noise = torch.Generator(device=device).manual_seed(99 + rank)
        old = cur0 + 0.01 * torch.randn(cur0.shape, device=device, generator=noise)
        ref = cur0 + 0.01 * torch.randn(cur0.shape, device=device, generator=noise)

        def barrier():
            if world > 1:
                dist.barrier()
            torch.cuda.synchronize()

        for _ in range(args.warmup):
            step(host_ids, host_rewards, mask_host, old, ref)
        barrier()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0 = time.perf_counter()
        start.record()
        last = None
        for _ in range(args.steps):
            last = float(step(host_ids, host_rewards, mask_host, old, ref).item())
        stop.record()
        barrier()
        wall = time.perf_counter() - t0
        ms = start.elapsed_time(stop)
    except Exception as exc:  # noqa: BLE001
        unavailable(f"reference step failed: {type(exc).__name__}: {exc}")

    if world > 1:
        t = torch.tensor([ms, wall], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, wall = float(t[0]), float(t[1])
    tokens = group * COMPLETION_LEN
    if rank == 0:
        print(json.dumps({
            "metric": "grpo_step_tokens_per_sec", "value": round(tokens * args.steps / (ms / 1e3), 1), "unit": "tokens/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms / args.steps, 3),
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "impl": "reference",
            "config": {
                "model": "llama3-8b", "layers": layers, "global_batch": group, "seq_len": PROMPT_LEN + COMPLETION_LEN,
                "parallelism": "single" if world == 1 else f"dp{world}-nccl-allreduce",
                "attention": attn_impl, "linear_logp_backend": type(linear_logp).__name__, "micro_batch": MICRO_BATCH,
                "tokens_counted": "completion tokens (G x 512) per step",
                "dev_overrides": bool(args.dev_layers or args.dev_group),
            },
            "e2e": {"value": round(tokens * args.steps / wall, 1), "unit": "tokens/s",
                    "h2d_bytes_per_step": host_ids.numel() * 8 + host_rewards.numel() * 4 + mask_host.numel(),
                    "d2h_bytes_per_step": 4, "last_loss": last},
        }), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
