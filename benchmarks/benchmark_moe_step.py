"""GRPO step of a Qwen3-30B-A3B-shaped mixture-of-experts model under data + expert parallelism.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29630 \
        benchmarks/benchmark_moe_step.py            # 48 layers, 128 experts top-8, G = 64 completions of 1024 tokens

Every rank trains on ``G / W`` completions of the group (data parallel for attention, norms, router, embedding and LM
head, whose gradients go through the fused reduce-scatter + AdamW + all-gather kernel) and owns ``128 / W`` experts of
every layer; MoE layers send each token to the ranks that own its eight experts and fetch the results back through peer
stores / loads in symmetric memory (``rl_engine.parallel.expert_parallel``).  The step includes the optimiser.  Device time
with CUDA events, max over ranks, one JSON line on rank 0.  Random-init bf16 weights, uniform token ids; the router sees
the model's own hidden states (the benchmark configuration asks for N(0,1) router logits: with random weights and
normalised inputs the logits are near-Gaussian, and the load per expert is reported).
"""

from __future__ import annotations

import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from common import peaks  # noqa: E402,F401  (also puts the repository root on sys.path)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--group", type=int, default=64)
    ap.add_argument("--prompt-len", type=int, default=128)
    ap.add_argument("--completion-len", type=int, default=1024)
    ap.add_argument("--layers", type=int, default=0, help="development: fewer layers than 48")
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=2)
    args = ap.parse_args()
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)

    from rl_engine.kernels.ops.base import check_device_errors
    from rl_engine.models.config import qwen3_30b_a3b
    from rl_engine.models.grpo import GRPOBatch, synthetic_batch
    from rl_engine.models.llama import LlamaModel
    from rl_engine.parallel.expert_parallel import expert_parallel_trainer

    cfg = qwen3_30b_a3b()
    if args.layers:
        cfg = cfg.with_layers(args.layers)
    if args.group % world:
        raise SystemExit("the group must divide over the ranks")
    per_rank = args.group // world
    model = LlamaModel(cfg, dtype=torch.bfloat16, device=dev, seed=0, max_positions=args.prompt_len + args.completion_len,
                       expert_shard=(rank, world))
    tokens_per_pass = args.prompt_len + per_rank * args.completion_len
    trainer = expert_parallel_trainer(model, max_tokens=tokens_per_pass, lr=1e-6, clip_eps=0.2, beta=0.04, micro_group=None)
    full = synthetic_batch(cfg.vocab_size, args.prompt_len, args.group, args.completion_len, seed=31).to(dev)
    sl = slice(rank * per_rank, (rank + 1) * per_rank)
    trainer.set_group_slice(sl)
    gen = torch.Generator(device=dev).manual_seed(7 + rank)
    shape = (per_rank, args.completion_len)
    old = -2.0 + 0.1 * torch.randn(shape, device=dev, generator=gen)
    batch = GRPOBatch(full.prompt_ids, full.completion_ids[sl].contiguous(), full.rewards, old, old.clone(),
                      full.completion_mask[sl].contiguous())
    for _ in range(args.warmup):
        trainer.step_device(batch)
    torch.cuda.synchronize()
    dist.barrier()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    loss = None
    for _ in range(args.steps):
        loss = trainer.step_device(batch)
    b.record()
    torch.cuda.synchronize()
    t = torch.tensor([a.elapsed_time(b) / args.steps], device=dev, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    trainer.check()
    trainer.expert_context.mem.check()
    check_device_errors(local)
    mean_loss = loss.float().reshape(1).clone()
    dist.all_reduce(mean_loss, op=dist.ReduceOp.AVG)
    peak = torch.tensor([torch.cuda.max_memory_allocated(dev) / 2**30], device=dev)
    dist.all_reduce(peak, op=dist.ReduceOp.MAX)
    if rank == 0:
        ms = float(t)
        tokens = args.group * args.completion_len
        active = cfg.num_layers * (cfg.hidden_size * (cfg.q_dim + 2 * cfg.kv_dim) + cfg.q_dim * cfg.hidden_size
                                   + cfg.experts_per_token * 3 * cfg.hidden_size * cfg.moe_ffn_size
                                   + cfg.hidden_size * cfg.num_experts) + cfg.vocab_size * cfg.hidden_size
        flops = 6.0 * active * (tokens + world * args.prompt_len)
        print(json.dumps({
            "benchmark": "moe_grpo_step", "model": cfg.name, "layers": cfg.num_layers, "world": world,
            "parallelism": f"dp{world} + ep{world} ({cfg.num_experts // world} experts per rank), fused zero1 step for replicated parameters",
            "experts": cfg.num_experts, "top_k": cfg.experts_per_token, "group": args.group, "prompt_len": args.prompt_len,
            "completion_len": args.completion_len, "ms_per_step": round(ms, 1),
            "completion_tokens_per_s": round(tokens / (ms * 1e-3), 1),
            "model_tflops_per_gpu": round(flops / (ms * 1e-3) / 1e12 / world, 1),
            "flops_counted": "6 x active parameters x tokens (recomputation of the MoE layers not counted)",
            "params_total_b": round(cfg.param_count() / 1e9, 2), "params_per_rank_b": round(model.flat.numel() / 1e9, 2),
            "loss": float(mean_loss), "peak_allocated_gb_max_rank": round(float(peak), 1), "steps": args.steps,
            "warmup": args.warmup, "dtype": "bf16", "data": "synthetic",
        }), flush=True)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
