"""Long-context GRPO step under context parallelism, followed by the trainer -> rollout weight sync.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29620 \
        benchmarks/benchmark_long_context.py                      # Llama-3-8B, G = 8 x 32 768 after a 4 096-token prompt

Every sequence (prompt + completion = 36 864 tokens) is sharded over the ranks in zig-zag chunks
(``ContextParallelGRPOTrainer``): causal attention exchanges keys / values over NVLink peer stores, all other layers work
on the local rows, the optimiser step is the fused reduce-scatter + AdamW + all-gather kernel.  After the timed steps the
bf16 weights (16 GB) go from rank 0 to every rank's window through ``NVLinkBroadcastBridge.sync`` (relay mode), which is
timed as well.  Device time with CUDA events for the steps, host wall clock around the sync collective, max over ranks.
One JSON line on rank 0.  Synthetic token ids, random-init weights.
"""

from __future__ import annotations

import argparse
import json
import os
import sys
import time

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from common import peaks  # noqa: E402,F401  (also puts the repository root on sys.path)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--group", type=int, default=8)
    ap.add_argument("--prompt-len", type=int, default=4096)
    ap.add_argument("--completion-len", type=int, default=32768)
    ap.add_argument("--layers", type=int, default=0, help="development: fewer layers than the 32 of Llama-3-8B")
    ap.add_argument("--steps", type=int, default=2)
    ap.add_argument("--warmup", type=int, default=1)
    ap.add_argument("--no-sync", action="store_true")
    args = ap.parse_args()
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)

    from rl_engine.executors.bridge import NVLinkBroadcastBridge
    from rl_engine.kernels.ops.base import check_device_errors
    from rl_engine.models.config import llama3_8b
    from rl_engine.models.grpo import synthetic_batch
    from rl_engine.models.llama import LlamaModel
    from rl_engine.parallel.long_context import ContextParallelGRPOTrainer
    from rl_engine.parallel.symmetric import SymmetricMemory

    cfg = llama3_8b()
    if args.layers:
        cfg = cfg.with_layers(args.layers)
    s = args.prompt_len + args.completion_len
    model = LlamaModel(cfg, dtype=torch.bfloat16, device=dev, seed=0, max_positions=s)
    trainer = ContextParallelGRPOTrainer(model, lr=1e-6, clip_eps=0.2, beta=0.04)
    host = synthetic_batch(cfg.vocab_size, args.prompt_len, args.group, args.completion_len, seed=77)
    batch = host.to(dev)
    # rollout-time log-probs: N(-2, 0.1) placeholders are enough for timing (no extra forward over 8 x 36 864 tokens)
    gen = torch.Generator(device=dev).manual_seed(5)
    batch.old_logps = -2.0 + 0.1 * torch.randn(batch.old_logps.shape, device=dev, generator=gen)
    batch.ref_logps = batch.old_logps.clone()
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
    step_ms = float(t)
    trainer.check()
    check_device_errors(local)
    peak_gb = torch.cuda.max_memory_allocated(dev) / 2**30
    kept = model.kept_layers()

    sync = None
    if not args.no_sync:
        nbytes = model.flat.numel() * 2 + 256 * (len(model.named_views()) + 1)
        mem = SymmetricMemory(nbytes + (1 << 20), device=dev)
        bridge = NVLinkBroadcastBridge(mem, nbytes)
        times = []
        for it in range(3):
            torch.cuda.synchronize()
            dist.barrier()
            t0 = time.perf_counter()
            manifest, tensors = bridge.sync(model.state_dict_views() if rank == 0 else None, weight_version=it + 1)
            torch.cuda.synchronize()
            tt = torch.tensor([time.perf_counter() - t0], device=dev, dtype=torch.float64)
            dist.all_reduce(tt, op=dist.ReduceOp.MAX)
            times.append(float(tt) * 1e3)
            if it < 2:
                bridge.release(manifest.update_id)
        same = torch.tensor([int(torch.equal(tensors["lm_head"], model.view("lm_head").detach()))], device=dev)
        dist.all_reduce(same, op=dist.ReduceOp.MIN)  # every rank trained the same weights: its window must equal them
        mem.check()
        size = model.flat.numel() * 2
        roof = size / (770.0 * 1e6) if world > 1 else size * 2 / (peaks()["hbm_gbs"] * 1e6)
        sync = {"ms": round(min(times[1:]), 2), "first_ms": round(times[0], 2), "gbytes": round(size / 2**30, 2),
                "tensors": len(manifest.tensors), "mode": "relay" if bridge.relay else "direct",
                "roofline_ms": round(roof, 2), "frac_of_roofline": round(roof / min(times[1:]), 3),
                "verified_on_all_ranks": bool(same.item()),
                "roofline": "the update's bytes leave the source's NVLink port once at 770 GB/s"}
    if rank == 0:
        tokens = args.group * args.completion_len
        print(json.dumps({
            "benchmark": "long_context_grpo_step", "model": cfg.name, "layers": cfg.num_layers, "world": world,
            "parallelism": f"cp{world}-zigzag + replicated weights, fused zero1 step",
            "group": args.group, "prompt_len": args.prompt_len, "completion_len": args.completion_len,
            "ms_per_step": round(step_ms, 1), "completion_tokens_per_s": round(tokens / (step_ms * 1e-3), 1),
            "sequence_tokens_per_s": round(args.group * s / (step_ms * 1e-3), 1), "steps": args.steps,
            "warmup": args.warmup, "loss": float(loss), "kept_layers": kept, "peak_allocated_gb": round(peak_gb, 1),
            "weight_sync": sync, "dtype": "bf16", "data": "synthetic",
        }), flush=True)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
