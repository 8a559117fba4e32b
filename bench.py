"""Headline benchmark: GRPO optimisation-step throughput on Llama-3-8B (random-init bf16).

    python bench.py --gpus 1 --steps 3 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port P bench.py --gpus N --steps K --warmup W
    python bench.py --impl reference ...      # the unmodified reference through its own API

One step = forward of the policy over one prompt group (G = 256 completions of 512 tokens sharing a
1024-token prompt), fused linear->log-prob over the 128 256-entry vocabulary, the GRPO clipped
surrogate + KL loss with group-normalised N(0,1) rewards, backward through everything, and an AdamW
update of all 8 B parameters.  Throughput counts completion tokens (G x 512) per second for the
whole job.  N > 1 splits the G completions over N data-parallel ranks (total work fixed: strong
scaling) and replaces the optimizer by the fused reduce-scatter + AdamW + all-gather kernel that
works over NVLink peer memory.

Timing: W untimed steps, then K steps between CUDA events with a barrier + synchronize on both
sides, max over ranks.  Model state (16 GB of weights alone) is far larger than L2, so no explicit
L2 flush is needed between steps.  SM clocks and throttle reasons are sampled through NVML during
the timed region.  The ``e2e`` entry times the same K steps through the public
``GRPOTrainer.step(host_batch)`` call, which copies the step's inputs from pinned host memory and
reads the loss back every step.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))

PROMPT_LEN, GROUP, COMPLETION_LEN = 1024, 256, 512
METRIC = "grpo_step_tokens_per_sec"


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    # dp: completions split over the ranks, fused ZeRO-1 step (default, fastest for an 8B model on 180 GB GPUs);
    # tp: tensor + sequence parallel layers and vocabulary-parallel LM head, every rank sees the whole group
    ap.add_argument("--parallelism", choices=["dp", "tp"], default="dp")
    # development switches; any use marks the run as not comparable
    ap.add_argument("--dev-layers", type=int, default=0)
    ap.add_argument("--dev-group", type=int, default=0)
    ap.add_argument("--dev-micro-group", type=int, default=0,
                    help="development only: fix the completions per forward/backward pass instead of planning them")
    return ap.parse_args()


class ClockSampler:
    """Samples SM clock and throttle reasons of this process's GPU every 200 ms through NVML."""

    def __init__(self, index: int) -> None:
        self.samples, self.reasons, self.max_mhz = [], set(), 0
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml

            pynvml.nvmlInit()
            self._nv = pynvml
            self._h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self._nv = None

    def _run(self):
        nv = self._nv
        names = {
            nv.nvmlClocksThrottleReasonHwSlowdown: "hw_slowdown",
            nv.nvmlClocksThrottleReasonHwThermalSlowdown: "hw_thermal_slowdown",
            nv.nvmlClocksThrottleReasonSwThermalSlowdown: "sw_thermal_slowdown",
            nv.nvmlClocksThrottleReasonSwPowerCap: "sw_power_cap",
            nv.nvmlClocksThrottleReasonHwPowerBrakeSlowdown: "hw_power_brake",
        }
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self._h, nv.NVML_CLOCK_SM))
                mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self._h)
                self.reasons.update(n for bit, n in names.items() if mask & bit)
            except Exception:
                pass
            self._stop.wait(0.2)

    def __enter__(self):
        if self._nv is not None:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2)

    def summary(self):
        return {
            "sm_mhz": statistics.median(self.samples) if self.samples else None,
            "sm_max_mhz": self.max_mhz or None,
            "reasons": sorted(self.reasons),
        }


def physical_gpu_index(local_rank: int) -> int:
    visible = os.environ.get("CUDA_VISIBLE_DEVICES")
    if visible:
        ids = [v for v in visible.split(",") if v.strip()]
        try:
            return int(ids[local_rank])
        except (ValueError, IndexError):
            return local_rank
    return local_rank


def run_reference(args) -> None:
    """Re-exec into the reference arm so that the reference's own ``rl_engine`` package is imported."""
    script = os.path.join(ROOT, "baseline", "reference_arm.py")
    ref_pkg = os.path.join(ROOT, "baseline", "_ref", "rl_engine")
    if not os.path.isdir(ref_pkg):
        if int(os.environ.get("RANK", "0")) == 0:
            print(json.dumps({"impl": "reference", "unavailable": "reference is not installed under baseline/_ref"}))
        return
    argv = [sys.executable, script, "--gpus", str(args.gpus), "--steps", str(args.steps), "--warmup", str(args.warmup)]
    if args.dev_layers:
        argv += ["--dev-layers", str(args.dev_layers)]
    if args.dev_group:
        argv += ["--dev-group", str(args.dev_group)]
    env = dict(os.environ)
    env.pop("PYTHONPATH", None)
    os.execve(sys.executable, argv, env)


def main() -> None:
    args = parse_args()
    if args.impl == "reference":
        run_reference(args)
        return

    sys.path.insert(0, ROOT)
    import torch
    import torch.distributed as dist

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.gpus != world:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}; launch with torch.distributed.run for N > 1")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)

    from rl_engine.kernels.ops.base import check_device_errors, require_ext
    from rl_engine.models.config import llama3_8b
    from rl_engine.models.grpo import GRPOTrainer, synthetic_batch
    from rl_engine.models.llama import LlamaModel

    ext = require_ext()
    cfg = llama3_8b()
    group = args.dev_group or GROUP
    if args.dev_layers:
        cfg = cfg.with_layers(args.dev_layers)
    if group % world:
        raise SystemExit("the group size must be divisible by the number of GPUs")
    tensor_parallel = args.parallelism == "tp" and world > 1
    local_group = group if tensor_parallel else group // world

    micro = args.dev_micro_group or "auto"
    model = LlamaModel(cfg, dtype=torch.bfloat16, device=device, seed=0, max_positions=PROMPT_LEN + COMPLETION_LEN)
    if tensor_parallel:
        from rl_engine.parallel.tp_linear import TensorParallelLinears
        from rl_engine.parallel.tp_model import TensorParallelGRPOTrainer, TensorParallelLlama

        tp_model = TensorParallelLlama(model, TensorParallelLinears(group=dist.group.WORLD, device=device))
        del model  # only this rank's shards stay resident
        torch.cuda.empty_cache()
        trainer = TensorParallelGRPOTrainer(tp_model, lr=1e-6, clip_eps=0.2, beta=0.04)
        parallelism = f"tp{world}-sequence-parallel-fused"
    elif world > 1:
        from rl_engine.parallel.data_parallel import ShardedGRPOTrainer

        trainer = ShardedGRPOTrainer(model, lr=1e-6, clip_eps=0.2, beta=0.04, micro_group=micro)
        parallelism = f"dp{world}-zero1-fused"
    else:
        trainer = GRPOTrainer(model, lr=1e-6, clip_eps=0.2, beta=0.04, micro_group=micro)
        parallelism = "single"

    # the same global batch on every run; each rank takes its slice of the G completions
    full = synthetic_batch(cfg.vocab_size, PROMPT_LEN, group, COMPLETION_LEN, seed=1234)
    sl = slice(0, group) if tensor_parallel else slice(rank * local_group, (rank + 1) * local_group)
    host = type(full)(
        prompt_ids=full.prompt_ids, completion_ids=full.completion_ids[sl].contiguous(), rewards=full.rewards,
        old_logps=full.old_logps[sl].contiguous(), ref_logps=full.ref_logps[sl].contiguous(),
        completion_mask=full.completion_mask[sl].contiguous(),
    )
    if world > 1 and not tensor_parallel:
        trainer.set_group_slice(sl)
    # old / reference log-probs = current log-probs + N(0, 0.01), as a rollout would have produced them
    with torch.no_grad():
        cur = trainer.policy_logps(host.to(device)).float().cpu()
    gen = torch.Generator().manual_seed(99 + (0 if tensor_parallel else rank))
    host.old_logps = cur + 0.01 * torch.randn(cur.shape, generator=gen)
    host.ref_logps = cur + 0.01 * torch.randn(cur.shape, generator=gen)
    host = host.pin()
    dev_batch = host.to(device)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        trainer.step_device(dev_batch)
    barrier()

    sampler = ClockSampler(physical_gpu_index(local_rank))
    launches0 = ext.launch_count()
    with sampler:
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        start.record()
        for _ in range(args.steps):
            trainer.step_device(dev_batch)
        stop.record()
        barrier()
    launches = ext.launch_count() - launches0
    ms = start.elapsed_time(stop)

    # end to end through the public API: pinned host inputs in, loss value out, every step
    barrier()
    t0 = time.perf_counter()
    loss_value = 0.0
    for _ in range(args.steps):
        loss_value = trainer.step(host)
    barrier()
    e2e_s = time.perf_counter() - t0
    check_device_errors(local_rank)

    if world > 1:
        t = torch.tensor([ms, e2e_s], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, e2e_s = float(t[0]), float(t[1])
    tokens = group * COMPLETION_LEN
    value = tokens * args.steps / (ms / 1e3)
    mem_free, mem_total = torch.cuda.mem_get_info(device)
    kept = trainer.model.kept_layers()
    activation_note = (f"{kept} of {cfg.num_layers} layers keep their activations, the others are recomputed in "
                       "the backward pass (planned from free device memory)")
    if rank == 0:
        line = {
            "metric": METRIC, "value": round(value, 1), "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": round(ms / args.steps, 3), "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "impl": "ours",
            "config": {
                "model": cfg.name, "layers": cfg.num_layers, "global_batch": group, "seq_len": PROMPT_LEN + COMPLETION_LEN,
                "prompt_len": PROMPT_LEN, "completion_len": COMPLETION_LEN, "parallelism": parallelism,
                "tokens_counted": "completion tokens (G x 512) per step",
                "optimizer": "AdamW (fp32 moments) over all parameters, inside the timed region",
                "l2": "inputs larger than L2 (16 GB of weights streamed every step); no explicit flush",
                "activation_memory": activation_note,
                "peak_torch_allocated_gb": round(torch.cuda.max_memory_allocated(device) / 2**30, 1),
                "device_memory_in_use_gb": round((mem_total - mem_free) / 2**30, 1),
                "dev_overrides": bool(args.dev_layers or args.dev_group or args.dev_micro_group),
            },
            "clocks": sampler.summary(),
            "e2e": {
                "value": round(tokens * args.steps / e2e_s, 1), "unit": "tokens/s",
                "h2d_bytes_per_step": host.nbytes(), "d2h_bytes_per_step": 4, "last_loss": loss_value,
            },
            "gpu_launches": int(launches),
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
