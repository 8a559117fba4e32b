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

The same line also carries the other two thirds of the headline metric, measured after the step timing
with the trainer's memory released (``ops``): the fused linear -> log-prob op forward + backward at
``[131072, 4096] x [128256, 4096]`` with 4096-token chunks (vocabulary-parallel over the N ranks when
N > 1) as TFLOP/s, its extra device memory at G = 64 / 128 / 256 completions of 512 tokens, and the
sampler's latency at ``[256, 151936]`` logits with temperature 0.7, top-k 50, top-p 0.9.
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
    # data parallel only: "on" splits the shared prompt's forward/backward pass over the ranks, "off" (default, faster at
    # this prompt length) runs it on every rank
    ap.add_argument("--prompt-shard", choices=["on", "off"], default="off")
    ap.add_argument("--skip-ops", action="store_true", help="leave out the per-operator measurements after the step")
    # development switches; any use marks the run as not comparable
    ap.add_argument("--dev-layers", type=int, default=0)
    ap.add_argument("--dev-group", type=int, default=0)
    ap.add_argument("--dev-no-overlap", action="store_true",
                    help="development only: data-parallel optimiser step after the backward pass instead of overlapped with it")
    ap.add_argument("--dev-layers-per-bucket", type=int, default=0,
                    help="development only: layers per bucket of the data-parallel optimiser step (library default 4)")
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


OPS_DEADLINE_S = 300
LOGP_HIDDEN, LOGP_VOCAB, LOGP_CHUNK = 4096, 128256, 4096
SAMPLER_ROWS, SAMPLER_VOCAB = 256, 151936


def _median_ms(fn, iters: int, warmup: int = 1):
    """Median device time of ``fn`` in ms (one CUDA-event pair per call, on the launching stream)."""
    import torch

    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    times = []
    for _ in range(iters):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        b.synchronize()
        times.append(a.elapsed_time(b))
    return statistics.median(times)


def measure_fused_logp(device, rank: int, world: int, iters: int = 20):
    """Fused linear -> log-prob, forward + backward, at G x 512 tokens for G = 64 / 128 / 256; timing at G = 256.

    With ``world`` > 1 every rank holds ``V / world`` rows of the LM head and the same tokens (vocabulary parallel);
    times are the max over ranks.  ``extra_vram_mb`` = peak allocated during the call minus the inputs (hidden states,
    weights, targets, upstream gradient) and minus what the call returns (log-probs; gradients), i.e. the op's
    workspaces and temporaries."""
    import torch
    import torch.distributed as dist

    from rl_engine.kernels.registry import kernel_registry

    op = kernel_registry.get_op("linear_logp")
    d, v = LOGP_HIDDEN, LOGP_VOCAB
    v_local = v // world
    v0 = rank * v_local
    if rank == world - 1:
        v_local = v - v0
    torch.cuda.synchronize()
    floor = torch.cuda.memory_allocated(device)  # nothing of this measurement exists yet
    gen = torch.Generator(device=device).manual_seed(7)  # the same tokens on every rank
    shard_gen = torch.Generator(device=device).manual_seed(11 + rank)
    weight = (torch.randn(v_local, d, device=device, generator=shard_gen) * 0.02).to(torch.bfloat16).requires_grad_(True)
    kw = {} if world == 1 else {"tp_group": dist.group.WORLD, "vocab_start_index": v0, "global_vocab_size": v}
    nbytes = lambda *ts: sum(t.numel() * t.element_size() for t in ts)
    extra, times = {}, {}
    for group in (64, 128, 256):
        n = group * 512
        hidden = torch.randn(n, d, device=device, generator=gen).to(torch.bfloat16).requires_grad_(True)
        targets = torch.randint(0, v, (n,), device=device, generator=gen)
        grad_out = torch.randn(n, device=device, generator=gen)

        def fwd():
            with torch.no_grad():
                return op(hidden, weight, targets, None, **kw)

        def fwd_bwd():
            hidden.grad = None
            weight.grad = None
            op(hidden, weight, targets, None, **kw).backward(grad_out)

        # everything above ``floor`` that is not an input or a returned tensor counts as extra, including the
        # workspaces that the op keeps between calls (created at the first call, they do not grow with G)
        inputs = nbytes(hidden, weight, targets, grad_out)
        hidden.grad = None
        weight.grad = None  # left over from the previous G: not part of this call
        torch.cuda.synchronize()
        torch.cuda.reset_peak_memory_stats(device)
        fwd()
        torch.cuda.synchronize()
        peak_fwd = torch.cuda.max_memory_allocated(device) - floor - inputs - n * 4
        torch.cuda.reset_peak_memory_stats(device)
        fwd_bwd()
        torch.cuda.synchronize()
        peak_bwd = torch.cuda.max_memory_allocated(device) - floor - inputs - nbytes(hidden.grad, weight.grad)
        extra[f"G{group}"] = {"fwd": round(peak_fwd / 2**20, 1), "fwd_bwd": round(peak_bwd / 2**20, 1)}
        if group == 256:
            times = {"fwd_ms": _median_ms(fwd, iters), "fwd_bwd_ms": _median_ms(fwd_bwd, iters)}
        del hidden, targets, grad_out
    if world > 1:
        t = torch.tensor([times["fwd_ms"], times["fwd_bwd_ms"]], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        times = {"fwd_ms": float(t[0]), "fwd_bwd_ms": float(t[1])}
    n = 256 * 512
    return {
        "shape": f"[{n},{d}]x[{v},{d}]", "tp": world, "chunk_tokens": LOGP_CHUNK, "iters": iters,
        "backend": type(op).__name__,
        "fwd_ms": round(times["fwd_ms"], 3), "fwd_bwd_ms": round(times["fwd_bwd_ms"], 3),
        "tflops_fwd": round(2.0 * n * d * v / (times["fwd_ms"] * 1e-3) / 1e12, 1),
        "tflops_fwd_bwd": round(6.0 * n * d * v / (times["fwd_bwd_ms"] * 1e-3) / 1e12, 1),
        "flops_counted": "2*N*D*V forward, 6*N*D*V forward+backward (the recomputation in backward is not counted)",
        "extra_vram_mb": extra,
        "l2": "inputs larger than L2 (1 GB of hidden states and 1 GB of weights per call)",
    }


def measure_sampler(device, iters: int = 30):
    """Temperature 0.7 / top-k 50 / top-p 0.9 sampling of one token per row of ``[256, 151936]`` fp32 logits; two
    input buffers alternate so that no call finds its logits in L2."""
    import torch

    from rl_engine.kernels.sampling import SamplerBackend

    sampler = SamplerBackend(seed=5)
    gen = torch.Generator(device=device).manual_seed(3)
    buffers = [torch.randn(SAMPLER_ROWS, SAMPLER_VOCAB, device=device, generator=gen) for _ in range(2)]
    state = {"i": 0}

    def call():
        state["i"] += 1
        return sampler.sample(buffers[state["i"] % 2], top_k=50, top_p=0.9, temperature=0.7)

    ids = call()
    assert ids.shape == (SAMPLER_ROWS,) and int(ids.min()) >= 0 and int(ids.max()) < SAMPLER_VOCAB
    return {"shape": [SAMPLER_ROWS, SAMPLER_VOCAB], "dtype": "fp32", "temperature": 0.7, "top_k": 50, "top_p": 0.9,
            "ms": round(_median_ms(call, iters, warmup=3), 4), "iters": iters, "backend": sampler.backend,
            "l2": "two 155 MB logit buffers alternate (each larger than L2)"}


def measure_tp_step(device, rank: int, world: int, warmup: int = 1, steps: int = 2):
    """The same GRPO step with the model tensor + sequence parallel over all ``world`` ranks (every rank sees the whole
    group of 256 completions; layers on the fused all-gather -> GEMM / GEMM -> reduce-scatter kernels, vocabulary-parallel
    LM head): the configuration the benchmark's config names as TP=N.  Data parallel stays the headline because it is
    faster for an 8 B model on 180 GB GPUs; this entry puts the TP number beside it."""
    import gc

    import torch
    import torch.distributed as dist

    from rl_engine.models.config import llama3_8b
    from rl_engine.models.grpo import synthetic_batch
    from rl_engine.models.llama import LlamaModel
    from rl_engine.parallel.tp_linear import TensorParallelLinears
    from rl_engine.parallel.tp_model import TensorParallelGRPOTrainer, TensorParallelLlama

    cfg = llama3_8b()
    model = LlamaModel(cfg, dtype=torch.bfloat16, device=device, seed=0, max_positions=PROMPT_LEN + COMPLETION_LEN)
    tp_model = TensorParallelLlama(model, TensorParallelLinears(group=dist.group.WORLD, device=device))
    del model
    gc.collect()
    torch.cuda.empty_cache()
    trainer = TensorParallelGRPOTrainer(tp_model, lr=1e-6, clip_eps=0.2, beta=0.04)
    host = synthetic_batch(cfg.vocab_size, PROMPT_LEN, GROUP, COMPLETION_LEN, seed=1234)
    batch = host.to(device)
    with torch.no_grad():
        cur = trainer.policy_logps(batch).float()
    gen = torch.Generator(device=device).manual_seed(99)
    batch.old_logps = cur + 0.01 * torch.randn(cur.shape, device=device, generator=gen)
    batch.ref_logps = cur + 0.01 * torch.randn(cur.shape, device=device, generator=gen)
    for _ in range(warmup):
        trainer.step_device(batch)
    torch.cuda.synchronize()
    dist.barrier()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(steps):
        loss = trainer.step_device(batch)
    b.record()
    torch.cuda.synchronize()
    t = torch.tensor([a.elapsed_time(b)], device=device, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t[0]) / steps
    from rl_engine.kernels.ops.base import check_device_errors

    check_device_errors(device.index or 0)
    out = {"parallelism": f"tp{world}-sequence-parallel-fused", "ms_per_step": round(ms, 3),
           "value": round(GROUP * COMPLETION_LEN / (ms * 1e-3), 1), "unit": "tokens/s", "steps": steps, "warmup": warmup,
           "global_batch": GROUP, "kept_layers": tp_model.kept_layers(), "last_loss": float(loss)}
    del trainer, tp_model, batch
    gc.collect()
    torch.cuda.empty_cache()
    return out


def measure_ops(device, rank: int, world: int, out=None):
    """The per-operator part of the headline metric (and, on more than one GPU, the tensor-parallel form of the step);
    a failure is reported in place of the numbers.  Results are added to ``out`` as they complete."""
    out = {} if out is None else out
    parts = [("fused_logp", lambda: measure_fused_logp(device, rank, world)), ("sampler", lambda: measure_sampler(device))]
    if world > 1 and os.environ.get("RLK_BENCH_TP", "1") != "0":
        parts.append(("tp_step", lambda: measure_tp_step(device, rank, world)))
    for name, fn in parts:
        try:
            out[name] = fn()
        except Exception as exc:  # noqa: BLE001 - the headline line must still be printed
            out[name] = {"error": f"{type(exc).__name__}: {exc}"[:300]}
    return out


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
    if not torch.cuda.is_available() or torch.cuda.device_count() <= local_rank:
        raise SystemExit("bench.py measures the training step on B200 GPUs: no CUDA device "
                         f"{local_rank} is visible to this process")
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

        shard = args.prompt_shard == "on"
        dev_kw = {}
        if args.dev_no_overlap:
            dev_kw["overlap"] = False
        if args.dev_layers_per_bucket:
            dev_kw["layers_per_bucket"] = args.dev_layers_per_bucket
        trainer = ShardedGRPOTrainer(model, lr=1e-6, clip_eps=0.2, beta=0.04, micro_group=micro, shard_prompt=shard,
                                     **dev_kw)
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
    if hasattr(trainer, "check"):
        trainer.check()  # bounded peer waits of the symmetric-memory barriers report here, not in the global word

    if world > 1:
        t = torch.tensor([ms, e2e_s], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, e2e_s = float(t[0]), float(t[1])
        if not tensor_parallel:  # every rank's loss is the mean over its own completions: report the group's mean
            mean_loss = torch.tensor([loss_value], device=device, dtype=torch.float64)
            dist.all_reduce(mean_loss, op=dist.ReduceOp.AVG)
            loss_value = float(mean_loss[0])
    tokens = group * COMPLETION_LEN
    value = tokens * args.steps / (ms / 1e3)
    mem_free, mem_total = torch.cuda.mem_get_info(device)
    peak_allocated = torch.cuda.max_memory_allocated(device)
    kept = trainer.model.kept_layers()
    master = ("fp32 master weights (bf16 parameter + 16-bit residual per element)" if getattr(trainer.opt, "residual", None)
              is not None else "fp32 master weights" if getattr(trainer.opt, "master", None) is not None else "none")
    line = {}
    emitted = threading.Event()

    def emit(ops):
        if emitted.is_set():
            return
        emitted.set()
        if rank == 0:
            line["ops"] = ops
            print(json.dumps(line), flush=True)
    activation_note = (f"{kept} of {cfg.num_layers} layers keep their activations, the others are recomputed in "
                       "the backward pass (planned from free device memory)")
    line.update({
        "metric": METRIC, "value": round(value, 1), "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": round(ms / args.steps, 3), "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "impl": "ours",
        "config": {
            "model": cfg.name, "layers": cfg.num_layers, "global_batch": group, "seq_len": PROMPT_LEN + COMPLETION_LEN,
            "prompt_len": PROMPT_LEN, "completion_len": COMPLETION_LEN, "parallelism": parallelism,
            "tokens_counted": "completion tokens (G x 512) per step",
            "optimizer": "AdamW (fp32 moments) over all parameters, inside the timed region",
            "master_weights": master,
            "l2": "inputs larger than L2 (16 GB of weights streamed every step); no explicit flush",
            "activation_memory": activation_note,
            "prompt_pass": ("split over the ranks (zig-zag context parallel), keys / values gathered by peer stores"
                            if getattr(trainer, "_prompt_shards", None) else "once per rank"),
            "peak_torch_allocated_gb": round(peak_allocated / 2**30, 1),
            "device_memory_in_use_gb": round((mem_total - mem_free) / 2**30, 1),
            "dev_overrides": bool(args.dev_layers or args.dev_group or args.dev_micro_group or args.dev_no_overlap
                                  or args.dev_layers_per_bucket),
        },
        "clocks": sampler.summary(),
        "e2e": {
            "value": round(tokens * args.steps / e2e_s, 1), "unit": "tokens/s",
            "h2d_bytes_per_step": host.nbytes(), "d2h_bytes_per_step": 4, "last_loss": loss_value,
        },
        "gpu_launches": int(launches),
    })

    # The per-operator numbers need a few GB: release the trainer first.  If that part does not finish in time the
    # line is printed without it, so the step result is never lost.
    ops = {}

    def watchdog():
        emit({**ops, "error": f"operator measurements did not finish within {OPS_DEADLINE_S} s"})
        os._exit(0)

    timer = threading.Timer(OPS_DEADLINE_S, watchdog)
    timer.daemon = True
    timer.start()
    if args.skip_ops:
        ops["skipped"] = "--skip-ops"
    elif (args.dev_layers or args.dev_group) and os.environ.get("RLK_BENCH_OPS") != "1":
        ops["skipped"] = "development overrides in use"
    else:
        if hasattr(trainer, "mem"):
            torch.cuda.synchronize()
            trainer.close() if hasattr(trainer, "close") else trainer.mem.close()
        del trainer, dev_batch, host, full
        model = tp_model = None  # noqa: F841 - drop the last references to the parameters
        import gc

        gc.collect()
        torch.cuda.empty_cache()
        if tensor_parallel:
            os.environ["RLK_BENCH_TP"] = "0"  # the step above already was the tensor-parallel one
        measure_ops(device, rank, world, ops)
    timer.cancel()
    emit(ops)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
