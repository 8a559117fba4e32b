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
completion`` sequence (G x 1536 tokens per step), processed in micro-batches.  Activations are kept
(no gradient checkpointing) with the largest micro-batch of 8 / 4 / 2 sequences that fits the device;
only if none fits is checkpointing switched on.  ``config.memory_plan`` records which variant ran.
Same metric, same counting (completion tokens per second), same JSON line as ``bench.py`` with
``"impl": "reference"``.

The line also carries ``ops``: the reference's ``linear_logp`` op (its stock dispatch: the Triton
forward + chunked PyTorch backward on this GPU), forward + backward at ``[G x 512, 4096] x [128256,
4096]`` for G = 64 / 128 / 256 with extra device memory and time, vocabulary-parallel over its NCCL
all-reduces when N > 1; and ``SamplerBackend.sample`` at ``[256, 151936]``, T = 0.7, k = 50, p = 0.9.
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
# (gradient checkpointing, sequences per micro-batch), tried in this order; the first that fits runs
MEMORY_PLANS = [(False, 8), (False, 4), (False, 2), (True, 8)]
OPS_TIME_LIMIT_S = 150.0  # the operator measurements stop taking new samples after this many seconds


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
    if not torch.cuda.is_available() or torch.cuda.device_count() <= local_rank:
        unavailable(f"no CUDA device {local_rank} is visible to this process")
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
    plan = {"checkpointing": False, "micro_batch": 8}

    def completion_logps(ids):
        # hidden state at position t predicts token t + 1
        base = model.model(input_ids=ids, use_cache=False).last_hidden_state
        hidden = base[:, PROMPT_LEN - 1 : PROMPT_LEN + COMPLETION_LEN - 1]
        targets = ids[:, PROMPT_LEN:]
        return linear_logp(hidden, model.lm_head.weight, targets, None)

    def step(ids_host, rewards_host, mask_h, old, ref):
        micro = plan["micro_batch"]
        ids = ids_host.to(device, non_blocking=True)
        rew = rewards_host.to(device, non_blocking=True)
        mask = mask_h.to(device, non_blocking=True)
        optimizer.zero_grad(set_to_none=True)
        adv = grpo.group_advantages(rew.float(), samples_per_prompt=group)[sl]
        total = torch.zeros((), device=device)
        n_micro = (local_group + micro - 1) // micro
        for i in range(n_micro):
            rows = slice(i * micro, min((i + 1) * micro, local_group))
            cur = completion_logps(ids[rows])
            ratio = compute_policy_ratio(cur, old[rows], mask[rows])
            a = adv[rows].float()[:, None]
            policy = -torch.minimum(ratio * a, torch.clamp(ratio, 0.8, 1.2) * a)
            kl = compute_reference_kl(cur, ref[rows], mask[rows])
            loss = masked_mean(policy + 0.04 * kl, mask[rows]) / n_micro
            loss.backward()
            total += loss.detach()
        if world > 1:
            # stands in for DeepSpeed's bucketed gradient all-reduce (one NCCL call per parameter, averaged)
            for p in model.parameters():
                if p.grad is not None:
                    dist.all_reduce(p.grad, op=dist.ReduceOp.AVG)
        optimizer.step()
        return total

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    try:
        with torch.no_grad():
            cur0 = torch.cat([
                completion_logps(host_ids[i : i + 8].to(device)).float() for i in range(0, local_group, 8)
            ])
        noise = torch.Generator(device=device).manual_seed(99 + rank)
        old = cur0 + 0.01 * torch.randn(cur0.shape, device=device, generator=noise)
        ref = cur0 + 0.01 * torch.randn(cur0.shape, device=device, generator=noise)

        # Pick the memory plan: keep activations with the largest micro-batch that fits; all ranks take the same one.
        tried = []

        def probe(micro):
            ids = host_ids[:micro].to(device)
            cur = completion_logps(ids)
            (cur.float().mean() * 0.0).backward()
            optimizer.step()

        for checkpointing, micro in MEMORY_PLANS:
            plan.update(checkpointing=checkpointing, micro_batch=micro)
            if checkpointing:
                model.gradient_checkpointing_enable()
            else:
                model.gradient_checkpointing_disable()
            fits = 1
            torch.cuda.reset_peak_memory_stats(device)
            try:
                # two micro-batches with an optimiser step in between, no collective: the second one runs with the
                # gradients and the optimiser state allocated, which is the step's peak
                for _ in range(2):
                    probe(micro)
            except torch.cuda.OutOfMemoryError:
                fits = 0
            # leave headroom for the step's own temporaries (loss tail, group statistics, allocator fragmentation)
            if torch.cuda.max_memory_reserved(device) > 0.93 * torch.cuda.get_device_properties(device).total_memory:
                fits = 0
            optimizer.zero_grad(set_to_none=True)
            torch.cuda.empty_cache()
            if world > 1:
                agreed = torch.tensor([fits], device=device)
                dist.all_reduce(agreed, op=dist.ReduceOp.MIN)
                fits = int(agreed.item())
            tried.append({"checkpointing": checkpointing, "micro_batch": micro, "fits": bool(fits)})
            if fits:
                break
        else:
            unavailable("reference step does not fit the device in any memory plan")

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
    peak_gb = round(torch.cuda.max_memory_allocated(device) / 2**30, 1)

    # the per-operator part of the metric, with the model's memory released
    del model, optimizer, old, ref, cur0
    import gc

    gc.collect()
    torch.cuda.empty_cache()
    ops = {"skipped": "development overrides in use"}
    if not (args.dev_layers or args.dev_group) or os.environ.get("RLK_BENCH_OPS") == "1":
        ops = measure_ops(torch, dist, kernel_registry, device, rank, world)

    tokens = group * COMPLETION_LEN
    if rank == 0:
        print(json.dumps({
            "metric": "grpo_step_tokens_per_sec", "value": round(tokens * args.steps / (ms / 1e3), 1), "unit": "tokens/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms / args.steps, 3),
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "impl": "reference",
            "config": {
                "model": "llama3-8b", "layers": layers, "global_batch": group, "seq_len": PROMPT_LEN + COMPLETION_LEN,
                "prompt_len": PROMPT_LEN, "completion_len": COMPLETION_LEN,
                "parallelism": "single" if world == 1 else f"dp{world}-nccl-allreduce",
                "attention": attn_impl, "linear_logp_backend": type(linear_logp).__name__,
                "micro_batch": plan["micro_batch"], "gradient_checkpointing": plan["checkpointing"],
                "memory_plan": tried, "peak_torch_allocated_gb": peak_gb,
                "tokens_counted": "completion tokens (G x 512) per step",
                "optimizer": "torch.optim.AdamW(fused=True) on bf16 parameters (no fp32 master), inside the timed region",
                "dev_overrides": bool(args.dev_layers or args.dev_group),
            },
            "e2e": {"value": round(tokens * args.steps / wall, 1), "unit": "tokens/s",
                    "h2d_bytes_per_step": host_ids.numel() * 8 + host_rewards.numel() * 4 + mask_host.numel(),
                    "d2h_bytes_per_step": 4, "last_loss": last},
            "ops": ops,
        }), flush=True)
    if world > 1:
        dist.destroy_process_group()


def _median_ms(torch, fn, iters, deadline):
    """Median device time over up to ``iters`` calls (at least one), stopping early at ``deadline``."""
    times = []
    for _ in range(iters):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        b.synchronize()
        times.append(a.elapsed_time(b))
        if time.perf_counter() > deadline:
            break
    times.sort()
    return times[len(times) // 2], len(times)


def measure_ops(torch, dist, kernel_registry, device, rank, world):
    """Same shapes, inputs, counting and memory accounting as ``measure_ops`` of ``bench.py``, through the
    reference's own ``kernel_registry`` / ``SamplerBackend``."""
    out = {}
    deadline = time.perf_counter() + OPS_TIME_LIMIT_S
    try:
        op = kernel_registry.get_op("linear_logp")
        d, v = 4096, 128256
        v_local = v // world
        v0 = rank * v_local
        if rank == world - 1:
            v_local = v - v0
        torch.cuda.synchronize()
        floor = torch.cuda.memory_allocated(device)
        gen = torch.Generator(device=device).manual_seed(7)
        shard_gen = torch.Generator(device=device).manual_seed(11 + rank)
        weight = (torch.randn(v_local, d, device=device, generator=shard_gen) * 0.02).to(torch.bfloat16).requires_grad_(True)
        kw = {} if world == 1 else {"tp_group": dist.group.WORLD, "vocab_start_index": v0, "global_vocab_size": v}
        nbytes = lambda *ts: sum(t.numel() * t.element_size() for t in ts)
        extra, times, counts = {}, {}, {}
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
                times["fwd_ms"], counts["fwd"] = _median_ms(torch, fwd, 20, deadline)
                times["fwd_bwd_ms"], counts["fwd_bwd"] = _median_ms(torch, fwd_bwd, 20, deadline)
            del hidden, targets, grad_out
        if world > 1:
            t = torch.tensor([times["fwd_ms"], times["fwd_bwd_ms"]], device=device, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            times = {"fwd_ms": float(t[0]), "fwd_bwd_ms": float(t[1])}
        n = 256 * 512
        out["fused_logp"] = {
            "shape": f"[{n},{d}]x[{v},{d}]", "tp": world, "iters": counts, "backend": type(op).__name__,
            "fwd_ms": round(times["fwd_ms"], 3), "fwd_bwd_ms": round(times["fwd_bwd_ms"], 3),
            "tflops_fwd": round(2.0 * n * d * v / (times["fwd_ms"] * 1e-3) / 1e12, 1),
            "tflops_fwd_bwd": round(6.0 * n * d * v / (times["fwd_bwd_ms"] * 1e-3) / 1e12, 1),
            "flops_counted": "2*N*D*V forward, 6*N*D*V forward+backward",
            "extra_vram_mb": extra,
        }
        del weight
    except Exception as exc:  # noqa: BLE001
        out["fused_logp"] = {"error": f"{type(exc).__name__}: {exc}"[:300]}
    try:
        from rl_engine.kernels.sampling import SamplerBackend

        torch.cuda.empty_cache()
        sampler = SamplerBackend()
        gen = torch.Generator(device=device).manual_seed(3)
        buffers = [torch.randn(256, 151936, device=device, generator=gen) for _ in range(2)]
        state = {"i": 0}

        def call():
            state["i"] += 1
            return sampler.sample(buffers[state["i"] % 2], top_k=50, top_p=0.9, temperature=0.7)

        for _ in range(3):
            ids = call()
        torch.cuda.synchronize()
        assert ids.numel() == 256
        ms, count = _median_ms(torch, call, 30, time.perf_counter() + 30.0)
        out["sampler"] = {"shape": [256, 151936], "dtype": "fp32", "temperature": 0.7, "top_k": 50, "top_p": 0.9,
                          "ms": round(ms, 4), "iters": count, "backend": str(getattr(sampler, "backend", "?"))}
    except Exception as exc:  # noqa: BLE001
        out["sampler"] = {"error": f"{type(exc).__name__}: {exc}"[:300]}
    return out


if __name__ == "__main__":
    main()
