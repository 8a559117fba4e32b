"""Per-operator comparison against the reference library on the same GPU, through both libraries' PUBLIC API.

    python benchmarks/benchmark_vs_reference.py                 # runs both arms, prints one markdown table
    python benchmarks/benchmark_vs_reference.py --impl ours     # one arm: one JSON line per workload
    python benchmarks/benchmark_vs_reference.py --impl reference

Both arms execute THIS file; only ``sys.path`` differs: the ``ours`` arm imports ``rl_engine`` from the repository, the
``reference`` arm from ``baseline/_ref`` (the unmodified reference installed there, with its own CUDA extension built
from its default sources).  Because the reference's registry / sampler / operator classes and this library's share one
public API, the workload code below is the same for both: ``kernel_registry.get_op(...)``, ``SamplerBackend`` and the
prefix-shared attention op.  Whatever backend each library's stock dispatch picks on this GPU is what gets timed (the
line records its class name).

Workloads are the shapes of the reference's published tables (its README and operator docs): fused linear->log-prob
forward and forward+backward, log-prob over materialised logits, temperature/top-k/top-p sampling, ratio/KL forward,
GRPO loss forward and forward+backward, prefix-shared attention.  Timing: CUDA events, median of ``--repeat`` after
``--warmup``, an L2-sized buffer written between repetitions; peak extra device memory of one call.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)


# ------------------------------------------------------------------------------------------ one arm
def _setup_path(impl: str) -> None:
    drop = {os.path.abspath(p) for p in (ROOT, HERE)}
    sys.path[:] = [p for p in sys.path if os.path.abspath(p or ".") not in drop]
    sys.path.insert(0, ROOT if impl == "ours" else os.path.join(ROOT, "baseline", "_ref"))


def run_arm(args) -> None:
    _setup_path(args.impl)
    import torch

    import rl_engine

    want = "baseline" if args.impl == "reference" else ""
    origin = os.path.abspath(rl_engine.__file__)
    if (args.impl == "reference") != ("baseline" in origin):
        raise SystemExit(f"rl_engine resolved to {origin}, not the {args.impl} arm {want}")
    from rl_engine.kernels.registry import kernel_registry
    from rl_engine.kernels.sampling import SamplerBackend

    dev = torch.device("cuda", 0)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

    def measure(fn):
        for _ in range(args.warmup):
            fn()
        torch.cuda.synchronize()
        times = []
        for _ in range(args.repeat):
            flush.zero_()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            fn()
            b.record()
            b.synchronize()
            times.append(a.elapsed_time(b))
        torch.cuda.synchronize()
        base = torch.cuda.memory_allocated(dev)
        torch.cuda.reset_peak_memory_stats(dev)
        fn()
        torch.cuda.synchronize()
        return statistics.median(times), (torch.cuda.max_memory_allocated(dev) - base) / 2**20

    def emit(op, shape, fn, backend, flops=None, nbytes=None):
        try:
            ms, extra_mb = measure(fn)
            line = {"op": op, "shape": shape, "ms": round(ms, 4), "extra_mb": round(extra_mb, 1), "backend": backend}
            if flops:
                line["tflops"] = round(flops / (ms * 1e-3) / 1e12, 1)
            if nbytes:
                line["gbs"] = round(nbytes / (ms * 1e-3) / 1e9, 1)
        except Exception as exc:  # noqa: BLE001 - a workload one library cannot run is a result, not a crash
            line = {"op": op, "shape": shape, "error": f"{type(exc).__name__}: {exc}"[:200], "backend": backend}
            torch.cuda.empty_cache()
        line["impl"] = args.impl
        print(json.dumps(line), flush=True)

    gen = torch.Generator(device=dev).manual_seed(0)
    randn = lambda *s, dtype=torch.bfloat16, scale=1.0: (torch.randn(*s, device=dev, generator=gen) * scale).to(dtype)
    selected = set(args.ops.split(",")) if args.ops != "all" else None
    on = lambda name: selected is None or name in selected

    # ---- fused linear -> log-prob (reference docs: N = 4096, D = 2048, V = 32768 / 131072, bf16) ----------------
    if on("linear_logp"):
        op = kernel_registry.get_op("linear_logp")
        for v in (32768, 131072):
            n, d = 4096, 2048
            h = randn(n, d).requires_grad_(True)
            w = randn(v, d, scale=0.02).requires_grad_(True)
            t = torch.randint(0, v, (n,), device=dev, generator=gen)
            g = randn(n, dtype=torch.float32)

            def fwd():
                with torch.no_grad():
                    op(h, w, t, None)

            def fwd_bwd():
                h.grad = w.grad = None
                op(h, w, t, None).backward(g)

            shape = f"N={n} D={d} V={v} bf16"
            emit("linear_logp fwd", shape, fwd, type(op).__name__, flops=2.0 * n * d * v)
            emit("linear_logp fwd+bwd", shape, fwd_bwd, type(op).__name__, flops=6.0 * n * d * v)
            del h, w

    # ---- log-prob over materialised logits (reference README: vocab 128256, 512 tokens x G, fp16) -------------
    if on("logp"):
        op = kernel_registry.get_op("logp")
        for gsz in (8, 32):
            rows, v = gsz * 512, 128256
            logits = randn(rows, v, dtype=torch.float16)
            ids = torch.randint(0, v, (rows,), device=dev, generator=gen)
            emit("logp (selected-token log-prob over logits)", f"rows={rows} V={v} fp16", lambda: op.apply(logits, ids),
                 type(op).__name__, nbytes=rows * v * 2.0)
            del logits

    # ---- sampling (reference README: vocab 128256, top-k 50, top-p 0.9; benchmark config: [256, 151936], T 0.7) -
    if on("sampling"):
        sampler = SamplerBackend()
        for rows, v, temp in ((32, 128256, 1.0), (256, 128256, 1.0), (256, 151936, 0.7)):
            logits = randn(rows, v, dtype=torch.float32)
            emit("sample top-k 50 / top-p 0.9", f"rows={rows} V={v} T={temp} fp32",
                 lambda: sampler.sample(logits, top_k=50, top_p=0.9, temperature=temp), str(getattr(sampler, "backend", "?")),
                 nbytes=rows * v * 4.0)
            del logits

    # ---- ratio / KL forward (reference docs: B = 16, T = 512, fp16) ---------------------------------------------
    if on("ratio_kl"):
        op = kernel_registry.get_op("ratio_kl")
        for v in (32768, 131072):
            b, t = 16, 512
            pol, ref = randn(b, t, v, dtype=torch.float16), randn(b, t, v, dtype=torch.float16)
            ids = torch.randint(0, v, (b, t), device=dev, generator=gen)
            mask = torch.ones(b, t, dtype=torch.bool, device=dev)
            old = randn(b, t, dtype=torch.float32)

            def fwd():
                with torch.no_grad():
                    op(pol, ref, ids, mask, old)

            emit("ratio_kl fwd", f"B={b} T={t} V={v} fp16", fwd, type(op).__name__, nbytes=2.0 * b * t * v * 2)
            del pol, ref

    # ---- GRPO loss from logits (reference docs: B = 32, T = 256, fp16) -------------------------------------------
    if on("grpo_loss"):
        op = kernel_registry.get_op("grpo_loss")
        for v in (32768, 131072):
            b, t = 32, 256
            pol = randn(b, t, v, dtype=torch.float16).requires_grad_(True)
            ref = randn(b, t, v, dtype=torch.float16)
            ids = torch.randint(0, v, (b, t), device=dev, generator=gen)
            mask = torch.ones(b, t, dtype=torch.bool, device=dev)
            old = randn(b, t, dtype=torch.float32)
            rewards = randn(b, dtype=torch.float32)
            kw = dict(clip_eps=0.2, beta=0.04, samples_per_prompt=8)

            def fwd():
                with torch.no_grad():
                    op(pol, ref, ids, old, rewards, mask, **kw)

            def fwd_bwd():
                pol.grad = None
                out = op(pol, ref, ids, old, rewards, mask, **kw)
                (out[0] if isinstance(out, (tuple, list)) else out).backward()

            shape = f"B={b} T={t} V={v} fp16"
            emit("grpo_loss fwd", shape, fwd, type(op).__name__, nbytes=2.0 * b * t * v * 2)
            emit("grpo_loss fwd+bwd", shape, fwd_bwd, type(op).__name__)
            del pol, ref

    # ---- prefix-shared attention (reference benchmark: bs 1, G 64, len_q 512, D 128, len_kv 1k..16k) ------------
    if on("attention"):
        if args.impl == "reference":
            from rl_engine.kernels.ops.cuda.attention.prefix_shared_attn import PrefixSharedAttentionOp

            attn = PrefixSharedAttentionOp()
            backend = "PrefixSharedAttentionOp" + ("" if getattr(attn, "has_hardware_op", False) else " (SDPA fallback)")
        else:
            attn = kernel_registry.get_op("prefix_shared_attn")
            backend = type(attn).__name__
        for len_kv in (1024, 4096, 16384):
            bs, g, len_q, d = 1, 64, 512, 128
            q, k, v_ = randn(bs, g, len_q, d), randn(bs, len_kv, d), randn(bs, len_kv, d)

            def fwd():
                with torch.no_grad():
                    attn(q, k, v_)

            emit("prefix_shared_attention fwd", f"bs={bs} G={g} len_q={len_q} len_kv={len_kv} D={d} bf16", fwd, backend,
                 flops=4.0 * bs * g * len_q * len_kv * d)


# ------------------------------------------------------------------------------------------ driver
def run_both(args) -> None:
    rows = {}
    for impl in ("reference", "ours"):
        if impl == "reference" and not os.path.isdir(os.path.join(ROOT, "baseline", "_ref", "rl_engine")):
            print("reference is not installed under baseline/_ref; only this library is measured", file=sys.stderr)
            continue
        env = dict(os.environ)
        env.pop("PYTHONPATH", None)
        cmd = [sys.executable, os.path.abspath(__file__), "--impl", impl, "--ops", args.ops, "--warmup", str(args.warmup),
               "--repeat", str(args.repeat)]
        done = subprocess.run(cmd, env=env, text=True, capture_output=True, timeout=args.timeout, check=False)
        if done.returncode != 0:
            print(f"[{impl}] arm exited {done.returncode}: {done.stderr[-1500:]}", file=sys.stderr)
        for line in done.stdout.splitlines():
            if line.startswith("{"):
                rec = json.loads(line)
                rows.setdefault((rec["op"], rec["shape"]), {})[impl] = rec
                print(line, flush=True)
    fmt = lambda r, key, unit="": "-" if r is None else (r.get("error", "")[:40] if "error" in r else f"{r[key]}{unit}")
    print("\n| op | shape | ours ms | reference ms | reference / ours | ours extra MB | reference extra MB | backends (ours / reference) |")
    print("|---|---|---|---|---|---|---|---|")
    for (op, shape), rec in rows.items():
        o, r = rec.get("ours"), rec.get("reference")
        ratio = "-"
        if o and r and "ms" in o and "ms" in r:
            ratio = f"{r['ms'] / o['ms']:.2f}x"
        print(f"| {op} | {shape} | {fmt(o, 'ms')} | {fmt(r, 'ms')} | {ratio} | {fmt(o, 'extra_mb')} | {fmt(r, 'extra_mb')} | "
              f"{(o or {}).get('backend', '-')} / {(r or {}).get('backend', '-')} |")


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--impl", choices=["both", "ours", "reference"], default="both")
    ap.add_argument("--ops", default="all", help="comma-separated subset of linear_logp,logp,sampling,ratio_kl,grpo_loss,attention")
    ap.add_argument("--warmup", type=int, default=2)
    ap.add_argument("--repeat", type=int, default=10)
    ap.add_argument("--timeout", type=int, default=900)
    args = ap.parse_args()
    if args.impl == "both":
        run_both(args)
    else:
        run_arm(args)


if __name__ == "__main__":
    main()
