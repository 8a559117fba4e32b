"""Vocabulary-parallel ``linear_logp`` under ``torchrun``: correctness, determinism and a timed stress phase.

    torchrun --nproc-per-node 4 --master-addr 127.0.0.1 tests/multigpu/linear_logp_tp.py                 # defaults
    torchrun --nproc-per-node 8 ... linear_logp_tp.py --stress --stress-tokens 131072 --stress-hidden 4096 \
        --stress-vocab 128256 --stress-iters 10                                                         # config-3 shape

NCCL + the fused sm_100a op when CUDA is present, Gloo + the PyTorch op on CPU (``--backend`` overrides).  Phases:

* correctness: every rank holds an uneven slice of the LM head; output, ``grad_hidden``, ``grad_weight`` and
  ``grad_bias`` are compared with autograd through materialised fp32 logits of the full vocabulary;
* determinism: the forward is repeated and must reproduce its bits, and all ranks must hold identical bits;
* stress (``--stress``): warm-up, then ``--stress-iters`` forward+backward steps timed on the device (CUDA events) or
  the host (CPU); reports the max over ranks of the median step time and of the peak memory, plus a finite check.

The process exits non-zero if any phase fails on any rank.  The reference's harness of the same name
(``tests/linear_logp_tp.py:228-423``) has the correctness and stress phases; determinism is added here because
bitwise reproducibility is part of this op's contract.
"""

from __future__ import annotations

import argparse
import os
import statistics
import sys
import time

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

DTYPES = {"bf16": torch.bfloat16, "fp16": torch.float16, "fp32": torch.float32}
TOLERANCE = {torch.bfloat16: 3e-2, torch.float16: 1e-2, torch.float32: 2e-4}  # relative to the reference's peak


def shard_bounds(vocab: int, world: int, uneven: bool):
    """Contiguous shards that tile [0, vocab); ``uneven`` moves every other boundary by a few multiples of 8."""
    cuts = [0]
    for r in range(1, world):
        cut = vocab * r // world // 8 * 8
        if uneven and r % 2:
            cut = min(vocab - 8 * (world - r), cut + 24)
        cuts.append(max(cut, cuts[-1] + 8))
    return cuts + [vocab]


def all_ranks(flag: bool, device) -> bool:
    t = torch.tensor([1 if flag else 0], device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MIN)
    return bool(t.item())


def max_over_ranks(value: float, device) -> float:
    t = torch.tensor([value], device=device, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def pick_op(name: str, device):
    if name == "native" or device.type == "cpu":
        from rl_engine.kernels.ops.pytorch.loss.linear_logp import NativeLinearLogpOp

        return NativeLinearLogpOp()
    from rl_engine.kernels.registry import kernel_registry

    return kernel_registry.get_op("linear_logp")


def relative_error(got: torch.Tensor, want: torch.Tensor) -> float:
    return float((got.float() - want.float()).abs().max() / want.float().abs().max().clamp_min(1e-12))


def correctness(args, rank, world, device, op) -> bool:
    dtype = DTYPES[args.dtype]
    bounds = shard_bounds(args.vocab, world, not args.even_shards)
    v0, v1 = bounds[rank], bounds[rank + 1]
    gen = torch.Generator(device=device).manual_seed(args.seed)  # identical tensors on every rank
    hidden = torch.randn(args.tokens, args.hidden, device=device, generator=gen).to(dtype)
    weight = (torch.randn(args.vocab, args.hidden, device=device, generator=gen) * 0.05).to(dtype)
    bias = None if args.no_bias else (torch.randn(args.vocab, device=device, generator=gen) * 0.1).to(dtype)
    target = torch.randint(0, args.vocab, (args.tokens,), device=device, generator=gen)
    upstream = torch.randn(args.tokens, device=device, generator=gen)

    # oracle: fp32 logits of the whole vocabulary, log-softmax, gather
    ref = [t.detach().float().requires_grad_(True) for t in (hidden, weight)] + (
        [] if bias is None else [bias.detach().float().requires_grad_(True)])
    logits = ref[0] @ ref[1].t() + (0 if bias is None else ref[2])
    want = torch.log_softmax(logits, dim=-1).gather(-1, target[:, None]).squeeze(-1)
    want.backward(upstream)

    h = hidden.detach().clone().requires_grad_(True)
    w = weight[v0:v1].detach().clone().requires_grad_(True)
    b = None if bias is None else bias[v0:v1].detach().clone().requires_grad_(True)
    kw = dict(tp_group=dist.group.WORLD, vocab_start_index=v0, global_vocab_size=args.vocab)
    got = op(h, w, target, b, **kw)
    got.backward(upstream)

    tol = args.tol if args.tol is not None else TOLERANCE[dtype]
    errors = {"output": relative_error(got, want), "grad_hidden": relative_error(h.grad, ref[0].grad),
              "grad_weight": relative_error(w.grad, ref[1].grad[v0:v1])}
    if bias is not None:
        errors["grad_bias"] = relative_error(b.grad, ref[2].grad[v0:v1])
    ok = all(e <= tol for e in errors.values())

    again = op(h.detach(), w.detach(), target, None if b is None else b.detach(), **kw)
    reproducible = torch.equal(again, got.detach())
    gathered = [torch.empty_like(got.detach()) for _ in range(world)]
    dist.all_gather(gathered, got.detach().contiguous())
    same_on_all_ranks = all(torch.equal(gathered[0], g) for g in gathered)
    worst = {k: max_over_ranks(v, device) for k, v in errors.items()}
    ok_all = all_ranks(ok, device)
    rep_all = all_ranks(reproducible and same_on_all_ranks, device)
    if rank == 0:
        print(f"[correctness] tokens={args.tokens} hidden={args.hidden} vocab={args.vocab} dtype={args.dtype} "
              f"shards={bounds} op={type(op).__name__}")
        for k, v in worst.items():
            print(f"  {k:12s} max relative error over ranks {v:.3e}  (limit {tol:.1e})")
        print(f"  correctness={'PASS' if ok_all else 'FAIL'}")
        print(f"[determinism] repeat bitwise equal and identical on all ranks: {'PASS' if rep_all else 'FAIL'}")
    return ok_all and rep_all


def stress(args, rank, world, device, op) -> bool:
    dtype = DTYPES[args.dtype]
    bounds = shard_bounds(args.stress_vocab, world, not args.even_shards)
    v0, v1 = bounds[rank], bounds[rank + 1]
    shared = torch.Generator(device=device).manual_seed(args.seed + 1000)
    own = torch.Generator(device=device).manual_seed(args.seed + 2000 + rank)
    hidden = torch.randn(args.stress_tokens, args.stress_hidden, device=device, generator=shared).to(dtype).requires_grad_(True)
    target = torch.randint(0, args.stress_vocab, (args.stress_tokens,), device=device, generator=shared)
    weight = (torch.randn(v1 - v0, args.stress_hidden, device=device, generator=own) * 0.02).to(dtype).requires_grad_(True)
    kw = dict(tp_group=dist.group.WORLD, vocab_start_index=v0, global_vocab_size=args.stress_vocab)
    out = None

    def step():
        nonlocal out
        hidden.grad = None
        weight.grad = None
        out = op(hidden, weight, target, None, **kw)
        out.float().mean().backward()

    cuda = device.type == "cuda"
    for _ in range(args.stress_warmup):
        step()
    if cuda:
        torch.cuda.synchronize(device)
        torch.cuda.reset_peak_memory_stats(device)
    dist.barrier()
    times = []
    for _ in range(args.stress_iters):
        if cuda:
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            step()
            b.record()
            b.synchronize()
            times.append(a.elapsed_time(b))
        else:
            t0 = time.perf_counter()
            step()
            times.append((time.perf_counter() - t0) * 1e3)
    finite = bool(torch.isfinite(out).all() and torch.isfinite(hidden.grad).all() and torch.isfinite(weight.grad).all())
    finite = all_ranks(finite, device)
    ms = max_over_ranks(statistics.median(times), device)
    peak = max_over_ranks(torch.cuda.max_memory_allocated(device) / 2**30 if cuda else 0.0, device)
    if rank == 0:
        flops = 6.0 * args.stress_tokens * args.stress_hidden * args.stress_vocab
        print(f"[stress] tokens={args.stress_tokens} hidden={args.stress_hidden} vocab={args.stress_vocab} "
              f"dtype={args.dtype} world={world} shards={bounds}")
        print(f"  finite={'PASS' if finite else 'FAIL'}")
        print(f"  max_rank_median_ms={ms:.3f}  ({args.stress_iters} timed steps after {args.stress_warmup} warm-up)")
        print(f"  aggregate_tflops_fwd_bwd={flops / (ms * 1e-3) / 1e12:.1f}  (6*N*D*V per step)")
        if cuda:
            print(f"  max_rank_peak_memory_gb={peak:.3f}")
    return finite


def build_parser() -> argparse.ArgumentParser:
    p = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    p.add_argument("--backend", choices=["auto", "nccl", "gloo"], default="auto")
    p.add_argument("--op", choices=["registry", "native"], default="registry")
    p.add_argument("--dtype", choices=sorted(DTYPES), default=None, help="default: bf16 on CUDA, fp32 on CPU")
    p.add_argument("--tokens", type=int, default=296)
    p.add_argument("--hidden", type=int, default=256)
    p.add_argument("--vocab", type=int, default=12040)
    p.add_argument("--even-shards", action="store_true")
    p.add_argument("--no-bias", action="store_true")
    p.add_argument("--tol", type=float, default=None)
    p.add_argument("--seed", type=int, default=2024)
    p.add_argument("--skip-correctness", action="store_true")
    p.add_argument("--stress", action="store_true")
    p.add_argument("--stress-tokens", type=int, default=4096)
    p.add_argument("--stress-hidden", type=int, default=2048)
    p.add_argument("--stress-vocab", type=int, default=32768)
    p.add_argument("--stress-warmup", type=int, default=2)
    p.add_argument("--stress-iters", type=int, default=5)
    return p


def main() -> int:
    args = build_parser().parse_args()
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    use_cuda = torch.cuda.is_available() and args.backend != "gloo"
    device = torch.device("cuda", local) if use_cuda else torch.device("cpu")
    if use_cuda:
        torch.cuda.set_device(device)
    backend = ("nccl" if use_cuda else "gloo") if args.backend == "auto" else args.backend
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29541")
    dist.init_process_group(backend, rank=rank, world_size=world, **({"device_id": device} if use_cuda else {}))
    if args.dtype is None:
        args.dtype = "bf16" if use_cuda else "fp32"
    op = pick_op(args.op, device)
    ok = True
    try:
        if not args.skip_correctness:
            ok = correctness(args, rank, world, device, op) and ok
        if args.stress:
            ok = stress(args, rank, world, device, op) and ok
        if use_cuda:
            from rl_engine.kernels.ops.base import _EXT_AVAILABLE, check_device_errors

            if _EXT_AVAILABLE:
                check_device_errors(local)
    finally:
        dist.barrier()
        dist.destroy_process_group()
    if rank == 0:
        print("RESULT", "PASS" if ok else "FAIL", flush=True)
    return 0 if ok else 1


if __name__ == "__main__":
    sys.exit(main())
