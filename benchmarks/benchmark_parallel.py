"""Multi-GPU benchmarks of the fused compute+communication paths, one JSON line per path (printed by rank 0).

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port 29600 \
        benchmarks/benchmark_parallel.py --paths all

Every number is device time (CUDA events around the launches on each rank, barrier before), the MAXIMUM over ranks,
median of ``--repeat`` repetitions after ``--warmup`` warm-ups.  Each line carries the path's roofline: the slower of
(FLOPs / measured bf16 GEMM peak) and (bytes that must enter this GPU over NVLink / 770 GB/s, the measured peer-copy
bandwidth per direction), and ``frac_of_roofline = roofline_ms / ms``.

Paths: ``tp_ag_gemm`` (all-gather -> QKV/up GEMM), ``tp_gemm_rs`` (down/out GEMM -> reduce-scatter), ``linear_logp_tp``
(vocabulary-parallel LM head with the in-kernel merge, forward and backward), ``cp_attention`` (context-parallel causal
attention forward+backward), ``ep_moe`` (expert-parallel MoE layer forward+backward), ``zero1`` (fused reduce-scatter +
AdamW + all-gather), ``weight_broadcast`` (trainer -> all ranks with fp32 -> bf16 cast), ``weight_sync`` (the whole weight
update protocol over ``NVLinkBroadcastBridge``, relay and direct).
"""

from __future__ import annotations

import argparse
import datetime
import json
import os
import statistics
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from common import peaks  # noqa: E402  (also puts the repository root on sys.path)

NVLINK_GBS = 770.0


def timed(fn, warmup: int, repeat: int):
    """Median over repetitions of the max-over-ranks device time of ``fn`` (ms)."""
    for _ in range(warmup):
        fn()
    samples = []
    for _ in range(repeat):
        torch.cuda.synchronize()
        dist.barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        t = torch.tensor([a.elapsed_time(b)], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        samples.append(float(t))
    return statistics.median(samples)


def emit(rank, name, ms, flops, nvlink_bytes, **extra):
    pk = peaks()
    compute_ms = flops / (pk["bf16_tflops"] * 1e9) if flops else 0.0
    link_ms = nvlink_bytes / (NVLINK_GBS * 1e6) if nvlink_bytes else 0.0
    roof = max(compute_ms, link_ms)
    if rank == 0:
        line = {"path": name, "world": dist.get_world_size(), "ms": round(ms, 4),
                "tflops_per_gpu": round(flops / ms / 1e9, 1) if flops else None,
                "nvlink_in_gbs_per_gpu": round(nvlink_bytes / ms / 1e6, 1) if nvlink_bytes else None,
                "roofline_ms": round(roof, 4), "bound": "compute" if compute_ms >= link_ms else "nvlink",
                "frac_of_roofline": round(roof / ms, 3) if ms > 0 else None, "peaks": pk["source"], **extra}
        print(json.dumps(line), flush=True)


def rnd(shape, scale=1.0, seed=0, dtype=torch.bfloat16):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return (torch.randn(shape, device="cuda", generator=g) * scale).to(dtype)


def bench_tp(args, rank, world):
    from rl_engine.parallel.tp_linear import TensorParallelLinears

    tp = TensorParallelLinears(device=torch.device("cuda", torch.cuda.current_device()))
    t, h, f = args.tokens // (128 * world) * 128 * world, 4096, 14336
    rows = t // world
    x_local = rnd((rows, h), seed=rank)
    w_up = rnd((2 * f // world, h), 0.02, 100 + rank)          # this rank's [gate | up] shard
    ms = timed(lambda: tp.ag_gemm(x_local, w_up), args.warmup, args.repeat)
    emit(rank, "tp_ag_gemm", ms, 2.0 * t * h * (2 * f // world), (world - 1) * rows * h * 2.0,
         shape=[t, 2 * f // world, h], note="all-gather of the token rows fused into the gate/up GEMM")
    act = rnd((t, f // world), seed=3)
    w_down = rnd((h, f // world), 0.02, 200 + rank)
    ms = timed(lambda: tp.gemm_rs(act, w_down), args.warmup, args.repeat)
    emit(rank, "tp_gemm_rs", ms, 2.0 * t * h * (f // world), (world - 1) * rows * h * 2.0,
         shape=[t, h, f // world], note="down GEMM with the reduce-scatter fused (bf16 partial tiles stored to the owners)")
    tp.check()


def bench_linear_logp(args, rank, world):
    from rl_engine.kernels.ops.sm100.linear_logp import FusedLinearLogpSM100Op

    n, d, v = args.logp_tokens, 4096, 128256
    bounds = [v * i // world // 8 * 8 for i in range(world)] + [v]
    v0, v1 = bounds[rank], bounds[rank + 1]
    hidden = rnd((n, d), seed=1).requires_grad_(True)           # same tokens on every rank
    w = rnd((v1 - v0, d), 0.02, 10 + rank).requires_grad_(True)
    tgt = torch.randint(0, v, (n,), device="cuda", generator=torch.Generator(device="cuda").manual_seed(2))
    op = FusedLinearLogpSM100Op(check_targets=False)
    group = dist.group.WORLD if world > 1 else None
    kw = dict(tp_group=group, vocab_start_index=v0, global_vocab_size=v) if world > 1 else {}

    def fwd():
        with torch.no_grad():
            return op(hidden, w, tgt, **kw)

    ms = timed(fwd, args.warmup, args.repeat)
    a, b = fwd(), fwd()
    same = torch.equal(a, b)
    gathered = [torch.empty_like(a) for _ in range(world)]
    dist.all_gather(gathered, a)
    ranks_equal = all(torch.equal(gathered[0], g) for g in gathered)
    # training == rollout: the first 1000 rows scored alone must give the same bits as inside the full batch
    with torch.no_grad():
        small = op(hidden[:1000], w, tgt[:1000], **kw)
    emit(rank, "linear_logp_tp_fwd", ms, 2.0 * n * d * (v1 - v0), n * 16.0 * (world - 1) * max(1, (v1 - v0) // 8192),
         shape=[n, d, v], vocab_shard=v1 - v0, run_to_run_bitwise=bool(same), ranks_bitwise_equal=bool(ranks_equal),
         batch_invariant_bitwise=bool(torch.equal(small, a[:1000])))

    def fwd_bwd():
        hidden.grad = w.grad = None
        op(hidden, w, tgt, **kw).sum().backward()

    ms = timed(fwd_bwd, max(1, args.warmup - 1), max(1, args.repeat // 2))
    emit(rank, "linear_logp_tp_fwd_bwd", ms, 8.0 * n * d * (v1 - v0), n * d * 4.0 * (world - 1) / world if world > 1 else 0.0,
         shape=[n, d, v], note="forward + recompute backward; grad_hidden summed over the vocabulary shards through peer memory")


def bench_cp(args, rank, world):
    from rl_engine.parallel.context_parallel import ContextParallelAttention

    hq, hkv = 32, 8
    s = args.cp_tokens // (256 * world) * 256 * world
    cp = ContextParallelAttention(s, hkv, device=torch.device("cuda", torch.cuda.current_device()))
    local = s // world
    q, k, v = (rnd((local, h, 128), seed=5 + i + 10 * rank).requires_grad_(True) for i, h in enumerate((hq, hkv, hkv)))
    do = rnd((local, hq, 128), seed=99 + rank)

    def fwd_bwd():
        q.grad = k.grad = v.grad = None
        cp(q, k, v).backward(do)

    ms = timed(fwd_bwd, args.warmup, args.repeat)
    flops = 4.5 * 4.0 * hq * 128 * (s / world) * (s + 1) / 2          # fwd 1x + bwd 3.5x of the causal QK^T + PV work
    kv_bytes = 2 * (world - 1) * local * hkv * 128 * 2.0               # K and V from every peer ...
    emit(rank, "cp_attention_fwd_bwd", ms, flops, 2 * kv_bytes + kv_bytes,  # ... twice (fwd, bwd re-gather) + dK/dV partials
         shape=[s, hq, hkv], note="zig-zag shards; K/V gathered by peer stores; dK/dV reduced by peer loads in rank order")
    cp.mem.check()


def bench_ep(args, rank, world):
    from rl_engine.parallel.expert_parallel import ExpertParallelContext, ExpertParallelMoE

    e, k, h, f = 128, 8, 2048, 768
    t = args.moe_tokens
    ctx = ExpertParallelContext(h, e, k, max_tokens=t, device=torch.device("cuda", torch.cuda.current_device()),
                                capacity_factor=2.0 if world > 1 else None)
    op = ExpertParallelMoE(ctx)
    el = e // world
    x = rnd((t, h), seed=rank).requires_grad_(True)
    router = rnd((e, h), 1.0 / 45.0, 7).requires_grad_(True)            # router logits ~ N(0, 1)
    w1 = rnd((el * 2 * f, h), 0.02, 20 + rank).requires_grad_(True)
    w2 = rnd((el * h, f), 0.02, 40 + rank).requires_grad_(True)
    do = rnd((t, h), seed=60 + rank)

    def fwd_bwd():
        x.grad = router.grad = w1.grad = w2.grad = None
        op(x, router, w1, w2).backward(do)

    ms = timed(fwd_bwd, args.warmup, args.repeat)
    flops = 3.0 * 2.0 * t * k * (h * 2 * f + f * h)                      # fwd + dgrad + wgrad of both expert GEMMs
    moved = 4.0 * t * k * h * 2.0 * (world - 1) / world                   # dispatch + combine, forward and backward
    emit(rank, "ep_moe_layer_fwd_bwd", ms, flops, moved, shape=[t, h, e, k, f],
         note="Qwen3-30B-A3B layer shapes; routed rows stored to the owners, expert outputs read back from the peers")
    ctx.mem.check()


def bench_zero1(args, rank, world):
    from rl_engine.kernels.ops.base import require_ext
    from rl_engine.parallel.symmetric import SymmetricMemory

    ext = require_ext()
    n = args.zero1_params // (8 * world) * 8 * world
    mem = SymmetricMemory(4 * n + (1 << 20))
    params, grads = mem.alloc((n,), torch.bfloat16), mem.alloc((n,), torch.bfloat16)
    params.local.normal_()
    grads.local.normal_()
    per = n // world
    lo, hi = rank * per, (rank + 1) * per
    m, v = torch.zeros(per, device="cuda"), torch.zeros(per, device="cuda")
    master = params.local[lo:hi].float()
    step = [0]

    def run():
        step[0] += 1
        mem.barrier()
        ext.zero1_fused_step(grads.ptrs, params.ptrs, lo, hi, m, v, master, 1e-6, 0.9, 0.95, 1e-8, 0.0, step[0], 1.0 / world, rank, None, 0)
        mem.barrier()

    ms = timed(run, args.warmup, args.repeat)
    link = (world - 1) * per * 2.0 * 2                                   # read peers' gradient shards + write parameters to peers
    if rank == 0:
        hbm = (per * (2.0 * world + 4 * 3 * 2) + n * 2.0) / ms / 1e6
        print(json.dumps({"path": "zero1_fused_step", "world": world, "ms": round(ms, 4), "params": n,
                          "nvlink_gbs_per_gpu": round(link / ms / 1e6, 1) if world > 1 else None,
                          "local_hbm_gbs": round(hbm, 1), "roofline_ms": round(link / (NVLINK_GBS * 1e6), 4) if world > 1 else None,
                          "frac_of_roofline": round(link / (NVLINK_GBS * 1e6) / ms, 3) if world > 1 else None}), flush=True)
    mem.check()


def bench_broadcast(args, rank, world):
    from rl_engine.kernels.ops.base import require_ext
    from rl_engine.parallel.symmetric import SymmetricMemory

    ext = require_ext()
    n = args.broadcast_params
    mem = SymmetricMemory(2 * n + (1 << 20))
    window = mem.alloc((n,), torch.bfloat16)
    src = torch.randn(n, device="cuda") if rank == 0 else None

    def run():
        mem.barrier()
        if rank == 0:
            ext.cast_broadcast(src, window.ptrs, 1)
        mem.barrier()

    ms = timed(run, args.warmup, args.repeat)
    ok = True
    if rank == 0:
        ok = torch.equal(window.local, src.to(torch.bfloat16))
    sent = (world - 1) * n * 2.0
    if rank == 0:
        print(json.dumps({"path": "weight_broadcast_cast", "world": world, "ms": round(ms, 4), "params": n,
                          "egress_gbs": round(sent / ms / 1e6, 1) if world > 1 else None,
                          "roofline_ms": round(max(sent / (NVLINK_GBS * 1e6), n * 4.0 / (peaks()["hbm_gbs"] * 1e6)), 4),
                          "frac_of_roofline": round(max(sent / (NVLINK_GBS * 1e6), n * 4.0 / (peaks()["hbm_gbs"] * 1e6)) / ms, 3),
                          "verified": bool(ok),
                          "note": "fp32 trainer weights read once, cast to bf16, stored into every rank's window"}), flush=True)
    mem.check()


def bench_weight_sync(args, rank, world):
    """The whole trainer -> rollout weight update through ``NVLinkBroadcastBridge.sync`` at the size of a model state
    (``--sync-gb`` of bf16 in ``--sync-tensors`` tensors): cast + stores, relay hop, manifest shipped with
    ``broadcast_object_list``, import, digest validation and acknowledge on every rank.  Times are host wall clock around
    the collective call with a device synchronise on both sides, max over ranks (the call contains host work)."""
    import time

    from rl_engine.executors.bridge import NVLinkBroadcastBridge
    from rl_engine.parallel.symmetric import SymmetricMemory

    total = int(args.sync_gb * (1 << 30))
    count = args.sync_tensors
    per = total // count // 512 * 256  # bf16 elements per tensor
    nbytes = per * 2 * count + 256 * count
    mem = SymmetricMemory((2 if world > 2 else 1) * (nbytes + 4096) + (1 << 20))  # one window per measured mode
    results = {}
    for relay in ((True, False) if world > 2 else (False,)):
        bridge = NVLinkBroadcastBridge(mem, nbytes, relay=relay, stores=args.sync_stores)
        state = None
        if rank == 0:
            flat = torch.empty(per * count, dtype=torch.bfloat16, device="cuda").normal_()
            state = {f"t{i}": flat[i * per:(i + 1) * per] for i in range(count)}
        samples = []
        for it in range(args.warmup + args.repeat):
            torch.cuda.synchronize()
            dist.barrier()
            t0 = time.perf_counter()
            manifest, tensors = bridge.sync(state, weight_version=it + 1)
            torch.cuda.synchronize()
            t = torch.tensor([time.perf_counter() - t0], device="cuda", dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            if it >= args.warmup:
                samples.append(float(t) * 1e3)
            if it + 1 < args.warmup + args.repeat:
                bridge.release(manifest.update_id)
        ok = torch.tensor([1], device="cuda")
        if rank == 0:
            ok[0] = int(torch.equal(tensors["t0"], state["t0"]) and torch.equal(tensors[f"t{count - 1}"], state[f"t{count - 1}"]))
        check = tensors[f"t{count // 2}"].float().sum().reshape(1).double()
        lo, hi = check.clone(), check.clone()
        dist.all_reduce(lo, op=dist.ReduceOp.MIN)
        dist.all_reduce(hi, op=dist.ReduceOp.MAX)
        results[relay] = (statistics.median(samples), bool(ok.item()) and float(lo) == float(hi))
        mem.check()
        del bridge, state
        torch.cuda.empty_cache()
    if rank == 0:
        size = per * 2 * count
        for relay, (ms, ok) in results.items():
            # unique bytes must leave the source once (relay) or once per peer (direct); every peer must receive all
            roof = (size if relay else size * (world - 1)) / (NVLINK_GBS * 1e6) if world > 1 else size * 2 / (peaks()["hbm_gbs"] * 1e6)
            print(json.dumps({"path": "weight_sync_bridge", "mode": "relay" if relay else "direct", "world": world,
                              "stores": args.sync_stores, "ms": round(ms, 3), "gbytes": round(size / 2**30, 2), "tensors": count,
                              "delivered_gbs_per_rank": round(size / ms / 1e6, 1), "roofline_ms": round(roof, 3),
                              "frac_of_roofline": round(roof / ms, 3), "verified_identical_on_all_ranks": ok,
                              "note": "publish + manifest broadcast + import + device digest check + acknowledge"}), flush=True)
    mem.close()


PATHS = {"tp": bench_tp, "linear_logp": bench_linear_logp, "cp": bench_cp, "ep": bench_ep, "zero1": bench_zero1,
         "broadcast": bench_broadcast, "weight_sync": bench_weight_sync}


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--paths", default="all", help=f"comma-separated subset of {sorted(PATHS)} or 'all'")
    ap.add_argument("--tokens", type=int, default=16384, help="token rows for the TP linears")
    ap.add_argument("--logp-tokens", type=int, default=8192)
    ap.add_argument("--cp-tokens", type=int, default=36864, help="sequence length for context-parallel attention")
    ap.add_argument("--moe-tokens", type=int, default=8192, help="tokens per rank for the MoE layer")
    ap.add_argument("--zero1-params", type=int, default=1 << 29)
    ap.add_argument("--broadcast-params", type=int, default=1 << 29)
    ap.add_argument("--sync-gb", type=float, default=1.0, help="bytes of bf16 state for the weight_sync path (16 = Llama-3-8B)")
    ap.add_argument("--sync-stores", choices=["copy-engine", "kernel"], default="copy-engine",
                    help="weight_sync path: table-driven cast + copy-engine transfers, or one fused cast + peer-store kernel per tensor")
    ap.add_argument("--sync-tensors", type=int, default=291, help="number of tensors the state is split into")
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--repeat", type=int, default=5)
    args = ap.parse_args()
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    if "MASTER_ADDR" not in os.environ:
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT="29600")
    # a short collective timeout: a rank that failed alone ends the run with an error instead of stalling the others
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", local),
                            timeout=datetime.timedelta(seconds=180))
    names = sorted(PATHS) if args.paths == "all" else [p.strip() for p in args.paths.split(",") if p.strip()]
    for name in names:
        try:
            PATHS[name](args, rank, world)
        except Exception as exc:  # one path failing must not hide the others
            if rank == 0:
                print(json.dumps({"path": name, "status": "blocked", "notes": (str(exc).splitlines() or [type(exc).__name__])[0]}), flush=True)
        torch.cuda.empty_cache()
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
