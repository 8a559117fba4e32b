"""Multi-rank checks, launched as ``torchrun --nproc-per-node N tests/multigpu/run_parallel_checks.py``.

Covers: symmetric heap mapping + device barrier, vocab-parallel fused linear_logp (forward bitwise
equal on all ranks and close to the single-GPU op, backward vs autograd), the fused
reduce-scatter + AdamW + all-gather step vs a single-process AdamW, and the weight broadcast+cast.
Every rank prints ``OK <name>`` lines; rank 0 prints ``ALL OK`` at the end.
"""

import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))


def main() -> None:
    rank = int(os.environ["RANK"])
    local = int(os.environ["LOCAL_RANK"])
    world = int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)

    from rl_engine.kernels.ops.base import check_device_errors, require_ext
    from rl_engine.kernels.ops.sm100.linear_logp import FusedLinearLogpSM100Op
    from rl_engine.parallel.symmetric import SymmetricMemory

    ext = require_ext()

    # ---- symmetric heap + barrier -------------------------------------------------------------
    mem = SymmetricMemory(1 << 22, device=dev)
    buf = mem.alloc((1024,), torch.float32)
    buf.local.fill_(float(rank + 1))
    mem.barrier()
    for r in range(world):
        assert float(buf.peer(r)[7]) == r + 1, "peer mapping shows the wrong data"
    mem.barrier()
    mem.check()
    print(f"[{rank}] OK symmetric heap", flush=True)

    # ---- weight broadcast + cast ---------------------------------------------------------------
    dst = mem.alloc((4096,), torch.bfloat16)
    src = torch.arange(4096, device=dev, dtype=torch.float32) * 0.25 + 1000 * 0
    if rank == 0:
        ext.cast_broadcast(src, dst.ptrs, 1)
    mem.barrier()
    assert torch.equal(dst.local.float(), src.to(torch.bfloat16).float())
    mem.check()
    print(f"[{rank}] OK cast_broadcast", flush=True)

    # ---- vocab-parallel fused linear_logp -------------------------------------------------------
    g = torch.Generator(device=dev).manual_seed(5)  # same data on all ranks
    N, D, V = 600, 256, 20000 + 8 * 37
    h = torch.randn(N, D, device=dev, generator=g).to(torch.bfloat16)
    w = (torch.randn(V, D, device=dev, generator=g) * 0.05).to(torch.bfloat16)
    t = torch.randint(0, V, (N,), device=dev, generator=g)
    gl = torch.randn(N, device=dev, generator=g)
    bounds = [0] + [int(V * (i + 1) / world) // 8 * 8 + (3 * 8 if i % 2 == 0 else 0) for i in range(world - 1)] + [V]
    v0, v1 = bounds[rank], bounds[rank + 1]
    op = FusedLinearLogpSM100Op()
    hs = h.clone().requires_grad_(True)
    ws = w[v0:v1].clone().requires_grad_(True)
    lp = op(hs, ws, t, tp_group=dist.group.WORLD, vocab_start_index=v0, global_vocab_size=V)
    lp.backward(gl)
    hf = h.clone().requires_grad_(True)
    wf = w.clone().requires_grad_(True)
    full = op(hf, wf, t)
    full.backward(gl)
    assert torch.allclose(lp, full, atol=2e-3, rtol=1e-3), (lp - full).abs().max()
    gathered = [torch.empty_like(lp) for _ in range(world)]
    dist.all_gather(gathered, lp.detach())
    assert all(torch.equal(gathered[0], x) for x in gathered), "ranks disagree bitwise"
    sc = hf.grad.float().abs().max()
    assert (hs.grad.float() - hf.grad.float()).abs().max() / sc < 2e-2
    scw = wf.grad.float().abs().max()
    assert (ws.grad.float() - wf.grad[v0:v1].float()).abs().max() / scw < 2e-2
    lp2 = op(h, w[v0:v1].contiguous(), t, tp_group=dist.group.WORLD, vocab_start_index=v0, global_vocab_size=V)
    assert torch.equal(lp2, lp.detach()), "TP forward is not run-to-run deterministic"
    check_device_errors(local)
    print(f"[{rank}] OK tp linear_logp (max |tp - full| = {(lp - full).abs().max().item():.2e})", flush=True)

    # ---- fused reduce-scatter + AdamW + all-gather ----------------------------------------------
    n = 8 * 1000 * world + 8 * 13
    params = mem.alloc((n,), torch.bfloat16)
    grads = mem.alloc((n,), torch.bfloat16)
    gp = torch.Generator(device=dev).manual_seed(11)
    p0 = torch.randn(n, device=dev, generator=gp)
    params.local.copy_(p0.to(torch.bfloat16))
    gr = torch.Generator(device=dev).manual_seed(100 + rank)
    grads.local.copy_(torch.randn(n, device=dev, generator=gr).to(torch.bfloat16))
    per = ((n + world - 1) // world + 7) // 8 * 8
    lo, hi = min(rank * per, n), min(rank * per + per, n)
    m = torch.zeros(hi - lo, device=dev)
    v = torch.zeros(hi - lo, device=dev)
    master = params.local[lo:hi].float()
    all_grads = [torch.randn(n, device=dev, generator=torch.Generator(device=dev).manual_seed(100 + r)).to(torch.bfloat16)
                 for r in range(world)]
    mem.barrier()
    ext.zero1_fused_step(grads.ptrs, params.ptrs, lo, hi, m, v, master, 1e-2, 0.9, 0.95, 1e-8, 0.1, 1, 1.0 / world)
    mem.barrier()
    ref = params.local.new_empty(n, dtype=torch.float32).copy_(p0.to(torch.bfloat16).float()).requires_grad_(True)
    opt = torch.optim.AdamW([ref], lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    gsum = torch.zeros(n, device=dev)
    for r in range(world):
        gsum += all_grads[r].float()
    ref.grad = gsum / world
    opt.step()
    assert torch.allclose(params.local.float(), ref.detach(), atol=2e-2, rtol=2e-2)
    both = [torch.empty_like(params.local) for _ in range(world)]
    dist.all_gather(both, params.local)
    assert all(torch.equal(both[0], x) for x in both), "parameters diverged between ranks"
    mem.check()
    print(f"[{rank}] OK zero1 fused step", flush=True)

    dist.barrier()
    if rank == 0:
        print("ALL OK", flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
