"""Multi-rank checks, launched as ``torchrun --nproc-per-node N tests/multigpu/run_parallel_checks.py``.

Covers: symmetric heap mapping + device barrier, vocab-parallel fused linear_logp (forward bitwise
equal on all ranks and close to the single-GPU op, backward vs autograd), the fused
reduce-scatter + AdamW + all-gather step vs a single-process AdamW, one data-parallel GRPO step (bucketed and
overlapped with backward) vs the single-GPU trainer on the same batch, the weight broadcast+cast, the
tensor-parallel linears fused with their all-gather / reduce-scatter, the context-parallel causal attention
(zig-zag shards) against full-sequence attention, and the expert-parallel MoE (peer-store dispatch / peer-load combine) against the single-GPU fused MoE.
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
    mem = SymmetricMemory(1 << 23, device=dev)
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

    # ---- the weight-update protocol over symmetric memory, relay and direct -----------------------------
    from rl_engine.executors.bridge import NVLinkBroadcastBridge

    for relay in (True, False):
        bridge = NVLinkBroadcastBridge(mem, 1 << 20, target_dtype=torch.bfloat16, relay=relay)
        state = None
        if rank == 0:
            gs = torch.Generator(device=dev).manual_seed(8)
            state = {"a.weight": torch.randn(300, 257, device=dev, generator=gs), "b.bias": torch.randn(19, device=dev, generator=gs),
                     "steps": torch.tensor([3, 4, 5], device=dev)}
        manifest, views = bridge.sync(state, weight_version=1)
        want = torch.randn(300, 257, device=dev, generator=torch.Generator(device=dev).manual_seed(8)).to(torch.bfloat16)
        assert torch.equal(views["a.weight"], want), f"weight sync (relay={relay}): wrong bytes on rank {rank}"
        assert views["steps"].tolist() == [3, 4, 5] and bridge.active_weight_version == 1
        assert manifest.metadata["weight_bridge"]["relay"] == (relay and world > 1)
    mem.check()
    print(f"[{rank}] OK weight sync bridge (relay + direct)", flush=True)

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
    ext.zero1_fused_step(grads.ptrs, params.ptrs, lo, hi, m, v, master, 1e-2, 0.9, 0.95, 1e-8, 0.1, 1, 1.0 / world, rank, None, 0)
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

    # ---- expert-parallel MoE over peer stores / loads ----------------------------------------------
    from rl_engine.kernels.ops.sm100.moe import FusedMoESM100Op
    from rl_engine.parallel.expert_parallel import ExpertParallelContext, ExpertParallelMoE

    E, K, H, F, T = 4 * world, 2, 256, 128, 300 + 17 * rank
    gw = torch.Generator(device=dev).manual_seed(21)  # same weights on all ranks
    router = (torch.randn(E, H, device=dev, generator=gw) * 0.3).to(torch.bfloat16)
    w1 = (torch.randn(E * 2 * F, H, device=dev, generator=gw) * 0.06).to(torch.bfloat16)
    w2 = (torch.randn(E * H, F, device=dev, generator=gw) * 0.09).to(torch.bfloat16)
    gx = torch.Generator(device=dev).manual_seed(300 + rank)  # own tokens
    x = torch.randn(T, H, device=dev, generator=gx).to(torch.bfloat16)
    dout = torch.randn(T, H, device=dev, generator=gx).to(torch.bfloat16)
    el = E // world
    ctx = ExpertParallelContext(H, E, K, max_tokens=300 + 17 * world, group=dist.group.WORLD, device=dev)
    ep_op = ExpertParallelMoE(ctx)
    xe = x.clone().requires_grad_(True)
    re_ = router.clone().requires_grad_(True)
    w1l = w1.view(E, 2 * F, H)[rank * el:(rank + 1) * el].reshape(-1, H).clone().requires_grad_(True)
    w2l = w2.view(E, H, F)[rank * el:(rank + 1) * el].reshape(-1, F).clone().requires_grad_(True)
    out_ep = ep_op(xe, re_, w1l, w2l)
    out_ep.backward(dout)
    xf = x.clone().requires_grad_(True)
    rf = router.clone().requires_grad_(True)
    w1f = w1.clone().requires_grad_(True)
    w2f = w2.clone().requires_grad_(True)
    out_full = FusedMoESM100Op()(xf, rf, w1f, w2f, K)
    out_full.backward(dout)

    def close(a, b, tol, what):
        scale = b.float().abs().max().clamp_min(1e-6)
        err_ = ((a.float() - b.float()).abs().max() / scale).item()
        assert err_ < tol, f"expert parallel {what}: relative error {err_:.3e}"

    close(out_ep, out_full, 2e-2, "output")
    close(xe.grad, xf.grad, 2e-2, "dx")
    close(re_.grad, rf.grad, 3e-2, "router grad")
    g1 = w1f.grad.float().clone()
    g2 = w2f.grad.float().clone()
    dist.all_reduce(g1)
    dist.all_reduce(g2)
    close(w1l.grad, g1.view(E, 2 * F, H)[rank * el:(rank + 1) * el].reshape(-1, H), 2e-2, "dW1")
    close(w2l.grad, g2.view(E, H, F)[rank * el:(rank + 1) * el].reshape(-1, F), 2e-2, "dW2")
    out_again = ep_op(x, router, w1l.detach(), w2l.detach())
    assert torch.equal(out_again, out_ep.detach()), "expert-parallel forward is not run-to-run deterministic"
    ctx.mem.check()
    check_device_errors(local)
    print(f"[{rank}] OK expert-parallel MoE", flush=True)

    # ---- a whole Llama layer under tensor + sequence parallelism vs the single-GPU layer ---------------
    from rl_engine.kernels.ops.sm100.attention import make_layout
    from rl_engine.models.config import ModelConfig
    from rl_engine.models.llama import LlamaModel
    from rl_engine.parallel.tp_linear import TensorParallelLinears as _TPL
    from rl_engine.parallel.tp_transformer import TensorParallelLlamaLayer, shard_layer_weights

    tp_layer = _TPL(group=dist.group.WORLD, device=dev)

    cfg = ModelConfig("tp-check", 1024, 512, 1, 4 * world, 2 * world, 128, 512 * world)
    full = LlamaModel(cfg, dtype=torch.bfloat16, device=dev, seed=9, activation_checkpointing=False)
    TT = 256 * world
    gl_ = torch.Generator(device=dev).manual_seed(901)
    xin = torch.randn(TT, cfg.hidden_size, device=dev, generator=gl_).to(torch.bfloat16)
    dout_l = torch.randn(TT, cfg.hidden_size, device=dev, generator=gl_).to(torch.bfloat16)
    pos = torch.arange(TT, device=dev)
    lay = make_layout([(0, TT, 0, 0, 0, TT)], True, dev)
    xf = xin.clone().requires_grad_(True)
    yf = full._layer(xf, 0, pos, lay)
    yf.backward(dout_l)
    shard = {k: v.requires_grad_(True) for k, v in shard_layer_weights(full, 0, rank, world).items()}
    layer = TensorParallelLlamaLayer(cfg, shard, tp_layer, full.rope_cos, full.rope_sin)
    tok = slice(rank * 256, (rank + 1) * 256)
    xl_ = xin[tok].clone().requires_grad_(True)
    yl = layer(xl_, pos, lay)
    yl.backward(dout_l[tok].contiguous())
    close(yl, yf.detach()[tok], 3e-2, "tp layer output")
    close(xl_.grad, xf.grad[tok], 3e-2, "tp layer dx")
    hq_l, d_ = cfg.num_heads // world, cfg.head_dim
    close(shard["wo"].grad, full.params[full._index["l0.wo"]].grad[:, rank * hq_l * d_:(rank + 1) * hq_l * d_], 3e-2, "tp layer dWo")
    f_l = cfg.ffn_size // world
    close(shard["w_down"].grad, full.params[full._index["l0.w_down"]].grad[:, rank * f_l:(rank + 1) * f_l], 3e-2, "tp layer dWdown")
    gq = full.params[full._index["l0.wqkv"]].grad[: cfg.q_dim].view(cfg.num_heads, d_, -1)[rank * hq_l:(rank + 1) * hq_l]
    close(shard["wqkv"].grad[: hq_l * d_], gq.reshape(hq_l * d_, -1), 3e-2, "tp layer dWq")
    norm_g = shard["mlp_norm"].grad.float().clone()
    dist.all_reduce(norm_g)
    close(norm_g, full.params[full._index["l0.mlp_norm"]].grad, 3e-2, "tp layer d(mlp_norm), summed over ranks")
    tp_layer.check()
    print(f"[{rank}] OK tensor-parallel Llama layer", flush=True)

    # ---- a whole GRPO step under tensor parallelism vs the single-GPU trainer ---------------------------
    from rl_engine.models.grpo import GRPOTrainer, synthetic_batch
    from rl_engine.parallel.tp_model import TensorParallelGRPOTrainer, TensorParallelLlama

    mcfg = ModelConfig("tp-model", 2048, 512, 2, max(8, 2 * world), max(4, world), 128, 1024)
    ref_model = LlamaModel(mcfg, dtype=torch.bfloat16, device=dev, seed=21)
    tp_model = TensorParallelLlama(ref_model, _TPL(group=dist.group.WORLD, device=dev))
    hb = synthetic_batch(mcfg.vocab_size, prompt_len=256, group=4, completion_len=192, seed=3)
    ref_tr = GRPOTrainer(ref_model, lr=1e-3)
    tp_tr = TensorParallelGRPOTrainer(tp_model, lr=1e-3)
    db = hb.to(dev)
    with torch.no_grad():
        lp_ref = ref_tr.policy_logps(db)
        lp_tp = tp_model.policy_logps(db)
    assert torch.allclose(lp_tp, lp_ref, atol=5e-2, rtol=5e-2), (lp_tp - lp_ref).abs().max()
    allg = [torch.empty_like(lp_tp) for _ in range(world)]
    dist.all_gather(allg, lp_tp)
    assert all(torch.equal(allg[0], t_) for t_ in allg), "TP log-probs differ between ranks"
    loss_ref = [ref_tr.step(hb) for _ in range(3)]
    loss_tp = [tp_tr.step(hb) for _ in range(3)]
    assert abs(loss_tp[0] - loss_ref[0]) < 2e-2 * max(1.0, abs(loss_ref[0])), (loss_tp, loss_ref)
    assert loss_tp[-1] < loss_tp[0], f"TP training does not reduce the loss: {loss_tp}"
    close(tp_model.params["final_norm"], ref_model.view("final_norm"), 2e-2, "tp model final_norm after 3 steps")
    hq_m = mcfg.num_heads // world * mcfg.head_dim
    close(tp_model.params["l1.wo"], ref_model.view("l1.wo")[:, rank * hq_m:(rank + 1) * hq_m], 5e-2, "tp model wo shard after 3 steps")
    check_device_errors(local)
    print(f"[{rank}] OK tensor-parallel GRPO step (loss {loss_tp[0]:.4f} -> {loss_tp[-1]:.4f}, single GPU {loss_ref[0]:.4f} -> {loss_ref[-1]:.4f})", flush=True)

    # ---- data-parallel GRPO step (bucketed fused reduce-scatter + AdamW + all-gather, overlapped with the last
    # ---- backward pass) vs the single-GPU trainer on the same batch ------------------------------------------
    from rl_engine.models.grpo import GRPOBatch
    from rl_engine.parallel.data_parallel import ShardedGRPOTrainer

    dcfg = ModelConfig("dp-check", 2048, 512, 3, 8, 4, 128, 1024)
    per_rank = 2
    G_dp = per_rank * world
    hb_dp = synthetic_batch(dcfg.vocab_size, prompt_len=256, group=G_dp, completion_len=192, seed=5)
    single = LlamaModel(dcfg, dtype=torch.bfloat16, device=dev, seed=33, activation_checkpointing=False)
    start = single.flat.clone()
    single_tr = GRPOTrainer(single, lr=1e-3, micro_group=None)
    with torch.no_grad():
        cur = single_tr.policy_logps(hb_dp.to(dev)).float()
    gn = torch.Generator(device=dev).manual_seed(71)  # the same noise on every rank
    hb_dp.old_logps = (cur + 0.01 * torch.randn(cur.shape, device=dev, generator=gn)).cpu()
    hb_dp.ref_logps = (cur + 0.01 * torch.randn(cur.shape, device=dev, generator=gn)).cpu()
    full_dev = hb_dp.to(dev)
    loss_single = [float(single_tr.step_device(full_dev)) for _ in range(2)]
    sl = slice(rank * per_rank, (rank + 1) * per_rank)
    local_dev = GRPOBatch(full_dev.prompt_ids, full_dev.completion_ids[sl].contiguous(), full_dev.rewards,
                          full_dev.old_logps[sl].contiguous(), full_dev.ref_logps[sl].contiguous(),
                          full_dev.completion_mask[sl].contiguous())
    results = {}
    for name, kw in (("one pass, overlapped", dict(micro_group=None, overlap=True, shard_prompt=False)),
                     ("one pass, not overlapped", dict(micro_group=None, overlap=False, shard_prompt=False)),
                     ("prompt pass + micro-batches, overlapped", dict(micro_group=1, overlap=True, shard_prompt=False)),
                     ("sharded prompt pass + one pass", dict(micro_group=None, overlap=True, shard_prompt=True)),
                     ("sharded prompt pass + micro-batches", dict(micro_group=1, overlap=False, shard_prompt=True))):
        model_dp = LlamaModel(dcfg, dtype=torch.bfloat16, device=dev, seed=33, activation_checkpointing=False)
        assert torch.equal(model_dp.flat, start)
        dp_tr = ShardedGRPOTrainer(model_dp, lr=1e-3, layers_per_bucket=1, **kw)
        dp_tr.set_group_slice(sl)
        losses = []
        for _ in range(2):
            l_ = dp_tr.step_device(local_dev).float().reshape(1)
            dist.all_reduce(l_, op=dist.ReduceOp.AVG)
            losses.append(float(l_))
        dp_tr.check()
        check_device_errors(local)
        every = [torch.empty_like(model_dp.flat) for _ in range(world)]
        dist.all_gather(every, model_dp.flat.contiguous())
        assert all(torch.equal(every[0], e_) for e_ in every), f"data parallel ({name}): parameters differ between ranks"
        assert abs(losses[0] - loss_single[0]) < 2e-2 * max(1.0, abs(loss_single[0])), (name, losses, loss_single)
        d_dp = model_dp.flat.float() - start.float()
        d_one = single.flat.float() - start.float()
        moved = d_one.abs() > 0
        assert moved.float().mean() > 0.5, "the single-GPU reference step did not move the parameters"
        # AdamW's first steps are close to lr * sign(gradient): compare the updates, not just the parameters
        rel = ((d_dp - d_one).abs().mean() / d_one.abs().mean()).item()
        agree = (torch.sign(d_dp[moved]) == torch.sign(d_one[moved])).float().mean().item()
        assert rel < 0.25 and agree > 0.9, f"data parallel ({name}): update differs from the single-GPU step: {rel:.3f}, {agree:.3f}"
        results[name] = model_dp.flat.clone()
        assert bool(dp_tr._prompt_shards) == ("sharded" in name), (name, "prompt sharding was not what the case asked for")
        dp_tr.close()
    assert torch.equal(results["one pass, overlapped"], results["one pass, not overlapped"]), \
        "overlapping the gradient exchange with backward changed the result"
    print(f"[{rank}] OK data-parallel GRPO step == single-GPU step (loss {losses[0]:.4f} vs {loss_single[0]:.4f})", flush=True)

    # ---- context-parallel causal attention (zig-zag shards, peer-store K/V gather, peer_sum dK/dV) ----
    from rl_engine.kernels.ops.sm100.attention import FlashAttentionSM100Op
    from rl_engine.parallel.context_parallel import ContextParallelAttention, shard_sequence

    HQ, HKV, C = 4, 2, 192
    S = 2 * world * C
    ga = torch.Generator(device=dev).manual_seed(77)  # same full sequence on all ranks
    qa = torch.randn(S, HQ, 128, device=dev, generator=ga).to(torch.bfloat16)
    ka = torch.randn(S, HKV, 128, device=dev, generator=ga).to(torch.bfloat16)
    va = torch.randn(S, HKV, 128, device=dev, generator=ga).to(torch.bfloat16)
    da = torch.randn(S, HQ, 128, device=dev, generator=ga).to(torch.bfloat16)
    cp = ContextParallelAttention(S, HKV, group=dist.group.WORLD, device=dev)
    ql, kl, vl = (shard_sequence(t, rank, world).clone().requires_grad_(True) for t in (qa, ka, va))
    out_cp = cp(ql, kl, vl)
    out_cp.backward(shard_sequence(da, rank, world))
    qf_, kf_, vf_ = (t.clone().requires_grad_(True) for t in (qa, ka, va))
    full_out = FlashAttentionSM100Op()(qf_[None], kf_[None], vf_[None], causal=True)[0]
    full_out.backward(da)
    close(out_cp, shard_sequence(full_out.detach(), rank, world), 2e-2, "cp output")
    close(ql.grad, shard_sequence(qf_.grad, rank, world), 2e-2, "cp dq")
    close(kl.grad, shard_sequence(kf_.grad, rank, world), 2e-2, "cp dk")
    close(vl.grad, shard_sequence(vf_.grad, rank, world), 2e-2, "cp dv")
    out_cp2 = cp(ql.detach(), kl.detach(), vl.detach())
    assert torch.equal(out_cp2, out_cp.detach()), "context-parallel forward is not run-to-run deterministic"
    cp.mem.check()
    check_device_errors(local)
    print(f"[{rank}] OK context-parallel attention", flush=True)

    # ---- mixture-of-experts model: data parallel + expert parallel GRPO step vs the single-GPU model with all experts ----
    from rl_engine.parallel.expert_parallel import expert_parallel_trainer

    ecfg = ModelConfig("ep-model", vocab_size=2048, hidden_size=256, num_layers=2, num_heads=4, num_kv_heads=2, head_dim=128,
                       ffn_size=512, rms_eps=1e-6, rope_theta=1e6, num_experts=4 * world, experts_per_token=2,
                       moe_ffn_size=128, qk_norm=True)
    full_moe = LlamaModel(ecfg, dtype=torch.bfloat16, device=dev, seed=55)
    shard_moe = LlamaModel(ecfg, dtype=torch.bfloat16, device=dev, seed=55, expert_shard=(rank, world))
    el_m, fe_m, hm = ecfg.num_experts // world, ecfg.moe_ffn_size, ecfg.hidden_size
    with torch.no_grad():  # replicated parameters from the full model, experts: this rank's slice
        for name, dst in shard_moe.named_views().items():
            src = full_moe.view(name)
            if name.endswith("w_gate_up"):
                src = src.view(ecfg.num_experts, 2 * fe_m, hm)[rank * el_m:(rank + 1) * el_m].reshape(-1, hm)
            elif name.endswith("w_down"):
                src = src.view(ecfg.num_experts, hm, fe_m)[rank * el_m:(rank + 1) * el_m].reshape(-1, fe_m)
            dst.copy_(src)
    per_rank_m = 2
    hb_m = synthetic_batch(ecfg.vocab_size, prompt_len=128, group=per_rank_m * world, completion_len=128, seed=6)
    full_tr = GRPOTrainer(full_moe, lr=1e-3, micro_group=None)
    with torch.no_grad():
        cur_m = full_tr.policy_logps(hb_m.to(dev)).float()
    gm = torch.Generator(device=dev).manual_seed(73)
    hb_m.old_logps = (cur_m + 0.01 * torch.randn(cur_m.shape, device=dev, generator=gm)).cpu()
    hb_m.ref_logps = (cur_m + 0.01 * torch.randn(cur_m.shape, device=dev, generator=gm)).cpu()
    db_m = hb_m.to(dev)
    start_m = {n: t.detach().clone() for n, t in shard_moe.named_views().items()}
    ep_tr = expert_parallel_trainer(shard_moe, max_tokens=128 + per_rank_m * 128, lr=1e-3, micro_group=None)
    sl_m = slice(rank * per_rank_m, (rank + 1) * per_rank_m)
    ep_tr.set_group_slice(sl_m)
    local_m = GRPOBatch(db_m.prompt_ids, db_m.completion_ids[sl_m].contiguous(), db_m.rewards, db_m.old_logps[sl_m].contiguous(),
                        db_m.ref_logps[sl_m].contiguous(), db_m.completion_mask[sl_m].contiguous())
    with torch.no_grad():
        lp_ep = ep_tr.policy_logps(local_m).float()
    assert torch.allclose(lp_ep, cur_m[sl_m], atol=5e-2, rtol=5e-2), (lp_ep - cur_m[sl_m]).abs().max()
    loss_full = float(full_tr.step_device(db_m))
    l_ep = ep_tr.step_device(local_m).float().reshape(1)
    dist.all_reduce(l_ep, op=dist.ReduceOp.AVG)
    ep_tr.check()
    ep_tr.expert_context.mem.check()
    check_device_errors(local)
    assert abs(float(l_ep) - loss_full) < 2e-2 * max(1.0, abs(loss_full)), (float(l_ep), loss_full)

    def update_matches(name, got_after, want_after, got_before):
        d_got, d_want = got_after.float() - got_before.float(), want_after.float() - got_before.float()
        moved_ = d_want.abs() > 0
        if moved_.float().mean() < 0.2:
            return  # a parameter that hardly receives gradient (e.g. rows of experts no token was routed to)
        rel_ = ((d_got - d_want).abs().mean() / d_want.abs().mean().clamp_min(1e-12)).item()
        assert rel_ < 0.35, f"expert-parallel step: update of {name} differs from the single-GPU step ({rel_:.3f})"

    for name, after in shard_moe.named_views().items():
        want = full_moe.view(name).detach()
        if name.endswith("w_gate_up"):
            want = want.view(ecfg.num_experts, 2 * fe_m, hm)[rank * el_m:(rank + 1) * el_m].reshape(-1, hm)
        elif name.endswith("w_down"):
            want = want.view(ecfg.num_experts, hm, fe_m)[rank * el_m:(rank + 1) * el_m].reshape(-1, fe_m)
        update_matches(name, after.detach(), want, start_m[name])
    dense_names = [n for n in shard_moe.named_views() if not n.endswith(("w_gate_up", "w_down"))]
    blob = torch.cat([shard_moe.view(n).detach().reshape(-1) for n in dense_names])
    every = [torch.empty_like(blob) for _ in range(world)]
    dist.all_gather(every, blob)
    assert all(torch.equal(every[0], e_) for e_ in every), "expert parallel: replicated parameters differ between ranks"
    ep_tr.mem.close()
    print(f"[{rank}] OK expert-parallel MoE GRPO step == single-GPU step (loss {float(l_ep):.4f} vs {loss_full:.4f})", flush=True)

    # ---- long-context GRPO step: sequences sharded over the ranks (context parallel) vs the single-GPU trainer ----
    from rl_engine.parallel.long_context import ContextParallelGRPOTrainer

    P_cp, L_cp = 128 * world, 128 * world * 3                 # S = 512 * world: chunks of 256 tokens
    hb_cp = synthetic_batch(dcfg.vocab_size, prompt_len=P_cp, group=2, completion_len=L_cp, seed=9)
    hb_cp.completion_mask[1, -37:] = False                    # a ragged completion
    one = LlamaModel(dcfg, dtype=torch.bfloat16, device=dev, seed=44, activation_checkpointing=False)
    start_cp = one.flat.clone()
    one_tr = GRPOTrainer(one, lr=1e-3, micro_group=None)
    with torch.no_grad():
        cur_cp = one_tr.policy_logps(hb_cp.to(dev)).float()
    gcp = torch.Generator(device=dev).manual_seed(72)
    hb_cp.old_logps = (cur_cp + 0.01 * torch.randn(cur_cp.shape, device=dev, generator=gcp)).cpu()
    hb_cp.ref_logps = (cur_cp + 0.01 * torch.randn(cur_cp.shape, device=dev, generator=gcp)).cpu()
    db_cp = hb_cp.to(dev)
    cp_model = LlamaModel(dcfg, dtype=torch.bfloat16, device=dev, seed=44, activation_checkpointing=False)
    cp_tr = ContextParallelGRPOTrainer(cp_model, lr=1e-3, layers_per_bucket=1)
    with torch.no_grad():
        lp_cp = cp_tr.policy_logps(db_cp)
    assert torch.allclose(lp_cp, cur_cp, atol=5e-2, rtol=5e-2), (lp_cp - cur_cp).abs().max()
    loss_one = float(one_tr.step_device(db_cp))
    loss_cp = float(cp_tr.step_device(db_cp))
    cp_tr.check()
    check_device_errors(local)
    assert abs(loss_cp - loss_one) < 2e-2 * max(1.0, abs(loss_one)), (loss_cp, loss_one)
    every = [torch.empty_like(cp_model.flat) for _ in range(world)]
    dist.all_gather(every, cp_model.flat.contiguous())
    assert all(torch.equal(every[0], e_) for e_ in every), "context parallel: parameters differ between ranks"
    d_cp, d_one = cp_model.flat.float() - start_cp.float(), one.flat.float() - start_cp.float()
    moved = d_one.abs() > 0
    rel = ((d_cp - d_one).abs().mean() / d_one.abs().mean()).item()
    agree = (torch.sign(d_cp[moved]) == torch.sign(d_one[moved])).float().mean().item()
    assert rel < 0.25 and agree > 0.9, f"context-parallel step differs from the single-GPU step: {rel:.3f}, {agree:.3f}"
    cp_tr.mem.close()
    print(f"[{rank}] OK context-parallel GRPO step == single-GPU step (loss {loss_cp:.4f} vs {loss_one:.4f}, update diff {rel:.3f})", flush=True)

    # ---- tensor-parallel linears: all-gather -> GEMM and GEMM -> reduce-scatter in one kernel ---------
    from rl_engine.parallel.tp_linear import TensorParallelLinears

    tp = TensorParallelLinears(group=dist.group.WORLD, device=dev)
    RL, KK, NC, NR = 256, 512, 384 * world, 640
    MM = RL * world
    rows = slice(rank * RL, (rank + 1) * RL)
    for it in range(3):  # three rounds: both buffer parities and the monotonic counters get reused
        gt = torch.Generator(device=dev).manual_seed(500 + it)  # same full problem on all ranks
        X = torch.randn(MM, KK, device=dev, generator=gt).to(torch.bfloat16)
        WC = (torch.randn(NC, KK, device=dev, generator=gt) * 0.05).to(torch.bfloat16)
        DY = torch.randn(MM, NC, device=dev, generator=gt).to(torch.bfloat16)
        ncol = slice(rank * NC // world, (rank + 1) * NC // world)
        xl = X[rows].clone().requires_grad_(True)
        wl = WC[ncol].clone().requires_grad_(True)
        y = tp.column_parallel(xl, wl)
        y.backward(DY[:, ncol].contiguous())
        close(y, X.float() @ WC[ncol].float().t(), 1e-2, f"column-parallel output (round {it})")
        close(xl.grad, (DY.float() @ WC.float())[rows], 2e-2, f"column-parallel dx (round {it})")
        close(wl.grad, DY[:, ncol].float().t() @ X.float(), 1e-2, f"column-parallel dw (round {it})")

        KL = KK // world
        kcol = slice(rank * KL, (rank + 1) * KL)
        WR = (torch.randn(NR, KK, device=dev, generator=gt) * 0.05).to(torch.bfloat16)
        DY2 = torch.randn(MM, NR, device=dev, generator=gt).to(torch.bfloat16)
        x2 = X[:, kcol].clone().requires_grad_(True)
        w2l = WR[:, kcol].clone().requires_grad_(True)
        y2 = tp.row_parallel(x2, w2l)
        y2.backward(DY2[rows].contiguous())
        close(y2, (X.float() @ WR.float().t())[rows], 2e-2, f"row-parallel output (round {it})")
        close(x2.grad, DY2.float() @ WR[:, kcol].float(), 1e-2, f"row-parallel dx (round {it})")
        close(w2l.grad, DY2.float().t() @ X[:, kcol].float(), 1e-2, f"row-parallel dw (round {it})")
        y2b = tp.row_parallel(x2.detach(), w2l.detach())
        assert torch.equal(y2b, y2.detach()), "GEMM -> reduce-scatter is not run-to-run deterministic"
    tp.check()
    print(f"[{rank}] OK tensor-parallel fused linears", flush=True)

    dist.barrier()
    if rank == 0:
        print("ALL OK", flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
