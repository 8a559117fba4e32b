"""Mixture-of-experts kernels vs the PyTorch oracle: routing, grouped GEMMs, full FFN forward/backward."""

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _rand(shape, seed, scale=1.0):
    g = torch.Generator(device=DEV).manual_seed(seed)
    return (torch.randn(shape, device=DEV, generator=g) * scale).to(torch.bfloat16)


def test_topk_routing_matches_torch():
    from rl_engine.kernels.ops.base import require_ext

    g = torch.Generator(device=DEV).manual_seed(0)
    logits = torch.randn(1000, 128, device=DEV, generator=g)
    logits[5, 7] = logits[5, 3]  # an exact tie: the lower expert id wins
    idx, w = require_ext().moe_topk(logits, 8)
    probs = torch.softmax(logits, -1)
    want = torch.sort(probs, dim=-1, descending=True, stable=True)
    assert torch.equal(idx.long(), want.indices[:, :8])
    ref_w = want.values[:, :8] / want.values[:, :8].sum(-1, keepdim=True)
    assert torch.allclose(w, ref_w, atol=1e-6, rtol=1e-5)


@pytest.mark.parametrize("experts,k", [(128, 8), (8, 2), (60, 4)])
def test_router_weights_gradient_matches_torch(experts, k):
    """``route_topk`` on the GPU (one forward kernel, one backward kernel) against softmax -> gather -> renormalise
    spelled with PyTorch ops in fp32: same ids, same weights, same gradient for the logits."""
    from rl_engine.kernels.ops.sm100.moe import route_topk

    g = torch.Generator(device=DEV).manual_seed(3)
    logits = torch.randn(777, experts, device=DEV, generator=g)
    dw = torch.randn(777, k, device=DEV, generator=g)
    a = logits.clone().requires_grad_(True)
    idx, w = route_topk(a, k)
    (w * dw).sum().backward()
    b = logits.clone().requires_grad_(True)
    probs = torch.softmax(b, dim=-1)
    picked = probs.gather(1, idx.long())
    w_ref = picked / picked.sum(-1, keepdim=True)
    (w_ref * dw).sum().backward()
    assert torch.equal(idx.long(), torch.sort(probs.detach(), dim=-1, descending=True, stable=True).indices[:, :k])
    assert torch.allclose(w, w_ref, atol=1e-6, rtol=1e-5)
    assert torch.allclose(a.grad, b.grad, atol=2e-6, rtol=1e-4)
    assert not idx.requires_grad


def test_grouped_gemm_modes():
    from rl_engine.kernels.ops.base import require_ext
    from rl_engine.kernels.ops.sm100.moe import build_dispatch_plan

    ext = require_ext()
    E, T, K, H, N = 6, 700, 2, 256, 384
    g = torch.Generator(device=DEV).manual_seed(1)
    idx = torch.stack([torch.randperm(E, device=DEV, generator=g)[:K] for _ in range(T)]).to(torch.int32)
    idx[:, 0] = torch.where(idx[:, 0] == 4, torch.zeros_like(idx[:, 0]), idx[:, 0])  # expert 4 nearly starved
    plan = build_dispatch_plan(idx, E)
    x = _rand((T, H), 2)
    w = _rand((E * N, H), 3, 0.05)
    xs = ext.moe_gather_rows(x, plan.src_row)
    y = ext.grouped_gemm(xs, w, 1, plan.tile_group, E, False, False)
    dy = _rand(tuple(y.shape), 4)
    dy[plan.src_row < 0] = 0
    dxs = ext.grouped_gemm(dy, w, 1, plan.tile_group, E, True, False)
    dw = ext.grouped_gemm(dy, xs, 2, plan.offsets, E, True, True)
    off = plan.offsets.tolist()
    for e in range(E):
        rows = slice(off[e], off[e + 1])
        we = w[e * N : (e + 1) * N].float()
        want = xs[rows].float() @ we.t()
        assert (y[rows].float() - want).abs().max().item() / (want.abs().max().item() + 1e-6) < 1e-2
        want_dx = dy[rows].float() @ we
        assert (dxs[rows].float() - want_dx).abs().max().item() / (want_dx.abs().max().item() + 1e-6) < 1e-2
        want_dw = dy[rows].float().t() @ xs[rows].float()
        assert (dw[e * N : (e + 1) * N] - want_dw).abs().max().item() / (want_dw.abs().max().item() + 1e-6) < 1e-2
    # every assignment landed in a slot of its expert, in token order
    slot = plan.slot.long()
    assert torch.equal(plan.src_row[slot.reshape(-1)].view(T, K), torch.arange(T, device=DEV, dtype=torch.int32)[:, None].expand(T, K))
    owner = torch.searchsorted(plan.offsets[1:].long().contiguous(), slot.reshape(-1), right=True).view(T, K)
    assert torch.equal(owner, idx.long())


@pytest.mark.parametrize("T,E,k,H,F", [(300, 8, 2, 256, 128), (1000, 16, 4, 512, 192)])
def test_moe_ffn_forward_backward_vs_oracle(T, E, k, H, F):
    from rl_engine.kernels.ops.sm100.moe import FusedMoESM100Op, NativeMoEOp

    x = _rand((T, H), 5)
    router = _rand((E, H), 6, 0.2)
    w1 = _rand((E * 2 * F, H), 7, 0.05)
    w2 = _rand((E * H, F), 8, 0.05)
    dout = _rand((T, H), 9)
    fused_in = [t.clone().requires_grad_(True) for t in (x, router, w1, w2)]
    out = FusedMoESM100Op()(*fused_in, k)
    out.backward(dout)
    ref_in = [t.clone().float().requires_grad_(True) for t in (x, router, w1, w2)]
    ref = NativeMoEOp()(*ref_in, k)
    ref.backward(dout.float())
    assert (out.float() - ref).abs().max().item() / ref.abs().max().item() < 2e-2
    for name, a, b in zip(("x", "router", "w1", "w2"), fused_in, ref_in):
        scale = b.grad.abs().max().item() + 1e-8
        assert (a.grad.float() - b.grad).abs().max().item() / scale < 4e-2, name
    again = [t.clone().requires_grad_(True) for t in (x, router, w1, w2)]
    out2 = FusedMoESM100Op()(*again, k)
    out2.backward(dout)
    assert torch.equal(out, out2) and all(torch.equal(a.grad, b.grad) for a, b in zip(fused_in, again))


def test_expert_parallel_single_rank_matches_fused_op(tmp_path):
    """World size 1: dispatch / combine run through the peer kernels on this GPU's own buffers, and a
    capacity smaller than the worst case leaves skipped tiles at the tail of the slot buffer."""
    import torch.distributed as dist

    from rl_engine.kernels.ops.sm100.moe import FusedMoESM100Op
    from rl_engine.parallel.expert_parallel import ExpertParallelContext, ExpertParallelMoE

    created = not dist.is_initialized()
    if created:
        dist.init_process_group("gloo", store=dist.FileStore(str(tmp_path / "store"), 1), rank=0, world_size=1)
    try:
        E, K, H, F, T = 8, 2, 256, 128, 500
        x = _rand((T, H), 31)
        router, w1, w2 = _rand((E, H), 32, 0.3), _rand((E * 2 * F, H), 33, 0.06), _rand((E * H, F), 34, 0.09)
        dout = _rand((T, H), 35)
        ctx = ExpertParallelContext(H, E, K, max_tokens=2048, device=torch.device(DEV))
        leaves = [t.clone().requires_grad_(True) for t in (x, router, w1, w2)]
        out = ExpertParallelMoE(ctx)(*leaves)
        out.backward(dout)
        ref_leaves = [t.clone().requires_grad_(True) for t in (x, router, w1, w2)]
        ref = FusedMoESM100Op()(*ref_leaves, K)
        ref.backward(dout)
        assert torch.equal(out, ref), "same kernels, same slot order: the outputs must agree bitwise"
        for a, b in zip(leaves, ref_leaves):
            assert torch.allclose(a.grad.float(), b.grad.float(), atol=1e-3, rtol=1e-2)
        ctx.mem.check()
    finally:
        if created:
            dist.destroy_process_group()


def test_qwen3_style_moe_model_grpo_steps():
    """A small Qwen3-MoE-shaped decoder (q/k norm, router + experts in every layer) trains through the fused path:
    the loss is finite, decreases over a few steps, every parameter family receives gradient, and the first-step
    loss matches the same model evaluated with the PyTorch MoE oracle."""
    from rl_engine.kernels.ops.base import check_device_errors
    from rl_engine.kernels.registry import kernel_registry
    from rl_engine.models.config import ModelConfig
    from rl_engine.models.grpo import GRPOTrainer, synthetic_batch
    from rl_engine.models.llama import LlamaModel

    cfg = ModelConfig("qwen3-moe-test", vocab_size=2048, hidden_size=256, num_layers=2, num_heads=4, num_kv_heads=2,
                      head_dim=128, ffn_size=512, rms_eps=1e-6, rope_theta=1e6, num_experts=8, experts_per_token=2,
                      moe_ffn_size=128, qk_norm=True)
    model = LlamaModel(cfg, dtype=torch.bfloat16, device=DEV, seed=3)
    trainer = GRPOTrainer(model, lr=2e-3)
    batch = synthetic_batch(cfg.vocab_size, prompt_len=128, group=4, completion_len=128, seed=5).pin()
    losses = [trainer.step(batch) for _ in range(4)]
    assert all(l == l and abs(l) < 1e4 for l in losses), losses
    assert losses[-1] < losses[0], losses
    flat_grad = model.ensure_flat_grad()
    for name in ("l0.router", "l0.w_gate_up", "l0.w_down", "l0.q_norm", "l1.k_norm", "l1.wqkv"):
        off, n = model._offsets[name], 1
        for d in model._shapes[name]:
            n *= d
        assert float(flat_grad[off:off + n].float().abs().sum()) > 0, f"no gradient reached {name}"
    assert type(kernel_registry.get_op("moe")).__name__ == "FusedMoESM100Op"
    check_device_errors(0)


def test_device_dispatch_plan_matches_portable_plan():
    """The three-kernel plan builder must reproduce the framework-op plan exactly (same slots, same padding)."""
    from rl_engine.kernels.ops.sm100 import moe

    g = torch.Generator(device=DEV).manual_seed(9)
    for t, k, e in ((700, 2, 6), (4096, 8, 128), (33, 1, 4), (1000, 4, 64)):
        idx = torch.stack([torch.randperm(e, device=DEV, generator=g)[:k] for _ in range(t)]).to(torch.int32)
        if e > 3:
            idx[idx == 3] = 0  # an expert that receives nothing keeps one padded block
        fast = moe.build_dispatch_plan(idx, e)
        slow = moe.build_dispatch_plan(idx.cpu(), e)
        assert torch.equal(fast.slot.cpu(), slow.slot) and torch.equal(fast.src_row.cpu(), slow.src_row)
        assert torch.equal(fast.offsets.cpu(), slow.offsets) and torch.equal(fast.counts.cpu(), slow.counts)
        assert torch.equal(fast.tile_group.cpu(), slow.tile_group) and fast.num_slots == slow.num_slots
