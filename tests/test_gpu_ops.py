"""sm_100a kernels vs plain PyTorch fp32 references (numerics, masks, determinism)."""

import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda"


def _gen(seed):
    return torch.Generator(device=DEV).manual_seed(seed)


# ------------------------------------------------------------------------------ logp rows
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("V", [300, 32000, 128256])
def test_logp_rows_all_methods(dtype, V):
    from rl_engine.kernels.ops.pytorch.loss.logp import NativeLogpOp
    from rl_engine.kernels.ops.sm100.logp import FusedLogpSM100Op

    g = _gen(V)
    logits = (torch.randn(3, 5, V, device=DEV, generator=g) * 3).to(dtype)
    ids = torch.randint(0, V, (3, 5), device=DEV, generator=g)
    fused, native = FusedLogpSM100Op(), NativeLogpOp()
    want32 = native.apply_fp32(logits, ids)
    tol = 2e-5 if dtype == torch.float32 else 2e-5  # fp32 math on the same quantised inputs
    assert torch.allclose(fused.apply_fp32(logits, ids), want32, atol=tol, rtol=1e-5)
    assert fused.apply(logits, ids).dtype == dtype
    out = torch.full((3, 5), 7.0, device=DEV)
    rows = torch.tensor([1, 4, 9, 14], device=DEV)
    fused.indexed_out(logits, ids, rows, out)
    flat = out.view(-1)
    assert torch.allclose(flat[rows], want32.view(-1)[rows], atol=tol, rtol=1e-5)
    untouched = torch.ones(15, dtype=torch.bool, device=DEV)
    untouched[rows] = False
    assert bool((flat[untouched] == 7.0).all())
    idx32 = fused.online_indexed_fp32(logits, ids, rows)
    assert bool((idx32.view(-1)[untouched] == 0).all())
    assert torch.equal(fused.apply_fp32(logits, ids), fused.online_fp32(logits, ids))  # bitwise repeatable
    with pytest.raises(ValueError):
        fused.indexed_fp32(logits, ids, torch.tensor([15], device=DEV))


def test_logp_rows_out_of_range_id_gives_zero():
    from rl_engine.kernels.ops.sm100.logp import FusedLogpSM100Op

    logits = torch.randn(4, 50, device=DEV)
    ids = torch.tensor([0, -1, 50, 3], device=DEV)
    out = FusedLogpSM100Op().apply_fp32(logits, ids)
    assert out[1] == 0 and out[2] == 0 and out[0] < 0


# -------------------------------------------------------------------------- linear_logp
def _ll_ref(h, w, t, b=None):
    z = h.float() @ w.float().t()
    if b is not None:
        z = z + b.float()
    lp = torch.log_softmax(z, -1)
    return lp.gather(-1, t[..., None]).squeeze(-1), -(lp.exp() * lp).sum(-1)


@pytest.mark.parametrize("N,D,V", [(96, 128, 500), (40, 80, 300), (300, 256, 9000), (1024, 512, 33000)])
@pytest.mark.parametrize("use_bias", [False, True])
def test_linear_logp_forward_backward(N, D, V, use_bias):
    from rl_engine.kernels.ops.sm100.linear_logp import FusedLinearLogpSM100Op

    g = _gen(N + V)
    h = (torch.randn(N, D, device=DEV, generator=g)).to(torch.bfloat16).requires_grad_(True)
    w = (torch.randn(V, D, device=DEV, generator=g) * 0.05).to(torch.bfloat16).requires_grad_(True)
    b = (torch.randn(V, device=DEV, generator=g) * 0.1).to(torch.bfloat16).requires_grad_(True) if use_bias else None
    t = torch.randint(0, V, (N,), device=DEV, generator=g)
    op = FusedLinearLogpSM100Op()
    lp, ent = op.with_entropy(h, w, t, b)
    want_lp, want_ent = _ll_ref(h.detach(), w.detach(), t, None if b is None else b.detach())
    assert torch.allclose(lp, want_lp, atol=2e-3, rtol=1e-3)
    assert torch.allclose(ent, want_ent, atol=2e-3, rtol=1e-3)
    gl = torch.randn(N, device=DEV, generator=g)
    lp.backward(gl)
    hf = h.detach().float().requires_grad_(True)
    wf = w.detach().float().requires_grad_(True)
    bf = None if b is None else b.detach().float().requires_grad_(True)
    ref_lp, _ = _ll_ref(hf, wf, t, bf)
    ref_lp.backward(gl)
    for got, want in ((h.grad, hf.grad), (w.grad, wf.grad)) + (((b.grad, bf.grad),) if use_bias else ()):
        scale = want.abs().max().item() + 1e-8
        assert (got.float() - want).abs().max().item() / scale < 2e-2


def test_linear_logp_bitwise_deterministic_and_batch_invariant():
    from rl_engine.kernels.ops.sm100.linear_logp import FusedLinearLogpSM100Op

    g = _gen(7)
    N, D, V = 700, 256, 20000
    h = torch.randn(N, D, device=DEV, generator=g).to(torch.bfloat16)
    w = (torch.randn(V, D, device=DEV, generator=g) * 0.05).to(torch.bfloat16)
    t = torch.randint(0, V, (N,), device=DEV, generator=g)
    op = FusedLinearLogpSM100Op()
    a = op(h, w, t)
    b = op(h, w, t)
    assert torch.equal(a, b)
    # a row's value must not depend on which other rows are in the batch (train == rollout layouts)
    part = op(h[100:357], w, t[100:357])
    assert torch.equal(part, a[100:357])
    shaped = op(h.view(7, 100, D), w, t.view(7, 100))
    assert torch.equal(shaped.view(-1), a)
    # backward determinism
    hg = h.clone().requires_grad_(True)
    wg = w.clone().requires_grad_(True)
    op(hg, wg, t).sum().backward()
    h2 = h.clone().requires_grad_(True)
    w2 = w.clone().requires_grad_(True)
    op(h2, w2, t).sum().backward()
    assert torch.equal(hg.grad, h2.grad) and torch.equal(wg.grad, w2.grad)


def test_linear_logp_rejects_out_of_range_targets():
    """``sync`` mode raises at the call; the default mode checks on the device: no host read-back per call, the bad
    rows come back NaN and the next ``check_device_errors`` raises."""
    from rl_engine.kernels.ops.base import check_device_errors
    from rl_engine.kernels.ops.sm100.linear_logp import FusedLinearLogpSM100Op

    h = torch.randn(8, 64, device=DEV).to(torch.bfloat16)
    w = torch.randn(100, 64, device=DEV).to(torch.bfloat16)
    with pytest.raises(ValueError):
        FusedLinearLogpSM100Op(check_targets="sync")(h, w, torch.full((8,), -100, device=DEV))
    op = FusedLinearLogpSM100Op()
    assert op.check_targets == "device"
    good = torch.arange(8, device=DEV)
    clean = op(h, w, good)
    check_device_errors(torch.cuda.current_device())  # valid ids leave the error word alone
    bad = good.clone()
    bad[3], bad[5] = 100, -1
    out = op(h, w, bad)
    with pytest.raises(RuntimeError, match="bad argument"):
        check_device_errors(torch.cuda.current_device())
    assert torch.isnan(out[[3, 5]]).all() and torch.equal(out[[0, 1, 2, 4, 6, 7]], clean[[0, 1, 2, 4, 6, 7]])
    check_device_errors(torch.cuda.current_device())  # the word was reset by the raise
    assert torch.isfinite(FusedLinearLogpSM100Op(check_targets="off")(h, w, bad)[[0, 1]]).all()
    check_device_errors(torch.cuda.current_device())


# ------------------------------------------------------------------------ ratio_kl / grpo
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_ratio_kl_and_grpo_loss_match_native(dtype):
    from rl_engine.kernels.ops.pytorch.loss.grpo_loss import NativeGRPOLossOp
    from rl_engine.kernels.ops.pytorch.loss.ratio_kl import NativeRatioKLOp
    from rl_engine.kernels.ops.sm100.grpo_loss import FusedGRPOLossSM100Op
    from rl_engine.kernels.ops.sm100.ratio_kl import FusedRatioKLSM100Op

    g = _gen(11)
    B, T, V = 8, 16, 777
    pol = torch.randn(B, T, V, device=DEV, generator=g).to(dtype)
    ref = (pol.float() + 0.1 * torch.randn(B, T, V, device=DEV, generator=g)).to(dtype)
    ids = torch.randint(0, V, (B, T), device=DEV, generator=g)
    mask = torch.rand(B, T, device=DEV, generator=g) > 0.3
    ids = torch.where(mask, ids, torch.full_like(ids, -100))  # garbage at masked positions
    old = torch.log_softmax(pol.float(), -1).gather(-1, ids.clamp(min=0)[..., None]).squeeze(-1)
    old = old + 0.05 * torch.randn(B, T, device=DEV, generator=g)
    rewards = torch.randn(B, device=DEV, generator=g)

    p1 = pol.clone().requires_grad_(True)
    p2 = pol.clone().float().requires_grad_(True)
    r1, k1 = FusedRatioKLSM100Op()(p1, ref, ids, mask, old)
    r2, k2 = NativeRatioKLOp()(p2, ref.float(), ids, mask, old)
    assert torch.allclose(r1, r2, atol=1e-4, rtol=1e-4) and torch.allclose(k1, k2, atol=1e-4, rtol=1e-3)
    assert bool((r1[~mask] == 1).all()) and bool((k1[~mask] == 0).all())
    gr = torch.randn(B, T, device=DEV, generator=g)
    gk = torch.randn(B, T, device=DEV, generator=g)
    (r1 * gr + k1 * gk).sum().backward()
    (r2 * gr + k2 * gk).sum().backward()
    tol = 1e-4 if dtype == torch.float32 else 2e-2
    assert (p1.grad.float() - p2.grad).abs().max().item() < tol
    assert bool((p1.grad[~mask] == 0).all())

    fused, native = FusedGRPOLossSM100Op(), NativeGRPOLossOp()
    p1 = pol.clone().requires_grad_(True)
    p2 = pol.clone().float().requires_grad_(True)
    got = fused(p1, ref, ids, old, rewards, mask, clip_eps=0.2, beta=0.04, samples_per_prompt=4)
    want = native(p2, ref.float(), ids, old, rewards, mask, clip_eps=0.2, beta=0.04, samples_per_prompt=4)
    for a, b in zip(got, want):
        assert torch.allclose(a, b, atol=2e-4, rtol=1e-3)
    got[0].backward()
    want[0].backward()
    assert (p1.grad.float() - p2.grad).abs().max().item() < (1e-5 if dtype == torch.float32 else 2e-3)
    with pytest.raises(ValueError):
        bad = ids.clone()
        bad[mask] = V
        FusedRatioKLSM100Op()(pol, ref, bad, mask, old)


def test_group_advantages_uniform_and_csr():
    from rl_engine.kernels.ops.pytorch.loss.grpo_loss import NativeGRPOLossOp
    from rl_engine.kernels.ops.sm100.grpo_loss import FusedGRPOLossSM100Op

    r = torch.randn(48, device=DEV)
    f, n = FusedGRPOLossSM100Op(), NativeGRPOLossOp()
    assert torch.allclose(f.group_advantages(r, samples_per_prompt=8), n.group_advantages(r, samples_per_prompt=8), atol=1e-5)
    bounds = [0, 3, 7, 12, 48]
    assert torch.allclose(f.group_advantages(r, group_boundaries=bounds), n.group_advantages(r, group_boundaries=bounds), atol=1e-5)
    const = torch.ones(8, device=DEV)
    assert torch.isfinite(f.group_advantages(const, samples_per_prompt=4)).all()
    with pytest.raises(ValueError):
        f.group_advantages(r, samples_per_prompt=1)


def test_logp_space_losses_match_native():
    from rl_engine.kernels.ops.pytorch.loss.grpo_loss import NativeGRPOLossOp
    from rl_engine.kernels.ops.pytorch.loss.policy_losses import NativeDPOLossOp, NativePPOLossOp
    from rl_engine.kernels.ops.sm100.grpo_loss import FusedGRPOLossSM100Op
    from rl_engine.kernels.ops.sm100.policy_losses import FusedDPOLossSM100Op, FusedPPOLossSM100Op

    g = _gen(5)
    B, T = 16, 33
    lp = (-torch.rand(B, T, device=DEV, generator=g) * 3)
    ref = lp + 0.1 * torch.randn(B, T, device=DEV, generator=g)
    old = lp + 0.3 * torch.randn(B, T, device=DEV, generator=g)
    mask = torch.rand(B, T, device=DEV, generator=g) > 0.2
    adv_s = torch.randn(B, device=DEV, generator=g)
    adv_t = torch.randn(B, T, device=DEV, generator=g)
    a = lp.clone().requires_grad_(True)
    b = lp.clone().requires_grad_(True)
    got = FusedGRPOLossSM100Op().apply_from_logps(a, ref, old, adv_s, mask, clip_eps=0.2, beta=0.04)
    want = NativeGRPOLossOp().apply_from_logps(b, ref, old, adv_s, mask, clip_eps=0.2, beta=0.04)
    for x, y in zip(got, want):
        assert torch.allclose(x, y, atol=1e-5, rtol=1e-4)
    (got[0] + 2 * got[1] - got[2]).backward()
    (want[0] + 2 * want[1] - want[2]).backward()
    assert torch.allclose(a.grad, b.grad, atol=1e-6, rtol=1e-4)
    again = FusedGRPOLossSM100Op().apply_from_logps(lp, ref, old, adv_s, mask, clip_eps=0.2, beta=0.04)
    assert all(torch.equal(x.detach(), y) for x, y in zip(got, again))
    a = lp.clone().requires_grad_(True)
    b = lp.clone().requires_grad_(True)
    got = FusedPPOLossSM100Op()(a, old, adv_t, mask, ref_logps=ref, clip_eps=0.1, beta=0.01)
    want = NativePPOLossOp()(b, old, adv_t, mask, ref_logps=ref, clip_eps=0.1, beta=0.01)
    for x, y in zip(got, want):
        assert torch.allclose(x, y, atol=1e-5, rtol=1e-4)
    got[0].backward()
    want[0].backward()
    assert torch.allclose(a.grad, b.grad, atol=1e-6, rtol=1e-4)
    pc, pr, rc, rr = (torch.randn(12, device=DEV, generator=g) for _ in range(4))
    x = pc.clone().requires_grad_(True)
    y = pc.clone().requires_grad_(True)
    xr = pr.clone().requires_grad_(True)
    yr = pr.clone().requires_grad_(True)
    got = FusedDPOLossSM100Op()(x, xr, rc, rr, beta=0.3, label_smoothing=0.1)
    want = NativeDPOLossOp()(y, yr, rc, rr, beta=0.3, label_smoothing=0.1)
    for u, v in zip(got, want):
        assert torch.allclose(u, v, atol=1e-5, rtol=1e-4)
    got[0].backward()
    want[0].backward()
    assert torch.allclose(x.grad, y.grad, atol=1e-6, rtol=1e-4) and torch.allclose(xr.grad, yr.grad, atol=1e-6, rtol=1e-4)


# ----------------------------------------------------------------------------- model ops
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_rmsnorm_swiglu_rope_embedding(dtype):
    from rl_engine.kernels.ops.pytorch.activation.swiglu import NativeSiLUOp, NativeSwiGLUOp
    from rl_engine.kernels.ops.pytorch.linear.rope import NativeRoPEOp
    from rl_engine.kernels.ops.pytorch.norm.rms_norm import NativeRMSNormOp
    from rl_engine.kernels.ops.sm100.model_ops import (
        FusedEmbeddingSM100Op, FusedRMSNormSM100Op, FusedRoPESM100Op, FusedSiLUSM100Op, FusedSwiGLUSM100Op,
    )

    g = _gen(3)
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    x = torch.randn(5, 37, 200, device=DEV, generator=g).to(dtype)
    w = torch.randn(200, device=DEV, generator=g).to(dtype)
    f, n = FusedRMSNormSM100Op(), NativeRMSNormOp()
    assert torch.allclose(f.forward_fp32(x, w), n.forward_fp32(x, w), atol=1e-5, rtol=1e-5)
    assert torch.equal(f(x, w)[2:4], f(x[2:4], w))  # batch invariance, bitwise
    xa, wa = x.clone().requires_grad_(True), w.clone().requires_grad_(True)
    xb, wb = x.clone().float().requires_grad_(True), w.clone().float().requires_grad_(True)
    dy = torch.randn_like(x)
    f(xa, wa).backward(dy)
    n.forward_fp32(xb, wb).backward(dy.float())
    assert (xa.grad.float() - xb.grad).abs().max().item() < tol * 5
    assert (wa.grad.float() - wb.grad).abs().max().item() / wb.grad.abs().max().item() < tol
    with pytest.raises(ValueError):
        f(x, w[:-1])

    gate = torch.randn(7, 19, 96, device=DEV, generator=g).to(dtype)
    up = torch.randn(7, 19, 96, device=DEV, generator=g).to(dtype)
    fs, ns = FusedSwiGLUSM100Op(), NativeSwiGLUOp()
    assert torch.allclose(fs.forward_fp32(gate, up), ns.forward_fp32(gate, up), atol=1e-5, rtol=1e-5)
    ga, ua = gate.clone().requires_grad_(True), up.clone().requires_grad_(True)
    gb, ub = gate.clone().float().requires_grad_(True), up.clone().float().requires_grad_(True)
    dy = torch.randn_like(gate)
    fs(ga, ua).backward(dy)
    ns.forward_fp32(gb, ub).backward(dy.float())
    assert (ga.grad.float() - gb.grad).abs().max().item() < tol * 5 and (ua.grad.float() - ub.grad).abs().max().item() < tol * 5
    assert torch.allclose(FusedSiLUSM100Op().forward_fp32(gate), NativeSiLUOp().forward_fp32(gate), atol=1e-5)
    with pytest.raises(ValueError):
        fs(gate, up[:, :, :-1])

    q = torch.randn(2, 50, 4, 64, device=DEV, generator=g).to(dtype)
    pos = torch.arange(50, device=DEV).expand(2, 50) + 3
    fr, nr = FusedRoPESM100Op(), NativeRoPEOp()
    assert (fr(q, pos).float() - nr.forward_fp32(q, pos)).abs().max().item() < tol
    qa = q.clone().requires_grad_(True)
    qb = q.clone().float().requires_grad_(True)
    dy = torch.randn_like(q)
    fr(qa, pos).backward(dy)
    nr.forward_fp32(qb, pos).backward(dy.float())
    assert (qa.grad.float() - qb.grad).abs().max().item() < tol * 2

    table = torch.randn(300, 72, device=DEV, generator=g).to(dtype)
    ids = torch.randint(0, 300, (4, 25), device=DEV, generator=g)
    ids[0, :5] = 17  # repeated id exercises the ordered segment sum
    fe = FusedEmbeddingSM100Op()
    ta = table.clone().requires_grad_(True)
    tb = table.clone().float().requires_grad_(True)
    out = fe(ids, ta)
    assert torch.equal(out, table[ids])
    dy = torch.randn(4, 25, 72, device=DEV, generator=g).to(dtype)
    out.backward(dy)
    torch.nn.functional.embedding(ids, tb).backward(dy.float())
    assert (ta.grad.float() - tb.grad).abs().max().item() < tol * 4


def test_adamw_matches_torch():
    from rl_engine.kernels.ops.base import require_ext

    g = _gen(9)
    p = torch.randn(10000, device=DEV, generator=g)
    grad = torch.randn(10000, device=DEV, generator=g)
    ref = p.clone().requires_grad_(True)
    opt = torch.optim.AdamW([ref], lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    pb = p.to(torch.bfloat16)
    master = p.clone()
    m, v = torch.zeros_like(p), torch.zeros_like(p)
    for step in range(1, 4):
        ref.grad = grad.clone()
        opt.step()
        require_ext().adamw(pb, master, grad.to(torch.bfloat16).float(), m, v, 1e-2, 0.9, 0.95, 1e-8, 0.1, step, 1.0)
    assert torch.allclose(master, ref.detach(), atol=2e-4, rtol=1e-3)
    assert torch.allclose(pb.float(), master, atol=1e-2, rtol=1e-2)


@pytest.mark.parametrize("lr", [1e-6, 1e-2])
@pytest.mark.parametrize("offset", [0, 1])
def test_adamw_split_master_is_the_fp32_master_bit_for_bit(lr, offset):
    """bf16 parameter + 16-bit residual carries the same fp32 master as a separate fp32 copy (vector path, scalar
    tail, and the scalar path of an unaligned buffer)."""
    from rl_engine.kernels.ops.base import require_ext
    from rl_engine.models.grpo import join_master, split_master

    ext = require_ext()
    g = _gen(21)
    n = 100003
    base = (torch.randn(n + 8, device=DEV, generator=g) * 0.02).to(torch.bfloat16)
    pa, pb = base.clone()[offset : offset + n], base.clone()[offset : offset + n]
    master = pa.float()
    residual = torch.zeros(n + 8, dtype=torch.int16, device=DEV)[offset : offset + n]
    ma, va = torch.zeros(n + 8, device=DEV)[offset : offset + n], torch.zeros(n + 8, device=DEV)[offset : offset + n]
    mb, vb = torch.zeros(n + 8, device=DEV)[offset : offset + n], torch.zeros(n + 8, device=DEV)[offset : offset + n]
    start = pa.clone()
    for step in range(1, 6):
        grad = torch.randn(n + 8, device=DEV, generator=g).to(torch.bfloat16)[offset : offset + n]
        ext.adamw(pa, master, grad, ma, va, lr, 0.9, 0.95, 1e-8, 0.01, step, 0.5)
        ext.adamw(pb, residual, grad, mb, vb, lr, 0.9, 0.95, 1e-8, 0.01, step, 0.5)
        assert torch.equal(join_master(pb, residual).view(torch.int32), master.view(torch.int32))
    assert torch.equal(ma, mb) and torch.equal(va, vb)
    want_param, want_residual = split_master(master)
    assert torch.equal(pb, want_param) and torch.equal(residual, want_residual)
    # the two roundings of the same master differ only on exact ties, by one bf16 step
    differ = pa != pb
    assert differ.float().mean().item() < 1e-3
    if lr == 1e-6:
        assert (pb != start).float().mean().item() < 0.2  # bf16 weights barely move in five such steps ...
        assert (master != start.float()).float().mean().item() > 0.99  # ... the master always does


# -------------------------------------------------------------------------------- sampler
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_sampler_matches_host_restatement(dtype):
    from rl_engine.kernels.ops.sm100.sampler import sample_reference, sample_topk_topp

    g = _gen(21)
    logits = (torch.randn(16, 5000, device=DEV, generator=g) * 2).to(dtype)
    for (k, p, temp) in [(50, 0.9, 0.7), (1, 1.0, 1.0), (8, 0.5, 1.3), (1024, 0.95, 1.0)]:
        got, lp = sample_topk_topp(logits, top_k=k, top_p=p, temperature=temp, seed=123, offset=4, return_logprob=True)
        want = sample_reference(logits, k, p, temp, 123, 4)
        agree = (got.cpu() == want).float().mean().item()
        assert agree >= 0.9, (k, p, temp, agree)  # float rounding at cut boundaries may flip a rare row
        again, _ = sample_topk_topp(logits, top_k=k, top_p=p, temperature=temp, seed=123, offset=4)
        assert torch.equal(got, again)
        assert bool((lp <= 1e-6).all())
    greedy, _ = sample_topk_topp(logits, top_k=1, top_p=1.0, temperature=1.0, seed=0, offset=0)
    assert torch.equal(greedy, logits.float().argmax(-1))


def test_sampler_distribution():
    from rl_engine.kernels.ops.sm100.sampler import sample_topk_topp

    z = torch.tensor([2.0, 1.0, 0.5, 0.0, -1.0, -3.0], device=DEV).repeat(20000, 1)
    ids, _ = sample_topk_topp(z, top_k=4, top_p=1.0, temperature=1.0, seed=99, offset=0)
    freq = torch.bincount(ids, minlength=6).float() / ids.numel()
    want = torch.softmax(z[0, :4], 0)
    assert freq[4:].sum() == 0 and torch.allclose(freq[:4], want, atol=0.015)


def test_swiglu_packed_and_rmsnorm_wide_rows():
    from rl_engine.kernels.ops.sm100.model_ops import FusedRMSNormSM100Op, swiglu_packed

    g = _gen(31)
    gu = torch.randn(3, 50, 2 * 1408, device=DEV, generator=g).to(torch.bfloat16)
    dy = torch.randn(3, 50, 1408, device=DEV, generator=g).to(torch.bfloat16)
    a = gu.clone().requires_grad_(True)
    b = gu.clone().float().requires_grad_(True)
    out = swiglu_packed(a)
    ref = torch.nn.functional.silu(b[..., :1408]) * b[..., 1408:]
    assert (out.float() - ref).abs().max().item() < 3e-2
    out.backward(dy)
    ref.backward(dy.float())
    assert (a.grad.float() - b.grad).abs().max().item() < 6e-2

    x = torch.randn(300, 4096, device=DEV, generator=g).to(torch.bfloat16)
    w = torch.randn(4096, device=DEV, generator=g).to(torch.bfloat16)
    f = FusedRMSNormSM100Op()
    xa, wa = x.clone().requires_grad_(True), w.clone().requires_grad_(True)
    xb, wb = x.clone().float().requires_grad_(True), w.clone().float().requires_grad_(True)
    y = f(xa, wa, eps=1e-5)
    yr = xb * torch.rsqrt(xb.square().mean(-1, keepdim=True) + 1e-5) * wb
    assert (y.float() - yr).abs().max().item() < 5e-2
    assert torch.equal(f(x[17:33], w, eps=1e-5), y[17:33].detach())
    d = torch.randn_like(x)
    y.backward(d)
    yr.backward(d.float())
    assert (xa.grad.float() - xb.grad).abs().max().item() < 0.1
    assert (wa.grad.float() - wb.grad).abs().max().item() / wb.grad.abs().max().item() < 2e-2


def test_device_stamps_and_phase_timer():
    from rl_engine.utils.tracing import DeviceStamps, PhaseTimer

    stamps = DeviceStamps(4)
    timer = PhaseTimer()
    a = torch.randn(4096, 4096, device="cuda")
    stamps.stamp(0)
    with timer.phase("matmul"):
        for _ in range(10):
            a @ a
    stamps.stamp(1)
    ms = stamps.elapsed_ms(0, 1)
    s = timer.summary()
    assert ms > 0 and s["matmul"]["total_ms"] > 0
    assert abs(ms - s["matmul"]["total_ms"]) < 0.5 * ms + 1.0  # two clocks, same interval


def test_outputs_do_not_overrun_canary_padded_buffers():
    """Kernels that write into caller-provided outputs must stay inside them: the outputs are carved out of
    a larger buffer filled with a sentinel, which must be intact afterwards."""
    from rl_engine.kernels.ops.sm100.gemm import gemm
    from rl_engine.kernels.ops.sm100.logp import FusedLogpSM100Op

    pad = 4096
    m, n, k = 200, 328, 136
    a = (torch.randn(m, k, device="cuda") * 0.5).to(torch.bfloat16)
    b = (torch.randn(n, k, device="cuda") * 0.5).to(torch.bfloat16)
    for pair in (False, True):
        buf = torch.full((pad + m * n + pad,), 12345.0, device="cuda")
        out = buf[pad:pad + m * n].view(m, n)
        gemm(a, b, out=out, out_dtype=torch.float32, pair=pair)
        assert bool((buf[:pad] == 12345.0).all()) and bool((buf[-pad:] == 12345.0).all())
        assert torch.allclose(out, a.float() @ b.float().t(), atol=2e-2, rtol=2e-3)
    rows, v = 333, 1000
    logits = torch.randn(rows, v, device="cuda").to(torch.bfloat16)
    ids = torch.randint(0, v, (rows,), device="cuda")
    buf = torch.full((pad + rows + pad,), 777.0, device="cuda")
    FusedLogpSM100Op().out(logits, ids, buf[pad:pad + rows])
    assert bool((buf[:pad] == 777.0).all()) and bool((buf[-pad:] == 777.0).all())
    want = torch.log_softmax(logits.float(), -1).gather(1, ids[:, None]).squeeze(1)
    assert torch.allclose(buf[pad:pad + rows], want, atol=1e-3, rtol=1e-3)


def test_full_vocab_nucleus_sampler_matches_oracle_and_distribution():
    """top_k=None goes to the full-vocabulary nucleus kernel: cut by probability mass, draw in index order."""
    from rl_engine.kernels.ops.sm100.sampler import nucleus_reference, sample_topk_topp

    g = torch.Generator(device="cuda").manual_seed(3)
    rows, v = 96, 5000
    logits = torch.randn(rows, v, device="cuda", generator=g) * 2.5
    for top_p, temp in ((0.9, 0.8), (0.5, 1.0), (1.0, 1.3)):
        ids, lp = sample_topk_topp(logits, top_k=None, top_p=top_p, temperature=temp, seed=11, offset=5, return_logprob=True)
        again, _ = sample_topk_topp(logits, top_k=None, top_p=top_p, temperature=temp, seed=11, offset=5)
        assert torch.equal(ids, again)
        want = nucleus_reference(logits, top_p, temp, 11, 5)
        # __expf vs exp: a draw that lands within a few ulp of a boundary may move to the neighbouring token
        assert (ids.cpu() == want).float().mean() > 0.97
        # every draw lies inside the nucleus: its probability is at least the smallest kept probability
        probs = torch.softmax(logits / temp, -1)
        sorted_p, _ = probs.sort(dim=-1, descending=True)
        cum = sorted_p.cumsum(-1)
        n_keep = (cum < top_p - 1e-6).sum(-1).clamp(max=v - 1)
        floor = sorted_p.gather(1, n_keep[:, None]).squeeze(1)
        picked = probs.gather(1, ids[:, None]).squeeze(1)
        assert bool((picked >= floor * (1 - 1e-3)).all())
        kept_mass = torch.where(probs >= floor[:, None] * (1 - 1e-6), probs, torch.zeros_like(probs)).sum(-1)
        assert torch.allclose(lp.exp(), picked / kept_mass, rtol=2e-2, atol=1e-6)
    # a tiny nucleus is the arg-max
    ids, _ = sample_topk_topp(logits, top_k=None, top_p=1e-6, temperature=1.0, seed=1, offset=0)
    assert torch.equal(ids, logits.argmax(-1))
    # distribution: the same row 4096 times (different row index -> different uniform)
    row = torch.tensor([2.0, 1.0, 0.0, -1.0, 0.5, 1.5, -3.0, 0.2], device="cuda")
    many = row.expand(4096, 8).contiguous()
    ids, _ = sample_topk_topp(many, top_k=None, top_p=0.8, temperature=1.0, seed=5, offset=0)
    p = torch.softmax(row, -1)
    keep = torch.zeros(8, dtype=torch.bool, device="cuda")
    order = p.argsort(descending=True)
    mass = 0.0
    for i in order.tolist():
        keep[i] = True
        mass += float(p[i])
        if mass >= 0.8:
            break
    target = torch.where(keep, p, torch.zeros_like(p))
    target = target / target.sum()
    freq = torch.bincount(ids, minlength=8).float() / 4096
    assert bool((freq[~keep] == 0).all()) and (freq - target).abs().max() < 0.03


def test_sampler_backend_uses_the_fused_kernels_without_top_k():
    from rl_engine.kernels.ops.base import require_ext
    from rl_engine.kernels.sampling import SamplerBackend

    ext = require_ext()
    sampler = SamplerBackend(seed=3)
    logits = torch.randn(32, 3000, device="cuda")
    before = ext.launch_count()
    a = sampler.sample(logits, top_k=None, top_p=0.9, temperature=0.7)
    b = sampler.sample(logits, top_k=None, top_p=None, temperature=1.0)
    assert ext.launch_count() - before == 2, "both calls must run one native kernel each"
    assert a.shape == (32,) and b.shape == (32,) and int(a.min()) >= 0 and int(b.max()) < 3000


def test_kept_and_recomputed_activations_give_identical_gradients_and_oom_falls_back(monkeypatch):
    """Recomputation replays the same deterministic kernels, so keeping a layer's activations or recomputing them
    must not change one bit of the gradient.  An out-of-memory error in the forward/backward (raised here by a fake,
    not by exhausting the device) makes the trainer recompute four more layers and repeat the step."""
    from rl_engine.models.config import ModelConfig
    from rl_engine.models.grpo import GRPOTrainer, synthetic_batch
    from rl_engine.models.llama import LlamaModel

    cfg = ModelConfig("ckpt", 1024, 256, 6, 2, 1, 128, 512)
    batch = synthetic_batch(cfg.vocab_size, prompt_len=64, group=4, completion_len=64, seed=5).to("cuda")
    grads = {}
    for mode in (True, False, "auto"):
        model = LlamaModel(cfg, dtype=torch.bfloat16, device="cuda", seed=8, activation_checkpointing=mode)
        trainer = GRPOTrainer(model, lr=1e-3)
        trainer.opt.zero_grad()
        loss, _, _ = trainer.loss(batch)
        loss.backward()
        grads[mode] = model.flat_grad.clone()
        if mode == "auto":
            assert model.plan_checkpointing(batch.prompt_ids.numel() + batch.completion_ids.numel()) == 6
    assert torch.equal(grads[True], grads[False]) and torch.equal(grads[True], grads["auto"])

    model = LlamaModel(cfg, dtype=torch.bfloat16, device="cuda", seed=8)
    trainer = GRPOTrainer(model, lr=1e-3)
    trainer.step_device(batch)  # makes the plan: all six layers fit
    real_loss, calls = trainer.loss, []

    def flaky_loss(b):
        calls.append(model.kept_layers())
        if len(calls) == 1:
            raise torch.cuda.OutOfMemoryError("injected")
        return real_loss(b)

    monkeypatch.setattr(trainer, "loss", flaky_loss)
    out = trainer.step_device(batch)
    assert torch.isfinite(out) and calls == [6, 2] and model.kept_layers() == 2


def test_lean_blocks_match_the_unfused_composition_bitwise_and_the_fp32_reference():
    """``norm_linear`` / ``swiglu_linear`` recompute the cheap op's output in backward; forward values and all gradients
    must be the bits of rms_norm -> matmul / swiglu -> matmul, and close to a plain fp32 PyTorch restatement."""
    from rl_engine.kernels.ops.sm100.gemm import matmul_nt
    from rl_engine.kernels.ops.sm100.lean_blocks import norm_linear, swiglu_linear
    from rl_engine.kernels.ops.sm100.model_ops import swiglu_packed
    from rl_engine.kernels.registry import kernel_registry

    g = torch.Generator(device="cuda").manual_seed(11)
    rows, h, n, f = 384, 512, 640, 768
    x = torch.randn(rows, h, device="cuda", generator=g).to(torch.bfloat16)
    nw = (1 + 0.1 * torch.randn(h, device="cuda", generator=g)).to(torch.bfloat16)
    w = (0.05 * torch.randn(n, h, device="cuda", generator=g)).to(torch.bfloat16)
    dy = torch.randn(rows, n, device="cuda", generator=g).to(torch.bfloat16)

    def run(fn):
        leaves = [t.clone().requires_grad_(True) for t in (x, nw, w)]
        y = fn(*leaves)
        y.backward(dy)
        return [y.detach()] + [t.grad for t in leaves]

    lean = run(lambda a, b, c: norm_linear(a, b, c, 1e-5))
    plain = run(lambda a, b, c: matmul_nt(kernel_registry.get_op("rms_norm")(a, b, eps=1e-5), c))
    for a, b in zip(lean, plain):
        assert torch.equal(a, b)
    xf, nwf, wf = (t.float().requires_grad_(True) for t in (x, nw, w))
    ref = (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-5) * nwf) @ wf.t()
    ref.backward(dy.float())
    for got, want in zip(lean, (ref.detach(), xf.grad, nwf.grad, wf.grad)):
        assert (got.float() - want).abs().max() / want.abs().max() < 2e-2

    gu = torch.randn(rows, 2 * f, device="cuda", generator=g).to(torch.bfloat16)
    w2 = (0.05 * torch.randn(h, f, device="cuda", generator=g)).to(torch.bfloat16)
    dy2 = torch.randn(rows, h, device="cuda", generator=g).to(torch.bfloat16)

    def run2(fn):
        leaves = [t.clone().requires_grad_(True) for t in (gu, w2)]
        y = fn(*leaves)
        y.backward(dy2)
        return [y.detach()] + [t.grad for t in leaves]

    lean2 = run2(swiglu_linear)
    plain2 = run2(lambda a, b: matmul_nt(swiglu_packed(a), b))
    for a, b in zip(lean2, plain2):
        assert torch.equal(a, b)
    guf, w2f = gu.float().requires_grad_(True), w2.float().requires_grad_(True)
    ref2 = (torch.nn.functional.silu(guf[:, :f]) * guf[:, f:]) @ w2f.t()
    ref2.backward(dy2.float())
    for got, want in zip(lean2, (ref2.detach(), guf.grad, w2f.grad)):
        assert (got.float() - want).abs().max() / want.abs().max() < 2e-2


@pytest.mark.parametrize("prompt_len,completion_len", [(128, 128), (100, 72)])
def test_prompt_cached_micro_batches_match_the_single_pass(prompt_len, completion_len):
    """The shared prompt runs once; micro-batches of completions attend to its cached keys / values and send their
    gradients back through fp32 leaves.  Log-probs must equal the single pass (bitwise when the prompt and completion
    lengths are multiples of the 128-row tile, so that every row sees the same tiles in the same order), and the
    accumulated gradients must agree with the single pass to bf16 rounding."""
    from rl_engine.models.config import ModelConfig
    from rl_engine.models.grpo import (GRPOTrainer, _PromptPass, policy_logps, policy_logps_after_prefix,
                                       synthetic_batch)
    from rl_engine.models.llama import LlamaModel

    cfg = ModelConfig("prefix", 1024, 256, 3, 4, 2, 128, 512)
    host = synthetic_batch(cfg.vocab_size, prompt_len=prompt_len, group=6, completion_len=completion_len, seed=9)
    host.completion_mask[2, completion_len // 2:] = False
    batch = host.to("cuda")
    model = LlamaModel(cfg, dtype=torch.bfloat16, device="cuda", seed=12)
    assert model.supports_prefix_cache()
    with torch.no_grad():
        full = policy_logps(model, batch)
        prefix = _PromptPass(model, batch.prompt_ids)
        parts = [policy_logps_after_prefix(model, batch.completions(i, i + 2), *prefix.inputs()) for i in (0, 2, 4)]
    cached = torch.cat(parts)
    if prompt_len % 128 == 0 and completion_len % 128 == 0:
        assert torch.equal(cached, full)
    else:
        assert torch.allclose(cached, full, atol=2e-2, rtol=2e-2)
    gen = torch.Generator(device="cuda").manual_seed(1)
    batch.old_logps = full + 0.05 * torch.randn(full.shape, device="cuda", generator=gen)
    batch.ref_logps = full + 0.05 * torch.randn(full.shape, device="cuda", generator=gen)

    results = {}
    for name, micro, cache in (("single", None, False), ("micro", 2, False), ("cached", 2, True)):
        m = LlamaModel(cfg, dtype=torch.bfloat16, device="cuda", seed=12)
        trainer = GRPOTrainer(m, lr=1e-3, micro_group=micro)
        trainer.cache_prompt = cache
        trainer.opt.zero_grad()
        loss = trainer.forward_backward(batch)
        results[name] = (float(loss), m.flat_grad.float().clone())
    ref_loss, ref_grad = results["single"]
    for name in ("micro", "cached"):
        loss, grad = results[name]
        assert abs(loss - ref_loss) < 2e-3 * max(1.0, abs(ref_loss)), (name, loss, ref_loss)
        rel = (grad - ref_grad).norm() / ref_grad.norm()
        assert float(rel) < 2e-2, (name, float(rel))
    # the embedding rows of prompt tokens receive gradient only through the prompt pass
    emb = results["cached"][1][: cfg.vocab_size * cfg.hidden_size].view(cfg.vocab_size, cfg.hidden_size)
    assert float(emb[host.prompt_ids.unique().cuda()].abs().sum()) > 0


def test_kv_cached_decode_matches_the_packed_forward_and_rollout_engine_runs():
    """Teacher-forced: hidden states from ``decode_step`` (one new token per completion against the key / value cache)
    must match the rows of the packed full forward.  The rollout engine on top of it is reproducible for a seed, with
    bf16 and with fp8 layer projections."""
    from rl_engine.executors.native_rollout import NativeRolloutEngine
    from rl_engine.kernels.ops.sm100.attention import grpo_group_layout
    from rl_engine.models.config import ModelConfig
    from rl_engine.models.llama import LlamaModel

    cfg = ModelConfig("decode", 1024, 256, 2, 4, 2, 128, 512)
    model = LlamaModel(cfg, dtype=torch.bfloat16, device="cuda", seed=31)
    p, g, l = 100, 3, 20
    gen = torch.Generator(device="cuda").manual_seed(3)
    prompt = torch.randint(0, cfg.vocab_size, (p,), device="cuda", generator=gen)
    comp = torch.randint(0, cfg.vocab_size, (g, l), device="cuda", generator=gen)
    with torch.no_grad():
        positions = torch.cat([torch.arange(p, device="cuda"), (p + torch.arange(l, device="cuda")).repeat(g)])
        full = model.hidden_states(torch.cat([prompt, comp.reshape(-1)]), positions, grpo_group_layout(p, g, l, "cuda"))
        last, prompt_kv = model.prefix_states(prompt)
        assert torch.allclose(last[0].float(), full[p - 1].float(), atol=3e-2, rtol=3e-2)
        cache = model.new_kv_cache(p + g * l)
        for (ck, cv), (pk, pv) in zip(cache, prompt_kv):
            ck[:p].copy_(pk)
            cv[:p].copy_(pv)
        base = p + torch.arange(g, device="cuda") * l
        prefix_layout, own_layout = model.decode_layouts(g, p, l)
        for t in range(l):
            pos = torch.full((g,), p + t, dtype=torch.long, device="cuda")
            hidden = model.decode_step(comp[:, t].contiguous(), pos, cache, base + t, prefix_layout, own_layout)
            own_layout.seqs[:, 5] += 1
            want = full[p + torch.arange(g, device="cuda") * l + t]
            assert torch.allclose(hidden.float(), want.float(), atol=4e-2, rtol=4e-2), t

    outs = [NativeRolloutEngine(model, seed=5).generate(prompt, num_generations=4, max_new_tokens=12, top_k=20)
            for _ in range(2)]
    assert outs[0]["completion_ids"].shape == (4, 12) and torch.equal(outs[0]["completion_ids"], outs[1]["completion_ids"])
    assert torch.isfinite(outs[0]["rollout_logps"]).all() and outs[0]["rollout_logps"].shape == (4, 12)
    eager = NativeRolloutEngine(model, seed=5, use_cuda_graph=False).generate(prompt, num_generations=4, max_new_tokens=12, top_k=20)
    assert torch.equal(eager["completion_ids"], outs[0]["completion_ids"])  # the captured step replays the same kernels
    stateless = NativeRolloutEngine(model, seed=5, use_kv_cache=False).generate(
        prompt, num_generations=4, max_new_tokens=12, top_k=20)
    # same seed, same draws: the first token comes from the prompt pass, whose rows are the same bits on both paths
    # (later tokens may differ: a random-init model's logits are nearly flat, so bf16 rounding can flip a draw)
    assert torch.equal(stateless["completion_ids"][:, 0], outs[0]["completion_ids"][:, 0])
    fp8 = NativeRolloutEngine(model, seed=5, fp8_linears=True).generate(prompt, num_generations=4, max_new_tokens=12, top_k=20)
    assert fp8["completion_ids"].shape == (4, 12) and torch.isfinite(fp8["rollout_logps"]).all()
    model.enable_fp8_inference(False)


@pytest.mark.parametrize("tokens,hq,hkv", [(1, 4, 1), (37, 8, 2), (1000, 32, 4)])
def test_fused_qk_head_norm_matches_the_generic_ops(tokens, hq, hkv):
    """Per-head RMSNorm of q and k inside a packed qkv buffer (one kernel each way) against slices + generic RMSNorm +
    concatenation in fp32: output, gradient of the buffer and of both weights; v passes through untouched; a buffer
    with a row pitch larger than its width works; two runs give the same bits."""
    from rl_engine.models.llama import _QKHeadNorm

    g = torch.Generator(device=DEV).manual_seed(tokens)
    width = (hq + 2 * hkv) * 128
    wide = torch.randn(tokens, width + 64, device=DEV, generator=g).to(torch.bfloat16)
    qkv = wide[:, :width]
    wq = (1.0 + 0.1 * torch.randn(128, device=DEV, generator=g)).to(torch.bfloat16)
    wk = (1.0 + 0.1 * torch.randn(128, device=DEV, generator=g)).to(torch.bfloat16)
    dout = torch.randn(tokens, width, device=DEV, generator=g).to(torch.bfloat16)
    eps = 1e-6

    a, aq, ak = qkv.clone().requires_grad_(True), wq.clone().requires_grad_(True), wk.clone().requires_grad_(True)
    x = a if tokens != 37 else None
    if x is None:  # non-contiguous rows
        holder = wide.clone().requires_grad_(True)
        x, a = holder[:, :width], holder
    out = _QKHeadNorm.apply(x, aq, ak, hq, hkv, eps)
    out.backward(dout)

    b, bq, bk = qkv.float().clone().requires_grad_(True), wq.float().clone().requires_grad_(True), wk.float().clone().requires_grad_(True)
    b3 = b.view(tokens, hq + 2 * hkv, 128)

    def norm(v, w):
        return v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + eps) * w

    ref = torch.cat([norm(b3[:, :hq], bq), norm(b3[:, hq:hq + hkv], bk), b3[:, hq + hkv:]], dim=1).reshape(tokens, width)
    ref.backward(dout.float())
    assert torch.allclose(out.float(), ref, atol=2e-2, rtol=2e-2)
    assert torch.equal(out[:, (hq + hkv) * 128:], qkv[:, (hq + hkv) * 128:])
    got_dx = a.grad[:, :width] if a.grad.shape[1] != width else a.grad
    assert torch.allclose(got_dx.float(), b.grad, atol=3e-2, rtol=3e-2)
    scale = max(1.0, float(bq.grad.abs().max()))
    assert torch.allclose(aq.grad.float(), bq.grad, atol=2e-2 * scale, rtol=2e-2)
    assert torch.allclose(ak.grad.float(), bk.grad, atol=2e-2 * max(1.0, float(bk.grad.abs().max())), rtol=2e-2)
    again = _QKHeadNorm.apply(x.detach(), wq, wk, hq, hkv, eps)
    assert torch.equal(again, out.detach())
