"""CPU tests: registry dispatch, PyTorch oracle operators, testing helpers, sampler front end."""

import importlib

import pytest
import torch


# ----------------------------------------------------------------------------------- registry
def test_registry_routes_cpu_to_pytorch_ops_and_caches():
    from rl_engine.kernels.registry import KernelRegistry, OpBackend

    reg = KernelRegistry()
    expected = {
        "logp": "NativeLogpOp", "logp_indexed": "NativeLogpOp", "logp_online": "NativeLogpOp",
        "logp_online_indexed": "NativeLogpOp", "attn": "NativeAttentionOp", "grpo_loss": "NativeGRPOLossOp",
        "linear_logp": "NativeLinearLogpOp", "ratio_kl": "NativeRatioKLOp", "rms_norm": "NativeRMSNormOp",
        "lm_head": "NativeLMHeadOp", "embedding": "NativeEmbeddingOp", "silu": "NativeSiLUOp",
        "swiglu": "NativeSwiGLUOp", "rope": "NativeRoPEOp", "ppo_loss": "NativePPOLossOp", "dpo_loss": "NativeDPOLossOp",
        "prefix_shared_attn": "NativePrefixSharedAttentionOp", "moe": "NativeMoEOp",
    }
    for op_type, cls in expected.items():
        op = reg.get_op(op_type)
        assert type(op).__name__ == cls
        assert reg.get_op(op_type) is op  # instance cache
    assert set(expected) == set(reg.op_types())
    with pytest.raises(ValueError, match="Supported backends"):
        OpBackend["NOT_A_BACKEND"]


def test_registry_missing_backend_falls_through_and_internal_bug_reraises(monkeypatch):
    from rl_engine.kernels import registry as regmod

    reg = regmod.KernelRegistry()

    class Fake:
        name = "FAKE"
        value = "rl_engine.kernels.ops.does_not_exist.Op"

    assert reg._load_backend(Fake) is None  # a missing backend module is not an error

    real_import = importlib.import_module

    def broken(name, *a, **k):
        if name == "rl_engine.kernels.ops.pytorch.loss.logp":
            raise ModuleNotFoundError("No module named 'rl_engine.some_internal_dep'", name="rl_engine.some_internal_dep")
        return real_import(name, *a, **k)

    monkeypatch.setattr(regmod.importlib, "import_module", broken)
    with pytest.raises(ModuleNotFoundError):
        reg._load_backend(regmod.OpBackend.PYTORCH_NATIVE)


def test_registry_failed_backend_is_remembered(monkeypatch):
    from rl_engine.kernels import registry as regmod

    reg = regmod.KernelRegistry()
    reg._priority_map["cpu"]["logp"] = [regmod.OpBackend.SM100_FUSED_LOGP, regmod.OpBackend.PYTORCH_NATIVE]
    calls = []
    real = reg._load_backend

    def spy(backend):
        calls.append(backend.name)
        return None if backend is regmod.OpBackend.SM100_FUSED_LOGP else real(backend)

    monkeypatch.setattr(reg, "_load_backend", spy)
    assert type(reg.get_op("logp")).__name__ == "NativeLogpOp"
    reg._instance_cache.clear()
    reg.get_op("logp")
    assert calls.count("SM100_FUSED_LOGP") == 1  # not retried once it failed


def test_force_backend_env(monkeypatch):
    from rl_engine.kernels import registry as regmod

    monkeypatch.setenv("RL_KERNEL_FORCE_BACKEND", "pytorch")
    reg = regmod.KernelRegistry()
    assert all(len(v) == 1 for v in reg._priority_map["cuda"].values())


def test_device_context_and_constants():
    from rl_engine.platforms import constants, device_ctx

    assert device_ctx.device_type in {"cpu", "cuda"} and device_ctx.is_rocm is False
    assert constants.DeviceType.CUDA.value == "cuda" and constants.BackendLib.SM100.value == "sm100"
    assert constants.CheckpointFormat.PT.value == "pt"


def test_logger_once_helpers(capsys):
    from rl_engine.utils.logger import init_logger

    log = init_logger("RL-Kernel-test")
    log.info_once("only %s", "once")
    log.info_once("only %s", "once")
    log.warn_once("careful")
    log.warn_once("careful")
    out = capsys.readouterr().out
    assert out.count("only once") == 1 and out.count("careful") == 1


# -------------------------------------------------------------------------------- logp family
def test_native_logp_nine_methods():
    from rl_engine.kernels.ops.pytorch.loss.logp import NativeLogpOp

    g = torch.Generator().manual_seed(0)
    logits = torch.randn(2, 5, 30, generator=g)
    ids = torch.randint(0, 30, (2, 5), generator=g)
    op = NativeLogpOp()
    want = torch.log_softmax(logits, -1).gather(-1, ids[..., None]).squeeze(-1)
    assert torch.allclose(op(logits, ids), want, atol=1e-6)
    assert torch.allclose(op.apply_fp32(logits.half(), ids), torch.log_softmax(logits.half().float(), -1).gather(-1, ids[..., None]).squeeze(-1), atol=1e-6)
    out = torch.full((2, 5), 9.0)
    rows = torch.tensor([0, 7])
    op.online_indexed_out(logits, ids, rows, out)
    flat = out.view(-1)
    assert torch.allclose(flat[rows], want.view(-1)[rows], atol=1e-6) and (flat[[1, 2, 3]] == 9).all()
    z = op.indexed_fp32(logits, ids, rows).view(-1)
    assert z[1] == 0 and torch.allclose(z[rows], want.view(-1)[rows], atol=1e-6)
    assert torch.allclose(op.online_out(logits, ids, torch.empty(2, 5)), want, atol=1e-6)
    with pytest.raises(ValueError):
        op(logits, ids[:, :4])
    with pytest.raises(ValueError):
        op.indexed_fp32(logits, ids, torch.tensor([10]))


# ------------------------------------------------------------------------------ linear_logp
def test_native_linear_logp_layout_invariance_and_grads():
    from rl_engine.kernels.ops.pytorch.loss.linear_logp import NativeLinearLogpOp, chunked_linear_logp_backward

    g = torch.Generator().manual_seed(1)
    N, D, V = 40, 80, 300
    h = torch.randn(N, D, generator=g, requires_grad=True)
    w = (torch.randn(V, D, generator=g) * 0.1).requires_grad_(True)
    b = torch.randn(V, generator=g).requires_grad_(True)
    t = torch.randint(0, V, (N,), generator=g)
    op = NativeLinearLogpOp()
    lp = op(h, w, t, b)
    want = torch.log_softmax(h @ w.t() + b, -1).gather(-1, t[:, None]).squeeze(-1)
    assert torch.allclose(lp, want, atol=1e-5)
    assert torch.equal(op(h.view(5, 8, D), w, t.view(5, 8), b).view(-1), lp)  # layout invariance
    perm = torch.randperm(N, generator=g)
    assert torch.allclose(op(h[perm], w, t[perm], b), lp[perm], atol=1e-6)
    gl = torch.randn(N, generator=g)
    lp.backward(gl)
    gh, gw, gb = chunked_linear_logp_backward(
        gl, h.detach(), w.detach(), t, b.detach(), has_bias=True, lead_shape=(N,), hidden_dtype=h.dtype,
        weight_dtype=w.dtype, bias_dtype=b.dtype, chunk_elems=7 * V,
    )
    assert torch.allclose(gh, h.grad, atol=1e-5) and torch.allclose(gw, w.grad, atol=1e-5) and torch.allclose(gb, b.grad, atol=1e-5)
    lp2, ent = op.with_entropy(h, w, t, b)
    p = torch.softmax(h @ w.t() + b, -1)
    assert torch.allclose(lp2, lp, atol=1e-6) and torch.allclose(ent, -(p * p.log()).sum(-1), atol=1e-5)
    with pytest.raises(ValueError):
        op(h, w[:, :-1], t)
    with pytest.raises(ValueError):
        op(h, w, t, torch.zeros(V + 1))
    with pytest.raises(ValueError):
        op(h, w, t, vocab_start_index=3)  # shard description without a group


# ------------------------------------------------------------------------ ratio_kl / grpo loss
def _rl_inputs(seed=2, B=6, T=7, V=40):
    g = torch.Generator().manual_seed(seed)
    pol = torch.randn(B, T, V, generator=g)
    ref = pol + 0.1 * torch.randn(B, T, V, generator=g)
    ids = torch.randint(0, V, (B, T), generator=g)
    mask = torch.rand(B, T, generator=g) > 0.3
    old = torch.log_softmax(pol, -1).gather(-1, ids[..., None]).squeeze(-1) + 0.05 * torch.randn(B, T, generator=g)
    rewards = torch.randn(B, generator=g)
    return pol, ref, ids, mask, old, rewards


def test_ratio_kl_mask_semantics():
    from rl_engine.kernels.ops.pytorch.loss.ratio_kl import NativeRatioKLOp

    pol, ref, ids, mask, old, _ = _rl_inputs()
    garbage = torch.where(mask, ids, torch.full_like(ids, -100))
    pol.requires_grad_(True)
    ratio, kl = NativeRatioKLOp()(pol, ref, garbage, mask, old)
    assert (ratio[~mask] == 1).all() and (kl[~mask] == 0).all() and (kl >= -1e-7).all()
    (ratio.sum() + kl.sum()).backward()
    assert (pol.grad[~mask] == 0).all()
    bad = ids.clone()
    bad[mask] = 40
    with pytest.raises(ValueError):
        NativeRatioKLOp()(pol.detach(), ref, bad, mask, old)


def test_grpo_loss_group_advantages_and_optimisation():
    from rl_engine.kernels.ops.pytorch.loss.grpo_loss import NativeGRPOLossOp

    pol, ref, ids, mask, old, rewards = _rl_inputs()
    op = NativeGRPOLossOp()
    adv = op.group_advantages(rewards, samples_per_prompt=3)
    r = rewards.view(2, 3)
    want = ((r - r.mean(1, keepdim=True)) / r.std(1, unbiased=False, keepdim=True)).view(-1)
    assert torch.allclose(adv, want, atol=1e-5)
    assert torch.allclose(op.group_advantages(rewards, group_boundaries=[0, 3, 6]), want, atol=1e-5)
    assert torch.isfinite(op.group_advantages(torch.ones(4), samples_per_prompt=2)).all()
    for kwargs in ({}, {"samples_per_prompt": 3, "group_boundaries": [0, 3, 6]}, {"samples_per_prompt": 1},
                   {"samples_per_prompt": 4}, {"group_boundaries": [0, 3]}, {"group_boundaries": [0, 3, 3, 6]}):
        with pytest.raises(ValueError):
            op.group_advantages(rewards, **kwargs)
    logits = pol.clone().requires_grad_(True)
    opt = torch.optim.SGD([logits], lr=0.5)
    losses = []
    for _ in range(5):
        opt.zero_grad()
        loss, pl, kl = op(logits, ref, ids, old, rewards, mask, clip_eps=0.2, beta=0.04, samples_per_prompt=3)
        assert torch.allclose(loss, pl + 0.04 * kl)
        loss.backward()
        opt.step()
        losses.append(float(loss))
    assert losses[-1] < losses[0]
    # logp-space entry point gives the same numbers as the logits entry point
    lp = torch.log_softmax(pol, -1).gather(-1, ids[..., None]).squeeze(-1)
    lr = torch.log_softmax(ref, -1).gather(-1, ids[..., None]).squeeze(-1)
    a = op.apply(pol, ref, ids, old, adv, mask, clip_eps=0.2, beta=0.04)
    b = op.apply_from_logps(lp, lr, old, adv, mask, clip_eps=0.2, beta=0.04)
    assert all(torch.allclose(x, y, atol=1e-6) for x, y in zip(a, b))


def test_ppo_and_dpo_oracles():
    from rl_engine.kernels.ops.pytorch.loss.policy_losses import NativeDPOLossOp, NativePPOLossOp

    g = torch.Generator().manual_seed(4)
    lp = -torch.rand(4, 6, generator=g)
    old = lp + 0.2 * torch.randn(4, 6, generator=g)
    adv = torch.randn(4, 6, generator=g)
    mask = torch.ones(4, 6, dtype=torch.bool)
    loss, pl, kl = NativePPOLossOp()(lp, old, adv, mask, clip_eps=0.2)
    r = torch.exp(lp - old)
    assert torch.allclose(pl, (-torch.minimum(r * adv, r.clamp(0.8, 1.2) * adv)).mean(), atol=1e-6) and kl == 0
    pc, pr, rc, rr = (torch.randn(5, generator=g) for _ in range(4))
    dl, cr, rj = NativeDPOLossOp()(pc, pr, rc, rr, beta=0.5)
    assert torch.allclose(dl, -torch.nn.functional.logsigmoid(0.5 * ((pc - pr) - (rc - rr))).mean(), atol=1e-6)
    assert torch.allclose(cr, 0.5 * (pc - rc)) and torch.allclose(rj, 0.5 * (pr - rr))
    tok = torch.randn(2, 4)
    m = torch.tensor([[1, 1, 0, 0], [1, 1, 1, 1]], dtype=torch.bool)
    assert torch.allclose(NativeDPOLossOp.sequence_logps(tok, m), (tok * m).sum(-1))


def test_expert_parallel_plan_is_a_consistent_partition():
    """Every rank derives its send slots from the same count matrix: together the assignments of all
    ranks fill each owner's expert blocks exactly once, in (source rank, assignment) order."""
    from rl_engine.parallel.expert_parallel import build_ep_plan

    world, experts, k = 4, 8, 2
    g = torch.Generator().manual_seed(0)
    idxs = [torch.stack([torch.randperm(experts, generator=g)[:k] for _ in range(40 + 7 * r)]).int() for r in range(world)]
    counts = torch.stack([torch.bincount(i.reshape(-1).long(), minlength=experts) for i in idxs])
    plans = [build_ep_plan(idxs[r], counts, r, world, 4096) for r in range(world)]
    el = experts // world
    for owner in range(world):
        taken = []
        for r in range(world):
            sel = plans[r].dest_rank == owner
            slots = plans[r].dest_slot[sel].long()
            exp = idxs[r].reshape(-1)[sel].long() - owner * el
            off = plans[owner].offsets.long()
            assert bool(((slots >= off[exp]) & (slots < off[exp + 1])).all())
            taken.append(slots)
        taken = torch.cat(taken)
        assert taken.unique().numel() == taken.numel()
        total = counts[:, owner * el:(owner + 1) * el].sum(0)
        off = plans[owner].offsets.long()
        for e in range(el):
            want = torch.arange(off[e], off[e] + total[e])
            got = taken[(taken >= off[e]) & (taken < off[e + 1])].sort().values
            assert torch.equal(got, want)
        tg = plans[owner].tile_group
        used_tiles = int(off[-1]) // 128
        assert bool((tg[:used_tiles] >= 0).all()) and bool((tg[used_tiles:] == -1).all())


def test_context_parallel_zigzag_shards_round_trip_and_balance():
    from rl_engine.parallel.context_parallel import local_layout_rows, shard_sequence, unshard_sequence, zigzag_chunks

    world, chunk = 4, 6
    x = torch.arange(2 * world * chunk * 3).view(2 * world * chunk, 3)
    parts = [shard_sequence(x, r, world) for r in range(world)]
    assert torch.equal(unshard_sequence(parts), x)
    assert sorted(c for r in range(world) for c in zigzag_chunks(r, world)) == list(range(2 * world))
    work = []
    for r in range(world):
        rows = local_layout_rows(r, world, chunk)
        assert [row[0] for row in rows] == [0, chunk] and all(row[1] == chunk and row[5] == chunk for row in rows)
        assert all(row[2] == 0 and row[3] == row[4] for row in rows)  # prefix = every key before the chunk
        work.append(sum(row[3] + row[5] / 2 for row in rows))
    assert max(work) == min(work)  # zig-zag gives every rank the same number of visible keys
    with pytest.raises(ValueError):
        shard_sequence(x[:-1], 0, world)


def test_phase_timer_and_trace_range_on_cpu():
    from rl_engine.utils.tracing import PhaseTimer, trace_range, traced

    timer = PhaseTimer(device="cpu")
    with trace_range("outer"):
        for _ in range(3):
            with timer.phase("matmul"):
                torch.randn(64, 64) @ torch.randn(64, 64)
        with timer.phase("other"):
            pass
    s = timer.summary()
    assert list(s) == ["matmul", "other"] and s["matmul"]["calls"] == 3 and s["matmul"]["total_ms"] > 0
    assert list(timer.max_over_ranks()) == ["matmul", "other"]

    @traced("labelled")
    def f(x):
        return x + 1

    assert f(1) == 2
    timer.reset()
    assert not timer.summary()


def test_alias_package_exposes_the_same_modules():
    import rl_kernel_b200

    assert rl_kernel_b200.ops.registry.kernel_registry is not None
    assert rl_kernel_b200.parallel.__name__ == "rl_engine.parallel"
    from rl_kernel_b200 import models, utils  # noqa: F401

    assert {"executors", "models", "ops", "parallel", "utils", "integrations"} <= set(dir(rl_kernel_b200))
    with pytest.raises(AttributeError):
        rl_kernel_b200.nothing_here


def test_debug_bounds_build_compiles(tmp_path):
    """``RLK_DEBUG_BOUNDS=1`` turns ``RLK_INDEX_OK`` into a checked access that reports to the error word; the
    kernels that take user indices must still compile for sm_100a with it switched on."""
    import os
    import shutil
    import subprocess

    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        pytest.skip("nvcc not available")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    src = os.path.join(root, "csrc", "kernels", "moe.cu")
    text = open(os.path.join(root, "csrc", "common", "ptx.cuh")).read()
    assert "RLK_DEBUG_BOUNDS" in text and "kErrBadIndex" in text
    out = subprocess.run(
        [nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-std=c++17", "-O1", "-DRLK_DEBUG_BOUNDS=1", "-c", src,
         "-o", str(tmp_path / "moe_debug.o")],
        capture_output=True, text=True, timeout=600,
    )
    assert out.returncode == 0, out.stderr[-2000:]


def test_poly_exp2_coefficients_are_accurate_enough_for_bf16_probabilities():
    """Host restatement of ``poly_exp2`` (csrc/common/ptx.cuh): round-to-nearest split through the 1.5 * 2^23 magic
    constant, cubic on [-0.5, 0.5], exponent add.  Relative error must stay far below bf16 resolution (3.9e-3)."""
    import re
    import struct

    root = __import__("os").path.dirname(__import__("os").path.dirname(__import__("os").path.abspath(__file__)))
    src = open(__import__("os").path.join(root, "csrc", "common", "ptx.cuh")).read()
    body = src[src.index("float poly_exp2(float x)"):]
    coeffs = [float(c) for c in re.findall(r"(0\.\d+)f", body[: body.index("return")])]
    assert len(coeffs) == 4, coeffs
    c3, c2, c1, c0 = coeffs

    def f32(v):
        return struct.unpack("f", struct.pack("f", v))[0]

    def poly_exp2(x):
        x = max(x, -126.0)
        t = f32(x + 12582912.0)
        f = f32(x - f32(t - 12582912.0))
        p = f32(f32(f * c3) + c2)
        p = f32(f32(p * f) + c1)
        p = f32(f32(p * f) + c0)
        bits = struct.unpack("I", struct.pack("f", p))[0] + ((struct.unpack("I", struct.pack("f", t))[0] << 23) & 0xFFFFFFFF)
        return struct.unpack("f", struct.pack("I", bits & 0xFFFFFFFF))[0]

    worst = 0.0
    for i in range(4001):
        x = -40.0 * i / 4000.0
        worst = max(worst, abs(poly_exp2(x) / 2.0 ** x - 1.0))
    assert worst < 2e-4, worst
    assert abs(poly_exp2(0.0) - 1.0) < 1e-4 and abs(poly_exp2(-1.0) - 0.5) < 1e-4


def test_extension_imports_in_a_fresh_interpreter_without_torch_preloaded():
    """The extension links against libtorch; the package has to load torch itself before importing it."""
    import glob
    import os
    import subprocess
    import sys

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    if not glob.glob(os.path.join(root, "rl_engine", "_C*.so")):
        pytest.skip("extension not built")
    code = "import rl_engine.kernels.ops.base as b; assert b._EXT_AVAILABLE, b._EXT_ERROR; print('ok')"
    out = subprocess.run([sys.executable, "-c", code], cwd=root, capture_output=True, text=True, timeout=300)
    assert out.returncode == 0 and "ok" in out.stdout, out.stderr[-2000:]
