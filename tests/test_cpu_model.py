"""CPU tests: model-side oracle ops (batch invariance + dtype-path accuracy), the tiny Llama GRPO step,
the sampler front end, model wrappers, and 4-rank Gloo vocab-parallel linear_logp."""

import os
import tempfile

import pytest
import torch
import torch.multiprocessing as mp


# ------------------------------------------------------------------- axis A / axis B contracts
def test_rmsnorm_swiglu_embedding_lmhead_contracts():
    from rl_engine.kernels.ops.pytorch.activation.swiglu import NativeSiLUOp, NativeSwiGLUOp
    from rl_engine.kernels.ops.pytorch.linear.embedding import NativeEmbeddingOp
    from rl_engine.kernels.ops.pytorch.linear.lm_head import NativeLMHeadOp
    from rl_engine.kernels.ops.pytorch.norm.rms_norm import NativeRMSNormOp

    g = torch.Generator().manual_seed(0)
    x = torch.randn(6, 9, 64, generator=g)
    w = torch.randn(64, generator=g)
    norm = NativeRMSNormOp()
    full = norm(x, w)
    assert torch.equal(full[2:4], norm(x[2:4], w))  # axis A: bitwise batch invariance
    want = x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + 1e-6) * w
    assert torch.allclose(full, want, atol=1e-6)
    xb = x.to(torch.bfloat16)
    assert norm(xb, w.to(torch.bfloat16)).dtype == torch.bfloat16 and norm.forward_fp32(xb, w).dtype == torch.float32
    assert torch.allclose(norm(xb, w.to(torch.bfloat16)).float(), norm.forward_fp32(xb, w.to(torch.bfloat16)), atol=5e-2)
    x_before = x.clone()
    norm(x, w)
    assert torch.equal(x, x_before)  # purity
    with pytest.raises(ValueError):
        norm(x, w[:-1])

    gate, up = torch.randn(4, 10, generator=g), torch.randn(4, 10, generator=g)
    sw = NativeSwiGLUOp()
    assert torch.allclose(sw(gate, up), torch.nn.functional.silu(gate) * up, atol=1e-6)
    # (CPU sigmoid takes a vector or a scalar path depending on alignment: compare to 1 ulp here; the
    #  bitwise batch-invariance contract is asserted on the GPU kernels)
    assert torch.allclose(sw(gate, up)[1:3], sw(gate[1:3], up[1:3]), atol=1e-7, rtol=1e-6)
    assert sw.forward_fp32(gate.half(), up.half()).dtype == torch.float32
    with pytest.raises(ValueError):
        sw(gate, up[:, :-1])
    assert torch.allclose(NativeSiLUOp()(gate), torch.nn.functional.silu(gate), atol=1e-6)

    table = torch.randn(50, 8, generator=g).to(torch.bfloat16)
    ids = torch.randint(0, 50, (3, 4), generator=g)
    emb = NativeEmbeddingOp()
    assert torch.equal(emb(ids, table), table[ids]) and emb.forward_fp32(ids.int(), table).dtype == torch.float32

    h, wt, b = torch.randn(5, 16, generator=g), torch.randn(30, 16, generator=g), torch.randn(30, generator=g)
    head = NativeLMHeadOp()
    assert torch.allclose(head(h, wt, bias=b), h @ wt.t() + b, atol=1e-5)
    prev = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = True
    with torch.autocast("cpu", dtype=torch.bfloat16):
        strict = head.forward_fp32(h.to(torch.bfloat16), wt.to(torch.bfloat16))
    assert strict.dtype == torch.float32 and torch.backends.cuda.matmul.allow_tf32 is True
    torch.backends.cuda.matmul.allow_tf32 = prev
    hg = h.clone().requires_grad_(True)
    head(hg, wt).sum().backward()
    assert torch.allclose(hg.grad, wt.sum(0).expand_as(h), atol=1e-5)  # closed form


def test_rope_oracle_properties():
    from rl_engine.kernels.ops.pytorch.linear.rope import NativeRoPEOp

    g = torch.Generator().manual_seed(1)
    x = torch.randn(2, 7, 3, 16, generator=g)
    pos = torch.arange(7).expand(2, 7)
    rope = NativeRoPEOp()
    y = rope(x, pos)
    assert torch.allclose(y.norm(dim=-1), x.norm(dim=-1), atol=1e-5)  # rotations preserve norms
    assert torch.allclose(rope(x, torch.zeros_like(pos)), x, atol=1e-6)
    # relative property: <R(p)q, R(p+d)k> depends only on d
    q, k = torch.randn(1, 1, 1, 16, generator=g), torch.randn(1, 1, 1, 16, generator=g)
    dots = [float((rope(q, torch.tensor([[p]])) * rope(k, torch.tensor([[p + 3]]))).sum()) for p in (0, 5, 11)]
    assert abs(dots[0] - dots[1]) < 1e-4 and abs(dots[0] - dots[2]) < 1e-4


def test_attention_oracles_gqa_and_prefix():
    from rl_engine.kernels.ops.pytorch.attention import (
        NativeAttentionOp, NativePrefixSharedAttentionOp, grouped_prefix_causal_attention_reference,
    )
    from rl_engine.models.llama import reference_packed_attention

    g = torch.Generator().manual_seed(2)
    q, k, v = torch.randn(2, 5, 4, 8, generator=g), torch.randn(2, 5, 2, 8, generator=g), torch.randn(2, 5, 2, 8, generator=g)
    out = NativeAttentionOp()(q, k, v, causal=True)
    rep = NativeAttentionOp()(q, k.repeat_interleave(2, 2), v.repeat_interleave(2, 2), causal=True)
    assert torch.allclose(out, rep, atol=1e-6)
    with pytest.raises(ValueError):
        NativeAttentionOp()(q, k[:, :, :1].expand(-1, -1, 3, -1), v[:, :, :1].expand(-1, -1, 3, -1))
    qs, ks, vs = torch.randn(1, 3, 4, 8, generator=g), torch.randn(1, 6, 8, generator=g), torch.randn(1, 6, 8, generator=g)
    shared = NativePrefixSharedAttentionOp()(qs, ks, vs)
    for i in range(3):
        s = torch.softmax(qs[0, i] @ ks[0].t() / 8**0.5, -1) @ vs[0]
        assert torch.allclose(shared[0, i], s, atol=1e-5)
    # packed reference (used by the CPU model) == explicit prefix + causal-suffix oracle
    P, G, L, hq, hkv = 5, 3, 4, 4, 2
    T = P + G * L
    q, k, v = (torch.randn(T, h, 8, generator=g) for h in (hq, hkv, hkv))
    seqs = [(0, P, 0, 0, 0, P)] + [(P + i * L, L, 0, P, P + i * L, L) for i in range(G)]
    packed = reference_packed_attention(q, k, v, seqs, True, 8**-0.5)
    want, _ = grouped_prefix_causal_attention_reference(
        q[P:].view(G, L, hq, 8), k[:P], v[:P], k[P:].view(G, L, hkv, 8), v[P:].view(G, L, hkv, 8))
    assert torch.allclose(packed[P:].view(G, L, hq, 8), want, atol=1e-5)


# --------------------------------------------------------------------- tiny Llama GRPO (config 1)
def test_cpu_fp32_grpo_step_on_tiny_llama():
    from rl_engine.kernels.registry import kernel_registry
    from rl_engine.models import LlamaModel, tiny_llama
    from rl_engine.models.grpo import GRPOTrainer, policy_logps, synthetic_batch

    cfg = tiny_llama()
    assert (cfg.num_layers, cfg.hidden_size, cfg.num_heads, cfg.head_dim, cfg.ffn_size, cfg.vocab_size) == (2, 256, 4, 64, 688, 32000)
    model = LlamaModel(cfg, dtype=torch.float32, device="cpu", seed=0)
    trainer = GRPOTrainer(model, lr=1e-3, clip_eps=0.2, beta=0.04)
    batch = synthetic_batch(cfg.vocab_size, prompt_len=64, group=8, completion_len=128, seed=0)
    with torch.no_grad():
        cur = policy_logps(model, batch)
        # fused_logp (registry "logp" op over materialised logits) vs the naive log_softmax gather
        tokens = torch.cat([batch.prompt_ids, batch.completion_ids.reshape(-1)])
        from rl_engine.models.grpo import group_geometry

        layout, positions, rows = group_geometry(64, 8, 128, "cpu")
        logits = model(tokens, positions, layout)[rows]
        naive = torch.log_softmax(logits, -1).gather(-1, batch.completion_ids.reshape(-1, 1)).squeeze(-1)
        fused = kernel_registry.get_op("logp").apply_fp32(logits, batch.completion_ids.reshape(-1))
    assert (fused - naive).abs().max() < 1e-5 and (cur.reshape(-1) - naive).abs().max() < 1e-4
    gen = torch.Generator().manual_seed(1)
    batch.old_logps = cur + 0.01 * torch.randn(cur.shape, generator=gen)
    batch.ref_logps = cur + 0.01 * torch.randn(cur.shape, generator=gen)
    before = model.flat.clone()
    l0 = trainer.step(batch)
    assert l0 == l0 and not torch.equal(before, model.flat)
    assert model.flat_grad.abs().sum() > 0
    # a second model with the same seed takes the bitwise same step
    model2 = LlamaModel(cfg, dtype=torch.float32, device="cpu", seed=0)
    assert GRPOTrainer(model2, lr=1e-3, clip_eps=0.2, beta=0.04).step(batch) == l0
    assert torch.equal(model.flat, model2.flat)


def test_model_presets():
    from rl_engine.models import llama3_8b, qwen3_30b_a3b

    c = llama3_8b()
    assert (c.num_layers, c.hidden_size, c.num_heads, c.num_kv_heads, c.head_dim, c.ffn_size, c.vocab_size) == (
        32, 4096, 32, 8, 128, 14336, 128256)
    assert 7.9e9 < c.param_count() < 8.2e9
    q = qwen3_30b_a3b()
    assert (q.num_layers, q.hidden_size, q.num_experts, q.experts_per_token, q.moe_ffn_size, q.vocab_size) == (
        48, 2048, 128, 8, 768, 151936)
    assert 29e9 < q.param_count() < 32e9


# ----------------------------------------------------------------------------------- sampler
def test_sampler_backend_cpu_paths_and_temperature_once():
    from rl_engine.kernels.sampling import SamplerBackend

    s = SamplerBackend()
    torch.manual_seed(0)
    logits = torch.tensor([[0.0, 5.0, 1.0, -2.0]]).repeat(200, 1)
    assert (s.sample(logits, top_k=1) == 1).all()
    picks = s.sample(logits, top_k=2, top_p=0.999, temperature=1.0)
    assert set(picks.tolist()) <= {1, 2}
    assert (s.sample(logits, top_p=0.5) == 1).all()  # the head token alone covers p
    # temperature must be applied exactly once: T = 2 on logits [0, 2 ln 3] gives p = (1/4, 3/4)
    two = torch.tensor([[0.0, 2 * torch.log(torch.tensor(3.0)).item()]]).repeat(20000, 1)
    freq = (s.sample(two, temperature=2.0) == 1).float().mean().item()
    assert abs(freq - 0.75) < 0.02
    with pytest.raises(ValueError):
        s.sample(logits, temperature=0.0)
    # top_k = 0 and top_p = 1 are the usual spellings of "off" (the fused kernel reads them that way too)
    off = s.sample(two, top_k=0, top_p=1.0)
    assert abs((off == 1).float().mean().item() - 0.9) < 0.02
    lp = s.compute_logp(torch.randn(3, 4, 9), torch.randint(0, 9, (3, 4)))
    assert lp.shape == (3, 4)


def test_host_philox_and_sample_reference_are_consistent():
    from rl_engine.kernels.ops.sm100.sampler import philox_uniform, sample_reference

    us = [philox_uniform(7, 3, r) for r in range(2000)]
    assert all(0.0 < u < 1.0 for u in us) and abs(sum(us) / len(us) - 0.5) < 0.03
    assert philox_uniform(7, 3, 0) == philox_uniform(7, 3, 0) != philox_uniform(7, 4, 0)
    z = torch.tensor([[3.0, 1.0, 2.0, -1.0]])
    assert sample_reference(z, top_k=1, top_p=1.0, temperature=1.0, seed=0, offset=0).tolist() == [0]


# ------------------------------------------------------------------------------ model wrappers
def test_model_wrappers_extract_and_score():
    from rl_engine.alignment import PolicyModelWrapper, ReferenceModelWrapper, extract_logits

    class Out:
        def __init__(self, logits):
            self.logits = logits

    t = torch.randn(2, 3, 5)
    assert extract_logits(t) is t and extract_logits({"logits": t}) is t and extract_logits(Out(t)) is t
    assert extract_logits((torch.tensor(1.0), t)) is t  # loss-first tuple
    for bad in ({"x": t}, object(), (torch.tensor(1.0),)):
        with pytest.raises(TypeError):
            extract_logits(bad)

    class Toy(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.e = torch.nn.Embedding(11, 6)
            self.h = torch.nn.Linear(6, 11)

        def forward(self, ids):
            return {"logits": self.h(self.e(ids))}

    toy = Toy()
    ids = torch.randint(0, 11, (2, 6))
    pol = PolicyModelWrapper(toy)
    mask = torch.tensor([[1, 1, 0, 0, 0], [1, 1, 1, 1, 0]], dtype=torch.bool)
    lp = pol.selected_logprobs(ids, ids[:, 1:], mask=mask, logits_end=-1, temperature=0.7)
    want = torch.log_softmax(toy(ids)["logits"][:, :-1] / 0.7, -1).gather(-1, ids[:, 1:, None]).squeeze(-1)
    assert torch.allclose(lp[mask], want[mask], atol=1e-6) and (lp[~mask] == 0).all() and lp.requires_grad
    ref = ReferenceModelWrapper(toy)
    assert not any(p.requires_grad for p in toy.parameters()) and not toy.training
    assert not ref.selected_logprobs(ids, ids[:, 1:], logits_end=-1).requires_grad


# ---------------------------------------------------------------- 4-rank Gloo vocab-parallel TP
def _tp_worker(rank, world, store_path, bounds, queue):
    import torch.distributed as dist

    from rl_engine.kernels.ops.pytorch.loss.linear_logp import NativeLinearLogpOp

    try:
        dist.init_process_group("gloo", init_method=f"file://{store_path}", rank=rank, world_size=world)
        g = torch.Generator().manual_seed(0)
        N, D, V = 9, 12, bounds[-1]
        h = torch.randn(N, D, generator=g)
        w = torch.randn(V, D, generator=g) * 0.3
        b = torch.randn(V, generator=g)
        t = torch.randint(0, V, (N,), generator=g)
        gl = torch.randn(N, generator=g)
        hf, wf, bf = h.clone().requires_grad_(True), w.clone().requires_grad_(True), b.clone().requires_grad_(True)
        NativeLinearLogpOp()(hf, wf, t, bf).backward(gl)
        v0, v1 = bounds[rank], bounds[rank + 1]
        hs, ws, bs = h.clone().requires_grad_(True), w[v0:v1].clone().requires_grad_(True), b[v0:v1].clone().requires_grad_(True)
        out = NativeLinearLogpOp()(hs, ws, t, bs, tp_group=dist.group.WORLD, vocab_start_index=v0, global_vocab_size=V)
        out.backward(gl)
        full = torch.log_softmax(h @ w.t() + b, -1).gather(-1, t[:, None]).squeeze(-1)
        errs = [
            (out - full).abs().max().item(), (hs.grad - hf.grad).abs().max().item(),
            (ws.grad - wf.grad[v0:v1]).abs().max().item(), (bs.grad - bf.grad[v0:v1]).abs().max().item(),
        ]
        bad_partition = False
        try:
            NativeLinearLogpOp()(h, w[v0:v1], t, tp_group=dist.group.WORLD, vocab_start_index=v0 + (1 if rank else 0),
                                 global_vocab_size=V)
        except ValueError:
            bad_partition = True
        queue.put((rank, max(errs), bad_partition))
        dist.destroy_process_group()
    except Exception as exc:  # pragma: no cover - reported to the parent
        queue.put((rank, f"{type(exc).__name__}: {exc}", False))


def test_vocab_parallel_linear_logp_four_gloo_ranks_uneven_shards():
    ctx = mp.get_context("spawn")
    queue = ctx.Queue()
    bounds = [0, 3, 7, 12, 16]
    with tempfile.TemporaryDirectory() as tmp:
        store = os.path.join(tmp, "store")
        procs = [ctx.Process(target=_tp_worker, args=(r, 4, store, bounds, queue)) for r in range(4)]
        for p in procs:
            p.start()
        results = []
        try:
            for _ in procs:
                results.append(queue.get(timeout=120))
        finally:
            for p in procs:
                p.join(timeout=10)
                if p.is_alive():
                    p.terminate()
    assert len(results) == 4
    for rank, err, bad_partition in results:
        assert isinstance(err, float), (rank, err)
        assert err < 1e-5 and bad_partition, (rank, err, bad_partition)


def test_activation_checkpoint_plan_modes_and_fallback():
    """``True`` recomputes every layer, ``False`` keeps every layer, ``"auto"`` on a CPU model recomputes (there is
    no device memory to plan against); an out-of-memory fallback lowers the number of kept layers by four."""
    from rl_engine.models.config import ModelConfig
    from rl_engine.models.llama import LlamaModel

    cfg = ModelConfig("plan", 256, 64, 6, 4, 2, 16, 128)
    assert LlamaModel(cfg, dtype=torch.float32, activation_checkpointing=True).plan_checkpointing(100) == 0
    keep_all = LlamaModel(cfg, dtype=torch.float32, activation_checkpointing=False)
    assert keep_all.plan_checkpointing(100) == 6
    assert LlamaModel(cfg, dtype=torch.float32).plan_checkpointing(100) == 0
    # per token: 2 H + qkv rows + q_dim + 2 F elements, plus the fp32 softmax statistics and two rstd
    per_token = 2 * 64 + (64 + 2 * 32) + 64 + 2 * 128
    assert keep_all.activation_bytes_per_layer(10) == 10 * (per_token * 4 + 4 * 4 + 8)
    assert keep_all.reduce_kept_layers(4) == 2 and keep_all.plan_checkpointing(100) == 2 and keep_all.kept_layers() == 2
    assert keep_all.reduce_kept_layers(4) == 0


def test_micro_batched_step_matches_the_single_pass_step():
    """Gradient accumulation over micro-batches of completions, each weighted by its share of the unmasked tokens,
    optimises the same token-mean loss as one pass over the whole group."""
    from rl_engine.models.config import ModelConfig
    from rl_engine.models.grpo import GRPOTrainer, choose_micro_group, policy_logps, synthetic_batch
    from rl_engine.models.llama import LlamaModel

    cfg = ModelConfig("micro", 512, 64, 2, 4, 2, 16, 128)
    batch = synthetic_batch(cfg.vocab_size, prompt_len=16, group=6, completion_len=12, seed=4)
    batch.completion_mask[1, 7:] = False  # uneven token counts between the micro-batches
    batch.completion_mask[4, 3:] = False
    results = []
    for micro in (None, 2, 4):  # 4: micro-batches of 4 and 2 completions
        model = LlamaModel(cfg, dtype=torch.float32, device="cpu", seed=2)
        with torch.no_grad():
            cur = policy_logps(model, batch)
        gen = torch.Generator().manual_seed(7)
        batch.old_logps = cur + 0.05 * torch.randn(cur.shape, generator=gen)
        batch.ref_logps = cur + 0.05 * torch.randn(cur.shape, generator=gen)
        trainer = GRPOTrainer(model, lr=1e-3, micro_group=micro)
        assert trainer.completions_per_pass(batch) == (6 if micro is None else micro)
        loss = trainer.step(batch)
        results.append((loss, model.flat_grad.clone()))
    for loss, grad in results[1:]:
        assert abs(loss - results[0][0]) < 1e-6
        assert (grad - results[0][1]).abs().max() < 1e-6 * max(1.0, float(results[0][1].abs().max()))

    # the chooser: everything fits -> one pass; all 32 layers fit at 17408 tokens but only 20 at 33792 -> 32 completions
    assert choose_micro_group(256, 1024, 512, 32, lambda tokens: 32) == 256
    gib = float(2**30)

    def kept(tokens, free=88.7):
        per, inp = tokens * 94344 / gib, tokens * 8192 / gib
        return (free - (32 * inp + 3 * per + 12)) // per

    assert choose_micro_group(256, 1024, 512, 32, kept) == 32
    assert choose_micro_group(32, 1024, 512, 32, kept) == 32
    assert choose_micro_group(6, 16, 12, 2, lambda tokens: 0) == 6  # short packed lengths are never split


def test_trainer_ignores_garbage_ids_at_masked_positions_and_rejects_them_at_active_ones():
    """Padding conventions put -100 or out-of-vocabulary ids at masked completion positions.  Completion tokens are model
    inputs too, so the trainer replaces them before use: loss and parameters are bit-identical to a clean batch.  The
    same values at ACTIVE positions are an error."""
    from rl_engine.models.config import ModelConfig
    from rl_engine.models.grpo import GRPOBatch, GRPOTrainer
    from rl_engine.models.llama import LlamaModel

    cfg = ModelConfig("t", 64, 32, 2, 2, 1, 16, 48)

    def run(garbage, at_active=False):
        model = LlamaModel(cfg, dtype=torch.float32, device="cpu", seed=1, max_positions=64)
        trainer = GRPOTrainer(model, lr=1e-2, micro_group=2)
        gen = torch.Generator().manual_seed(0)
        comp = torch.randint(0, 64, (4, 6), generator=gen)
        mask = torch.ones(4, 6, dtype=torch.bool)
        mask[1, 3:] = False
        mask[3, 1:] = False
        if garbage is not None:
            comp = torch.where(mask ^ at_active, comp, torch.full_like(comp, garbage))
        batch = GRPOBatch(prompt_ids=torch.randint(0, 64, (5,), generator=gen), completion_ids=comp, completion_mask=mask,
                          rewards=torch.tensor([1.0, 0.0, 0.5, -1.0]), old_logps=torch.full((4, 6), -4.0),
                          ref_logps=torch.full((4, 6), -4.0))
        return float(trainer.step_device(batch)), model.flat.clone()

    clean = run(None)
    for garbage in (-100, 9999):
        loss, flat = run(garbage)
        assert loss == clean[0] and torch.equal(flat, clean[1])
    with pytest.raises((IndexError, ValueError, RuntimeError)):
        run(9999, at_active=True)
