"""Pipeline parallelism on CPU ranks (Gloo): the 1F1B schedule over two and three stages of a tiny Llama gives the
losses and the parameter gradients of the unsplit model; stage cutting; misuse is refused."""

import os
import tempfile

import pytest
import torch
import torch.multiprocessing as mp


def _micro_batches(vocab, count, p=5, g=2, l=4):
    out = []
    for i in range(count):
        gen = torch.Generator().manual_seed(100 + i)
        prompt = torch.randint(0, vocab, (p,), generator=gen)
        completions = torch.randint(0, vocab, (g, l), generator=gen)
        out.append((prompt, completions))
    return out


def _loss(hidden, head_weight, completions, rows):
    from rl_engine.kernels.registry import kernel_registry

    picked = kernel_registry.get_op("embedding")(rows, hidden)
    logp = kernel_registry.get_op("linear_logp")(picked, head_weight, completions.reshape(-1))
    return -logp.mean()


def _worker(rank, world, store_path, layers, micro, queue):
    import torch.distributed as dist

    try:
        dist.init_process_group("gloo", init_method=f"file://{store_path}", rank=rank, world_size=world)
        from rl_engine.models.config import tiny_llama
        from rl_engine.models.grpo import group_geometry
        from rl_engine.models.llama import LlamaModel
        from rl_engine.parallel.pipeline_parallel import LlamaPipelineStage, PipelineSchedule

        cfg = tiny_llama(head_dim=32).with_layers(layers)
        full = LlamaModel(cfg, dtype=torch.float32, device="cpu", seed=3, activation_checkpointing=False)
        batches = _micro_batches(cfg.vocab_size, micro)
        geometry = [group_geometry(b[0].numel(), b[1].shape[0], b[1].shape[1], "cpu") for b in batches]

        # the unsplit model: mean of the micro-batches' losses
        ref_losses = []
        for (prompt, completions), (layout, positions, rows) in zip(batches, geometry):
            hidden = full.hidden_states(torch.cat([prompt, completions.reshape(-1)]), positions, layout)
            loss = _loss(hidden, full.lm_head_weight(), completions, rows)
            (loss / micro).backward()
            ref_losses.append(float(loss.detach()))

        stage = LlamaPipelineStage(cfg, rank, world, dtype=torch.float32, device="cpu", activation_checkpointing=False)
        stage.load_from(full)
        inputs = [torch.cat([p, c.reshape(-1)]) for p, c in batches]

        def stage_fn(x, i):
            layout, positions, _rows = geometry[i]
            return stage.forward(x, positions, layout)

        def loss_fn(hidden, i):
            return _loss(hidden, stage.model.lm_head_weight(), batches[i][1], geometry[i][2])

        schedule = PipelineSchedule(stage_fn, dtype=torch.float32)
        losses = schedule.run(inputs, loss_fn if rank == world - 1 else None)

        worst = 0.0
        if rank == world - 1:
            worst = max(abs(float(a) - b) for a, b in zip(losses, ref_losses))
        full_views, mine = full.named_views(), stage.model.named_views()
        checked = 0
        for name, p in mine.items():
            if name.startswith("l") and "." in name and name[1:name.index(".")].isdigit():
                src = full_views[f"l{stage.layers[int(name[1:name.index('.')])]}{name[name.index('.'):]}"]
            elif name == "embed" and rank == 0:
                src = full_views[name]
            elif name in ("final_norm", "lm_head") and rank == world - 1:
                src = full_views[name]
            else:
                continue  # a parameter this stage owns but does not use
            assert p.grad is not None and src.grad is not None, name
            worst = max(worst, float((p.grad - src.grad).abs().max()))
            checked += 1
        queue.put((rank, worst, checked, None if losses is None else len(losses)))
        dist.destroy_process_group()
    except Exception as exc:  # pragma: no cover - reported to the parent
        import traceback

        queue.put((rank, f"{type(exc).__name__}: {exc}\n{traceback.format_exc()}", 0, None))


@pytest.mark.parametrize("world,layers,micro", [(2, 4, 3), (3, 5, 2)])
def test_1f1b_pipeline_matches_the_unsplit_model(world, layers, micro):
    ctx = mp.get_context("spawn")
    queue = ctx.Queue()
    with tempfile.TemporaryDirectory() as tmp:
        store = os.path.join(tmp, "store")
        procs = [ctx.Process(target=_worker, args=(r, world, store, layers, micro, queue)) for r in range(world)]
        for p in procs:
            p.start()
        results = []
        try:
            for _ in procs:
                results.append(queue.get(timeout=240))
        finally:
            for p in procs:
                p.join(timeout=10)
                if p.is_alive():
                    p.terminate()
    assert len(results) == world
    for rank, err, checked, n_losses in results:
        assert isinstance(err, float), (rank, err)
        assert err < 2e-5 and checked >= 6, (rank, err, checked)
        assert n_losses == (micro if rank == world - 1 else None)


def test_stage_cutting_and_misuse():
    from rl_engine.parallel.pipeline_parallel import stage_layers

    assert [list(r) for r in stage_layers(5, 3)] == [[0, 1], [2, 3], [4]]
    assert [len(r) for r in stage_layers(32, 8)] == [4] * 8
    with pytest.raises(ValueError):
        stage_layers(2, 3)


def _trainer_worker(rank, world, store_path, queue):
    import torch.distributed as dist

    try:
        dist.init_process_group("gloo", init_method=f"file://{store_path}", rank=rank, world_size=world)
        from rl_engine.models.config import tiny_llama
        from rl_engine.models.grpo import GRPOTrainer, synthetic_batch
        from rl_engine.models.llama import LlamaModel
        from rl_engine.parallel.pipeline_parallel import LlamaPipelineStage, PipelineGRPOTrainer

        cfg = tiny_llama(head_dim=32).with_layers(4)
        full = LlamaModel(cfg, dtype=torch.float32, device="cpu", seed=5, activation_checkpointing=False)
        batch = synthetic_batch(cfg.vocab_size, prompt_len=6, group=4, completion_len=5, seed=9)
        gen = torch.Generator().manual_seed(1)
        batch.old_logps = -2.0 + 0.1 * torch.randn(4, 5, generator=gen)
        batch.ref_logps = -2.0 + 0.1 * torch.randn(4, 5, generator=gen)
        batch.completion_mask[1, 3:] = False

        stage = LlamaPipelineStage(cfg, rank, world, dtype=torch.float32, device="cpu", activation_checkpointing=False)
        stage.load_from(full)
        pp = PipelineGRPOTrainer(stage, micro_group=2, lr=1e-3)
        single = GRPOTrainer(full, lr=1e-3, micro_group=None)
        want_losses = [float(single.step_device(batch)) for _ in range(2)]
        got_losses = [pp.step_device(batch) for _ in range(2)]

        worst = 0.0
        if rank == world - 1:
            worst = max(abs(float(a) - b) for a, b in zip(got_losses, want_losses))
        else:
            assert all(x is None for x in got_losses)
        full_views, mine = full.named_views(), stage.model.named_views()
        for name, p in mine.items():
            if name.startswith("l") and "." in name and name[1:name.index(".")].isdigit():
                src = full_views[f"l{stage.layers[int(name[1:name.index('.')])]}{name[name.index('.'):]}"]
            elif (name == "embed" and rank == 0) or (name in ("final_norm", "lm_head") and rank == world - 1):
                src = full_views[name]
            else:
                continue
            worst = max(worst, float((p.detach() - src.detach()).abs().max()))
        queue.put((rank, worst))
        dist.destroy_process_group()
    except Exception as exc:  # pragma: no cover - reported to the parent
        import traceback

        queue.put((rank, f"{type(exc).__name__}: {exc}\n{traceback.format_exc()}"))


def test_pipeline_grpo_trainer_steps_like_the_single_model_trainer():
    """Two AdamW steps of the GRPO objective on two pipeline stages (micro-batches of two completions) leave every
    parameter where the single-model trainer leaves it, and report the same losses."""
    world = 2
    ctx = mp.get_context("spawn")
    queue = ctx.Queue()
    with tempfile.TemporaryDirectory() as tmp:
        store = os.path.join(tmp, "store")
        procs = [ctx.Process(target=_trainer_worker, args=(r, world, store, queue)) for r in range(world)]
        for p in procs:
            p.start()
        results = []
        try:
            for _ in procs:
                results.append(queue.get(timeout=240))
        finally:
            for p in procs:
                p.join(timeout=10)
                if p.is_alive():
                    p.terminate()
    assert len(results) == world
    for rank, err in results:
        assert isinstance(err, float), (rank, err)
        assert err < 5e-5, (rank, err)
