"""Trainer checkpoints: save -> mutate -> load restores weights, AdamW moments, master weights, the step count and the
sampler's stream position; sharded optimizer state is per rank and refuses a shard that is not its own."""

import os
import types

import pytest
import torch

from rl_engine.executors.checkpoint import load_checkpoint, save_checkpoint
from rl_engine.kernels.sampling import SamplerBackend
from rl_engine.models.config import ModelConfig
from rl_engine.models.grpo import FlatAdamW
from rl_engine.models.llama import LlamaModel


def tiny(dtype=torch.bfloat16, seed=0):
    cfg = ModelConfig(name="tiny", vocab_size=256, hidden_size=32, num_layers=2, num_heads=2, num_kv_heads=1,
                      head_dim=16, ffn_size=48)
    return LlamaModel(cfg, dtype=dtype, device="cpu", seed=seed, max_positions=32)


def _train(opt, steps, seed):
    g = torch.Generator().manual_seed(seed)
    for _ in range(steps):
        opt.grad.copy_(torch.randn(opt.grad.shape, generator=g).to(opt.grad.dtype))
        opt.step()


def test_save_mutate_load_restores_everything(tmp_path):
    model = tiny()
    opt = FlatAdamW(model, lr=1e-3)
    sampler = SamplerBackend(seed=17)
    sampler._offset = 5
    _train(opt, 3, seed=1)
    want = {"flat": model.flat.clone(), "m": opt.m.clone(), "v": opt.v.clone(), "master": opt.master.clone()}
    update_id = save_checkpoint(str(tmp_path), model, opt, weight_version=7, sampler=sampler, extra={"note": "x"})
    assert update_id and os.path.exists(tmp_path / "optimizer.pt") and os.path.exists(tmp_path / "state.json")

    _train(opt, 2, seed=2)                       # mutate everything
    sampler.manual_seed(99)
    assert not torch.equal(model.flat, want["flat"]) and opt.steps == 5

    state = load_checkpoint(str(tmp_path), model, opt, sampler=sampler)
    assert state["weight_version"] == 7 and state["extra"] == {"note": "x"} and state["world"] == 1
    assert torch.equal(model.flat, want["flat"]) and torch.equal(opt.m, want["m"]) and torch.equal(opt.v, want["v"])
    assert torch.equal(opt.master, want["master"]) and opt.steps == 3
    assert (sampler.seed, sampler._offset) == (17, 5)
    # the resumed run continues exactly like the uninterrupted one
    twin = tiny()
    twin_opt = FlatAdamW(twin, lr=1e-3)
    _train(twin_opt, 3, seed=1)
    _train(twin_opt, 1, seed=5)
    _train(opt, 1, seed=5)
    assert torch.equal(model.flat, twin.flat) and torch.equal(opt.master, twin_opt.master)


def test_checkpoint_into_a_fresh_process_state(tmp_path):
    model = tiny(seed=3)
    opt = FlatAdamW(model, lr=1e-3)
    _train(opt, 2, seed=4)
    save_checkpoint(str(tmp_path), model, opt, weight_version=1)
    other = tiny(seed=8)                          # different initial weights, fresh optimizer
    other_opt = FlatAdamW(other, lr=1e-3)
    load_checkpoint(str(tmp_path), other, other_opt)
    assert torch.equal(other.flat, model.flat) and torch.equal(other_opt.master, opt.master) and other_opt.steps == 2


def test_optimizer_file_is_loaded_without_unpickling_code(tmp_path):
    model = tiny()
    opt = FlatAdamW(model, lr=1e-3)
    save_checkpoint(str(tmp_path), model, opt, weight_version=1)

    class Evil:
        def __reduce__(self):
            return (os.system, ("true",))

    torch.save({"m": opt.m, "v": opt.v, "master": None, "steps": 1, "evil": Evil()}, tmp_path / "optimizer.pt")
    with pytest.raises(Exception):
        load_checkpoint(str(tmp_path), model, opt)


def test_missing_optimizer_shard_is_an_error_and_weights_load_at_any_world_size(tmp_path):
    model = tiny()
    opt = FlatAdamW(model, lr=1e-3)
    save_checkpoint(str(tmp_path), model, None, weight_version=1)
    with pytest.raises(FileNotFoundError):
        load_checkpoint(str(tmp_path), model, opt)
    # the weights are replicated: loading them alone works for any number of ranks
    assert load_checkpoint(str(tmp_path), model, None, world=2)["world"] == 1


def _sharded(model, rank, world):
    from rl_engine.parallel.data_parallel import ShardedFusedAdamW

    n = model.flat.numel()
    padded = (n + 7) // 8 * 8
    flat = torch.zeros(padded, dtype=model.flat.dtype)
    flat[:n].copy_(model.flat)
    holder = types.SimpleNamespace(local=flat, ptrs=[0] * world)
    mem = types.SimpleNamespace(rank=rank, world=world)
    return ShardedFusedAdamW(model, mem, holder, types.SimpleNamespace(local=torch.zeros_like(flat), ptrs=[0] * world),
                             lr=1e-3, overlap=False, layers_per_bucket=1)


def test_sharded_optimizer_state_round_trip_per_rank(tmp_path):
    model = tiny()
    world = 3                                      # does not divide the bucket sizes evenly
    shards = [_sharded(model, r, world) for r in range(world)]
    n_pad = shards[0].params.local.numel()
    covered = torch.zeros(n_pad, dtype=torch.int32)
    for sh in shards:
        for lo, hi, _ in sh.slices:
            assert lo % 8 == 0 and hi % 8 == 0 and hi >= lo
            covered[lo:hi] += 1
    assert bool((covered == 1).all())              # the ranks' slices tile the padded flat vector exactly once
    for r, sh in enumerate(shards):
        sh.m.uniform_(-1, 1)
        sh.v.uniform_(0, 1)
        sh.steps = 4
        save_checkpoint(str(tmp_path), model, sh, weight_version=2, rank=r, world=world)
    assert os.path.exists(tmp_path / "optimizer.rank2of3.pt") and not os.path.exists(tmp_path / "optimizer.pt")
    fresh = _sharded(model, 1, world)
    load_checkpoint(str(tmp_path), model, fresh, rank=1, world=world)
    assert torch.equal(fresh.m, shards[1].m) and torch.equal(fresh.v, shards[1].v) and fresh.steps == 4
    assert torch.equal(fresh.master, shards[1].master)
    # another rank's shard is refused
    wrong = torch.load(tmp_path / "optimizer.rank0of3.pt", weights_only=True)
    with pytest.raises(ValueError):
        fresh.load_state_dict(wrong)
    # a shard without master weights re-seeds them from the (restored) parameters
    state = torch.load(tmp_path / "optimizer.rank1of3.pt", weights_only=True)
    state["master"] = None
    fresh.params.local.fill_(0.5)
    fresh.load_state_dict(state)
    assert torch.equal(fresh.master, torch.full_like(fresh.master, 0.5))


def test_resume_with_another_world_size_recuts_the_optimizer_state(tmp_path):
    """Saved by 3 ranks, resumed by 2 ranks, by 1 (``FlatAdamW``), and back from 1 to 3: every element of the moments
    and the master weights lands at the same flat index."""
    from rl_engine.executors.checkpoint import OptimizerShardReader

    model = tiny()
    n = model.flat.numel()
    three = [_sharded(model, r, 3) for r in range(3)]
    n_pad = three[0].params.local.numel()
    truth = {k: torch.zeros(n_pad) for k in ("m", "v", "master")}
    gen = torch.Generator().manual_seed(5)
    for r, sh in enumerate(three):
        sh.m.copy_(torch.rand(sh.m.shape, generator=gen) - 0.5)
        sh.v.copy_(torch.rand(sh.v.shape, generator=gen))
        sh.master.add_(torch.rand(sh.master.shape, generator=gen) * 1e-3)
        sh.steps = 6
        for lo, hi, off in sh.slices:
            for k in truth:
                truth[k][lo:hi] = getattr(sh, k)[off : off + hi - lo]
        save_checkpoint(str(tmp_path / "w3"), model, sh, weight_version=3, rank=r, world=3)
    reader = OptimizerShardReader.from_directory(str(tmp_path / "w3"), 3)
    assert reader.steps == 6 and reader.numel == n_pad and reader.has("master") and not reader.has("master_residual")
    assert torch.equal(reader.read("m", 5, 77), truth["m"][5:77])
    # 3 -> 2
    for r in range(2):
        sh = _sharded(model, r, 2)
        state = load_checkpoint(str(tmp_path / "w3"), model, sh, rank=r, world=2)
        assert state["world"] == 3 and sh.steps == 6
        for lo, hi, off in sh.slices:
            for k in truth:
                assert torch.equal(getattr(sh, k)[off : off + hi - lo], truth[k][lo:hi]), (k, r)
    # 3 -> 1
    flat = FlatAdamW(model, lr=1e-3)
    load_checkpoint(str(tmp_path / "w3"), model, flat, world=1)
    assert torch.equal(flat.m, truth["m"][:n]) and torch.equal(flat.v, truth["v"][:n]) and flat.steps == 6
    # 1 -> 3: the flat state is one slice [0, n); padding past n keeps the parameter as its master
    flat.m.mul_(2.0)
    save_checkpoint(str(tmp_path / "w1"), model, flat, weight_version=4)
    for r in range(3):
        sh = _sharded(model, r, 3)
        load_checkpoint(str(tmp_path / "w1"), model, sh, rank=r, world=3)
        for lo, hi, off in sh.slices:
            top = min(hi, n)
            assert torch.equal(sh.m[off : off + top - lo], flat.m[lo:top])
            if flat.master is not None:
                assert torch.equal(sh.master[off : off + top - lo], flat.master[lo:top])
    # shards of different checkpoints are refused
    torch.save({"m": torch.zeros(4), "v": torch.zeros(4), "master": None, "steps": 1, "slices": [[0, 4]]}, tmp_path / "a.pt")
    with pytest.raises(ValueError, match="step count"):
        OptimizerShardReader([torch.load(tmp_path / "a.pt", weights_only=True),
                              {"m": torch.zeros(4), "v": torch.zeros(4), "steps": 2, "slices": [[4, 8]]}])
    with pytest.raises(ValueError, match="overlap"):
        OptimizerShardReader([{"m": torch.zeros(4), "v": torch.zeros(4), "steps": 1, "slices": [[0, 4]]},
                              {"m": torch.zeros(4), "v": torch.zeros(4), "steps": 1, "slices": [[2, 6]]}])
    # an optimizer that cannot take a re-cut state still gets the explicit error
    class Plain:
        def load_state_dict(self, state): raise AssertionError("must not be called")
    with pytest.raises(ValueError, match="written by 3"):
        load_checkpoint(str(tmp_path / "w3"), model, Plain(), world=2)
