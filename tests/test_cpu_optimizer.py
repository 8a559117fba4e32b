"""CPU tests of the optimiser plumbing: fp32-master defaults, the split (bf16 + 16-bit residual) master form, bucket
cuts of the flat parameter vector and the layer notifications that drive the overlapped gradient exchange."""

import torch

from rl_engine.models.config import ModelConfig
from rl_engine.models.grpo import FlatAdamW, GRPOTrainer, join_master, split_master, synthetic_batch
from rl_engine.models.llama import LlamaModel


def tiny(layers=3, dtype=torch.float32):
    cfg = ModelConfig(name="tiny", vocab_size=512, hidden_size=64, num_layers=layers, num_heads=2, num_kv_heads=1,
                      head_dim=32, ffn_size=96)
    return LlamaModel(cfg, dtype=dtype, device="cpu", seed=0, max_positions=64)


def test_split_master_round_trips_every_bit():
    g = torch.Generator().manual_seed(0)
    w = torch.randn(1 << 16, generator=g) * torch.logspace(-8, 4, 1 << 16)
    w[:6] = torch.tensor([0.0, -0.0, 1.0, -1.0, 3.0e-39, -65504.0])
    # exact ties (low half = 0x8000) in both signs
    ties = (torch.randint(0, 1 << 15, (64,), generator=g).to(torch.int32) << 16) + 0x8000
    w[6:70] = ties.view(torch.float32)
    w[70:134] = -ties.view(torch.float32)
    param, residual = split_master(w)
    assert param.dtype == torch.bfloat16 and residual.dtype == torch.int16
    assert torch.equal(join_master(param, residual).view(torch.int32), w.view(torch.int32))
    # the bf16 part is the nearest bf16 value (ties go away from zero)
    assert ((param.float() - w).abs() <= (w.to(torch.bfloat16).float() - w).abs() + 0).all()


def test_master_weights_are_the_default_and_small_updates_accumulate():
    model = tiny(dtype=torch.bfloat16)
    opt = FlatAdamW(model, lr=1e-6)
    assert opt.has_master and opt.master is not None and opt.master.dtype == torch.float32
    before_master, before_param = opt.master.clone(), model.flat.clone()
    opt.grad.copy_(torch.randn(opt.grad.shape, generator=torch.Generator().manual_seed(1)).to(opt.grad.dtype))
    opt.step()
    # one step at lr = 1e-6 is far below bf16 resolution: the master moves, the bf16 weights (mostly) do not
    assert (opt.master != before_master).float().mean() > 0.9
    assert (model.flat != before_param).float().mean() < 0.05
    for _ in range(400):
        opt.step()
    assert (model.flat != before_param).float().mean() > 0.2  # ... but the updates are not lost
    assert torch.equal(model.flat, opt.master.to(torch.bfloat16))
    # without a master the same 401 steps leave most weights where they were
    plain = tiny(dtype=torch.bfloat16)
    popt = FlatAdamW(plain, lr=1e-6, master_weights=False)
    popt.grad.copy_(opt.grad)
    start = plain.flat.clone()
    for _ in range(401):
        popt.step()
    assert (plain.flat != start).float().mean() < (model.flat != before_param).float().mean()


def test_trainers_default_to_master_weights():
    import inspect

    from rl_engine.parallel import data_parallel

    assert inspect.signature(GRPOTrainer.__init__).parameters["master_weights"].default is True
    assert inspect.signature(FlatAdamW.__init__).parameters["master_weights"].default is True
    assert inspect.signature(data_parallel.ShardedGRPOTrainer.__init__).parameters["master_weights"].default is True
    assert inspect.signature(data_parallel.ShardedFusedAdamW.__init__).parameters["master_weights"].default is True


def test_optimizer_state_round_trip_reseeds_missing_master():
    model = tiny(dtype=torch.bfloat16)
    opt = FlatAdamW(model, lr=1e-3)
    opt.grad.fill_(0.5)
    opt.step()
    state = {k: (v.clone() if torch.is_tensor(v) else v) for k, v in opt.state_dict().items()}
    weights = model.flat.clone()
    opt.step()
    model.flat.copy_(weights)
    opt.load_state_dict(state)
    assert opt.steps == 1 and torch.equal(opt.master, state["master"]) and torch.equal(opt.m, state["m"])
    # a checkpoint without master weights must not leave the old master in place
    model.flat.fill_(0.25)
    opt.load_state_dict({**state, "master": None, "master_residual": None})
    assert torch.equal(opt.master, torch.full_like(opt.master, 0.25))


def test_layer_buckets_tile_the_flat_vector():
    from rl_engine.parallel.data_parallel import layer_buckets

    model = tiny(layers=6)
    ranges, ready_at = layer_buckets(model, layers_per_bucket=2)
    assert ranges[0][0] == 0 and ranges[-1][1] == model.flat.numel()
    assert all(a[1] == b[0] for a, b in zip(ranges, ranges[1:]))
    assert len(ranges) == 4  # [embed + l0-1] [l2-3] [l4-5] [final norm + head]
    assert ready_at == {1: 2, 2: 4, 3: 6}
    off = model._offsets
    assert ranges[1] == (off["l2.attn_norm"], off["l4.attn_norm"]) and ranges[3][0] == off["final_norm"]
    # fewer layers than a bucket: embedding + all layers, then the head
    ranges, ready_at = layer_buckets(tiny(layers=1), layers_per_bucket=4)
    assert len(ranges) == 2 and ready_at == {1: 1}


def test_layer_grad_hook_reports_layers_from_last_to_first():
    model = tiny(layers=3)
    trainer = GRPOTrainer(model, lr=1e-3, micro_group=None)
    seen = []

    class Recording(GRPOTrainer):
        pass

    import contextlib

    @contextlib.contextmanager
    def final_pass():
        model.layer_grad_hook = seen.append
        try:
            yield
        finally:
            model.layer_grad_hook = None

    trainer.final_pass = final_pass
    batch = synthetic_batch(512, 8, 4, 6, seed=3)
    trainer.step_device(batch)
    assert seen == [3, 2, 1, 0]
    assert model.layer_grad_hook is None


def test_moe_parameter_ranges_split_replicated_and_expert_parameters():
    from rl_engine.parallel.expert_parallel import moe_parameter_ranges

    cfg = ModelConfig(name="tiny-moe", vocab_size=256, hidden_size=32, num_layers=3, num_heads=2, num_kv_heads=1,
                      head_dim=16, ffn_size=48, num_experts=8, experts_per_token=2, moe_ffn_size=16, qk_norm=True)
    full = LlamaModel(cfg, dtype=torch.float32, device="cpu", seed=0, max_positions=32)
    shard = LlamaModel(cfg, dtype=torch.float32, device="cpu", seed=0, max_positions=32, expert_shard=(1, 4))
    assert shard.view("l0.w_gate_up").shape[0] == full.view("l0.w_gate_up").shape[0] // 4
    assert shard.view("l0.router").shape == full.view("l0.router").shape          # the router scores all experts
    dense, ready_at, experts = moe_parameter_ranges(shard)
    pieces = sorted(dense + experts)
    assert pieces[0][0] == 0 and pieces[-1][1] == shard.flat.numel()
    assert all(a[1] == b[0] for a, b in zip(pieces, pieces[1:]))                  # together they tile the flat vector
    off = shard._offsets
    assert experts[1] == (off["l1.w_gate_up"], off["l2.attn_norm"]) and dense[1] == (off["l1.attn_norm"], off["l1.w_gate_up"])
    assert dense[-1][0] == off["final_norm"] and ready_at == {1: 1, 2: 2, 3: 3}
    import pytest

    with pytest.raises(ValueError):
        LlamaModel(cfg, dtype=torch.float32, device="cpu", expert_shard=(0, 3))
    with pytest.raises(RuntimeError, match="moe_op"):
        shard._ffn(torch.zeros(4, 32), 0, False)
