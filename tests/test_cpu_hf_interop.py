"""Hugging Face checkpoints <-> the native model, on CPU in fp32: a tiny random ``LlamaForCausalLM`` (and, where this
``transformers`` has them, ``Qwen3ForCausalLM`` and ``Qwen3MoeForCausalLM``) loaded into ``LlamaModel`` gives the same
logits; the Hugging Face views of the native parameters are zero-copy and round-trip; expert shards take their experts."""

import pytest
import torch

transformers = pytest.importorskip("transformers")


def _native_from(hf_model, **kw):
    from rl_engine.models.hf_interop import config_from_hf, load_hf_state_dict
    from rl_engine.models.llama import LlamaModel

    cfg = config_from_hf(hf_model.config)
    model = LlamaModel(cfg, dtype=torch.float32, device="cpu", seed=0, activation_checkpointing=False, max_positions=64, **kw)
    unused = load_hf_state_dict(model, hf_model.state_dict())
    return cfg, model, unused


def _compare_logits(hf_model, model, vocab, atol=2e-4):
    from rl_engine.models.causal_lm import PackedCausalLM

    ids = torch.randint(0, vocab, (2, 9), generator=torch.Generator().manual_seed(4))
    with torch.no_grad():
        want = hf_model(input_ids=ids, use_cache=False).logits.float()
        got = PackedCausalLM(model)(ids).logits.float()
    assert got.shape == want.shape
    assert torch.allclose(got, want, atol=atol, rtol=1e-3), float((got - want).abs().max())


def test_llama_checkpoint_loads_and_matches_transformers():
    from rl_engine.models.hf_interop import hf_state_dict_views

    config = transformers.LlamaConfig(
        vocab_size=97, hidden_size=64, intermediate_size=112, num_hidden_layers=2, num_attention_heads=4,
        num_key_value_heads=2, max_position_embeddings=64, rms_norm_eps=1e-5, rope_theta=10000.0, tie_word_embeddings=False,
        attention_bias=False, mlp_bias=False)
    torch.manual_seed(0)
    hf = transformers.LlamaForCausalLM(config).float().eval()
    cfg, model, unused = _native_from(hf)
    assert (cfg.hidden_size, cfg.num_layers, cfg.num_heads, cfg.num_kv_heads, cfg.head_dim, cfg.ffn_size) == (64, 2, 4, 2, 16, 112)
    assert not cfg.qk_norm and not cfg.num_experts and unused == []
    _compare_logits(hf, model, 97)
    views = hf_state_dict_views(model)
    theirs = hf.state_dict()
    assert set(views) == set(theirs)
    lo, hi = model.flat.data_ptr(), model.flat.data_ptr() + model.flat.numel() * 4
    for name, want in theirs.items():
        assert torch.equal(views[name], want), name
        assert lo <= views[name].data_ptr() < hi and views[name].is_contiguous(), name     # a view, not a copy
    with pytest.raises(KeyError):
        from rl_engine.models.hf_interop import load_hf_state_dict

        load_hf_state_dict(model, {k: v for k, v in theirs.items() if "k_proj" not in k})


def test_tied_embeddings_and_unsupported_configurations():
    from rl_engine.models.hf_interop import config_from_hf, load_hf_state_dict
    from rl_engine.models.llama import LlamaModel

    config = transformers.LlamaConfig(vocab_size=50, hidden_size=32, intermediate_size=48, num_hidden_layers=1,
                                      num_attention_heads=2, num_key_value_heads=2, tie_word_embeddings=True)
    torch.manual_seed(1)
    hf = transformers.LlamaForCausalLM(config).float().eval()
    cfg = config_from_hf(hf.config)
    model = LlamaModel(cfg, dtype=torch.float32, device="cpu", activation_checkpointing=False, max_positions=32)
    state = {k: v for k, v in hf.state_dict().items() if k != "lm_head.weight"}
    load_hf_state_dict(model, state)
    assert torch.equal(model.view("lm_head"), hf.model.embed_tokens.weight)
    _compare_logits(hf, model, 50)
    with pytest.raises(ValueError):
        config_from_hf({"hidden_size": 32, "num_attention_heads": 2, "num_hidden_layers": 1, "vocab_size": 10,
                        "intermediate_size": 8, "rope_scaling": {"rope_type": "longrope", "factor": 8.0}})
    with pytest.raises(ValueError):
        config_from_hf({"hidden_size": 32, "num_attention_heads": 2, "num_hidden_layers": 1, "vocab_size": 10,
                        "intermediate_size": 8, "attention_bias": True})


def test_qwen3_dense_checkpoint_with_head_norms():
    if not hasattr(transformers, "Qwen3ForCausalLM"):
        pytest.skip("this transformers has no Qwen3")
    config = transformers.Qwen3Config(
        vocab_size=83, hidden_size=64, intermediate_size=96, num_hidden_layers=2, num_attention_heads=4,
        num_key_value_heads=2, head_dim=32, max_position_embeddings=64, rms_norm_eps=1e-6, rope_theta=10000.0,
        tie_word_embeddings=False, attention_bias=False)
    torch.manual_seed(2)
    hf = transformers.Qwen3ForCausalLM(config).float().eval()
    with torch.no_grad():  # make the head norms non-trivial
        for layer in hf.model.layers:
            layer.self_attn.q_norm.weight.uniform_(0.5, 1.5)
            layer.self_attn.k_norm.weight.uniform_(0.5, 1.5)
    cfg, model, unused = _native_from(hf)
    assert cfg.qk_norm and cfg.head_dim == 32 and cfg.q_dim == 128 and unused == []
    _compare_logits(hf, model, 83)


def test_qwen3_moe_checkpoint_and_expert_shards():
    if not hasattr(transformers, "Qwen3MoeForCausalLM"):
        pytest.skip("this transformers has no Qwen3-MoE")
    from rl_engine.models.hf_interop import hf_state_dict_views

    config = transformers.Qwen3MoeConfig(
        vocab_size=71, hidden_size=64, intermediate_size=96, moe_intermediate_size=48, num_hidden_layers=2,
        num_attention_heads=4, num_key_value_heads=2, head_dim=16, num_experts=4, num_experts_per_tok=2,
        norm_topk_prob=True, decoder_sparse_step=1, mlp_only_layers=[], max_position_embeddings=64, rms_norm_eps=1e-6,
        rope_theta=10000.0, tie_word_embeddings=False, attention_bias=False, output_router_logits=False)
    torch.manual_seed(3)
    hf = transformers.Qwen3MoeForCausalLM(config).float().eval()
    state = hf.state_dict()
    stacked = "model.layers.0.mlp.experts.gate_up_proj" in state   # newer transformers: experts stacked per layer
    cfg, model, unused = _native_from(hf)
    assert cfg.num_experts == 4 and cfg.experts_per_token == 2 and cfg.moe_ffn_size == 48 and cfg.qk_norm and unused == []
    _compare_logits(hf, model, 71, atol=5e-4)
    # an expert shard takes its own experts (2 and 3 of 4); the per-expert checkpoint names come out as views
    _cfg, shard, unused = _native_from(hf, expert_shard=(1, 2))
    if not stacked:
        assert all(".experts.0." in k or ".experts.1." in k for k in unused) and len(unused) == 2 * 2 * 3
    views = hf_state_dict_views(shard)
    assert "model.layers.0.mlp.experts.2.gate_proj.weight" in views and "model.layers.0.mlp.experts.0.gate_proj.weight" not in views
    if stacked:
        want_down = state["model.layers.1.mlp.experts.down_proj"][3]
        want_gate = state["model.layers.0.mlp.experts.gate_up_proj"][2][:48]
    else:
        want_down = state["model.layers.1.mlp.experts.3.down_proj.weight"]
        want_gate = state["model.layers.0.mlp.experts.2.gate_proj.weight"]
    assert torch.equal(views["model.layers.1.mlp.experts.3.down_proj.weight"], want_down)
    assert torch.equal(views["model.layers.0.mlp.experts.2.gate_proj.weight"], want_gate)
    # a checkpoint with one tensor per expert (the on-disk format) loads to the same parameters
    per_expert = {k: v for k, v in state.items() if ".mlp.experts." not in k}
    full_views = hf_state_dict_views(model)
    per_expert.update({k: v.clone() for k, v in full_views.items() if ".mlp.experts." in k})
    from rl_engine.models.hf_interop import config_from_hf, load_hf_state_dict
    from rl_engine.models.llama import LlamaModel

    again = LlamaModel(config_from_hf(hf.config), dtype=torch.float32, device="cpu", seed=9, activation_checkpointing=False,
                       max_positions=64)
    assert load_hf_state_dict(again, per_expert) == []
    assert torch.equal(again.flat, model.flat)


def test_model_from_hf_and_publishing_checkpoint_names_through_a_bridge():
    """``model_from_hf`` builds and loads in one call; a weight bridge that is handed the Hugging Face views ships the
    checkpoint-format names an inference engine expects, and the consumer's tensors equal the Hugging Face weights."""
    from rl_engine.executors.bridge import LocalTensorCopyBridge
    from rl_engine.models.hf_interop import hf_state_dict_views, model_from_hf

    config = transformers.LlamaConfig(vocab_size=61, hidden_size=32, intermediate_size=48, num_hidden_layers=2,
                                      num_attention_heads=4, num_key_value_heads=2, max_position_embeddings=48,
                                      tie_word_embeddings=False)
    torch.manual_seed(3)
    hf = transformers.LlamaForCausalLM(config).float().eval()
    model = model_from_hf(hf, dtype=torch.float32, device="cpu", activation_checkpointing=False)
    assert model.cfg.num_layers == 2
    _compare_logits(hf, model, 61)
    bridge = LocalTensorCopyBridge()
    manifest = bridge.publish(hf_state_dict_views(model), weight_version=1)
    assert set(manifest.tensors) == set(hf.state_dict())
    got = bridge.import_update(manifest)
    for name, want in hf.state_dict().items():
        assert torch.equal(got[name], want), name
    bridge.acknowledge(manifest.update_id)


def test_checkpoint_directory_round_trip_with_transformers(tmp_path):
    """``save_hf_checkpoint`` writes a directory that ``transformers`` loads (same logits), sharded files carry an index,
    and ``model_from_hf_checkpoint`` streams it back bit for bit; a tied checkpoint omits and restores the head."""
    import json
    import os

    from rl_engine.models.config import ModelConfig
    from rl_engine.models.hf_interop import (
        checkpoint_files, load_hf_checkpoint, model_from_hf_checkpoint, save_hf_checkpoint,
    )
    from rl_engine.models.llama import LlamaModel

    cfg = ModelConfig("t", 71, 64, 2, 4, 2, 16, 112, rms_eps=1e-5, rope_theta=10000.0)
    model = LlamaModel(cfg, dtype=torch.float32, device="cpu", seed=5, activation_checkpointing=False, max_positions=64)
    one = tmp_path / "one"
    assert save_hf_checkpoint(model, one) == ["model.safetensors", "config.json"]
    hf = transformers.AutoModelForCausalLM.from_pretrained(one, dtype=torch.float32).eval()
    assert type(hf).__name__ == "LlamaForCausalLM" and hf.config.max_position_embeddings == 64
    _compare_logits(hf, model, 71)
    # sharded: several files and an index; streams back into a fresh model exactly
    many = tmp_path / "many"
    files = save_hf_checkpoint(model, many, max_shard_bytes=40_000)
    assert "model.safetensors.index.json" in files and len(checkpoint_files(many)) >= 3
    index = json.load(open(many / "model.safetensors.index.json"))
    assert index["metadata"]["total_size"] == cfg.param_count() * 4
    again = model_from_hf_checkpoint(many, dtype=torch.float32, device="cpu", seed=11, activation_checkpointing=False)
    assert torch.equal(again.flat, model.flat) and again.rope_cos.shape[0] == 64
    # tied: no head in the file, restored from the embedding on load
    with torch.no_grad():
        model.view("lm_head").copy_(model.view("embed"))
    tied = tmp_path / "tied"
    save_hf_checkpoint(model, tied, tie_word_embeddings=True)
    from safetensors import safe_open

    with safe_open(os.path.join(tied, "model.safetensors"), framework="pt") as f:
        assert "lm_head.weight" not in f.keys()
    fresh = LlamaModel(cfg, dtype=torch.float32, device="cpu", seed=3, activation_checkpointing=False, max_positions=64)
    assert load_hf_checkpoint(fresh, tied) == [] and torch.equal(fresh.flat, model.flat)
    # a checkpoint that lacks a tensor is an error, not a silently random parameter
    from safetensors.torch import load_file, save_file

    broken = tmp_path / "broken"
    os.makedirs(broken)
    state = load_file(os.path.join(one, "model.safetensors"))
    state.pop("model.layers.1.mlp.down_proj.weight")
    save_file(state, os.path.join(broken, "model.safetensors"))
    with pytest.raises(KeyError, match="down_proj"):
        load_hf_checkpoint(fresh, broken)


def test_qwen3_moe_checkpoint_directory(tmp_path):
    if not hasattr(transformers, "Qwen3MoeForCausalLM"):
        pytest.skip("this transformers has no Qwen3-MoE")
    from rl_engine.models.config import ModelConfig
    from rl_engine.models.hf_interop import hf_config_dict, model_from_hf_checkpoint, save_hf_checkpoint
    from rl_engine.models.llama import LlamaModel

    cfg = ModelConfig("m", 67, 64, 2, 4, 2, 32, 96, rms_eps=1e-6, rope_theta=10000.0, num_experts=4, experts_per_token=2,
                      moe_ffn_size=48, qk_norm=True)
    assert hf_config_dict(cfg)["model_type"] == "qwen3_moe"
    model = LlamaModel(cfg, dtype=torch.float32, device="cpu", seed=6, activation_checkpointing=False, max_positions=64)
    save_hf_checkpoint(model, tmp_path)                       # one tensor per expert: the on-disk convention
    hf = transformers.AutoModelForCausalLM.from_pretrained(tmp_path, dtype=torch.float32).eval()
    assert type(hf).__name__ == "Qwen3MoeForCausalLM"
    _compare_logits(hf, model, 67, atol=5e-4)
    shard = model_from_hf_checkpoint(tmp_path, dtype=torch.float32, device="cpu", expert_shard=(1, 2),
                                     activation_checkpointing=False)
    full_gate_up = model.view("l1.w_gate_up")
    assert torch.equal(shard.view("l1.w_gate_up"), full_gate_up[full_gate_up.shape[0] // 2 :])
    assert torch.equal(shard.view("l0.router"), model.view("l0.router"))


@pytest.mark.parametrize("scaling", [
    {"rope_type": "llama3", "factor": 4.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0, "original_max_position_embeddings": 16},
    {"rope_type": "linear", "factor": 2.0},
    {"rope_type": "yarn", "factor": 4.0, "original_max_position_embeddings": 16, "beta_fast": 4.0, "beta_slow": 1.0},
])
def test_rope_scaling_matches_transformers(scaling, tmp_path):
    """Llama-3.1-style and linear context extension: with 16 original positions and head_dim 16 the eight rotary
    frequencies fall into all three bands of the llama3 rule (kept, blended, divided), and 40 positions reach past the
    original range; logits must agree with ``transformers``, and the configuration must survive a save / load."""
    from rl_engine.models.hf_interop import config_from_hf, hf_config_dict, model_from_hf, save_hf_checkpoint

    config = transformers.LlamaConfig(vocab_size=59, hidden_size=32, intermediate_size=48, num_hidden_layers=2,
                                      num_attention_heads=2, num_key_value_heads=1, max_position_embeddings=64,
                                      rope_theta=10000.0, rope_scaling=dict(scaling), tie_word_embeddings=False)
    torch.manual_seed(8)
    hf = transformers.LlamaForCausalLM(config).float().eval()
    model = model_from_hf(hf, dtype=torch.float32, device="cpu", activation_checkpointing=False)
    assert model.cfg.rope_scaling is not None and model.cfg.rope_scaling[0] == scaling["rope_type"]
    from rl_engine.models.causal_lm import PackedCausalLM

    ids = torch.randint(0, 59, (2, 40), generator=torch.Generator().manual_seed(9))
    with torch.no_grad():
        want = hf(input_ids=ids, use_cache=False).logits.float()
        got = PackedCausalLM(model)(ids).logits.float()
    assert torch.allclose(got, want, atol=2e-4, rtol=1e-3), float((got - want).abs().max())
    # the scaling changes the result (the test would pass vacuously otherwise) ...
    from dataclasses import replace
    from rl_engine.models.llama import LlamaModel

    plain = LlamaModel(replace(model.cfg, rope_scaling=None), dtype=torch.float32, device="cpu", activation_checkpointing=False,
                       max_positions=64)
    plain.flat.data.copy_(model.flat.data)
    with torch.no_grad():
        assert float((PackedCausalLM(plain)(ids).logits.float() - want).abs().max()) > 1e-4
    # ... and survives config.json
    assert config_from_hf(hf_config_dict(model.cfg)).rope_scaling == model.cfg.rope_scaling
    save_hf_checkpoint(model, tmp_path)
    again = transformers.AutoModelForCausalLM.from_pretrained(tmp_path, dtype=torch.float32).eval()
    with torch.no_grad():
        assert torch.allclose(again(input_ids=ids, use_cache=False).logits.float(), want, atol=1e-5)


def test_presets_describe_the_published_architectures():
    from rl_engine.models import llama3_70b, llama3_8b, llama31_8b, qwen3_8b, qwen3_30b_a3b, qwen3_32b

    billions = lambda cfg: cfg.param_count() / 1e9  # noqa: E731
    assert 7.9 < billions(llama3_8b()) < 8.1 and 69 < billions(llama3_70b()) < 72
    assert 8.0 < billions(qwen3_8b()) < 8.4 and 32 < billions(qwen3_32b()) < 33.5 and 30 < billions(qwen3_30b_a3b()) < 31
    assert llama31_8b().rope_scaling == ("llama3", 8.0, 1.0, 4.0, 8192) and llama31_8b().param_count() == llama3_8b().param_count()


def test_tied_embeddings_stay_tied_through_training_and_round_trip(tmp_path):
    """A tied Hugging Face model (small Llama-3.2 / Qwen3 style) keeps ``embed == lm_head`` bit for bit over optimiser
    steps: both get the summed gradient.  The saved checkpoint omits the head and ``transformers`` ties it again."""
    from dataclasses import replace

    from rl_engine.models.grpo import GRPOBatch, GRPOTrainer
    from rl_engine.models.hf_interop import model_from_hf, save_hf_checkpoint
    from rl_engine.models.config import require_untied

    config = transformers.LlamaConfig(vocab_size=53, hidden_size=32, intermediate_size=48, num_hidden_layers=2,
                                      num_attention_heads=2, num_key_value_heads=1, max_position_embeddings=48,
                                      tie_word_embeddings=True)
    torch.manual_seed(10)
    hf = transformers.LlamaForCausalLM(config).float().eval()
    model = model_from_hf(hf, dtype=torch.float32, device="cpu", activation_checkpointing=False)
    assert model.cfg.tie_word_embeddings and torch.equal(model.view("embed"), model.view("lm_head"))
    trainer = GRPOTrainer(model, lr=1e-2, micro_group=2)
    gen = torch.Generator().manual_seed(11)
    start = model.view("embed").detach().clone()
    seen = {}
    real_tie = trainer.opt._tie_gradients

    def spy():
        seen["embed"] = model._slice(trainer.opt.grad, "embed").clone()
        seen["head"] = model._slice(trainer.opt.grad, "lm_head").clone()
        real_tie()
        seen["tied"] = model._slice(trainer.opt.grad, "embed").clone()

    trainer.opt._tie_gradients = spy
    for _ in range(3):
        batch = GRPOBatch(prompt_ids=torch.randint(0, 53, (6,), generator=gen),
                          completion_ids=torch.randint(0, 53, (4, 5), generator=gen),
                          completion_mask=torch.ones(4, 5, dtype=torch.bool), rewards=torch.randn(4, generator=gen),
                          old_logps=torch.full((4, 5), -4.0), ref_logps=torch.full((4, 5), -4.0))
        trainer.step_device(batch)
        assert torch.equal(model.view("embed"), model.view("lm_head"))
    assert not torch.equal(model.view("embed"), start)
    assert torch.equal(seen["tied"], seen["embed"] + seen["head"]) and float(seen["head"].abs().max()) > 0
    # untied configuration of the same model: the two matrices drift apart (so the tie above is doing the work)
    free = model_from_hf(hf, dtype=torch.float32, device="cpu", activation_checkpointing=False)
    free.cfg = replace(free.cfg, tie_word_embeddings=False)
    other = GRPOTrainer(free, lr=1e-2, micro_group=2)
    other.step_device(batch)
    assert not torch.equal(free.view("embed"), free.view("lm_head"))
    # checkpoint: head left out, transformers ties it again, logits agree
    files = save_hf_checkpoint(model, tmp_path)
    from safetensors import safe_open

    with safe_open(str(tmp_path / files[0]), framework="pt") as f:
        assert "lm_head.weight" not in f.keys()
    again = transformers.AutoModelForCausalLM.from_pretrained(tmp_path, dtype=torch.float32).eval()
    assert again.config.tie_word_embeddings
    _compare_logits(again, model, 53)
    with pytest.raises(ValueError, match="tied embeddings"):
        require_untied(model.cfg, "ShardedFusedAdamW")


def test_qwen2_checkpoint_with_biased_qkv_projections(tmp_path):
    """Qwen2 / Qwen2.5: q, k and v carry a bias.  Logits match ``transformers``, the bias trains (gradient = column sum
    of the qkv gradient), the views and a saved directory carry the three HF bias tensors."""
    if not hasattr(transformers, "Qwen2ForCausalLM"):
        pytest.skip("this transformers has no Qwen2")
    from rl_engine.models.hf_interop import hf_state_dict_views, model_from_hf, model_from_hf_checkpoint, save_hf_checkpoint
    from rl_engine.models import qwen25_7b
    from rl_engine.models.config import require_no_qkv_bias

    config = transformers.Qwen2Config(vocab_size=67, hidden_size=64, intermediate_size=96, num_hidden_layers=2,
                                      num_attention_heads=4, num_key_value_heads=2, max_position_embeddings=64,
                                      rms_norm_eps=1e-6, rope_theta=10000.0, tie_word_embeddings=False, use_sliding_window=False)
    torch.manual_seed(12)
    hf = transformers.Qwen2ForCausalLM(config).float().eval()
    with torch.no_grad():
        for layer in hf.model.layers:
            for proj in (layer.self_attn.q_proj, layer.self_attn.k_proj, layer.self_attn.v_proj):
                proj.bias.uniform_(-0.5, 0.5)
    model = model_from_hf(hf, dtype=torch.float32, device="cpu", activation_checkpointing=False)
    assert model.cfg.qkv_bias and not model.cfg.qk_norm and model.view("l1.bqkv").shape == (64 + 2 * 32,)
    _compare_logits(hf, model, 67)
    views = hf_state_dict_views(model)
    assert torch.equal(views["model.layers.1.self_attn.k_proj.bias"], hf.model.layers[1].self_attn.k_proj.bias)
    assert set(views) == set(hf.state_dict())
    # gradients reach the bias
    from rl_engine.models.causal_lm import PackedCausalLM

    ids = torch.randint(0, 67, (2, 7), generator=torch.Generator().manual_seed(13))
    model.ensure_flat_grad().zero_()
    PackedCausalLM(model)(ids).logits.float().square().mean().backward()
    hf.zero_grad()
    hf(input_ids=ids, use_cache=False).logits.float().square().mean().backward()
    want = torch.cat([hf.model.layers[0].self_attn.q_proj.bias.grad, hf.model.layers[0].self_attn.k_proj.bias.grad,
                      hf.model.layers[0].self_attn.v_proj.bias.grad])
    assert torch.allclose(model.view("l0.bqkv").grad, want, atol=1e-6) and float(want.abs().max()) > 0
    # directory round trip, written as Qwen2
    save_hf_checkpoint(model, tmp_path)
    again = transformers.AutoModelForCausalLM.from_pretrained(tmp_path, dtype=torch.float32).eval()
    assert type(again).__name__ == "Qwen2ForCausalLM"
    _compare_logits(again, model, 67)
    back = model_from_hf_checkpoint(tmp_path, dtype=torch.float32, device="cpu", activation_checkpointing=False)
    assert torch.equal(back.flat, model.flat)
    assert 7.5 < qwen25_7b().param_count() / 1e9 < 7.8
    with pytest.raises(ValueError, match="biased q/k/v"):
        require_no_qkv_bias(model.cfg, "TensorParallelLlama")


def test_mistral_checkpoint_is_the_llama_architecture():
    if not hasattr(transformers, "MistralForCausalLM"):
        pytest.skip("this transformers has no Mistral")
    from rl_engine.models.hf_interop import config_from_hf

    config = transformers.MistralConfig(vocab_size=61, hidden_size=64, intermediate_size=96, num_hidden_layers=2,
                                        num_attention_heads=4, num_key_value_heads=2, max_position_embeddings=64,
                                        rms_norm_eps=1e-5, rope_theta=10000.0, sliding_window=None, tie_word_embeddings=False)
    torch.manual_seed(14)
    hf = transformers.MistralForCausalLM(config).float().eval()
    cfg, model, unused = _native_from(hf)
    assert not cfg.qkv_bias and not cfg.qk_norm and unused == []
    _compare_logits(hf, model, 61)
    windowed = transformers.MistralConfig(vocab_size=61, hidden_size=64, intermediate_size=96, num_hidden_layers=1,
                                          num_attention_heads=4, num_key_value_heads=2, max_position_embeddings=64, sliding_window=16)
    with pytest.raises(ValueError, match="sliding-window"):
        config_from_hf(windowed)
    with pytest.raises(ValueError, match="model_type 'gpt2'"):
        config_from_hf(transformers.GPT2Config(vocab_size=10, n_embd=8, n_layer=1, n_head=1))


def test_padded_batches_match_transformers_for_right_and_left_padding():
    """``PackedCausalLM`` drops padding from the pack: logits at the real tokens of right- and left-padded rows equal
    what ``transformers`` computes with the same attention mask; padded slots come back as zeros; a mask with a hole is
    refused."""
    from rl_engine.models.causal_lm import PackedCausalLM
    from rl_engine.models.hf_interop import model_from_hf

    config = transformers.LlamaConfig(vocab_size=47, hidden_size=32, intermediate_size=48, num_hidden_layers=2,
                                      num_attention_heads=2, num_key_value_heads=1, max_position_embeddings=32,
                                      tie_word_embeddings=False)
    torch.manual_seed(15)
    hf = transformers.LlamaForCausalLM(config).float().eval()
    lm = PackedCausalLM(model_from_hf(hf, dtype=torch.float32, device="cpu", activation_checkpointing=False))
    ids = torch.randint(0, 47, (3, 8), generator=torch.Generator().manual_seed(16))
    right = torch.tensor([[1] * 8, [1] * 5 + [0] * 3, [1] * 2 + [0] * 6])
    left = torch.tensor([[1] * 8, [0] * 3 + [1] * 5, [0] * 6 + [1] * 2])
    for mask in (right, left):
        with torch.no_grad():
            want = hf(input_ids=ids, attention_mask=mask, use_cache=False).logits.float()
            got = lm(ids, attention_mask=mask).logits.float()
        keep = mask.bool()
        assert torch.allclose(got[keep], want[keep], atol=2e-4, rtol=1e-3), float((got[keep] - want[keep]).abs().max())
        assert float(got[~keep].abs().max()) == 0.0
    with pytest.raises(ValueError, match="contiguous run"):
        lm(ids, attention_mask=torch.tensor([[1, 1, 0, 1, 1, 1, 1, 1]] * 3))


def test_mixtral_checkpoint_names_and_logits(tmp_path):
    """Mixtral: experts without q/k norms, ``block_sparse_moe`` / ``w1`` ``w3`` ``w2`` names on disk (newer
    ``transformers`` hold them stacked under ``mlp`` in memory); both spellings load, logits match, a saved directory
    loads back into ``transformers`` as ``MixtralForCausalLM``."""
    if not hasattr(transformers, "MixtralForCausalLM"):
        pytest.skip("this transformers has no Mixtral")
    from rl_engine.models.hf_interop import hf_state_dict_views, model_from_hf_checkpoint, save_hf_checkpoint

    config = transformers.MixtralConfig(vocab_size=67, hidden_size=64, intermediate_size=48, num_hidden_layers=2,
                                        num_attention_heads=4, num_key_value_heads=2, num_local_experts=4, num_experts_per_tok=2,
                                        max_position_embeddings=64, sliding_window=None, rms_norm_eps=1e-5, rope_theta=10000.0,
                                        tie_word_embeddings=False)
    torch.manual_seed(17)
    hf = transformers.MixtralForCausalLM(config).float().eval()
    cfg, model, unused = _native_from(hf)
    assert cfg.num_experts == 4 and cfg.experts_per_token == 2 and cfg.moe_ffn_size == 48 and not cfg.qk_norm and unused == []
    _compare_logits(hf, model, 67, atol=5e-4)
    views = hf_state_dict_views(model)
    assert "model.layers.1.block_sparse_moe.experts.3.w2.weight" in views and "model.layers.0.block_sparse_moe.gate.weight" in views
    assert views["model.layers.0.block_sparse_moe.experts.0.w3.weight"].shape == (48, 64)
    save_hf_checkpoint(model, tmp_path)
    again = transformers.AutoModelForCausalLM.from_pretrained(tmp_path, dtype=torch.float32).eval()
    assert type(again).__name__ == "MixtralForCausalLM"
    _compare_logits(again, model, 67, atol=5e-4)
    back = model_from_hf_checkpoint(tmp_path, dtype=torch.float32, device="cpu", activation_checkpointing=False)
    assert torch.equal(back.flat, model.flat)
