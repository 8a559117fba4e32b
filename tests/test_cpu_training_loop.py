"""The RL loop on the real stack, CPU-sized: native rollout -> stateless reference scoring -> GRPO training worker
(``GRPOTrainer`` on a ``LlamaModel``) -> publish -> ``RolloutExecutor.update_weights`` -> the next rollout runs on the
new version.  Plus the hidden-state extraction rules of the training workers and the DeepSpeed worker's ZeRO-3
publication against a fake DeepSpeed module."""

import types

import pytest
import torch

from rl_engine.executors.bridge import make_weight_bridge
from rl_engine.executors.hidden_states import extract_hidden_states
from rl_engine.executors.rollout import RolloutExecutor
from rl_engine.executors.stateless_executor import StatelessForwardConfig, StatelessForwardExecutor, StatelessForwardInputs
from rl_engine.executors.trainer import GRPOTrainingConfig, GRPOTrainingWorker, NativeTrainingConfig, NativeTrainingWorker
from rl_engine.executors.training_contract import make_rollout_result
from rl_engine.models.causal_lm import PackedCausalLM
from rl_engine.models.config import ModelConfig
from rl_engine.models.llama import LlamaModel


def tiny(seed):
    cfg = ModelConfig(name="tiny", vocab_size=128, hidden_size=32, num_layers=2, num_heads=2, num_kv_heads=1,
                      head_dim=16, ffn_size=48)
    return LlamaModel(cfg, dtype=torch.float32, device="cpu", seed=seed, max_positions=64)


# ----------------------------------------------------------------------------------- the loop
def test_rollout_score_train_publish_update_loop():
    policy, rollout_copy, reference = tiny(1), tiny(2), tiny(1)
    bridge = make_weight_bridge("local-clone", source_worker="trainer")
    worker = GRPOTrainingWorker(GRPOTrainingConfig(lr=5e-3, device="cpu", dtype=torch.float32, vocab_size=128),
                                model=policy, weight_bridge=bridge)
    executor = RolloutExecutor({"num_generations": 4}, weight_bridge=bridge, policy_model=rollout_copy)
    scorer = StatelessForwardExecutor(PackedCausalLM(reference),
                                      StatelessForwardConfig(mode="reference", attention_backend="model_default"))
    # version 0: the rollout side starts from the trainer's weights
    executor.update_weights(worker.publish_weights(0))
    assert executor.active_weight_version == 0 and torch.equal(rollout_copy.flat, policy.flat)

    prompt = torch.arange(5, 13)
    versions, losses = [], []
    for iteration in range(2):
        out = executor.execute_rollout(prompt, num_generations=4, max_new_tokens=6, temperature=1.0, top_k=20, top_p=0.95)
        assert out["status"] == "success" and out["weight_version"] == iteration
        comp = out["completion_ids"]
        assert comp.shape == (4, 6) and out["rollout_logps"].shape == (4, 6)
        # stateless scoring of the frozen reference policy over [prompt | completion] rows
        ids = torch.cat([prompt.expand(4, -1), comp], dim=1)
        comp_mask = torch.zeros_like(ids, dtype=torch.bool)
        comp_mask[:, prompt.numel():] = True
        scored = scorer.score(StatelessForwardInputs(ids, torch.ones_like(ids, dtype=torch.bool), comp_mask))
        assert scored.metrics["zero_kv_cache"] is True
        ref_logps = scored.reference_logps[:, prompt.numel():]
        payload = {"prompt_ids": prompt, "completion_ids": comp, "rollout_logps": out["rollout_logps"],
                   "reference_logps": ref_logps, "rewards": comp.float().mean(1) / 128.0}
        before = policy.flat.clone()
        result = worker.train(make_rollout_result(iteration=iteration, weight_version=out["weight_version"], payload=payload))
        m = result.metrics
        assert m["training_backend"] == "GRPOTrainer" and m["training_data_source"] == "rollout_payload"
        assert m["reward_source"] == "payload_rewards" and m["reference_logp_source"] == "payload_reference_logps"
        assert m["active_tokens"] == 24 and m["master_weights"] in (True, False)
        assert not torch.equal(policy.flat, before)                      # the real model was stepped
        assert result.consumed_weight_version == iteration and result.published_weight_version == iteration + 1
        manifest = worker.publish_weights(result.published_weight_version)
        assert set(manifest.tensors) == set(policy.named_views())
        executor.update_weights(manifest)
        assert executor.active_weight_version == iteration + 1
        assert torch.equal(rollout_copy.flat, policy.flat)               # ... and the rollout side now serves it
        versions.append(executor.active_weight_version)
        losses.append(m["loss"])
    assert versions == [1, 2] and all(torch.isfinite(torch.tensor(losses)))
    # the first iteration's reference scores came from a model equal to the policy: rollout == reference log-probs
    # (checked on the stored first payload through a fresh rollout at fixed weights)
    frozen = RolloutExecutor({"num_generations": 2}, weight_bridge=bridge, policy_model=tiny(1))
    out = frozen.execute_rollout(prompt, num_generations=2, max_new_tokens=4)
    ids = torch.cat([prompt.expand(2, -1), out["completion_ids"]], dim=1)
    mask = torch.zeros_like(ids, dtype=torch.bool)
    mask[:, prompt.numel():] = True
    again = scorer.score(StatelessForwardInputs(ids, torch.ones_like(ids, dtype=torch.bool), mask))
    assert torch.allclose(again.reference_logps[:, prompt.numel():], out["rollout_logps"], atol=1e-4)


def test_grpo_worker_accepts_reference_payload_parser_and_synthetic_fallback():
    worker = GRPOTrainingWorker(
        GRPOTrainingConfig(lr=1e-3, device="cpu", dtype=torch.float32, vocab_size=128, num_prompts=2, samples_per_prompt=3,
                           prompt_len=4, completion_len=5), model=tiny(3))
    start = worker.model.flat.clone()
    result = worker.train(make_rollout_result(iteration=0, weight_version=0, payload=None))
    assert result.metrics["training_data_source"] == "synthetic_fallback" and result.metrics["optimizer_steps"] == 1
    assert not torch.equal(worker.model.flat, start)
    vllm_style = {"outputs": [[{"token_ids": [1, 2, 3]}, {"token_ids": [4, 5]}], [{"token_ids": [7, 8, 9, 10]}, {"token_ids": [3]}]]}
    result = worker.train(make_rollout_result(iteration=1, weight_version=1, payload=vllm_style))
    assert result.metrics["training_data_source"] == "rollout_payload" and result.metrics["rollout_prompt_groups"] == 2
    with pytest.raises(TypeError):
        GRPOTrainingWorker(model=torch.nn.Linear(2, 2))


def test_grpo_worker_checkpoint_round_trip(tmp_path):
    worker = GRPOTrainingWorker(
        GRPOTrainingConfig(lr=1e-3, device="cpu", dtype=torch.float32, vocab_size=128, num_prompts=1, samples_per_prompt=4,
                           prompt_len=3, completion_len=4), model=tiny(4))
    worker.train(make_rollout_result(iteration=0, weight_version=0, payload=None))
    worker.publish_weights(1)
    worker.save_checkpoint(str(tmp_path))
    saved = worker.model.flat.clone()
    worker.train(make_rollout_result(iteration=1, weight_version=1, payload=None))
    assert not torch.equal(worker.model.flat, saved)
    state = worker.load_checkpoint(str(tmp_path))
    assert torch.equal(worker.model.flat, saved) and worker.trainer.opt.steps == 1 and state["weight_version"] == 1
    worker.publish_weights()  # versions continue after the restored one
    assert worker.health_check()["published_weight_version"] == 2


# ------------------------------------------------------------------------- hidden-state extraction
class _Out:
    def __init__(self, **kw):
        self.__dict__.update(kw)


def test_extract_hidden_states_rules():
    h = torch.randn(2, 5, 8)
    other = torch.randn(2, 5, 16)
    assert extract_hidden_states(h) is h
    assert extract_hidden_states({"last_hidden_state": h, "logits": other}, hidden_dim=8) is h
    assert extract_hidden_states(_Out(hidden=h)) is h
    layers = (torch.randn(2, 5, 8), torch.randn(2, 5, 8), h)
    assert extract_hidden_states(_Out(hidden_states=layers, logits=other), hidden_dim=8) is h      # the LAST layer
    assert extract_hidden_states({"hidden_states": list(layers)}) is h
    # tuples: (loss, states, cache-like list) -> the one qualifying tensor; hidden_dim disambiguates
    loss = torch.tensor(0.5)
    assert extract_hidden_states((loss, h, [torch.randn(3)])) is h
    assert extract_hidden_states((other, h), hidden_dim=8) is h
    # ambiguous tensors: the single deepest one wins; named fields inside a tuple win over bare tensors
    flat2d = torch.randn(10, 8)
    assert extract_hidden_states((flat2d, h)) is h
    assert extract_hidden_states((other, _Out(last_hidden_state=h))) is h
    assert extract_hidden_states(((loss, {"hidden": h}),)) is h                                    # nested containers
    with pytest.raises(TypeError, match="hidden-state"):
        extract_hidden_states((loss, torch.randn(4)))
    with pytest.raises(TypeError):
        extract_hidden_states({"logits": other}, hidden_dim=8)
    with pytest.raises(TypeError):
        extract_hidden_states((torch.randn(2, 5, 8), torch.randn(2, 5, 8)))                       # two equal candidates


def test_native_worker_trains_a_backbone_that_returns_a_model_output():
    class Backbone(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.embed = torch.nn.Embedding(64, 16)
            self.lm_head = torch.nn.Linear(16, 64, bias=False)

        def forward(self, ids):
            h = self.embed(ids)
            return _Out(logits=None, hidden_states=(h * 0, h), past_key_values=None)

    cfg = NativeTrainingConfig(device="cpu", dtype=torch.float32, vocab_size=64, hidden_dim=16, num_prompts=1,
                               samples_per_prompt=2, prompt_len=2, completion_len=3, lr=1e-2)
    worker = NativeTrainingWorker(cfg, model=Backbone())
    before = worker.model.embed.weight.detach().clone()
    out = worker.train(make_rollout_result(iteration=0, weight_version=0, payload=None))
    assert out.metrics["training_backend"] == "native" and not torch.equal(worker.model.embed.weight, before)


# ------------------------------------------------------------------------- DeepSpeed ZeRO-3 publish
class _FakeEngine:
    def __init__(self, model, rank, world):
        self.module, self.global_rank, self.world_size = model, rank, world

    def __call__(self, *args, **kwargs):
        return self.module(*args, **kwargs)

    def backward(self, loss):
        loss.backward()

    def step(self):
        pass


def _fake_deepspeed(rank=0, world=2, with_gather=True, log=None):
    class Gathered:
        def __init__(self, params, modifier_rank=None):
            self.n, self.modifier_rank = len(list(params)), modifier_rank

        def __enter__(self):
            (log if log is not None else []).append(("enter", self.n, self.modifier_rank))

        def __exit__(self, *exc):
            (log if log is not None else []).append(("exit",))
            return False

    def initialize(model=None, optimizer=None, config=None):
        return _FakeEngine(model, rank, world), optimizer, None, None

    zero = types.SimpleNamespace(GatheredParameters=Gathered) if with_gather else types.SimpleNamespace()
    return types.SimpleNamespace(initialize=initialize, zero=zero)


def test_deepspeed_zero3_publishes_a_rank0_gathered_clone():
    from rl_engine.executors.bridge import WeightBridgeUnavailableError
    from rl_engine.executors.deepspeed_trainer import DeepSpeedTrainingConfig, DeepSpeedTrainingWorker

    cfg = DeepSpeedTrainingConfig(device="cpu", dtype=torch.float32, vocab_size=32, hidden_dim=8, zero_stage=3)
    log = []
    worker = DeepSpeedTrainingWorker(cfg, deepspeed_module=_fake_deepspeed(log=log))
    manifest = worker.publish_weights(1)
    layout = manifest.metadata["layout"]
    assert layout["kind"] == "full-state" and layout["zero_stage"] == 3 and layout["world_size"] == 2 and layout["rank"] == 0
    export = manifest.metadata["deepspeed_zero3_full_state_export"]
    assert export["method"] == "deepspeed.zero.GatheredParameters" and export["tensor_count"] == len(manifest.tensors) == 3   # embedding, head weight, head bias
    assert log[0] == ("enter", 3, 0) and log[1] == ("exit",)          # cloned inside the gather context, modifier rank 0
    # the published tensors are a clone: later training does not change what the consumer imports
    imported = worker.bridge.import_update(manifest)
    snapshot = {k: v.clone() for k, v in imported.items()}
    with torch.no_grad():
        for p in worker.model.parameters():
            p.add_(1.0)
    assert all(torch.equal(imported[k], snapshot[k]) for k in snapshot)
    assert isinstance(worker.model, torch.nn.Module) and hasattr(worker.model, "lm_head")          # live model restored
    # other ranks and runtimes without a gather API refuse instead of publishing a shard
    with pytest.raises(WeightBridgeUnavailableError, match="rank 0"):
        DeepSpeedTrainingWorker(cfg, deepspeed_module=_fake_deepspeed(rank=1)).publish_weights(1)
    with pytest.raises(WeightBridgeUnavailableError, match="GatheredParameters"):
        DeepSpeedTrainingWorker(cfg, deepspeed_module=_fake_deepspeed(with_gather=False)).publish_weights(1)
    solo = DeepSpeedTrainingWorker(cfg, deepspeed_module=_fake_deepspeed(world=1, with_gather=False)).publish_weights(1)
    assert solo.metadata["deepspeed_zero3_full_state_export"]["method"] == "single-rank-state-dict"


def test_cuda_home_discovery(tmp_path, monkeypatch):
    from rl_engine.executors import deepspeed_trainer as ds

    toolkit = tmp_path / "nvidia" / "cu13"
    (toolkit / "bin").mkdir(parents=True)
    (toolkit / "include").mkdir()
    (toolkit / "lib64").mkdir()
    (toolkit / "bin" / "nvcc").write_text("")
    (toolkit / "include" / "cuda.h").write_text("")
    (tmp_path / "nvidia" / "cu12").mkdir()                                # older and incomplete: skipped
    monkeypatch.setattr(ds.sysconfig, "get_paths", lambda: {"purelib": str(tmp_path), "platlib": str(tmp_path)})
    import torch.utils.cpp_extension as ext

    monkeypatch.setattr(ext, "CUDA_HOME", ext.CUDA_HOME)                 # restored after the test
    env = {"PATH": "/usr/bin"}
    assert ds.configure_cuda_home(env) == str(toolkit)
    assert env["CUDA_HOME"] == str(toolkit) and env["PATH"].split(":")[0] == str(toolkit / "bin")
    assert env["LD_LIBRARY_PATH"] == str(toolkit / "lib64") and ext.CUDA_HOME == str(toolkit)
    explicit = {"CUDA_HOME": "/opt/cuda-x"}
    assert ds.configure_cuda_home(explicit) == "/opt/cuda-x" and "PATH" not in explicit


def test_worker_publishes_hugging_face_names_and_the_native_rollout_side_installs_them():
    """``weight_names="hf"``: the manifest carries the names of the Hugging Face checkpoint of the architecture (what a
    vLLM weight loader takes); the native rollout executor recognises them and fills its packed parameters."""
    policy, rollout_copy = tiny(7), tiny(8)
    bridge = make_weight_bridge("local-clone", source_worker="trainer")
    worker = GRPOTrainingWorker(GRPOTrainingConfig(lr=1e-3, device="cpu", dtype=torch.float32, vocab_size=128,
                                                   weight_names="hf"), model=policy, weight_bridge=bridge)
    manifest = worker.publish_weights(0)
    assert "model.layers.1.self_attn.k_proj.weight" in manifest.tensors and "l1.wqkv" not in manifest.tensors
    assert manifest.tensors["model.layers.0.mlp.up_proj.weight"].shape == (48, 32)
    executor = RolloutExecutor({"num_generations": 2}, weight_bridge=bridge, policy_model=rollout_copy)
    executor.update_weights(manifest)
    assert torch.equal(rollout_copy.flat, policy.flat) and executor.active_weight_version == 0
    with pytest.raises(ValueError):
        policy.state_dict_views(names="onnx")


def test_native_worker_trains_hugging_face_causal_lms_below_their_vocabulary_projection():
    """``NativeTrainingWorker(model=<HF ...ForCausalLM>)``: the decoder (``base_model``) is called directly, so the
    LM head's ``forward`` never runs and no ``[B, S, V]`` logits exist; the step changes the head through ``linear_logp``
    and the published names are the checkpoint's."""
    transformers = pytest.importorskip("transformers")
    from rl_engine.executors.hidden_states import backbone_hidden_states, output_head

    cfg = NativeTrainingConfig(lr=1e-2, device="cpu", dtype=torch.float32, vocab_size=64, num_prompts=2, samples_per_prompt=3,
                               prompt_len=4, completion_len=5)
    llama = transformers.LlamaForCausalLM(transformers.LlamaConfig(
        vocab_size=64, hidden_size=32, intermediate_size=48, num_hidden_layers=2, num_attention_heads=2, num_key_value_heads=1,
        max_position_embeddings=64, tie_word_embeddings=False)).float()
    gpt2 = transformers.GPT2LMHeadModel(transformers.GPT2Config(vocab_size=64, n_embd=32, n_layer=2, n_head=2, n_positions=64))
    for model in (llama, gpt2):
        head_calls = []
        model.lm_head.register_forward_hook(lambda *_: head_calls.append(1))
        worker = NativeTrainingWorker(cfg, model=model)
        before = model.lm_head.weight.detach().clone()
        result = worker.train(make_rollout_result(iteration=0, weight_version=0, payload=None))
        assert result.metrics["current_logp_path"] == "linear_logp" and torch.isfinite(torch.tensor(result.metrics["loss"]))
        assert not torch.equal(before, model.lm_head.weight) and head_calls == []
        assert set(worker.publish_weights(1).tensors) == set(model.state_dict())
    # a model that returns logits only is asked for its hidden states; one that cannot give any is an error
    class LogitsOnly(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.config = types.SimpleNamespace(output_hidden_states=False)
            self.embed, self.lm_head = torch.nn.Embedding(64, 16), torch.nn.Linear(16, 64, bias=False)

        def forward(self, ids, output_hidden_states=False):
            h = self.embed(ids)
            out = {"logits": self.lm_head(h)}
            if output_hidden_states:
                out["hidden_states"] = (h, h * 2.0)
            return out

    m = LogitsOnly()
    ids = torch.randint(0, 64, (2, 3))
    assert torch.equal(backbone_hidden_states(m, ids, hidden_dim=16), m.embed(ids) * 2.0)
    assert output_head(m) is m.lm_head
    with pytest.raises(TypeError):
        backbone_hidden_states(torch.nn.Embedding(64, 8), ids, hidden_dim=16)
    with pytest.raises(TypeError):
        output_head(torch.nn.Embedding(64, 8))
