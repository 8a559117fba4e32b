"""CPU tests: stateless scorer, paged-KV baseline, training contract, workers, vLLM/Ray/DeepSpeed fakes."""

import subprocess
import sys
import types

import pytest
import torch

from rl_engine.executors.paged_kv_baseline import PagedKVScoringBaseline, PagedKVScoringConfig
from rl_engine.executors.stateless_executor import (
    StatelessForwardConfig, StatelessForwardExecutor, StatelessForwardInputs, score_reference_logprobs,
    summarize_tensor_tree,
)
from rl_engine.executors.training_contract import (
    StatelessScoringWorker, TorchRLTrainingConfig, build_stateless_inputs_from_rollout_payload,
    extract_rollout_candidate_groups, extract_rollout_reference_logp_groups, extract_rollout_reward_groups,
    extract_rollout_token_groups, make_rollout_result,
)


class _Config:
    def __init__(self):
        self.use_cache = True
        self._attn_implementation = "sdpa"


class _TinyLM(torch.nn.Module):
    """HF-shaped causal LM: accepts attention_mask / use_cache and can return a KV cache."""

    def __init__(self, vocab=17, dim=8, leak_cache=False, fail_on_flash=False):
        super().__init__()
        self.config = _Config()
        self.emb = torch.nn.Embedding(vocab, dim)
        self.head = torch.nn.Linear(dim, vocab)
        self.leak_cache, self.fail_on_flash, self.calls = leak_cache, fail_on_flash, []

    def forward(self, input_ids, attention_mask=None, use_cache=None):
        self.calls.append({"use_cache": use_cache, "backend": self.config._attn_implementation, "training": self.training})
        if self.fail_on_flash and self.config._attn_implementation == "flash_attention_2":
            raise ImportError("flash_attn is not installed")
        h = self.emb(input_ids).cumsum(1)
        out = {"logits": self.head(h)}
        if use_cache or self.leak_cache:
            out["past_key_values"] = [(h, h)]
        return out


def _inputs(b=3, s=6, vocab=17, seed=0):
    g = torch.Generator().manual_seed(seed)
    ids = torch.randint(0, vocab, (b, s), generator=g)
    comp = torch.zeros(b, s, dtype=torch.bool)
    comp[:, 2:] = True
    comp[1, 5] = False
    return StatelessForwardInputs(ids, torch.ones(b, s, dtype=torch.bool), comp)


# ------------------------------------------------------------------------------ stateless scorer
def test_stateless_config_validation():
    for kwargs in ({"mode": "x"}, {"use_cache": True}, {"attention_backend": "magic"}, {"max_batch_size": 0}, {"temperature": 0.0}):
        with pytest.raises(ValueError):
            StatelessForwardConfig(**kwargs)


def test_stateless_reference_scores_and_policy_restore():
    model = _TinyLM().train()
    ex = StatelessForwardExecutor(model, StatelessForwardConfig(mode="reference", attention_backend="eager", return_token_scores=True))
    inputs = _inputs()
    res = ex.score(inputs)
    logits = model(inputs.input_ids)["logits"]
    want = torch.log_softmax(logits[:, :-1].float(), -1).gather(-1, inputs.input_ids[:, 1:, None]).squeeze(-1)
    got = res.reference_logps
    assert got.shape == (3, 6) and (got[:, 0] == 0).all() and (got[~inputs.completion_mask] == 0).all()
    assert torch.allclose(got[:, 1:][inputs.completion_mask[:, 1:]], want[inputs.completion_mask[:, 1:]], atol=1e-5)
    assert torch.equal(res.token_scores, got) and res.rewards is None and not got.requires_grad
    first = model.calls[0]
    assert first == {"use_cache": False, "backend": "eager", "training": False}
    assert model.config.use_cache is True and model.config._attn_implementation == "sdpa" and model.training  # restored
    m = res.metrics
    assert m["mode"] == "reference" and m["zero_kv_cache"] and m["use_cache_passed"] and m["active_completion_tokens"] == 11
    assert m["attention_backend"] == "eager" and m["attention_backend_fallback"] is False and m["kv_cache_output_mb"] == 0


def test_stateless_rejects_kv_cache_and_falls_back_from_flash():
    with pytest.raises(ValueError, match="KV-cache outputs"):
        StatelessForwardExecutor(_TinyLM(leak_cache=True), StatelessForwardConfig(mode="reference")).score(_inputs())
    tolerant = StatelessForwardExecutor(_TinyLM(leak_cache=True), StatelessForwardConfig(mode="reference", reject_kv_cache_outputs=False))
    assert tolerant.score(_inputs()).metrics["kv_cache_output_tensors"] == 2
    flaky = _TinyLM(fail_on_flash=True)
    res = StatelessForwardExecutor(flaky, StatelessForwardConfig(mode="reference")).score(_inputs())
    assert res.metrics["attention_backend_fallback"] is True and res.metrics["attention_backend_requested"] == "flash_attention_2"
    assert [c["backend"] for c in flaky.calls] == ["flash_attention_2", "eager"]

    class Broken(_TinyLM):
        def forward(self, input_ids, attention_mask=None, use_cache=None):
            raise RuntimeError("shape mismatch somewhere")

    with pytest.raises(RuntimeError, match="shape mismatch"):
        StatelessForwardExecutor(Broken(), StatelessForwardConfig(mode="reference")).score(_inputs())


def test_stateless_rewards_and_input_validation():
    class Reward(torch.nn.Module):
        def forward(self, input_ids):
            return {"logits": input_ids.float().mean(1, keepdim=True)}

    res = StatelessForwardExecutor(Reward(), StatelessForwardConfig(mode="reward", attention_backend="model_default")).score(_inputs())
    assert res.rewards.shape == (3,) and res.reference_logps is None and res.metrics["use_cache_passed"] is False
    bad_adapter = StatelessForwardExecutor(Reward(), StatelessForwardConfig(mode="reward"), reward_adapter=lambda o, i: torch.zeros(2))
    with pytest.raises(ValueError, match="batch size"):
        bad_adapter.score(_inputs())
    ins = _inputs()
    with pytest.raises(ValueError):
        StatelessForwardExecutor(_TinyLM(), StatelessForwardConfig(max_batch_size=2)).score(ins)
    starts_at_zero = StatelessForwardInputs(ins.input_ids, ins.attention_mask, torch.ones_like(ins.completion_mask))
    with pytest.raises(ValueError, match="position 0"):
        score_reference_logprobs(torch.zeros(3, 6, 17), starts_at_zero)
    assert summarize_tensor_tree({"a": [torch.zeros(2, 2), (torch.zeros(3),)], "b": None}).tensor_count == 2


def test_paged_kv_baseline_reserves_and_matches_stateless_scores():
    model = _TinyLM()
    inputs = _inputs()
    cfg = PagedKVScoringConfig(num_layers=2, num_kv_heads=2, head_dim=4, block_size=4, kv_cache_dtype=torch.float16)
    res = PagedKVScoringBaseline(model, cfg).score(inputs)
    stateless = StatelessForwardExecutor(model, StatelessForwardConfig(mode="reference", attention_backend="model_default")).score(inputs)
    assert torch.allclose(res.reference_logps, stateless.reference_logps, atol=1e-6)
    m = res.metrics
    assert m["paged_kv_required_blocks"] == 6 and m["paged_kv_blocks"] == 6 and m["use_cache"] is True
    payload = 2 * (2 * 6 * 4 * 2 * 4) * 2
    assert abs(m["paged_kv_cache_payload_mb"] - payload / 1048576) < 1e-9 and m["model_kv_cache_output_present"]
    assert m["baseline_kind"] == "generation_engine_paged_kv_reservation" and m["total_kv_cache_bytes"] > payload
    with pytest.raises(ValueError, match="cannot fit"):
        PagedKVScoringBaseline(model, PagedKVScoringConfig(block_size=4, kv_cache_blocks=2)).score(inputs)
    for kwargs in ({"use_cache": False}, {"num_layers": 0}, {"block_size": 0}, {"kv_cache_blocks": 0}):
        with pytest.raises(ValueError):
            PagedKVScoringConfig(**kwargs)


# --------------------------------------------------------------------------- training contract
class _Completion:
    def __init__(self, token_ids, reward=None):
        self.token_ids, self.text, self.finish_reason, self.cumulative_logprob = token_ids, "t", "stop", -1.5
        if reward is not None:
            self.reward = reward


class _Request:
    def __init__(self, token_ids, prompt=(1, 2), reward=None):
        self.request_id, self.prompt_token_ids, self.outputs = "r", list(prompt), [_Completion(token_ids, reward)]


def test_payload_extractors_accept_dicts_objects_and_nesting():
    payload = {"outputs": [[{"token_ids": [3, 4], "reward": 1.0, "ref_logps": [-1.0, -2.0]}, _Request([5], reward=0.5)],
                           [{"outputs": [{"token_ids": [6, 7, 8], "score": 2.0}]}]]}
    assert extract_rollout_candidate_groups(payload) == [[[3, 4], [5]], [[6, 7, 8]]]
    assert extract_rollout_token_groups(payload) == [[3, 4], [5], [6, 7, 8]]
    assert extract_rollout_reward_groups(payload) == [[1.0, 0.5], [2.0]]
    assert extract_rollout_reference_logp_groups(payload)[0][0] == [-1.0, -2.0]
    assert extract_rollout_candidate_groups({"token_groups": [[1, 2], [3]]}) == [[[1, 2]], [[3]]]
    assert extract_rollout_candidate_groups(None) == [] and extract_rollout_candidate_groups({"x": 1}) == []


def test_build_stateless_inputs_from_payload():
    payload = {"outputs": [[_Request([5, 6, 7], prompt=(9, 8)), _Request([4], prompt=(9, 8))]]}
    ins = build_stateless_inputs_from_rollout_payload(payload, prompt_len=None)
    assert ins.input_ids.tolist() == [[9, 8, 5, 6, 7], [9, 8, 4, 0, 0]]
    assert ins.completion_mask.tolist() == [[False, False, True, True, True], [False, False, True, False, False]]
    assert ins.attention_mask.tolist() == [[True] * 5, [True, True, True, False, False]]
    clipped = build_stateless_inputs_from_rollout_payload(payload, prompt_len=1, max_completion_len=2, prompt_token_id=3)
    assert clipped.input_ids.shape == (2, 3) and clipped.input_ids[0].tolist() == [9, 5, 6]
    for bad in ({"prompt_len": -1}, {"max_completion_len": 0}):
        with pytest.raises(ValueError):
            build_stateless_inputs_from_rollout_payload(payload, **bad)
    with pytest.raises(ValueError, match="candidate token ids"):
        build_stateless_inputs_from_rollout_payload({})


def test_scoring_worker_attaches_scores_to_candidates():
    payload = {"outputs": [[{"token_ids": [3, 4, 5]}, {"token_ids": [6]}]]}
    rollout = make_rollout_result(iteration=2, weight_version=7, payload=payload, metrics={"k": 1})

    class Both(_TinyLM):
        def forward(self, input_ids, attention_mask=None, use_cache=None):
            out = super().forward(input_ids, attention_mask, use_cache)
            out["rewards"] = input_ids.float().sum(1)
            return out

    worker = StatelessScoringWorker(
        StatelessForwardExecutor(Both(), StatelessForwardConfig(mode="both", attention_backend="model_default")),
        lambda r: build_stateless_inputs_from_rollout_payload(r.payload, prompt_len=1),
    )
    scored = worker.score(rollout)
    assert scored.iteration == 2 and scored.weight_version == 7 and scored.metrics["k"] == 1
    assert scored.metrics["scoring_backend"] == "stateless" and scored.metrics["scoring_zero_kv_cache"]
    cands = scored.payload["outputs"][0]
    assert isinstance(cands[0]["reward"], float) and len(cands[0]["reference_logps"]) == 3 and len(cands[1]["reference_logps"]) == 1
    assert scored.payload["stateless_scores"]["reference_logps"].shape == (2, 4)
    assert scored.duration_seconds >= 0


def test_native_training_worker_uses_payload_then_synthetic_and_publishes():
    from rl_engine.executors.rollout import RolloutExecutor
    from rl_engine.executors.trainer import NativeTrainingConfig, NativeTrainingWorker

    worker = NativeTrainingWorker(NativeTrainingConfig(vocab_size=32, hidden_dim=16, completion_len=4, lr=5e-2))
    payload = {"outputs": [[{"token_ids": [1, 2, 3], "reward": 1.0, "ref_logps": [-3.0, -3.0, -3.0]},
                            {"token_ids": [4, 5, 6, 7, 8], "reward": -1.0, "ref_logps": [-3.0] * 5}]]}
    res = worker.train(make_rollout_result(iteration=0, weight_version=0, payload=payload))
    m = res.metrics
    assert m["training_data_source"] == "rollout_payload" and m["reward_source"] == "payload_rewards"
    assert m["reference_logp_source"] == "payload_reference_logps" and m["rollout_sequences"] == 2 and m["active_tokens"] == 7
    assert m["current_logp_path"] == "linear_logp" and m["training_backend"] == "native" and res.published_weight_version == 1
    proxy = worker.train(make_rollout_result(iteration=1, weight_version=1, payload={"token_groups": [[1, 2], [3, 4]]}))
    assert proxy.metrics["reward_source"] == "token_id_proxy" and proxy.metrics["reference_logp_source"] == "synthetic_current_offset"
    synth = worker.train(make_rollout_result(iteration=2, weight_version=1, payload=None))
    assert synth.metrics["training_data_source"] == "synthetic_fallback" and synth.metrics["loss"] == synth.metrics["loss"]
    with pytest.raises(ValueError, match="token ids"):
        bad = NativeTrainingWorker(NativeTrainingConfig(vocab_size=32))
        bad.model.lm_head = torch.nn.Linear(32, 8, bias=False)
        bad.train(make_rollout_result(iteration=0, weight_version=0, payload={"token_groups": [[31, 30]]}))
    manifest = worker.publish_weights()
    assert manifest.weight_version == 0
    from rl_engine.executors.bridge import WeightManifestValidationError

    with pytest.raises(WeightManifestValidationError):
        worker.publish_weights(0)
    rollout_side = RolloutExecutor(weight_bridge=worker.bridge)
    tensors = rollout_side.update_weights(worker.publish_weights(5))
    assert torch.equal(tensors["lm_head.weight"], worker.model.lm_head.weight) and rollout_side.active_weight_version == 5
    assert TorchRLTrainingConfig().samples_per_prompt == 2


# ------------------------------------------------------------------------------------- fakes
class FakeSamplingParams:
    def __init__(self, **kwargs):
        self.kwargs = kwargs


class FakeLLM:
    instances = []

    def __init__(self, **kwargs):
        self.kwargs, self.seen = kwargs, []
        FakeLLM.instances.append(self)

    def generate(self, prompts, params):
        self.seen.append((list(prompts), params))
        return [_Request([i, i + 1], prompt=(7,)) for i, _ in enumerate(prompts)]


def test_vllm_sampler_repeats_prompts_contiguously_and_regroups():
    from rl_engine.executors.rollout import RolloutExecutor
    from rl_engine.executors.vllm_sampler import VLLMSamplerConfig, VLLMSharedPrefixSampler

    cfg = VLLMSamplerConfig.from_model_config(
        {"model": "m", "vllm": {"num_generations": 2, "engine_kwargs": {"dtype": "bf16"}}, "sampler": {"num_generations": 3},
         "sampling_params": {"temperature": 0.7}})
    assert cfg.num_generations == 3 and cfg.engine_kwargs == {"dtype": "bf16"} and cfg.enable_prefix_caching
    sampler = VLLMSharedPrefixSampler(cfg, llm_cls=FakeLLM, sampling_params_cls=FakeSamplingParams)
    out = sampler.generate(["a", "b"], sampling_params={"top_p": 0.9})
    engine = FakeLLM.instances[-1]
    assert engine.kwargs == {"dtype": "bf16", "model": "m", "enable_prefix_caching": True}
    prompts, params = engine.seen[0]
    assert prompts == ["a", "a", "a", "b", "b", "b"] and params.kwargs == {"temperature": 0.7, "top_p": 0.9}
    assert out["num_prompts"] == 2 and len(out["outputs"]) == 2 and len(out["outputs"][1]) == 3
    cand = out["normalized_outputs"][1][2]
    assert (cand.prompt_index, cand.candidate_index, cand.token_ids, cand.prompt_token_ids) == (1, 2, [5, 6], [7])
    assert "raw_output" not in cand.to_dict() and cand.to_dict()["finish_reason"] == "stop"
    assert extract_rollout_candidate_groups(out)[0] == [[0, 1], [1, 2], [2, 3]]  # feeds the trainer as is
    with pytest.raises(ValueError):
        VLLMSamplerConfig(num_generations=0)
    with pytest.raises(ValueError):
        VLLMSamplerConfig(backend="other")
    with pytest.raises(ValueError, match="model path"):
        VLLMSharedPrefixSampler(VLLMSamplerConfig(), llm_cls=FakeLLM, sampling_params_cls=FakeSamplingParams).generate("x")
    ex = RolloutExecutor({"model": "m", "num_generations": 2}, weight_transport="local-clone")
    ex.sampler = VLLMSharedPrefixSampler(VLLMSamplerConfig.from_model_config(ex.config), llm_cls=FakeLLM,
                                         sampling_params_cls=FakeSamplingParams)
    assert ex.generate_candidates("p")["num_generations"] == 2
    assert ex.execute_rollout(torch.tensor([1, 2]))["status"] == "no_policy_model"


class FakeObjectRef:
    def __init__(self, value):
        self.value = value


class FakeRay:
    def __init__(self):
        self.inited, self.killed, self.options_seen = [], [], []

    def is_initialized(self):
        return bool(self.inited)

    def init(self, **kwargs):
        self.inited.append(kwargs)

    def remote(self, cls):
        ray = self

        class RemoteClass:
            def __init__(self, opts=None):
                self.opts = opts

            def options(self, **opts):
                ray.options_seen.append(opts)
                return RemoteClass(opts)

            def remote(self, *args, **kwargs):
                instance = cls(*args, **kwargs)

                class Actor:
                    def __getattr__(self, name):
                        method = getattr(instance, name)
                        return types.SimpleNamespace(remote=lambda *a, **k: FakeObjectRef(method(*a, **k)))

                return Actor()

        return RemoteClass()

    def get(self, ref):
        return ref.value

    def kill(self, actor, no_restart=True):          # the signature of ``ray.kill``
        assert no_restart is True
        self.killed.append(actor)


def test_ray_actor_manager_with_fake_ray():
    from rl_engine.executors.ray_actor_manager import (
        RayActorManager, RayActorOptions, RayRuntimeConfig, RayUnavailableError, RayWorkerSpec, _load_ray,
    )
    from rl_engine.executors.rollout import RolloutExecutor
    from rl_engine.executors.trainer import NativeTrainingConfig, NativeTrainingWorker

    ray = FakeRay()
    with RayActorManager(RayRuntimeConfig(address="auto", namespace="rl"), ray_module=ray) as mgr:
        assert ray.inited == [{"ignore_reinit_error": True, "address": "auto", "namespace": "rl"}]
        trainer = mgr.create_training_worker(RayWorkerSpec(
            NativeTrainingWorker, kwargs={"config": NativeTrainingConfig(vocab_size=32, hidden_dim=8)},
            actor_options=RayActorOptions(name="trainer", num_gpus=1, max_restarts=2)))
        assert ray.options_seen[0] == {"name": "trainer", "num_gpus": 1, "max_restarts": 2}   # only what was set
        result = trainer.train(make_rollout_result(iteration=0, weight_version=0, payload=None))
        assert result.published_weight_version == 1
        manifest = trainer.publish_weights(weight_version=1)
        rollout = mgr.create_rollout_worker(RayWorkerSpec(RolloutExecutor, kwargs={"weight_transport": "local-clone"}))
        health = mgr.health_check()
        assert [h["worker_type"] for h in health] == ["NativeTrainingWorker", "RolloutExecutor"] and health[0]["published_weight_version"] == 1
        trainer.release_weights(manifest.update_id)
        assert rollout is not None
    assert len(ray.killed) == 2
    if "ray" not in sys.modules:
        try:
            import ray as _real  # noqa: F401
        except ImportError:
            with pytest.raises(RayUnavailableError):
                _load_ray()


class FakeDeepSpeedEngine:
    def __init__(self, model, optimizer):
        self.module, self.optimizer, self.steps, self.backwards, self.forwards = model, optimizer, 0, 0, 0

    def __call__(self, *args, **kwargs):          # DeepSpeedEngine.forward runs the wrapped module
        self.forwards += 1
        return self.module(*args, **kwargs)

    def zero_grad(self):
        self.optimizer.zero_grad()

    def backward(self, loss):
        self.backwards += 1
        loss.backward()

    def step(self):
        self.steps += 1
        self.optimizer.step()


def _fake_deepspeed(record):
    class Gathered:
        def __init__(self, params, modifier_rank=None):
            record.append(("gather", len(list(params)), modifier_rank))

        def __enter__(self):
            return self

        def __exit__(self, *a):
            return False

    def initialize(model=None, optimizer=None, config=None):
        record.append(("initialize", config))
        return FakeDeepSpeedEngine(model, optimizer), optimizer, None, None

    return types.SimpleNamespace(initialize=initialize, zero=types.SimpleNamespace(GatheredParameters=Gathered))


def test_deepspeed_worker_with_fake_module_and_zero3_gather():
    from rl_engine.executors.deepspeed_trainer import DeepSpeedTrainingConfig, DeepSpeedTrainingWorker, DeepSpeedUnavailableError, _load_deepspeed

    record = []
    cfg = DeepSpeedTrainingConfig(vocab_size=32, hidden_dim=8, zero_stage=3, deepspeed_config={"zero_optimization": {"overlap_comm": True}})
    worker = DeepSpeedTrainingWorker(cfg, deepspeed_module=_fake_deepspeed(record))
    ds_cfg = record[0][1]
    assert ds_cfg["zero_optimization"] == {"stage": 3, "overlap_comm": True} and ds_cfg["bf16"] == {"enabled": False}
    res = worker.train(make_rollout_result(iteration=0, weight_version=0, payload=None))
    assert res.metrics["training_backend"] == "deepspeed" and res.metrics["deepspeed_zero_stage"] == 3
    assert worker.engine.steps == 1 and worker.engine.backwards == 1 and worker.engine.forwards == 1   # through the engine
    assert ("gather", 2, None) in record                     # lm_head weight and bias, gathered around forward + backward
    manifest = worker.publish_weights()
    assert manifest.metadata["layout"]["zero_stage"] == 3 and record[-1][0] == "gather"
    try:
        import deepspeed  # noqa: F401
    except ImportError:
        with pytest.raises(DeepSpeedUnavailableError):
            _load_deepspeed()


def test_importing_executors_does_not_import_heavy_runtimes():
    code = (
        "import sys; import rl_engine.executors.rollout, rl_engine.executors.stateless_executor, "
        "rl_engine.executors.paged_kv_baseline, rl_engine.executors.ray_actor_manager, rl_engine.executors.deepspeed_trainer, "
        "rl_engine.executors.vllm_sampler, rl_engine.executors.training_contract, rl_engine.kernels.registry, rl_engine.kernels.sampling; "
        "bad = [m for m in ('vllm', 'ray', 'deepspeed', 'flash_attn', 'flashinfer', 'triton') if m in sys.modules]; "
        "print('BAD', bad)"
    )
    import os

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    out = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, cwd=root, timeout=300)
    assert out.returncode == 0, out.stderr[-2000:]
    assert "BAD []" in out.stdout, out.stdout[-500:]


def test_sampler_and_payload_parser_against_real_vllm_classes():
    """With vLLM installed: the sampler builds a real ``vllm.SamplingParams`` from its configuration, and real
    ``RequestOutput`` / ``CompletionOutput`` objects (returned by a stand-in engine, no GPU) are regrouped, normalised
    and parsed by the training contract exactly like the fakes used elsewhere."""
    try:
        from vllm import SamplingParams
        from vllm.outputs import CompletionOutput, RequestOutput
    except Exception as exc:  # noqa: BLE001  (not installed, or not importable on this machine)
        pytest.skip(f"vllm is not importable here: {type(exc).__name__}")
    from rl_engine.executors.training_contract import extract_rollout_candidate_groups
    from rl_engine.executors.vllm_sampler import VLLMSamplerConfig, VLLMSharedPrefixSampler

    seen = {}

    class Engine:
        def generate(self, prompts, params):
            seen["prompts"], seen["params"] = list(prompts), params
            out = []
            for i, prompt in enumerate(prompts):
                done = CompletionOutput(index=0, text=f"t{i}", token_ids=[i + 1, i + 2], cumulative_logprob=-0.5 * (i + 1),
                                        logprobs=None, finish_reason="length")
                out.append(RequestOutput(request_id=f"r{i}", prompt=prompt if isinstance(prompt, str) else None,
                                         prompt_token_ids=[7, 8, 9], prompt_logprobs=None, outputs=[done], finished=True))
            return out

    config = VLLMSamplerConfig.from_model_config({
        "model": "unused", "num_generations": 3,
        "sampling_params": {"temperature": 0.7, "top_p": 0.9, "top_k": 50, "max_tokens": 16, "seed": 1}})
    sampler = VLLMSharedPrefixSampler(config, engine=Engine(), sampling_params_cls=SamplingParams, llm_cls=object)
    result = sampler.generate(["alpha", "beta"])
    assert isinstance(seen["params"], SamplingParams) and seen["params"].top_k == 50 and seen["params"].max_tokens == 16
    assert seen["prompts"] == ["alpha"] * 3 + ["beta"] * 3                  # repeated back to back for the prefix cache
    assert result["num_prompts"] == 2 and result["num_generations"] == 3
    first = result["normalized_outputs"][1][2]
    assert first.request_id == "r5" and first.token_ids == [6, 7] and first.finish_reason == "length"
    assert first.prompt_token_ids == [7, 8, 9] and first.cumulative_logprob == -3.0 and first.text == "t5"
    groups = extract_rollout_candidate_groups(result)
    assert groups == [[[1, 2], [2, 3], [3, 4]], [[4, 5], [5, 6], [6, 7]]]
