"""Tooling around the operators: the single-GPU example as a subprocess (CPU smoke run; strict mode must refuse a
fallback), the profiler suite and its report writers, the synthetic RL batch fixture, and the stateless executor
driving real (tiny, random-init) Hugging Face models."""

import argparse
import json
import os
import subprocess
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "benchmarks"))


# ------------------------------------------------------------------------------ example CLI
def _run_example(*flags):
    env = dict(os.environ, PYTHONPATH=ROOT + os.pathsep + os.environ.get("PYTHONPATH", ""))
    return subprocess.run([sys.executable, "examples/grpo_single_gpu.py", "--device", "cpu", *flags], cwd=ROOT, env=env,
                          text=True, capture_output=True, check=False, timeout=600)


def test_example_runs_on_cpu():
    done = _run_example("--steps", "2", "--num-prompts", "1", "--samples-per-prompt", "2", "--prompt-len", "2",
                        "--completion-len", "3", "--vocab-size", "16", "--hidden-dim", "8")
    assert done.returncode == 0, done.stderr
    assert "completed grpo_single_gpu" in done.stdout and "device=cpu" in done.stdout


def test_example_strict_mode_refuses_the_cpu_fallback():
    done = _run_example("--steps", "1", "--num-prompts", "1", "--samples-per-prompt", "2", "--completion-len", "2",
                        "--vocab-size", "8", "--require-fused-logp")
    assert done.returncode != 0
    assert "--require-fused-logp" in done.stderr and "not the fused backend" in done.stderr


# ------------------------------------------------------------------------------ profiler suite
def _suite_args(workloads, **over):
    base = dict(device="cpu", dtype="float32", batch_sizes="2", seq_lens="4", vocab_sizes="32", workloads=workloads,
                top_k=4, top_p=0.9, seed=0, warmup=0, repeat=1, smoke=True, hidden=16)
    base.update(over)
    return argparse.Namespace(**base)


def test_profiler_suite_on_cpu_reports_pass_and_blocked():
    from profiler import available_workloads, build_arg_parser, run_automated_suite

    names = available_workloads()
    assert {"logp_native", "logp_fused", "sampling_native"} <= set(names)   # hyphenated spellings are accepted too
    assert build_arg_parser().parse_args([]).workloads == ",".join(names)   # the registry drives the CLI default
    metrics = run_automated_suite(_suite_args("logp-native,logp-fused,sampling-native")).get_metrics()
    by_name = {m.benchmark_name: m for m in metrics}
    assert by_name["logp_native"].status == "pass" and by_name["logp_native"].tokens_per_sec > 0
    assert by_name["sampling_native"].status == "pass"
    assert by_name["logp_fused"].status == "blocked"          # no GPU here: reported, not silently replaced
    with pytest.raises(ValueError, match="unsupported workloads: missing-op"):
        run_automated_suite(_suite_args("logp-native,missing-op"))


def test_profiler_report_writers_and_cli(tmp_path):
    from profiler import run_automated_suite

    prof = run_automated_suite(_suite_args("logp-native"))
    prof.save_csv(tmp_path / "p.csv")
    prof.save_json(tmp_path / "p.json")
    prof.save_csv(tmp_path / "p.csv")                          # the CSV writer appends: one header, two rows
    lines = (tmp_path / "p.csv").read_text().strip().splitlines()
    assert "tokens_per_sec" in lines[0] and len(lines) == 3
    report = json.loads((tmp_path / "p.json").read_text())
    assert report["report_version"] == "1.0" and report["metrics"][0]["benchmark_name"] == "logp_native"
    env = dict(os.environ, PYTHONPATH=ROOT)
    out = tmp_path / "cli.json"
    done = subprocess.run([sys.executable, "benchmarks/profiler.py", "--device", "cpu", "--smoke", "--workloads",
                           "logp-native,sampling-native", "--format", "json", "--output", str(out)], cwd=ROOT, env=env,
                          text=True, capture_output=True, check=False, timeout=600)
    assert done.returncode == 0, done.stderr
    assert {m["benchmark_name"] for m in json.loads(out.read_text())["metrics"]} == {"logp_native", "sampling_native"}


def test_profiler_timing_uses_warmup_then_median(monkeypatch):
    from profiler import PerformanceProfiler

    prof = PerformanceProfiler(device=torch.device("cpu"), warmup=2, repeat=3)
    calls = []
    result, latency_ms, std_ms = prof.time_fn(lambda: calls.append(1) or 4)
    assert result == 4 and len(calls) == 5 and latency_ms >= 0.0 and std_ms is not None


# ------------------------------------------------------------------------------ weight-sync benchmark modes
@pytest.mark.parametrize("mode", ["shared-memory", "file"])
def test_weight_sync_benchmark_cross_process_modes(mode):
    """The benchmark's consumer-process modes are integration tests of the transports: a separate process attaches to
    the published update, validates it against the manifest and acknowledges; after the publisher's release a fresh
    import is refused."""
    env = dict(os.environ, PYTHONPATH=ROOT)
    done = subprocess.run([sys.executable, "benchmark_weight_sync_bridge.py", "--mode", mode, "--cross-process", "--smoke"],
                          cwd=os.path.join(ROOT, "benchmarks"), env=env, text=True, capture_output=True, check=False, timeout=600)
    assert done.returncode == 0, done.stderr
    row = json.loads([ln for ln in done.stdout.splitlines() if ln.startswith("{")][-1])
    assert row["status"] == "pass" and row["cross_process"] is True and row["verified"] is True
    assert row["after_release"] == "stale import refused" and row["consumer_version"] == 1 and row["tensors"] == 8


def test_weight_sync_benchmark_in_process_and_blockers():
    env = dict(os.environ, PYTHONPATH=ROOT)
    for mode in ("local", "rollout-update", "runtime-blockers"):
        done = subprocess.run([sys.executable, "benchmark_weight_sync_bridge.py", "--mode", mode, "--smoke"],
                              cwd=os.path.join(ROOT, "benchmarks"), env=env, text=True, capture_output=True, check=False,
                              timeout=600)
        assert done.returncode == 0, done.stderr
        row = json.loads([ln for ln in done.stdout.splitlines() if ln.startswith("{")][-1])
        assert row["status"] == "pass", row
    assert "multi-node" in row and row["multi-node"].startswith("blocked")


# ------------------------------------------------------------------------------ fixture
def test_synthetic_batch_fixture_contract():
    from rl_engine.testing import make_synthetic_rl_kernel_batch

    kw = dict(num_prompts=2, samples_per_prompt=3, prompt_len=4, completion_len=5, vocab_size=128, valid_density=0.6,
              dtype=torch.float32, seed=7)
    a, b = make_synthetic_rl_kernel_batch(**kw), make_synthetic_rl_kernel_batch(**kw)
    assert a.batch_size == 6 and a.total_seq_len == 9 and a.prompt_len == 4 and a.completion_len == 5
    for name, shape in (("input_ids", (6, 9)), ("attention_mask", (6, 9)), ("prompt_mask", (6, 9)),
                        ("completion_mask", (6, 5)), ("token_ids", (6, 5)), ("advantages", (6, 5)),
                        ("old_logps", (6, 5)), ("ref_logps", (6, 5)), ("rewards", (6,))):
        assert tuple(getattr(a, name).shape) == shape
        assert torch.equal(getattr(a, name), getattr(b, name)), f"{name} is not reproducible from the seed"
    assert a.prompt_mask[:, :4].all() and not a.prompt_mask[:, 4:].any()
    assert torch.equal(a.attention_mask[:, 4:], a.completion_mask)
    assert a.valid_indices.numel() == round(6 * 5 * 0.6) == int(a.completion_mask.sum())
    # the samples of a prompt share its tokens; different prompts differ
    assert torch.equal(a.input_ids[0, :4], a.input_ids[2, :4]) and not torch.equal(a.input_ids[0, :4], a.input_ids[3, :4])
    assert not torch.equal(make_synthetic_rl_kernel_batch(**{**kw, "seed": 8}).token_ids, a.token_ids)
    # dense / compact views
    vals = torch.arange(30.0).reshape(6, 5)
    assert torch.equal(a.compact_completion_values(vals), vals.reshape(-1)[a.flat_completion_mask])
    assert torch.equal(a.compact_token_ids(), a.flat_token_ids[a.flat_completion_mask])
    with pytest.raises(ValueError, match="expected leading shape"):
        a.dense_completion_values(torch.zeros(5, 5))
    meta = a.benchmark_metadata()
    assert meta["valid_tokens"] == 18 and meta["num_prompts"] == 2 and meta["samples_per_prompt"] == 3
    for bad in (dict(num_prompts=0), dict(samples_per_prompt=0), dict(prompt_len=-1), dict(completion_len=0),
                dict(vocab_size=1), dict(valid_density=1.5)):
        with pytest.raises(ValueError):
            make_synthetic_rl_kernel_batch(**{**kw, **bad})


# ------------------------------------------------------------------------------ real HF models, stateless
transformers = pytest.importorskip("transformers")


def _inputs(device="cpu"):
    from rl_engine.executors.stateless_executor import StatelessForwardInputs

    ids = torch.tensor([[5, 6, 7, 8, 9], [9, 8, 7, 6, 5]], device=device)
    comp = torch.tensor([[0, 0, 1, 1, 1], [0, 0, 0, 1, 1]], dtype=torch.bool, device=device)
    return StatelessForwardInputs(ids, torch.ones_like(ids, dtype=torch.bool), comp)


def test_stateless_executor_scores_a_real_hf_causal_lm_without_kv_cache():
    from rl_engine.executors.stateless_executor import StatelessForwardConfig, StatelessForwardExecutor

    torch.manual_seed(47)
    cfg = transformers.GPT2Config(vocab_size=32, n_positions=16, n_embd=16, n_layer=1, n_head=2, use_cache=True)
    model = transformers.GPT2LMHeadModel(cfg).eval()
    executor = StatelessForwardExecutor(model, StatelessForwardConfig(mode="reference"))
    inputs = _inputs()
    result = executor.score(inputs)
    assert result.reference_logps.shape == (2, 5)
    assert torch.count_nonzero(result.reference_logps[~inputs.completion_mask]) == 0
    m = result.metrics
    assert m["use_cache_passed"] is True and m["zero_kv_cache"] is True and m["kv_cache_output_tensors"] == 0
    # flash attention cannot run an fp32 CPU model: the executor fell back to eager attention and says so
    assert m["attention_backend_fallback"] is True and m["attention_backend"] == "eager"
    assert model.config.use_cache is True                      # the caller's setting is restored after scoring
    # against the definition: log-softmax of the previous position's logits at the realised token
    with torch.no_grad():
        logits = model(input_ids=inputs.input_ids, use_cache=False).logits.float()
    want = torch.log_softmax(logits[:, :-1], -1).gather(-1, inputs.input_ids[:, 1:, None]).squeeze(-1)
    got = result.reference_logps[:, 1:]
    keep = inputs.completion_mask[:, 1:]
    assert torch.allclose(got[keep], want[keep], atol=1e-5)


def test_stateless_executor_scores_a_real_hf_sequence_classifier():
    from rl_engine.executors.stateless_executor import StatelessForwardConfig, StatelessForwardExecutor

    torch.manual_seed(48)
    cfg = transformers.BertConfig(vocab_size=32, hidden_size=16, num_hidden_layers=1, num_attention_heads=2,
                                  intermediate_size=32, max_position_embeddings=16, num_labels=1)
    model = transformers.BertForSequenceClassification(cfg).eval()
    result = StatelessForwardExecutor(model, StatelessForwardConfig(mode="reward")).score(_inputs())
    assert result.rewards.shape == (2,) and result.rewards.requires_grad is False
    assert result.metrics["zero_kv_cache"] is True


def test_rl_loop_example_learns_and_serves_the_trained_weights():
    """``examples/rl_loop.py`` on CPU: rollout -> stateless reference scoring -> GRPO worker -> publish -> update, 18
    times; the toy reward must climb and the rollout side must end on the last published version."""
    import importlib.util
    import os

    path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "examples", "rl_loop.py")
    spec = importlib.util.spec_from_file_location("rl_loop_example", path)
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    summary = module.main(["--iterations", "18"])
    assert summary["final_weight_version"] == 18 and summary["training_backend"] == "GRPOTrainer"
    assert summary["mean_reward_last3"] > summary["mean_reward_first3"] + 0.15
