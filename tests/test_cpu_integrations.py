"""TRL-style drop-ins on CPU: the selected-token log-softmax (values and gradients against plain PyTorch), the
no-logits variant through ``linear_logp``, the sampler wrapper, and patching / unpatching a stand-in ``trl`` module."""

import sys
import types

import pytest
import torch

from rl_engine.integrations import trl as drop_in


def _reference(logits, index):
    return torch.log_softmax(logits.float(), dim=-1).gather(-1, index.unsqueeze(-1)).squeeze(-1)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_selective_log_softmax_matches_log_softmax_gather_with_gradients(dtype):
    gen = torch.Generator().manual_seed(0)
    logits = torch.randn(3, 7, 50, generator=gen).to(dtype).requires_grad_(True)
    index = torch.randint(0, 50, (3, 7), generator=gen)
    got = drop_in.selective_log_softmax(logits, index)
    want = _reference(logits.detach().clone().requires_grad_(True), index)
    assert got.shape == (3, 7) and got.dtype == torch.float32
    assert torch.allclose(got, want, atol=1e-5 if dtype == torch.float32 else 2e-2)
    upstream = torch.randn(3, 7, generator=gen)
    got.backward(upstream)
    ref_logits = logits.detach().clone().requires_grad_(True)
    _reference(ref_logits, index).backward(upstream)
    assert torch.allclose(logits.grad.float(), ref_logits.grad.float(), atol=1e-5 if dtype == torch.float32 else 2e-2)
    with pytest.raises(ValueError):
        drop_in.selective_log_softmax(logits, index[:, :3])


def test_from_hidden_equals_the_logits_route():
    gen = torch.Generator().manual_seed(1)
    hidden = torch.randn(2, 5, 16, generator=gen, requires_grad=True)
    weight = torch.randn(40, 16, generator=gen, requires_grad=True)
    bias = torch.randn(40, generator=gen)
    index = torch.randint(0, 40, (2, 5), generator=gen)
    fused = drop_in.selective_log_softmax_from_hidden(hidden, weight, index, bias)
    plain = drop_in.selective_log_softmax(hidden @ weight.t() + bias, index)
    assert fused.shape == (2, 5) and torch.allclose(fused, plain, atol=1e-5)
    fused.sum().backward()
    assert hidden.grad is not None and weight.grad is not None


def test_sampler_wrapper_draws_valid_ids_and_restarts_with_a_seed():
    logits = torch.randn(6, 30, generator=torch.Generator().manual_seed(2))
    ids = drop_in.sample(logits, temperature=0.8, top_k=5, top_p=0.9, seed=3)
    assert ids.shape == (6,) and bool(((ids >= 0) & (ids < 30)).all())
    top5 = torch.topk(logits, 5).indices
    assert all(int(ids[i]) in top5[i].tolist() for i in range(6))


def test_patch_and_unpatch_a_trl_like_module(monkeypatch):
    original = lambda logits, index: "original"  # noqa: E731
    utils = types.ModuleType("trl.trainer.utils")
    utils.selective_log_softmax = original
    grpo = types.ModuleType("trl.trainer.grpo_trainer")
    grpo.selective_log_softmax = original            # trainers import the function by name
    other = types.ModuleType("trl.trainer.sft_trainer")
    for name, mod in (("trl", types.ModuleType("trl")), ("trl.trainer", types.ModuleType("trl.trainer")),
                      ("trl.trainer.utils", utils), ("trl.trainer.grpo_trainer", grpo), ("trl.trainer.sft_trainer", other)):
        monkeypatch.setitem(sys.modules, name, mod)
    done = drop_in.patch_trl()
    assert sorted(done) == ["trl.trainer.grpo_trainer.selective_log_softmax", "trl.trainer.utils.selective_log_softmax"]
    assert utils.selective_log_softmax is drop_in.selective_log_softmax is grpo.selective_log_softmax
    assert drop_in.patch_trl() == []                 # idempotent
    assert drop_in.unpatch_trl() == 2 and utils.selective_log_softmax is original and grpo.selective_log_softmax is original
    # an explicit module object (another stack)
    mine = types.SimpleNamespace(selective_log_softmax=original)
    assert len(drop_in.patch_trl(mine)) == 1 and mine.selective_log_softmax is drop_in.selective_log_softmax
    drop_in.unpatch_trl()
    assert mine.selective_log_softmax is original


def test_patch_without_trl_is_an_explicit_error(monkeypatch):
    monkeypatch.setitem(sys.modules, "trl", None)
    with pytest.raises(RuntimeError, match="trl is not installed"):
        drop_in.patch_trl()
