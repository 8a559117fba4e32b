"""Stand-ins that let the reference library's own test files run against this library.

The reference's tests exercise its public API (operators, executors, bridges, workers), which this library keeps, so
they double as a parity suite.  A few of them also import things that exist only there: its Triton operator modules
(their tests skip without a Triton GPU, but the import must succeed) and private helpers of its DeepSpeed worker.
Importing this module registers stand-ins for exactly those names, mapped to this library's equivalents, so that the
behaviour BEHIND the names is what gets tested.  Nothing else is patched.

Run from an empty directory, with a checkout of the reference at ``$REF`` and this repository at ``$REPO``::

    PYTHONPATH=$REPO:$REPO/tests/reference_compat python -m pytest $REF/tests/test_weight_sync_bridge.py \\
        -q -p no:cacheprovider --rootdir=.

``sitecustomize.py`` beside this file imports it in every interpreter started with that ``PYTHONPATH``, which also
covers the worker processes that some tests spawn.  Expected differences are listed in ``README.md`` here.
"""

import sys
import types

import torch

import rl_engine.executors.deepspeed_trainer as _deepspeed_trainer
from rl_engine.executors.hidden_states import extract_hidden_states as _extract
from rl_engine.executors.trainer import safe_token_ids as _safe_token_ids
from rl_engine.kernels.ops.pytorch.loss.grpo_loss import NativeGRPOLossOp
from rl_engine.kernels.ops.pytorch.loss.linear_logp import NativeLinearLogpOp
from rl_engine.kernels.ops.pytorch.loss.ratio_kl import NativeRatioKLOp


def _module(name: str, **attrs) -> types.ModuleType:
    mod = types.ModuleType(name)
    mod.__dict__.update(attrs)
    sys.modules[name] = mod
    return mod


# import paths of the reference's Triton operators (this library has no Triton): the test files import them at module
# level and skip the Triton cases without a Triton-capable GPU
_module("rl_engine.kernels.ops.triton")
_module("rl_engine.kernels.ops.triton.loss")
_module("rl_engine.kernels.ops.triton.loss.grpo_loss", TritonGRPOLossOp=NativeGRPOLossOp)
_module("rl_engine.kernels.ops.triton.loss.ratio_kl", TritonRatioKLOp=NativeRatioKLOp)
_module("rl_engine.kernels.ops.triton.loss.linear_logp", TritonLinearLogpOp=NativeLinearLogpOp)


class _EmbeddingLMHeadModel(torch.nn.Module):
    """The reference's toy policy under its private name (an embedding whose output is the hidden state, plus a head)."""

    def __init__(self, vocab_size, hidden_dim, bias=True, tie_weights=False):
        super().__init__()
        self.embedding = torch.nn.Embedding(vocab_size, hidden_dim)
        self.lm_head = torch.nn.Linear(hidden_dim, vocab_size, bias=bias)
        if tie_weights:
            self.lm_head.weight = self.embedding.weight

    def forward(self, token_ids):
        return self.embedding(token_ids)


def _extract_hidden_states(model_output, *, expected_hidden_dim=None):
    return _extract(model_output, hidden_dim=expected_hidden_dim)


_deepspeed_trainer._EmbeddingLMHeadModel = _EmbeddingLMHeadModel
_deepspeed_trainer._safe_token_ids = _safe_token_ids
_deepspeed_trainer._extract_hidden_states = _extract_hidden_states
