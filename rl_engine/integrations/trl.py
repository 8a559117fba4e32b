"""Drop-in operators for TRL-style trainers.

The reference advertises its log-prob and sampling operators as drop-in replacements for the ones in TRL or
DeepSpeed-Chat (``README.md:99``) and leaves the wiring to the user.  This module is that wiring:

* ``selective_log_softmax(logits, index)``: signature and semantics of ``trl.trainer.utils.selective_log_softmax``
  (log-softmax over the last dimension gathered at ``index``), differentiable, on the streaming log-prob kernels when
  the logits live on a GPU -- one pass over the logits forward, one backward, no ``[.., V]`` fp32 temporary;
* ``selective_log_softmax_from_hidden(hidden, lm_head_weight, index, bias=None)``: the same quantity without ever
  materialising logits (the registry's ``linear_logp``), for trainers that can hand over the last hidden states;
* ``sample(logits, ...)``: temperature / top-k / top-p sampling through ``SamplerBackend``;
* ``patch_trl()`` / ``unpatch_trl()``: swap the function into an importable ``trl`` (or any module object passed in).

Nothing imports ``trl`` unless ``patch_trl`` is called without a module.
"""

from __future__ import annotations

import importlib
import sys
from typing import Any, Dict, List, Optional, Tuple

import torch

_FUSED_DTYPES = (torch.bfloat16, torch.float16, torch.float32)
_PATCHED: Dict[Tuple[int, str], Tuple[Any, Any]] = {}   # (id(module), attribute) -> (module, original)


def _torch_selective_log_softmax(logits: torch.Tensor, index: torch.Tensor) -> torch.Tensor:
    picked = torch.gather(logits, dim=-1, index=index.unsqueeze(-1)).squeeze(-1).float()
    return (picked - torch.logsumexp(logits.float(), dim=-1)).to(logits.dtype if logits.dtype == torch.float64 else torch.float32)


def selective_log_softmax(logits: torch.Tensor, index: torch.Tensor) -> torch.Tensor:
    """``log_softmax(logits, -1)`` gathered at ``index`` (shape ``logits.shape[:-1]``), in fp32.  Ids must be in
    ``[0, V)``; on the GPU path an id outside the range is reported through the device error word, as for every
    operator of this library."""
    if index.shape != logits.shape[:-1]:
        raise ValueError(f"index has shape {tuple(index.shape)}, logits {tuple(logits.shape)}: expected {tuple(logits.shape[:-1])}")
    if logits.is_cuda and logits.dtype in _FUSED_DTYPES and logits.numel():
        from rl_engine.kernels.ops.sm100.logp_autograd import selected_logprobs

        keep = torch.ones(index.shape, dtype=torch.bool, device=logits.device)
        return selected_logprobs(logits, index, keep)
    return _torch_selective_log_softmax(logits, index.long())


def selective_log_softmax_from_hidden(hidden: torch.Tensor, lm_head_weight: torch.Tensor, index: torch.Tensor,
                                      bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Selected-token log-probs of ``hidden @ lm_head_weight.T (+ bias)`` without the logits (fused ``linear_logp``)."""
    from rl_engine.kernels.registry import kernel_registry

    lead = hidden.shape[:-1]
    if index.shape != lead:
        raise ValueError(f"index has shape {tuple(index.shape)}, hidden {tuple(hidden.shape)}: expected {tuple(lead)}")
    out = kernel_registry.get_op("linear_logp")(hidden.reshape(-1, hidden.shape[-1]), lm_head_weight, index.reshape(-1), bias)
    return out.reshape(lead)


_SAMPLER: Any = None


def sample(logits: torch.Tensor, *, temperature: float = 1.0, top_k: Optional[int] = None, top_p: Optional[float] = None,
           seed: Optional[int] = None) -> torch.Tensor:
    """Next-token ids ``[B]`` from ``[B, V]`` logits (``SamplerBackend``: one radix-select kernel on a GPU).  One
    sampler lives for the process, so successive calls draw from successive positions of its random stream; ``seed``
    restarts the stream."""
    global _SAMPLER
    if _SAMPLER is None:
        from rl_engine.kernels.sampling import SamplerBackend

        _SAMPLER = SamplerBackend()
    if seed is not None:
        _SAMPLER.manual_seed(seed)
    return _SAMPLER.sample(logits, top_k=top_k, top_p=top_p, temperature=temperature)


def patch_trl(module: Any = None, names: Tuple[str, ...] = ("selective_log_softmax",)) -> List[str]:
    """Replaces ``selective_log_softmax`` in ``trl.trainer.utils`` and in every already imported ``trl.trainer.*`` module
    that holds a reference to it (trainers import the function by name).  ``module``: patch this module object instead
    (tests, other stacks).  Returns the patched ``module.attribute`` names; ``unpatch_trl()`` restores them."""
    if module is None:
        try:
            targets = [importlib.import_module("trl.trainer.utils")]
        except ImportError as exc:
            raise RuntimeError("trl is not installed; pass the module that holds selective_log_softmax") from exc
        targets += [m for name, m in list(sys.modules.items()) if name.startswith("trl.trainer.") and m is not None
                    and m is not targets[0]]
    else:
        targets = [module]
    replacement = {"selective_log_softmax": selective_log_softmax}
    done = []
    for target in targets:
        for name in names:
            original = getattr(target, name, None)
            if original is None or original is replacement[name]:
                continue
            _PATCHED[(id(target), name)] = (target, original)
            setattr(target, name, replacement[name])
            done.append(f"{getattr(target, '__name__', type(target).__name__)}.{name}")
    return done


def unpatch_trl() -> int:
    """Puts back everything ``patch_trl`` replaced; returns how many attributes were restored."""
    count = 0
    for (_, name), (target, original) in list(_PATCHED.items()):
        setattr(target, name, original)
        count += 1
    _PATCHED.clear()
    return count
