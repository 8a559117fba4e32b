"""Find the final hidden states in whatever a backbone returns.

A training worker that scores with ``linear_logp`` needs ``[..., hidden_dim]`` states, not logits.  Backbones return
them in many shapes: a bare tensor, a Hugging Face ``ModelOutput`` (``last_hidden_state``, or the ``hidden_states``
tuple when ``output_hidden_states=True``), a dict with those keys, or a tuple such as ``(loss, states, cache)``.

Behavioural parity with the reference's worker (``rl_engine/executors/deepspeed_trainer.py:424-556``):

* a tensor qualifies if it has at least two dimensions and, when ``hidden_dim`` is given, that last dimension;
* named fields win over position: ``last_hidden_state`` / ``hidden`` first, then the LAST qualifying entry of
  ``hidden_states``;
* in a tuple / list, entries that carry such fields are looked at before bare tensors; among bare tensors a single
  qualifying one is taken, else the single one with the most dimensions; nested containers are searched last;
* nothing found -> ``TypeError`` naming the output's type.

The search is written as one walk that yields candidates in that priority order, instead of the reference's family
of mutually recursive helpers.
"""

from __future__ import annotations

from typing import Any, Iterator, Mapping, Optional, Sequence

import torch

_DIRECT_FIELDS = ("last_hidden_state", "hidden")
_STACK_FIELD = "hidden_states"
_MISSING = object()


def _field(obj: Any, name: str) -> Any:
    if isinstance(obj, Mapping):
        return obj.get(name, _MISSING)
    return getattr(obj, name, _MISSING)


def _names_hidden_states(obj: Any) -> bool:
    if isinstance(obj, (torch.Tensor, tuple, list)):
        return False
    return any(_field(obj, name) is not _MISSING for name in _DIRECT_FIELDS + (_STACK_FIELD,))


class _Search:
    def __init__(self, hidden_dim: Optional[int]) -> None:
        self.hidden_dim = None if hidden_dim is None else int(hidden_dim)

    def fits(self, t: Any) -> bool:
        return (isinstance(t, torch.Tensor) and t.ndim >= 2
                and (self.hidden_dim is None or int(t.shape[-1]) == self.hidden_dim))

    def walk(self, obj: Any) -> Iterator[torch.Tensor]:
        """Yields qualifying tensors of ``obj`` in priority order."""
        if obj is None or obj is _MISSING:
            return
        if isinstance(obj, torch.Tensor):
            if self.fits(obj):
                yield obj
            return
        if isinstance(obj, (tuple, list)):
            yield from self._walk_sequence(obj)
            return
        for name in _DIRECT_FIELDS:
            yield from self.walk(_field(obj, name))
        stack = _field(obj, _STACK_FIELD)
        if isinstance(stack, torch.Tensor):
            yield from self.walk(stack)
        elif isinstance(stack, (tuple, list)):
            for entry in reversed(stack):  # the last layer's states come last
                yield from self.walk(entry)

    def _walk_sequence(self, items: Sequence[Any]) -> Iterator[torch.Tensor]:
        for item in items:
            if _names_hidden_states(item):
                yield from self.walk(item)
        tensors = [t for t in items if self.fits(t)]
        if len(tensors) == 1:
            yield tensors[0]
        elif tensors:
            top = max(t.ndim for t in tensors)
            deepest = [t for t in tensors if t.ndim == top]
            if len(deepest) == 1:
                yield deepest[0]
        for item in items:
            if not isinstance(item, torch.Tensor) and not _names_hidden_states(item):
                yield from self.walk(item)


def extract_hidden_states(model_output: Any, *, hidden_dim: Optional[int] = None) -> torch.Tensor:
    """The final hidden states in ``model_output`` (see the module docstring for the rules)."""
    for found in _Search(hidden_dim).walk(model_output):
        return found
    want = "" if hidden_dim is None else f" with last dimension {hidden_dim}"
    raise TypeError(f"model output of type {type(model_output).__name__} exposes no hidden-state tensor{want}")


def output_head(model: Any) -> Any:
    """The module that maps hidden states to vocabulary logits: ``model.lm_head``, else what a Hugging Face model
    returns from ``get_output_embeddings()``.  It must have a 2-D ``weight``."""
    head = getattr(model, "lm_head", None)
    if head is None and callable(getattr(model, "get_output_embeddings", None)):
        head = model.get_output_embeddings()
    if head is None or getattr(head, "weight", None) is None or head.weight.ndim != 2:
        raise TypeError(f"{type(model).__name__} exposes no output projection (lm_head / get_output_embeddings())")
    return head


def backbone_hidden_states(model: Any, token_ids: torch.Tensor, *, hidden_dim: Optional[int] = None) -> torch.Tensor:
    """Final hidden states of ``model`` for ``token_ids`` ``[B, S]`` without running its vocabulary projection where
    that can be avoided.

    * A Hugging Face ``...ForCausalLM`` keeps its decoder under ``base_model`` (``model.model``, ``model.transformer``):
      that decoder is called directly (``use_cache=False``), so no ``[B, S, V]`` logits are ever built.
    * Anything else is called as ``model(token_ids)`` and its output searched (``extract_hidden_states``); a model
      that returns logits only is asked again with ``output_hidden_states=True``."""
    base = getattr(model, "base_model", None)
    if isinstance(base, torch.nn.Module) and base is not model and getattr(model, "lm_head", None) is not None:
        try:
            out = base(input_ids=token_ids, use_cache=False)
        except TypeError:                      # an encoder-style backbone has no cache switch
            out = base(input_ids=token_ids)
        return extract_hidden_states(out, hidden_dim=hidden_dim)
    out = model(token_ids)
    try:
        return extract_hidden_states(out, hidden_dim=hidden_dim)
    except TypeError:
        if not hasattr(getattr(model, "config", None), "output_hidden_states"):
            raise
    return extract_hidden_states(model(token_ids, output_hidden_states=True), hidden_dim=hidden_dim)
