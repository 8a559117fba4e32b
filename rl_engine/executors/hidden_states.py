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
