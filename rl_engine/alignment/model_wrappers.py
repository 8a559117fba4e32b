"""Adapters that turn "some model" into logits / selected-token log-probs for RL losses.

Parity: reference ``rl_engine/alignment/model_wrappers.py:14-160``: ``extract_logits`` accepts a
tensor, a mapping with ``"logits"``, an object with ``.logits`` or a (possibly loss-first)
tuple/list; ``PolicyModelWrapper.selected_logprobs(..., mask, logits_start, logits_end,
temperature, output_dtype)``; ``ReferenceModelWrapper`` freezes, switches to eval and runs
under ``no_grad``.

Difference: if the wrapped model exposes ``hidden_states_and_head(input_ids, **kw)`` returning
``(hidden, lm_head_weight)`` (the models in ``rl_engine.models`` do), ``selected_logprobs`` goes
through the registry's ``linear_logp`` so ``[B, T, V]`` logits are never materialised.
"""

from __future__ import annotations

from collections.abc import Mapping
from typing import Any, Optional

import torch

from rl_engine.testing import selected_logprobs_reference


def _logits_field(output: Any) -> Any:
    """The ``logits`` member of a mapping or an object, ``None`` when ``output`` has no such member."""
    if isinstance(output, Mapping):
        if "logits" not in output:
            raise TypeError("model output mapping does not contain a 'logits' entry")
        return output["logits"]
    return getattr(output, "logits", None)


def extract_logits(model_output: Any) -> torch.Tensor:
    """The logits tensor inside whatever a model returned.  A worklist walk instead of recursion: containers are
    opened in order, the first tensor with at least two dimensions found inside a container wins (so a scalar loss in
    front of the logits is skipped), and a bare tensor or a ``logits`` member is taken as it is."""
    if isinstance(model_output, torch.Tensor):
        return model_output
    pending, nested, problems = [model_output], False, []
    while pending:
        item = pending.pop(0)
        if isinstance(item, torch.Tensor):
            if not nested or item.ndim >= 2:
                return item
            problems.append(f"a {item.ndim}-d tensor has too few dimensions for logits")
            continue
        if isinstance(item, (tuple, list)):
            pending[:0], nested = list(item), True
            continue
        try:
            field = _logits_field(item)
        except TypeError as exc:
            if not nested:
                raise
            problems.append(str(exc))
            continue
        if field is None:
            problems.append(f"{type(item)!r} does not expose logits")
        elif not isinstance(field, torch.Tensor):
            problems.append(f"the 'logits' member of {type(item)!r} must be a torch.Tensor, got {type(field)!r}")
        elif nested and field.ndim < 2:
            problems.append("a 'logits' member has too few dimensions")
        else:
            return field
    raise TypeError("model output does not contain a logits tensor: " + ("; ".join(problems) or "it is empty"))


def _window(logits: torch.Tensor, start: Optional[int], end: Optional[int]) -> torch.Tensor:
    if start is None and end is None:
        return logits
    if logits.ndim < 2:
        raise ValueError("logits must have at least two dimensions to slice token positions")
    return logits[..., slice(start, end), :]


class PolicyModelWrapper(torch.nn.Module):
    def __init__(self, model: torch.nn.Module):
        super().__init__()
        self.model = model

    def forward(self, input_ids: torch.Tensor, **model_kwargs: Any) -> Any:
        return self.model(input_ids, **model_kwargs)

    def forward_logits(self, input_ids: torch.Tensor, **model_kwargs: Any) -> torch.Tensor:
        return extract_logits(self.forward(input_ids, **model_kwargs))

    def selected_logprobs(
        self,
        input_ids: torch.Tensor,
        token_ids: torch.Tensor,
        *,
        mask: Optional[torch.Tensor] = None,
        logits_start: Optional[int] = None,
        logits_end: Optional[int] = None,
        temperature: float = 1.0,
        output_dtype: torch.dtype = torch.float32,
        **model_kwargs: Any,
    ) -> torch.Tensor:
        fused = getattr(self.model, "hidden_states_and_head", None)
        if callable(fused) and temperature == 1.0:
            from rl_engine.kernels.registry import kernel_registry

            hidden, head = fused(input_ids, **model_kwargs)
            hidden = hidden[..., slice(logits_start, logits_end), :]
            ids = token_ids.long()
            if mask is not None:
                keep = mask.to(torch.bool)
                ids = torch.where(keep, ids, torch.zeros_like(ids))
            logp = kernel_registry.get_op("linear_logp")(hidden, head, ids)
            if mask is not None:
                logp = torch.where(keep, logp, torch.zeros_like(logp))
            return logp.to(output_dtype)
        logits = _window(self.forward_logits(input_ids, **model_kwargs), logits_start, logits_end)
        return selected_logprobs_reference(
            logits, token_ids, mask=mask, temperature=temperature, output_dtype=output_dtype
        )


class ReferenceModelWrapper(PolicyModelWrapper):
    def __init__(self, model: torch.nn.Module, *, freeze: bool = True, eval_mode: bool = True):
        super().__init__(model)
        if freeze:
            self.freeze()
        if eval_mode:
            self.eval()

    def freeze(self) -> "ReferenceModelWrapper":
        for p in self.model.parameters():
            p.requires_grad_(False)
        return self

    @torch.no_grad()
    def forward_logits(self, input_ids: torch.Tensor, **model_kwargs: Any) -> torch.Tensor:
        return super().forward_logits(input_ids, **model_kwargs)

    @torch.no_grad()
    def selected_logprobs(self, input_ids, token_ids, **kwargs: Any) -> torch.Tensor:
        return super().selected_logprobs(input_ids, token_ids, **kwargs)
