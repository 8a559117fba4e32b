"""``[B, S]`` causal-LM facade over the packed ``LlamaModel``.

Scoring executors, model wrappers and third-party loops call a policy the Hugging Face way:
``model(input_ids=[B, S], attention_mask=[B, S], use_cache=False, output_hidden_states=...)`` and read ``.logits`` or
``.last_hidden_state``.  ``LlamaModel`` works on ONE packed token axis with a layout that says who attends to whom.
``PackedCausalLM`` bridges the two: every row becomes one causal sequence of the packed axis (padding on either side is
dropped from the pack and comes back as zeros), the model runs once over all rows, and the outputs are scattered back to
``[B, S, ...]``.  Nothing is cached between calls (``use_cache=True`` is refused), which is what the stateless
scoring executor wants (reference: ``rl_engine/executors/stateless_executor.py:93-209`` drives HF models this way).
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

import torch
from torch import nn


@dataclass
class CausalLMOutput:
    logits: Optional[torch.Tensor]
    last_hidden_state: torch.Tensor
    hidden_states: Optional[Tuple[torch.Tensor, ...]] = None
    past_key_values: None = None


class _Config:
    """The few ``model.config`` fields that scoring code reads or toggles."""

    def __init__(self, cfg) -> None:
        self.use_cache = False
        self.vocab_size = cfg.vocab_size
        self.hidden_size = cfg.hidden_size
        self.num_hidden_layers = cfg.num_layers
        self._attn_implementation = "model_default"


class PackedCausalLM(nn.Module):
    def __init__(self, model, *, return_logits: bool = True) -> None:
        super().__init__()
        self.model = model
        self.config = _Config(model.cfg)
        self.return_logits = return_logits

    @property
    def lm_head(self):
        """Object with ``.weight`` / ``.bias`` like ``nn.Linear`` (for ``linear_logp`` callers)."""
        head = nn.Module()
        head.weight = self.model.lm_head_weight()
        head.bias = None
        return head

    def forward(self, input_ids: torch.Tensor, attention_mask: Optional[torch.Tensor] = None, use_cache: bool = False,
                output_hidden_states: bool = False, **_unused) -> CausalLMOutput:
        from rl_engine.kernels.ops.sm100.attention import make_layout
        from rl_engine.models.llama import linear

        if use_cache:
            raise ValueError("PackedCausalLM keeps no key/value cache; call it with use_cache=False")
        if input_ids.ndim != 2:
            raise ValueError(f"input_ids must be [B, S], got {tuple(input_ids.shape)}")
        b, s = input_ids.shape
        dev = self.model.flat.device
        ids = input_ids.to(dev).long()
        if attention_mask is None:
            lengths, firsts = [s] * b, [0] * b
        else:
            mask = attention_mask.to(dev).bool()
            lengths = [int(n) for n in mask.long().sum(1).tolist()]
            # a row's tokens must be one contiguous run (right padding, left padding as batched generation produces
            # it, or both); positions count from the first real token, as Hugging Face models do for padded rows
            firsts = [int(f) for f in mask.long().argmax(1).tolist()]
            column = torch.arange(s, device=dev)[None, :]
            first_t, len_t = torch.tensor(firsts, device=dev)[:, None], torch.tensor(lengths, device=dev)[:, None]
            if not torch.equal(mask, (column >= first_t) & (column < first_t + len_t)):
                raise ValueError("attention_mask must select one contiguous run of tokens in every row")
        seqs, starts, cursor = [], [], 0
        for n in lengths:
            starts.append(cursor)
            if n:
                seqs.append((cursor, n, 0, 0, cursor, n))
            cursor += n
        if cursor == 0:
            raise ValueError("attention_mask selects no token")
        layout = make_layout(seqs, True, dev)
        packed = torch.cat([ids[r, firsts[r] : firsts[r] + n] for r, n in enumerate(lengths) if n])
        positions = torch.cat([torch.arange(n, device=dev) for n in lengths if n])
        hidden = self.model.hidden_states(packed, positions, layout)            # [T, H], after the final norm
        out_hidden = hidden.new_zeros(b, s, hidden.shape[-1])
        for r, n in enumerate(lengths):
            if n:
                out_hidden[r, firsts[r] : firsts[r] + n] = hidden[starts[r] : starts[r] + n]
        logits = None
        if self.return_logits:
            flat_logits = linear(hidden, self.model.lm_head_weight())
            logits = flat_logits.new_zeros(b, s, flat_logits.shape[-1])
            for r, n in enumerate(lengths):
                if n:
                    logits[r, firsts[r] : firsts[r] + n] = flat_logits[starts[r] : starts[r] + n]
        return CausalLMOutput(logits=logits, last_hidden_state=out_hidden,
                              hidden_states=(out_hidden,) if output_hidden_states else None)
