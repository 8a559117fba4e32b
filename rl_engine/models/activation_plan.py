"""How many decoder layers keep their activations for the backward pass, and how many are recomputed.

A B200 has 180 GB of HBM3e; after parameters, gradients and optimiser state there is often room for the activations
of many (sometimes all) layers, and every layer that keeps them saves one forward pass of that layer per step.  The
plan is made once per packed length from the free device memory at the first training forward; an out-of-memory
error later lowers it (``reduce``), the trainer then repeats the forward/backward.

The reference has no equivalent: its training worker delegates memory policy to DeepSpeed
(``rl_engine/executors/deepspeed_trainer.py:73-311``).
"""

from __future__ import annotations

from typing import Optional, Tuple, Union

import torch

_NEVER_REPLAN = 1 << 62


class ActivationPlanner:
    """``mode``: ``True`` recompute every layer, ``False`` keep every layer, ``"auto"`` plan from free memory."""

    def __init__(self, layers: int, mode: Union[bool, str] = "auto", headroom_bytes: int = 12 << 30) -> None:
        if mode not in (True, False, "auto"):
            raise ValueError("activation_checkpointing must be True, False or 'auto'")
        self.layers, self.mode, self.headroom = layers, mode, headroom_bytes
        self._plan: Optional[Tuple[int, int]] = None  # (packed tokens the plan was made for, layers kept)

    def estimate(self, per_layer_bytes: int, layer_input_bytes: int, device: torch.device) -> int:
        """Layers that would fit right now (no caching).  The reserve is the inputs of all layers, the transients of
        three layers (one being recomputed plus its backward temporaries) and the head room."""
        if self.mode is True or device.type != "cuda":
            return 0
        if self.mode is False:
            return self.layers
        free, _total = torch.cuda.mem_get_info(device)
        cached = torch.cuda.memory_reserved(device) - torch.cuda.memory_allocated(device)
        per_layer = max(1, per_layer_bytes)
        reserve = self.layers * layer_input_bytes + 3 * per_layer + self.headroom
        return int(max(0, min(self.layers, (free + cached - reserve) // per_layer)))

    def kept(self, tokens: int, per_layer_bytes: int, layer_input_bytes: int, device: torch.device) -> int:
        """Trailing layers that keep their activations.  ``per_layer_bytes``: what autograd holds for one kept layer;
        ``layer_input_bytes``: the input every recomputed layer holds.  Planned once per packed length."""
        if self.mode is True:
            return 0
        if self.mode is False:
            return self.layers
        if self._plan is not None and tokens <= self._plan[0]:
            return self._plan[1]
        if device.type != "cuda":
            return 0
        self._plan = (tokens, self.estimate(per_layer_bytes, layer_input_bytes, device))
        return self._plan[1]

    def current(self) -> int:
        """The number of layers kept by the plan in force (all layers before any plan under ``False``)."""
        if self.mode is True:
            return 0
        if self._plan is not None:
            return self._plan[1]
        return self.layers if self.mode is False else 0

    def reduce(self, by: int = 4) -> int:
        """After an out-of-memory error: recompute ``by`` more layers from now on.  Returns the new number kept."""
        keep = self._plan[1] if self._plan is not None else self.layers
        if self.mode is not True:
            self.mode = "auto"
        self._plan = (_NEVER_REPLAN, max(0, keep - by))
        return self._plan[1]
