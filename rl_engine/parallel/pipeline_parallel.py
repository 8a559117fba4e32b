"""Pipeline parallelism: a one-forward-one-backward (1F1B) schedule over point-to-point messages.

The reference has no pipeline parallelism (only an enum name, ``rl_engine/platforms/constants.py:77``); an 8B model with
its optimiser state fits a 180 GB GPU, so the headline paths of this library are data / tensor / context / expert
parallel and this module is the optional fifth: layers are cut into ``S`` contiguous stages, one rank each, and ``M``
micro-batches flow through them.  Activations go downstream and their gradients upstream as ``torch.distributed``
point-to-point messages (NCCL between GPUs, Gloo between CPU ranks); sends are asynchronous (``isend``), so a stage's
send of micro-batch ``i`` overlaps its compute on micro-batch ``i + 1``.

Schedule of stage ``s`` (``PipelineSchedule.run``): ``min(S - 1 - s, M)`` warm-up forwards, then one forward and one
backward alternately, then the remaining backwards.  At most ``S - s`` micro-batches are alive on a stage, against ``M``
for the fill-drain schedule.  Every stage applies its micro-batches in index order, so gradient accumulation order, and
with it every bit of the result, is fixed.

``LlamaPipelineStage`` cuts a ``LlamaModel`` configuration into stages (embedding on the first, final norm on the last;
the caller's ``loss_fn`` owns the LM head on the last stage) for packed sequences with a caller-supplied layout.

Tested on CPU ranks (Gloo) against the unsplit model: losses and every parameter gradient agree.  Not measured on GPUs.
"""

from __future__ import annotations

from typing import Callable, List, Optional, Sequence

import torch
import torch.distributed as dist

_HEADER = 8  # int64 words: number of dimensions, then the sizes


class PipelineSchedule:
    """``run(micro_inputs, loss_fn)`` on every rank of ``group``; rank ``r`` of the group is stage ``r``.

    ``stage_fn(x, index)``: this stage's layers applied to micro-batch ``index``.  On the first stage ``x`` is
    ``micro_inputs[index]`` (anything the stage understands, e.g. token ids); on the others it is the activation
    received from the stage before, a tensor of ``dtype`` that requires grad.  ``loss_fn(y, index)`` runs on the last
    stage only and returns a scalar; the schedule back-propagates ``loss * weight[index]`` (``weights`` default to
    ``1 / M``).  Returns the list of detached losses on the last stage, ``None`` elsewhere."""

    def __init__(self, stage_fn: Callable, *, group=None, dtype: torch.dtype = torch.bfloat16, device=None) -> None:
        self.stage_fn = stage_fn
        self.group = group
        self.stage = dist.get_rank(group)
        self.stages = dist.get_world_size(group)
        self.dtype = dtype
        self.device = torch.device(device) if device is not None else torch.device("cpu")
        self._pending: List = []  # (work handle, tensor kept alive until the send has completed)

    # -- messages ----------------------------------------------------------------------------------------
    def _global(self, stage: int) -> int:
        return dist.get_global_rank(self.group, stage) if self.group is not None else stage

    def _isend(self, tensor: torch.Tensor, stage: int) -> None:
        t = tensor.contiguous()
        self._pending.append((dist.isend(t, self._global(stage), group=self.group), t))

    def _send_activation(self, y: torch.Tensor) -> None:
        if y.dtype != self.dtype:
            raise TypeError(f"stage output is {y.dtype}, the pipeline was built for {self.dtype}")
        if y.dim() + 1 > _HEADER:
            raise ValueError("activations of more than 7 dimensions are not supported")
        header = torch.zeros(_HEADER, dtype=torch.int64)
        header[0] = y.dim()
        header[1 : 1 + y.dim()] = torch.tensor(list(y.shape), dtype=torch.int64)
        self._isend(header.to(self.device), self.stage + 1)
        self._isend(y.detach(), self.stage + 1)

    def _recv_activation(self) -> torch.Tensor:
        header = torch.zeros(_HEADER, dtype=torch.int64, device=self.device)
        dist.recv(header, self._global(self.stage - 1), group=self.group)
        words = header.tolist()
        shape = [int(v) for v in words[1 : 1 + int(words[0])]]
        x = torch.empty(shape, dtype=self.dtype, device=self.device)
        dist.recv(x, self._global(self.stage - 1), group=self.group)
        return x.requires_grad_(True)

    def _drain(self) -> None:
        for work, _keep in self._pending:
            work.wait()
        self._pending.clear()

    # -- schedule ----------------------------------------------------------------------------------------
    def run(self, micro_inputs: Sequence, loss_fn: Optional[Callable] = None,
            weights: Optional[Sequence[float]] = None) -> Optional[List[torch.Tensor]]:
        m = len(micro_inputs)
        if m == 0:
            raise ValueError("a pipeline step needs at least one micro-batch")
        first, last = self.stage == 0, self.stage == self.stages - 1
        if last and loss_fn is None:
            raise ValueError("the last stage needs loss_fn")
        weights = [1.0 / m] * m if weights is None else [float(w) for w in weights]
        if len(weights) != m:
            raise ValueError("one weight per micro-batch")
        alive = {}   # micro-batch index -> (input activation or None, output tensor or loss)
        losses: List[torch.Tensor] = []

        def forward(i: int) -> None:
            x = micro_inputs[i] if first else self._recv_activation()
            y = self.stage_fn(x, i)
            if last:
                loss = loss_fn(y, i)
                losses.append(loss.detach())
                alive[i] = (None if first else x, loss * weights[i])
            else:
                self._send_activation(y)
                alive[i] = (None if first else x, y)

        def backward(i: int) -> None:
            x, out = alive.pop(i)
            if last:
                out.backward()
            else:
                grad = torch.empty_like(out)
                dist.recv(grad, self._global(self.stage + 1), group=self.group)
                torch.autograd.backward(out, grad)
            if x is not None:
                self._isend(x.grad, self.stage - 1)

        warmup = min(self.stages - 1 - self.stage, m)
        for i in range(warmup):
            forward(i)
        for i in range(m - warmup):
            forward(warmup + i)
            backward(i)
        for i in range(m - warmup, m):
            backward(i)
        self._drain()
        return losses if last else None


def stage_layers(num_layers: int, stages: int) -> List[range]:
    """Contiguous layer ranges, one per stage; the first ``num_layers % stages`` stages hold one layer more."""
    if stages < 1 or num_layers < stages:
        raise ValueError(f"{num_layers} layers cannot be cut into {stages} non-empty stages")
    base, extra = divmod(num_layers, stages)
    out, start = [], 0
    for s in range(stages):
        n = base + (1 if s < extra else 0)
        out.append(range(start, start + n))
        start += n
    return out


class LlamaPipelineStage:
    """Stage ``stage`` of ``stages`` of a ``LlamaModel`` configuration for packed sequences.

    ``model`` is a ``LlamaModel`` built with ``cfg.with_layers(len(self.layers))``: it owns this stage's decoder layers
    (renumbered from 0) plus an embedding and a final norm / LM head, of which only the first stage uses the embedding
    and only the last the final norm and the LM head.  ``load_from(full)`` copies this stage's parameters out of an unsplit
    model (tests, checkpoints).  ``forward(x, positions, layout)``: token ids on the first stage, hidden states
    ``[T, H]`` elsewhere; the last stage returns final-norm hidden states."""

    def __init__(self, cfg, stage: int, stages: int, *, dtype=torch.bfloat16, device="cpu", seed: int = 0, **model_kw) -> None:
        from rl_engine.models.llama import LlamaModel

        self.stage, self.stages = int(stage), int(stages)
        self.layers = stage_layers(cfg.num_layers, stages)[stage]
        self.model = LlamaModel(cfg.with_layers(len(self.layers)), dtype=dtype, device=device, seed=seed + stage, **model_kw)

    @torch.no_grad()
    def load_from(self, full) -> None:
        mine, theirs = self.model.named_views(), full.named_views()
        for name, dst in mine.items():
            if name.startswith("l") and "." in name and name[1 : name.index(".")].isdigit():
                local = int(name[1 : name.index(".")])
                src = theirs[f"l{self.layers[local]}{name[name.index('.'):]}"]
            else:
                src = theirs[name]
            dst.copy_(src)

    def forward(self, x: torch.Tensor, positions: torch.Tensor, layout) -> torch.Tensor:
        from rl_engine.kernels.registry import kernel_registry
        from rl_engine.models.llama import rms_norm

        model = self.model
        if self.stage == 0:
            x = kernel_registry.get_op("embedding")(x, model.view("embed"))
        for i in range(len(self.layers)):
            x = model._layer(x, i, positions, layout)
        if self.stage == self.stages - 1:
            x = rms_norm(x, model.view("final_norm"), model.cfg.rms_eps)
        return x
