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
        from rl_engine.models.config import require_untied
        from rl_engine.models.llama import LlamaModel

        if stages > 1:
            require_untied(cfg, type(self).__name__)      # the embedding and the head live on different stages
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


class PipelineGRPOTrainer:
    """One GRPO step of a Llama model cut into pipeline stages: every rank of ``group`` holds one
    ``LlamaPipelineStage`` and the whole prompt group (token ids, rewards, old / reference log-probs are small).

    The group's completions are split into micro-batches of ``micro_group`` completions that each re-process the shared
    prompt; every micro-batch's GRPO loss is weighted by its share of the unmasked tokens, so the step optimises the same
    token-mean loss as ``GRPOTrainer`` on the unsplit model (checked on Gloo ranks).  Advantages come from the whole
    group's rewards.  Every stage then steps its own parameters with the flat AdamW (fp32 masters by default).
    ``step_device`` returns the loss on the last stage and ``None`` elsewhere."""

    def __init__(self, stage: LlamaPipelineStage, *, micro_group: int, group=None, lr: float = 1e-6, clip_eps: float = 0.2,
                 beta: float = 0.04, adv_eps: float = 1e-6, weight_decay: float = 0.0, master_weights: bool = True) -> None:
        from rl_engine.models.grpo import FlatAdamW

        if micro_group < 1:
            raise ValueError("micro_group must be at least one completion")
        self.stage, self.micro_group = stage, int(micro_group)
        self.clip_eps, self.beta, self.adv_eps = clip_eps, beta, adv_eps
        flat = stage.model.flat
        self.schedule = PipelineSchedule(self._stage_fn, group=group, dtype=flat.dtype, device=flat.device)
        self.opt = FlatAdamW(stage.model, lr=lr, weight_decay=weight_decay, master_weights=master_weights)
        self._micro = []  # (batch part, layout, positions, rows, advantages) of the step in flight

    def _stage_fn(self, x, index: int) -> torch.Tensor:
        _part, layout, positions, _rows, _adv = self._micro[index]
        return self.stage.forward(x, positions, layout)

    def _loss_fn(self, hidden: torch.Tensor, index: int) -> torch.Tensor:
        from rl_engine.kernels.registry import kernel_registry

        part, _layout, _positions, rows, adv = self._micro[index]
        picked = kernel_registry.get_op("embedding")(rows, hidden)
        logp = kernel_registry.get_op("linear_logp")(picked, self.stage.model.lm_head_weight(), part.completion_ids.reshape(-1))
        loss, _policy, _kl = kernel_registry.get_op("grpo_loss").apply_from_logps(
            logp.reshape(part.completion_ids.shape), part.ref_logps, part.old_logps, adv, part.completion_mask,
            clip_eps=self.clip_eps, beta=self.beta)
        return loss

    def step_device(self, batch) -> Optional[torch.Tensor]:
        from rl_engine.kernels.registry import kernel_registry
        from rl_engine.models.grpo import group_geometry

        g = batch.completion_ids.shape[0]
        device = batch.completion_ids.device
        adv = kernel_registry.get_op("grpo_loss").group_advantages(batch.rewards.float(), samples_per_prompt=g, eps=self.adv_eps)
        unmasked = float(batch.completion_mask.sum().clamp_min(1))
        self._micro, inputs, weights = [], [], []
        for i0 in range(0, g, self.micro_group):
            part = batch.completions(i0, min(g, i0 + self.micro_group))
            m, l = part.completion_ids.shape
            layout, positions, rows = group_geometry(part.prompt_ids.numel(), m, l, device)
            self._micro.append((part, layout, positions, rows, adv[i0 : i0 + m].contiguous()))
            inputs.append(torch.cat([part.prompt_ids, part.completion_ids.reshape(-1)]))
            weights.append(float(part.completion_mask.sum()) / unmasked)
        self.opt.zero_grad()
        last = self.schedule.stage == self.schedule.stages - 1
        losses = self.schedule.run(inputs, self._loss_fn if last else None, weights)
        self._micro = []
        self.opt.step()
        if not last:
            return None
        return sum(loss * w for loss, w in zip(losses, weights))
