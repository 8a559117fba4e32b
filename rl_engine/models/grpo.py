"""One GRPO optimisation step on a packed prompt group, end to end.

``GRPOTrainer.step(batch)`` is the public training call: it takes host (pinned) tensors, copies
them to the device, runs forward -> fused ``linear_logp`` -> log-prob-space GRPO loss -> backward
-> fused AdamW, and returns the loss as a Python float (a device-to-host read).  ``step_device``
is the same step on tensors that already live on the device.

The reference's counterpart is ``DeepSpeedTrainingWorker.train``
(``rl_engine/executors/deepspeed_trainer.py:128-202``) on a toy model with DeepSpeed's optimiser.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Optional

import torch

from rl_engine.models.llama import LlamaModel


@dataclass
class GRPOBatch:
    """One prompt group.  ``completion_ids [G, L]``, ``prompt_ids [P]``, ``rewards [G]``,
    ``old_logps`` / ``ref_logps`` ``[G, L]`` (float32), ``completion_mask [G, L]`` (bool)."""

    prompt_ids: torch.Tensor
    completion_ids: torch.Tensor
    rewards: torch.Tensor
    old_logps: torch.Tensor
    ref_logps: torch.Tensor
    completion_mask: torch.Tensor

    def to(self, device, non_blocking: bool = True) -> "GRPOBatch":
        return GRPOBatch(*(t.to(device, non_blocking=non_blocking) for t in self.tensors()))

    def pin(self) -> "GRPOBatch":
        return GRPOBatch(*(t.pin_memory() for t in self.tensors()))

    def tensors(self):
        return (self.prompt_ids, self.completion_ids, self.rewards, self.old_logps, self.ref_logps, self.completion_mask)

    def nbytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in self.tensors())


def synthetic_batch(vocab: int, prompt_len: int, group: int, completion_len: int, seed: int = 0) -> GRPOBatch:
    """Seeded host batch: uniform token ids, N(0,1) rewards, old/ref = N(-2, 0.1) placeholders."""
    g = torch.Generator().manual_seed(seed)
    return GRPOBatch(
        prompt_ids=torch.randint(0, vocab, (prompt_len,), generator=g),
        completion_ids=torch.randint(0, vocab, (group, completion_len), generator=g),
        rewards=torch.randn(group, generator=g),
        old_logps=torch.zeros(group, completion_len),
        ref_logps=torch.zeros(group, completion_len),
        completion_mask=torch.ones(group, completion_len, dtype=torch.bool),
    )


class FlatAdamW:
    """AdamW over one flat parameter buffer; one fused kernel launch per step on the GPU."""

    def __init__(self, model, lr=1e-6, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.0,
                 master_weights: bool = False) -> None:
        self.model = model
        self.param = model.flat
        self.grad = model.ensure_flat_grad()
        param = self.param
        self.lr, self.betas, self.eps, self.weight_decay = lr, betas, eps, weight_decay
        self.m = torch.zeros(param.numel(), dtype=torch.float32, device=param.device)
        self.v = torch.zeros(param.numel(), dtype=torch.float32, device=param.device)
        self.master = param.detach().float().clone() if master_weights else None
        self.steps = 0

    def zero_grad(self) -> None:
        self.grad.zero_()

    @torch.no_grad()
    def step(self, grad_scale: float = 1.0) -> None:
        self.steps += 1
        p, g = self.param, self.grad
        if p.is_cuda:
            from rl_engine.kernels.ops.base import require_ext

            require_ext().adamw(p, self.master, g, self.m, self.v, self.lr, self.betas[0], self.betas[1], self.eps,
                                self.weight_decay, self.steps, grad_scale)
            return
        b1, b2 = self.betas
        gf = g.float() * grad_scale
        self.m.mul_(b1).add_(gf, alpha=1 - b1)
        self.v.mul_(b2).addcmul_(gf, gf, value=1 - b2)
        w = p.float() if self.master is None else self.master
        denom = (self.v / (1 - b2**self.steps)).sqrt_().add_(self.eps)
        w = w * (1 - self.lr * self.weight_decay) - self.lr * (self.m / (1 - b1**self.steps)) / denom
        if self.master is not None:
            self.master.copy_(w)
        p.copy_(w.to(p.dtype))

    def state_dict(self) -> Dict[str, object]:
        return {"m": self.m, "v": self.v, "master": self.master, "steps": self.steps}

    def load_state_dict(self, state: Dict[str, object]) -> None:
        self.m.copy_(state["m"])
        self.v.copy_(state["v"])
        if self.master is not None and state.get("master") is not None:
            self.master.copy_(state["master"])
        self.steps = int(state["steps"])


_GEOMETRY: Dict[tuple, tuple] = {}


def group_geometry(p: int, g: int, l: int, device):
    """(packed layout, positions [P + G*L], hidden row predicting each completion token [G*L])."""
    key = (p, g, l, str(device))
    hit = _GEOMETRY.get(key)
    if hit is None:
        from rl_engine.kernels.ops.sm100.attention import grpo_group_layout

        layout = grpo_group_layout(p, g, l, device)
        positions = torch.cat([torch.arange(p), (p + torch.arange(l)).repeat(g)]).to(device)
        rows = p + torch.arange(g)[:, None] * l + torch.arange(l)[None, :] - 1  # the token before (g, i)
        rows[:, 0] = p - 1
        if len(_GEOMETRY) > 32:
            _GEOMETRY.clear()
        hit = _GEOMETRY[key] = (layout, positions, rows.reshape(-1).to(device))
    return hit


def policy_logps(model: LlamaModel, batch: "GRPOBatch") -> torch.Tensor:
    """Selected-token log-probs ``[G, L]`` of the completions under ``model`` (differentiable).

    Used by the trainer and by the native rollout engine, so both paths run the same kernels in the
    same order: their log-probs for the same tokens and weights agree bitwise."""
    from rl_engine.kernels.registry import kernel_registry

    p, (g, l) = batch.prompt_ids.numel(), batch.completion_ids.shape
    layout, positions, rows = group_geometry(p, g, l, batch.prompt_ids.device)
    tokens = torch.cat([batch.prompt_ids, batch.completion_ids.reshape(-1)])
    hidden = model.hidden_states(tokens, positions, layout)
    # deterministic differentiable row gather (ordered segment sums in backward, no atomics)
    picked = kernel_registry.get_op("embedding")(rows, hidden)
    logp = kernel_registry.get_op("linear_logp")(picked, model.lm_head_weight(), batch.completion_ids.reshape(-1))
    return logp.reshape(g, l)


class GRPOTrainer:
    def __init__(self, model: LlamaModel, *, lr: float = 1e-6, clip_eps: float = 0.2, beta: float = 0.04,
                 adv_eps: float = 1e-6, weight_decay: float = 0.0, master_weights: bool = False) -> None:
        self.model = model
        self.clip_eps, self.beta, self.adv_eps = clip_eps, beta, adv_eps
        self.opt = FlatAdamW(model, lr=lr, weight_decay=weight_decay, master_weights=master_weights)

    def policy_logps(self, batch: GRPOBatch) -> torch.Tensor:
        return policy_logps(self.model, batch)

    def loss(self, batch: GRPOBatch):
        from rl_engine.kernels.registry import kernel_registry

        op = kernel_registry.get_op("grpo_loss")
        adv = op.group_advantages(batch.rewards.float(), samples_per_prompt=batch.rewards.numel(), eps=self.adv_eps)
        logp = self.policy_logps(batch)
        return op.apply_from_logps(
            logp, batch.ref_logps, batch.old_logps, adv, batch.completion_mask, clip_eps=self.clip_eps, beta=self.beta
        )

    def step_device(self, batch: GRPOBatch) -> torch.Tensor:
        """Forward, backward and optimiser step.  If the kept activations do not fit after all (the plan of
        ``LlamaModel.plan_checkpointing`` is an estimate), the forward/backward is repeated with four more layers
        recomputed; nothing has been applied to the parameters at that point."""
        while True:
            self.opt.zero_grad()
            loss = None
            try:
                loss, _pl, _kl = self.loss(batch)
                loss.backward()
                break
            except torch.cuda.OutOfMemoryError:
                if not hasattr(self.model, "kept_layers") or self.model.kept_layers() == 0:
                    raise
            loss = None
            torch.cuda.empty_cache()
            self.model.reduce_kept_layers(4)
        self.opt.step()
        return loss.detach()

    def step(self, host_batch: GRPOBatch) -> float:
        """Public end-to-end step: host (pinned) batch in, loss value out."""
        device = self.model.flat.device
        return float(self.step_device(host_batch.to(device)).item())
