"""One GRPO optimisation step on a packed prompt group, end to end.

``GRPOTrainer.step(batch)`` is the public training call: it takes host (pinned) tensors, copies
them to the device, runs forward -> fused ``linear_logp`` -> log-prob-space GRPO loss -> backward
-> fused AdamW, and returns the loss as a Python float (a device-to-host read).  ``step_device``
is the same step on tensors that already live on the device.

The reference's counterpart is ``DeepSpeedTrainingWorker.train``
(``rl_engine/executors/deepspeed_trainer.py:128-202``) on a toy model with DeepSpeed's optimiser.
"""

from __future__ import annotations

import contextlib
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

    def with_safe_ids(self) -> "GRPOBatch":
        """Completion ids at masked positions replaced by 0.  Completion tokens are model inputs as well as targets, and
        padding conventions put -100 or other out-of-vocabulary values there; their loss terms are masked anyway."""
        keep = self.completion_mask.to(torch.bool)
        ids = torch.where(keep, self.completion_ids, torch.zeros_like(self.completion_ids))
        return GRPOBatch(self.prompt_ids, ids, self.rewards, self.old_logps, self.ref_logps, self.completion_mask)

    def completions(self, begin: int, end: int) -> "GRPOBatch":
        """The same prompt with completions ``[begin, end)`` (``rewards`` stay those of the whole group)."""
        return GRPOBatch(self.prompt_ids, self.completion_ids[begin:end].contiguous(), self.rewards,
                         self.old_logps[begin:end].contiguous(), self.ref_logps[begin:end].contiguous(),
                         self.completion_mask[begin:end].contiguous())


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


def split_master(master: torch.Tensor):
    """fp32 ``master`` -> (bf16 parameter, int16 residual) with ``master_bits = (bf16_bits << 16) + residual``.
    The parameter is the master rounded to bf16 (ties away from zero in magnitude), so the pair holds every bit of
    the fp32 value at 2 extra bytes per parameter."""
    bits = master.contiguous().view(torch.int32)
    up = (bits + 0x8000) >> 16  # arithmetic shift keeps the sign bit in place for the narrowing below
    residual = (bits - (up << 16)).to(torch.int16)
    return up.to(torch.int16).view(torch.bfloat16), residual


def join_master(param: torch.Tensor, residual: torch.Tensor) -> torch.Tensor:
    """Inverse of ``split_master``: the fp32 master of a bf16 ``param`` and its int16 ``residual``."""
    bits = (param.contiguous().view(torch.int16).to(torch.int32) << 16) + residual.to(torch.int32)
    return bits.view(torch.float32)


class FlatAdamW:
    """AdamW over one flat parameter buffer; one fused kernel launch per step on the GPU.

    ``master_weights`` (default on): the update is applied to an fp32 master copy and the low-precision parameter is
    its rounding, as DeepSpeed's bf16 optimiser does for the reference (``rl_engine/executors/deepspeed_trainer.py:
    101-126``).  At a learning rate of 1e-6 an update is far below the bf16 spacing of a weight, so without a master
    nearly every update would round away.  For bf16 parameters on the GPU the master is kept as the parameter plus a
    16-bit residual (``split_master``): exact fp32 arithmetic for 2 extra bytes per parameter instead of 4, which is
    what lets an 8 B-parameter model keep all activations on one 180 GB device."""

    def __init__(self, model, lr=1e-6, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.0,
                 master_weights: bool = True) -> None:
        self.model = model
        self.param = model.flat
        self.grad = model.ensure_flat_grad()
        param = self.param
        self.lr, self.betas, self.eps, self.weight_decay = lr, betas, eps, weight_decay
        self.m = torch.zeros(param.numel(), dtype=torch.float32, device=param.device)
        self.v = torch.zeros(param.numel(), dtype=torch.float32, device=param.device)
        self.grad_scale = 1.0  # multiplies the accumulated gradient in ``step`` (1 / number of accumulated groups)
        self.master: Optional[torch.Tensor] = None     # fp32 master (CPU, or parameters that are not bf16)
        self.residual: Optional[torch.Tensor] = None   # int16 residuals of a bf16 parameter (GPU)
        if master_weights and param.dtype != torch.float32:
            if param.is_cuda and param.dtype == torch.bfloat16:
                self.residual = torch.zeros(param.numel(), dtype=torch.int16, device=param.device)
            else:
                self.master = param.detach().float().clone()
        self.steps = 0

    @property
    def has_master(self) -> bool:
        return self.master is not None or self.residual is not None

    def master_weights(self) -> torch.Tensor:
        """The fp32 values the optimiser works on (a copy when they are stored in split form)."""
        if self.residual is not None:
            return join_master(self.param.detach(), self.residual)
        return self.master if self.master is not None else self.param.detach().float()

    def zero_grad(self) -> None:
        self.grad.zero_()

    def _tie_gradients(self) -> None:
        """Tied embeddings: the embedding and the LM head are one matrix, so each gets the sum of both gradients.
        They start equal and see the same update from the same optimiser state, hence stay equal bit for bit."""
        cfg = getattr(self.model, "cfg", None)
        if cfg is None or not getattr(cfg, "tie_word_embeddings", False):
            return
        g_embed = self.model._slice(self.grad, "embed")
        g_head = self.model._slice(self.grad, "lm_head")
        g_embed.add_(g_head)
        g_head.copy_(g_embed)

    @torch.no_grad()
    def step(self, grad_scale: Optional[float] = None) -> None:
        grad_scale = self.grad_scale if grad_scale is None else float(grad_scale)
        self._tie_gradients()
        self.steps += 1
        p, g = self.param, self.grad
        if p.is_cuda:
            from rl_engine.kernels.ops.base import require_ext

            state = self.residual if self.residual is not None else self.master
            require_ext().adamw(p, state, g, self.m, self.v, self.lr, self.betas[0], self.betas[1], self.eps,
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
        """Tensors and ints only.  The master is saved in the form it is held in: ``master`` (fp32) or
        ``master_residual`` (int16, to be joined with the saved bf16 parameters), so saving allocates nothing large."""
        return {"m": self.m, "v": self.v, "master": self.master, "master_residual": self.residual, "steps": self.steps}

    accepts_resharded_state = True

    def load_state_dict(self, state) -> None:
        """Call after the parameters have been restored.  A checkpoint without a master re-seeds the master from
        the loaded parameters instead of keeping the values it had before.  ``state`` may be an
        ``OptimizerShardReader`` (a checkpoint written by several data-parallel ranks): the whole vectors are then
        gathered from the shards."""
        if hasattr(state, "read"):
            n = self.param.numel()
            if state.numel > (n + 7) // 8 * 8:
                raise ValueError(f"the checkpoint's optimizer state covers {state.numel} elements, this model has {n}")
            state = {"m": state.read("m", 0, n), "v": state.read("v", 0, n), "steps": state.steps,
                     "master": state.read("master", 0, n) if state.has("master") else None,
                     "master_residual": state.read("master_residual", 0, n) if state.has("master_residual") else None}
        self.m.copy_(state["m"])
        self.v.copy_(state["v"])
        self.steps = int(state["steps"])
        if not self.has_master:
            return
        saved, saved_residual = state.get("master"), state.get("master_residual")
        if self.residual is not None:
            if saved_residual is not None:      # same form: the restored parameters already are the rounded master
                self.residual.copy_(saved_residual)
            elif saved is not None:
                param, residual = split_master(saved.to(self.param.device, torch.float32))
                self.param.copy_(param)
                self.residual.copy_(residual)
            else:
                self.residual.zero_()           # master == loaded parameters
            return
        if saved is not None:
            master = saved.to(self.param.device, torch.float32)
        elif saved_residual is not None:
            master = join_master(self.param.detach(), saved_residual.to(self.param.device))
        else:
            master = self.param.detach().float()
        self.master.copy_(master)
        self.param.copy_(master.to(self.param.dtype))


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


def suffix_geometry(p: int, m: int, l: int, device):
    """Geometry of a pass that holds ``m`` completions of ``l`` tokens after a cached prompt of ``p`` tokens:
    (layout with queries in the pass's rows and keys in ``[prompt | pass]``, positions ``[m * l]``, for every
    completion token the row of ``[last prompt state | pass states]`` that predicts it ``[m * l]``)."""
    key = ("suffix", p, m, l, str(device))
    hit = _GEOMETRY.get(key)
    if hit is None:
        from rl_engine.kernels.ops.sm100.attention import make_layout

        layout = make_layout([(i * l, l, 0, p, p + i * l, l) for i in range(m)], True, device)
        positions = (p + torch.arange(l)).repeat(m).to(device)
        rows = torch.arange(m)[:, None] * l + torch.arange(l)[None, :]  # 1 + (i * l + j - 1)
        rows[:, 0] = 0                                                   # the prompt's last state
        if len(_GEOMETRY) > 32:
            _GEOMETRY.clear()
        hit = _GEOMETRY[key] = (layout, positions, rows.reshape(-1).to(device))
    return hit


def policy_logps_after_prefix(model: LlamaModel, batch: "GRPOBatch", last_state: torch.Tensor, kv) -> torch.Tensor:
    """``policy_logps`` for completions whose prompt was processed by ``model.prefix_states`` (``last_state``, ``kv``):
    same kernels and per-row arithmetic as the single pass, without re-processing the prompt."""
    from rl_engine.kernels.registry import kernel_registry

    p, (m, l) = batch.prompt_ids.numel(), batch.completion_ids.shape
    layout, positions, rows = suffix_geometry(p, m, l, batch.prompt_ids.device)
    hidden = model.hidden_states_after_prefix(batch.completion_ids.reshape(-1), positions, layout, kv)
    picked = kernel_registry.get_op("embedding")(rows, torch.cat([last_state, hidden]))
    logp = kernel_registry.get_op("linear_logp")(picked, model.lm_head_weight(), batch.completion_ids.reshape(-1))
    return logp.reshape(m, l)


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


def choose_micro_group(group: int, prompt_len: int, completion_len: int, layers: int, kept_for_tokens,
                       prompt_once: bool = False) -> int:
    """Completions per forward/backward pass that minimise the step's compute.

    Splitting the group into micro-batches re-processes the shared prompt once per micro-batch, but the smaller
    packed length lets more layers keep their activations, which saves their recomputation (a third of a layer's
    forward + backward work).  Cost model per candidate ``m`` (``group``, ``group / 2``, ... while even and the packed
    length stays above 4096 tokens): ``(group / m) * (prompt + m * completion) * (3 + recomputed / layers)``.
    ``kept_for_tokens(tokens)`` answers how many layers could keep their activations at that packed length.  With
    ``prompt_once`` the micro-batches attend to cached prompt keys / values: the prompt costs one extra pass of its own
    instead of one per micro-batch."""
    best, best_cost = group, None
    m = group
    while m >= 1:
        split_prompt = prompt_once and m != group  # the prompt is its own pass; micro-batches hold completions only
        tokens = m * completion_len + (0 if split_prompt else prompt_len)
        if m != group and tokens < 4096:
            break
        kept = min(layers, max(0, int(kept_for_tokens(tokens))))
        cost = (group // m) * tokens * (3.0 + (layers - kept) / max(1, layers)) + (3.0 * prompt_len if split_prompt else 0)
        if best_cost is None or cost < best_cost * 0.98:  # a smaller micro-batch has to pay for its extra launches
            best, best_cost = m, cost
        if m % 2:
            break
        m //= 2
    return best


class _PromptPass:
    """The shared prompt, processed once per step.  Micro-batches read its last hidden state and per-layer keys /
    values through fp32 leaves, which collect their gradients; ``backward`` then back-propagates the sums through the
    prompt pass once."""

    def __init__(self, model: LlamaModel, prompt_ids: torch.Tensor, **sharding) -> None:
        self.last_state, self.kv = model.prefix_states(prompt_ids, **sharding)
        leaf = lambda t: t.detach().float().requires_grad_(True)
        self.last_leaf = leaf(self.last_state)
        self.kv_leaves = [(leaf(k), leaf(v)) for k, v in self.kv]

    def inputs(self):
        dtype = self.last_state.dtype
        return self.last_leaf.to(dtype), [(k.to(dtype), v.to(dtype)) for k, v in self.kv_leaves]

    def backward(self) -> None:
        outputs, grads = [self.last_state], [self.last_leaf.grad]
        for (k, v), (k_leaf, v_leaf) in zip(self.kv, self.kv_leaves):
            outputs += [k, v]
            grads += [k_leaf.grad, v_leaf.grad]
        keep = [(o, g.to(o.dtype)) for o, g in zip(outputs, grads) if g is not None]
        torch.autograd.backward([o for o, _ in keep], [g for _, g in keep])


class GRPOTrainer:
    """``micro_group``: completions per forward/backward pass.  ``None`` runs the whole group in one pass, an integer
    fixes it, ``"auto"`` (default) picks it at the first step with ``choose_micro_group``.  Gradients of the
    micro-batches accumulate in the flat gradient buffer; each micro-batch's loss is weighted by its share of the
    unmasked tokens, so the step optimises the same token-mean loss as a single pass."""

    retry_on_out_of_memory = True
    # Optional ``rl_engine.parallel.liveness.RankLiveness``: checked on the host at the start of every step, before
    # anything is launched, so that a step whose peers have left raises ``RankLeftError`` instead of waiting on them.
    liveness = None
    _steps_started = 0
    cache_prompt = True  # micro-batches attend to the prompt's cached keys / values instead of re-processing it
    _last_group = True   # False while ``step_groups`` is accumulating a group that is not the step's last one

    def __init__(self, model: LlamaModel, *, lr: float = 1e-6, clip_eps: float = 0.2, beta: float = 0.04,
                 adv_eps: float = 1e-6, weight_decay: float = 0.0, master_weights: bool = True,
                 micro_group="auto") -> None:
        self.model = model
        self.clip_eps, self.beta, self.adv_eps = clip_eps, beta, adv_eps
        self.micro_group = micro_group
        self._micro_choice: Dict[tuple, int] = {}
        self.opt = FlatAdamW(model, lr=lr, weight_decay=weight_decay, master_weights=master_weights)

    def policy_logps(self, batch: GRPOBatch) -> torch.Tensor:
        return policy_logps(self.model, batch)

    def advantages(self, batch: GRPOBatch) -> torch.Tensor:
        """Group-normalised advantage of each completion of ``batch`` (``[G]``)."""
        from rl_engine.kernels.registry import kernel_registry

        op = kernel_registry.get_op("grpo_loss")
        return op.group_advantages(batch.rewards.float(), samples_per_prompt=batch.rewards.numel(), eps=self.adv_eps)

    def loss_with_advantages(self, batch: GRPOBatch, adv: torch.Tensor, prefix: Optional["_PromptPass"] = None):
        from rl_engine.kernels.registry import kernel_registry

        if prefix is None:
            logp = self.policy_logps(batch)
        else:
            logp = policy_logps_after_prefix(self.model, batch, *prefix.inputs())
        return kernel_registry.get_op("grpo_loss").apply_from_logps(
            logp, batch.ref_logps, batch.old_logps, adv, batch.completion_mask, clip_eps=self.clip_eps, beta=self.beta
        )

    def loss(self, batch: GRPOBatch):
        return self.loss_with_advantages(batch, self.advantages(batch))

    def completions_per_pass(self, batch: GRPOBatch) -> int:
        g, l = batch.completion_ids.shape
        if self.micro_group is None:
            return g
        if isinstance(self.micro_group, int):
            return max(1, min(g, self.micro_group))
        key = (g, l, batch.prompt_ids.numel())
        if key not in self._micro_choice:
            estimate = getattr(self.model, "estimate_kept_layers", None)
            layers = self.model.cfg.num_layers
            supported = getattr(self.model, "supports_prefix_cache", None)
            once = bool(self.cache_prompt and supported is not None and supported())
            self._micro_choice[key] = (g if estimate is None
                                       else choose_micro_group(g, key[2], l, layers, estimate, prompt_once=once))
        return self._micro_choice[key]

    def forward_backward(self, batch: GRPOBatch) -> torch.Tensor:
        """Accumulates the gradient of the group's token-mean loss into the flat gradient buffer; returns the loss."""
        g = batch.completion_ids.shape[0]
        m = self.completions_per_pass(batch)
        if m >= g and not self.force_prompt_pass(batch):
            with self.final_pass():
                loss, _pl, _kl = self.loss(batch)
            loss.backward()
            return loss.detach()
        adv = self.advantages(batch)
        unmasked = batch.completion_mask.sum().clamp_min(1).float()
        total = torch.zeros((), dtype=torch.float32, device=batch.completion_ids.device)
        with self.final_pass():  # the prompt's backward pass runs after those of all micro-batches
            prefix = self.prompt_pass(batch)
        for i0 in range(0, g, m):
            part = batch.completions(i0, min(g, i0 + m))
            last_without_prefix = prefix is None and i0 + m >= g
            with (self.final_pass() if last_without_prefix else contextlib.nullcontext()):
                loss, _pl, _kl = self.loss_with_advantages(part, adv[i0:i0 + m].contiguous(), prefix)
            weighted = loss * (part.completion_mask.sum().float() / unmasked)
            weighted.backward()
            total += weighted.detach()
        if prefix is not None:
            prefix.backward()
        return total

    def prompt_pass(self, batch: GRPOBatch) -> Optional["_PromptPass"]:
        """Runs the shared prompt once for all micro-batches if the model supports prefix-cached passes."""
        if not self.prompt_cacheable(batch):
            return None
        return _PromptPass(self.model, batch.prompt_ids)

    def force_prompt_pass(self, batch: GRPOBatch) -> bool:
        """True if the prompt-pass route is to be taken even though the whole group fits in one pass."""
        return False

    def prompt_cacheable(self, batch: GRPOBatch) -> bool:
        supported = getattr(self.model, "supports_prefix_cache", None)
        return bool(self.cache_prompt and supported is not None and supported())

    def final_pass(self):
        """Context manager around the FORWARD of the pass whose backward runs last in the step.  A trainer that
        overlaps its gradient exchange with that backward pass hooks in here; the plain trainer does nothing."""
        return contextlib.nullcontext()

    def before_optimizer_step(self) -> None:
        """Hook for trainers whose gradients need a reduction that the optimiser kernel does not do."""

    def step_device(self, batch: GRPOBatch) -> torch.Tensor:
        """Forward, backward and optimiser step.  If the kept activations do not fit after all (the plan of
        ``LlamaModel.plan_checkpointing`` is an estimate), the forward/backward is repeated with four more layers
        recomputed; nothing has been applied to the parameters at that point."""
        if self.liveness is not None:
            self.liveness.check(self._steps_started)
        self._steps_started += 1
        batch = batch.with_safe_ids()
        while True:
            self.opt.zero_grad()
            try:
                loss = self.forward_backward(batch)
                break
            except torch.cuda.OutOfMemoryError:
                applied = getattr(self.opt, "_launched", None)  # buckets an overlapped optimiser has already applied
                if (not self.retry_on_out_of_memory or not hasattr(self.model, "kept_layers")
                        or self.model.kept_layers() == 0 or (applied and any(applied))):
                    raise
            torch.cuda.empty_cache()
            self.model.reduce_kept_layers(4)
        self.before_optimizer_step()
        self.opt.step()
        return loss

    def step_groups(self, batches) -> torch.Tensor:
        """One optimiser step on several prompt groups (a sequence of device ``GRPOBatch``): the gradient is the mean
        over the groups of each group's token-mean loss.  Returns that mean loss.  No out-of-memory retry here."""
        batches = [b.with_safe_ids() for b in batches]
        if not batches:
            raise ValueError("step_groups needs at least one prompt group")
        self.opt.zero_grad()
        self.opt.grad_scale = 1.0 / len(batches)
        total = None
        try:
            for i, batch in enumerate(batches):
                self._last_group = i + 1 == len(batches)
                loss = self.forward_backward(batch)
                total = loss if total is None else total + loss
            self.before_optimizer_step()
            self.opt.step()
        finally:
            self._last_group = True
            self.opt.grad_scale = 1.0
        return total / len(batches)

    def step(self, host_batch: GRPOBatch) -> float:
        """Public end-to-end step: host (pinned) batch in, loss value out."""
        device = self.model.flat.device
        return float(self.step_device(host_batch.to(device)).item())
