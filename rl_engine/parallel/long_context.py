"""Long-context GRPO step: every sequence is sharded over the ranks (context parallelism), the weights are replicated.

One sequence = shared prompt + one completion (e.g. 4 096 + 32 768 tokens).  Its ``S`` tokens are cut into ``2 W`` chunks
and rank ``r`` holds chunks ``r`` and ``2 W - 1 - r`` (zig-zag, equal causal work per rank).  Everything but attention is
local to a token, so a rank runs the ordinary layers on its ``S / W`` rows; attention goes through
``ContextParallelAttention`` (keys / values exchanged by peer stores over NVLink, gradients of the owned keys / values
summed in rank order).  The selected-token log-probs come from the fused ``linear_logp`` on the local rows: the target of
row ``p`` is token ``p + 1``, which every rank knows because the token ids are replicated.

The G sequences of a group are processed one after the other (gradient accumulation); the loss of a rank's rows is
weighted by ``rows here / rows of the whole group``, so the sum over ranks and sequences is the group's token-mean GRPO
loss.  Parameter gradients are therefore SUMMED over the ranks: the fused reduce-scatter + AdamW + all-gather kernel of the
data-parallel trainer is reused with a scale of 1 instead of 1 / W, including its overlap with the last backward pass.

The reference has no sequence/context parallelism (it only avoids materialising logits and key/value caches:
``rl_engine/executors/stateless_executor.py:93-100``); the oracle is ``GRPOTrainer`` on one GPU with the same batch.
"""

from __future__ import annotations

import contextlib
from typing import Dict

import torch

from rl_engine.models.grpo import GRPOBatch
from rl_engine.models.llama import LlamaModel
from rl_engine.parallel.context_parallel import ContextParallelAttention, shard_sequence
from rl_engine.parallel.data_parallel import ShardedGRPOTrainer


class ContextParallelGRPOTrainer(ShardedGRPOTrainer):
    """``step(host_batch)`` with the same batch on every rank; ``prompt_len + completion_len`` must be a multiple of
    ``2 * world`` (of ``256 * world`` to keep whole attention tiles per chunk)."""

    retry_on_out_of_memory = False  # the ranks would have to agree on the retry; an error is raised instead

    def __init__(self, model: LlamaModel, *, group=None, **kw) -> None:
        kw.setdefault("micro_group", None)
        super().__init__(model, group=group, **kw)
        self.group = group
        self._cp: Dict[int, ContextParallelAttention] = {}
        self.opt.reduce = "sum"  # every rank holds the gradient of ITS rows' share of one loss: sum, not average

    def attention(self, seq_len: int) -> ContextParallelAttention:
        if seq_len not in self._cp:
            self._cp[seq_len] = ContextParallelAttention(seq_len, self.model.cfg.num_kv_heads, self.model.cfg.head_dim,
                                                         group=self.group, device=self.model.flat.device)
        return self._cp[seq_len]

    # -- one sequence -------------------------------------------------------------------------------------
    def sequence_logps(self, tokens: torch.Tensor) -> torch.Tensor:
        """Log-prob of token ``p + 1`` given the sequence up to ``p`` for this rank's rows ``p`` (zig-zag order,
        ``[S / W]``).  The row of the last position predicts nothing and carries a dummy target."""
        from rl_engine.kernels.registry import kernel_registry

        rank, world = self.mem.rank, self.mem.world
        s = tokens.numel()
        cp = self.attention(s)
        positions = shard_sequence(torch.arange(s, device=tokens.device), rank, world)
        local = shard_sequence(tokens, rank, world)
        targets = shard_sequence(torch.cat([tokens[1:], tokens[:1]]), rank, world)
        hidden = self.model.hidden_states(local, positions, cp)
        return kernel_registry.get_op("linear_logp")(hidden, self.model.lm_head_weight(), targets)

    def policy_logps(self, batch: GRPOBatch) -> torch.Tensor:
        """``[G, L]`` log-probs of the completions, gathered from all ranks (collective; for scoring and tests)."""
        import torch.distributed as dist

        from rl_engine.parallel.context_parallel import unshard_sequence

        p, (g, l) = batch.prompt_ids.numel(), batch.completion_ids.shape
        rows = []
        for i in range(g):
            local = self.sequence_logps(torch.cat([batch.prompt_ids, batch.completion_ids[i]]))
            parts = [torch.empty_like(local) for _ in range(self.mem.world)]
            if self.mem.world > 1:
                dist.all_gather(parts, local.detach().contiguous(), group=self.group)
            else:
                parts = [local.detach()]
            rows.append(unshard_sequence(parts)[p - 1 : p - 1 + l])
        return torch.stack(rows)

    def _scatter_completion_values(self, values: torch.Tensor, p: int, s: int, fill: float = 0.0) -> torch.Tensor:
        """Per-completion-token ``values [L]`` placed at the rows that predict those tokens (``p - 1 ...``), this
        rank's rows only."""
        full = torch.full((s,), fill, dtype=values.dtype, device=values.device)
        full[p - 1 : p - 1 + values.numel()] = values
        return shard_sequence(full, self.mem.rank, self.mem.world)

    # -- the step -----------------------------------------------------------------------------------------
    def forward_backward(self, batch: GRPOBatch) -> torch.Tensor:
        from rl_engine.kernels.registry import kernel_registry

        loss_op = kernel_registry.get_op("grpo_loss")
        p, (g, l) = batch.prompt_ids.numel(), batch.completion_ids.shape
        s = p + l
        adv = super(ShardedGRPOTrainer, self).advantages(batch)  # [G], the whole group on every rank
        total_tokens = batch.completion_mask.sum().clamp_min(1).float()
        total = torch.zeros((), dtype=torch.float32, device=batch.completion_ids.device)
        for i in range(g):
            mask = self._scatter_completion_values(batch.completion_mask[i], p, s, fill=False)
            old = self._scatter_completion_values(batch.old_logps[i].float(), p, s)
            ref = self._scatter_completion_values(batch.ref_logps[i].float(), p, s)
            tokens = torch.cat([batch.prompt_ids, batch.completion_ids[i]])
            last = i + 1 == g and self._last_group
            with (self.final_pass() if last else contextlib.nullcontext()):
                logp = self.sequence_logps(tokens)
            loss, _pl, _kl = loss_op.apply_from_logps(logp[None], ref[None], old[None], adv[i : i + 1].contiguous(),
                                                      mask[None], clip_eps=self.clip_eps, beta=self.beta)
            weighted = loss * (mask.sum().float() / total_tokens)
            weighted.backward()
            total += weighted.detach()
        return total

    def step_device(self, batch: GRPOBatch) -> torch.Tensor:
        """Returns the group's token-mean loss (summed over the ranks' shares)."""
        import torch.distributed as dist

        loss = super().step_device(batch)
        if self.mem.world > 1:
            loss = loss.clone()
            dist.all_reduce(loss, group=self.group)
        return loss

    def check(self) -> None:
        super().check()
        for cp in self._cp.values():
            cp.mem.check()
