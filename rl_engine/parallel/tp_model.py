"""A whole Llama decoder and GRPO step under tensor + sequence parallelism.

Every rank holds 1/W of each projection (heads / FFN columns), 1/W of the LM head (vocabulary rows) and its own copy
of the small replicated parameters (embedding table, RMSNorm weights).  Activations between the linears are sharded by
token rows (``[T / W, H]``); the layers are ``TensorParallelLlamaLayer`` (fused all-gather -> GEMM and GEMM ->
reduce-scatter kernels), the LM head is the vocabulary-parallel fused ``linear_logp`` whose cross-rank softmax merge
runs inside the GEMM kernel.  The loss is computed redundantly (and identically, bit for bit) on every rank from the
gathered final hidden states, so the gradient of a rank's own rows is just its slice of the hidden-state gradient.

Gradients of the sharded weights are complete on their rank.  Gradients of the replicated parameters are partial sums
over the rank's token rows and are summed over the ranks once per step (one all-reduce over a contiguous slice of the
flat gradient buffer).  Parameters and gradients live in flat buffers, so the optimiser is the same fused AdamW kernel as
on one GPU, run on the local shard: optimiser state is sharded 1/W by construction.

The reference has no tensor-parallel model; the oracle is ``LlamaModel`` + ``GRPOTrainer`` with the full weights.
"""

from __future__ import annotations

from typing import Dict, List, Tuple, Union

import torch
from torch.utils.checkpoint import checkpoint

from rl_engine.models.activation_plan import ActivationPlanner
from rl_engine.models.config import require_no_qkv_bias, require_untied
from rl_engine.models.grpo import GRPOBatch, GRPOTrainer, group_geometry
from rl_engine.models.llama import LlamaModel, rms_norm
from rl_engine.parallel.tp_linear import TensorParallelLinears
from rl_engine.parallel.tp_transformer import TensorParallelLlamaLayer, shard_layer_weights


class _GatherRows(torch.autograd.Function):
    """``[T / W, H]`` local rows -> ``[T, H]`` on every rank.  Backward: every rank already holds the full, identical
    gradient (the loss is replicated), so the local rows' gradient is a slice -- no reduction."""

    @staticmethod
    def forward(ctx, x_local, tp: TensorParallelLinears):
        ctx.rows, ctx.rank = x_local.shape[0], tp.rank
        return tp.all_gather_rows(x_local).clone()

    @staticmethod
    def backward(ctx, grad):
        return grad[ctx.rank * ctx.rows:(ctx.rank + 1) * ctx.rows].contiguous(), None


class TensorParallelLlama:
    """Built from a full ``LlamaModel`` (identical on all ranks); keeps only this rank's shards."""

    def __init__(self, full: LlamaModel, tp: TensorParallelLinears,
                 activation_checkpointing: Union[bool, str] = "auto") -> None:
        cfg = full.cfg
        require_untied(cfg, type(self).__name__)
        require_no_qkv_bias(cfg, type(self).__name__)
        self.cfg, self.tp = cfg, tp
        self.rank, self.world = tp.rank, tp.world
        self._planner = ActivationPlanner(cfg.num_layers, activation_checkpointing)
        # kept per token by a tensor-parallel layer, summed over the ranks: the layer input, both normalised inputs and
        # the mid-layer residual (row shards), qkv, the attention output, gate/up and the SwiGLU output (column shards)
        self._per_token_bytes = full.flat.element_size() * (
            4 * cfg.hidden_size + (cfg.q_dim + 2 * cfg.kv_dim) + cfg.q_dim + 3 * cfg.ffn_size) + 4 * cfg.num_heads + 8
        if cfg.vocab_size % (8 * self.world):
            raise ValueError("vocabulary must divide by 8 * TP size")
        v_local = cfg.vocab_size // self.world
        self.vocab_start = self.rank * v_local
        tensors: List[Tuple[str, torch.Tensor]] = [("embed", full.view("embed").detach()),
                                                   ("final_norm", full.view("final_norm").detach())]
        for i in range(cfg.num_layers):
            for n in ("attn_norm", "mlp_norm"):
                tensors.append((f"l{i}.{n}", full.view(f"l{i}.{n}").detach()))
        self._replicated = len(tensors)
        for i in range(cfg.num_layers):
            shard = shard_layer_weights(full, i, self.rank, self.world)
            for n in ("wqkv", "wo", "w_gate_up", "w_down"):
                tensors.append((f"l{i}.{n}", shard[n]))
        tensors.append(("lm_head", full.view("lm_head").detach()[self.vocab_start:self.vocab_start + v_local]))
        # one flat buffer, replicated parameters first (so that one all-reduce covers their gradients)
        offsets, total = {}, 0
        for name, t in tensors:
            offsets[name] = total
            total += (t.numel() + 127) // 128 * 128
            if name == tensors[self._replicated - 1][0]:
                self._replicated_numel = total
        dev, dtype = full.flat.device, full.flat.dtype
        self.flat = torch.empty(total, dtype=dtype, device=dev)
        self.flat_grad = torch.zeros(total, dtype=dtype, device=dev)
        self.params: Dict[str, torch.nn.Parameter] = {}
        for name, t in tensors:
            view = self.flat[offsets[name]:offsets[name] + t.numel()].view(t.shape)
            view.copy_(t)
            p = torch.nn.Parameter(view, requires_grad=True)
            p.grad = self.flat_grad[offsets[name]:offsets[name] + t.numel()].view(t.shape)
            self.params[name] = p
        self.rope_cos, self.rope_sin = full.rope_cos, full.rope_sin
        self.layers = [
            TensorParallelLlamaLayer(cfg, {n: self.params[f"l{i}.{n}"] for n in
                                           ("attn_norm", "mlp_norm", "wqkv", "wo", "w_gate_up", "w_down")},
                                     tp, self.rope_cos, self.rope_sin)
            for i in range(cfg.num_layers)
        ]

    def ensure_flat_grad(self) -> torch.Tensor:
        return self.flat_grad

    # -- activation memory (a rank holds 1/W of every activation of a layer: rows or columns) ----------
    def plan_checkpointing(self, tokens: int) -> int:
        """Layers kept, agreed by all ranks (the minimum of their plans): a recomputed layer re-runs the fused
        collectives in the backward pass, so every rank has to recompute the same layers."""
        import torch.distributed as dist

        before = self._planner._plan
        layer_input = tokens // self.world * self.cfg.hidden_size * self.flat.element_size()
        keep = self._planner.kept(tokens, tokens * self._per_token_bytes // self.world, layer_input, self.flat.device)
        if self._planner._plan is not before and self.world > 1:  # a new plan was made (on every rank: same tokens)
            agreed = torch.tensor([keep], device=self.flat.device)
            dist.all_reduce(agreed, op=dist.ReduceOp.MIN, group=self.tp.group)
            keep = int(agreed.item())
            self._planner._plan = (tokens, keep)
        return keep

    def estimate_kept_layers(self, tokens: int) -> int:
        """The ranks' minimum of what would fit for ``tokens`` packed tokens (collective: call on every rank)."""
        import torch.distributed as dist

        layer_input = tokens // self.world * self.cfg.hidden_size * self.flat.element_size()
        keep = self._planner.estimate(tokens * self._per_token_bytes // self.world, layer_input, self.flat.device)
        if self.world > 1:
            agreed = torch.tensor([keep], device=self.flat.device)
            dist.all_reduce(agreed, op=dist.ReduceOp.MIN, group=self.tp.group)
            keep = int(agreed.item())
        return keep

    def kept_layers(self) -> int:
        return self._planner.current()

    def reduce_kept_layers(self, by: int = 4) -> int:
        return self._planner.reduce(by)

    # -- forward ------------------------------------------------------------------------------------
    def hidden_states_local(self, token_ids: torch.Tensor, positions: torch.Tensor, layout) -> torch.Tensor:
        """Packed ``token_ids [T]`` -> final-norm hidden states of this rank's rows ``[T / W, H]``."""
        from rl_engine.kernels.registry import kernel_registry

        t = token_ids.numel()
        if t % (128 * self.world):
            raise ValueError(f"{t} packed tokens do not divide into {self.world} shards of 128-row tiles")
        rows = t // self.world
        mine = token_ids[self.rank * rows:(self.rank + 1) * rows]
        x = kernel_registry.get_op("embedding")(mine, self.params["embed"])
        training = torch.is_grad_enabled()
        first_kept = len(self.layers) - (self.plan_checkpointing(t) if training else 0)
        for i, layer in enumerate(self.layers):
            if training and i < first_kept:
                x = checkpoint(layer, x, positions, layout, use_reentrant=False)
            else:
                x = layer(x, positions, layout)
        return rms_norm(x, self.params["final_norm"], self.cfg.rms_eps)

    def policy_logps(self, batch: GRPOBatch) -> torch.Tensor:
        """Selected-token log-probs ``[G, L]`` of the completions; identical bits on every rank."""
        from rl_engine.kernels.registry import kernel_registry

        p, (g, l) = batch.prompt_ids.numel(), batch.completion_ids.shape
        layout, positions, rows = group_geometry(p, g, l, batch.prompt_ids.device)
        tokens = torch.cat([batch.prompt_ids, batch.completion_ids.reshape(-1)])
        hidden = _GatherRows.apply(self.hidden_states_local(tokens, positions, layout), self.tp)
        picked = kernel_registry.get_op("embedding")(rows, hidden)
        logp = kernel_registry.get_op("linear_logp")(
            picked, self.params["lm_head"], batch.completion_ids.reshape(-1), tp_group=self.tp.process_group(),
            vocab_start_index=self.vocab_start, global_vocab_size=self.cfg.vocab_size,
        )
        return logp.reshape(g, l)

    def sync_replicated_grads(self) -> None:
        """Sum the replicated parameters' gradients (partial over token rows) over the ranks."""
        import torch.distributed as dist

        if self.world > 1:
            dist.all_reduce(self.flat_grad[: self._replicated_numel], group=self.tp.group)


class TensorParallelGRPOTrainer(GRPOTrainer):
    """``step(host_batch) -> loss`` with the same contract as ``GRPOTrainer`` (the same batch on every rank).

    Every rank runs the same passes (micro-batch size and kept layers are agreed by the ranks, because a recomputed
    layer re-runs its fused collectives), so an out-of-memory error is not retried here: it is raised."""

    retry_on_out_of_memory = False

    def __init__(self, model: TensorParallelLlama, *, lr: float = 1e-6, clip_eps: float = 0.2, beta: float = 0.04,
                 adv_eps: float = 1e-6, weight_decay: float = 0.0, micro_group="auto") -> None:
        super().__init__(model, lr=lr, clip_eps=clip_eps, beta=beta, adv_eps=adv_eps, weight_decay=weight_decay,
                         micro_group=micro_group)

    def policy_logps(self, batch: GRPOBatch) -> torch.Tensor:
        return self.model.policy_logps(batch)

    def before_optimizer_step(self) -> None:
        self.model.sync_replicated_grads()
