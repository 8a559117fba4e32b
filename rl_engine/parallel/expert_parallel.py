"""Expert parallelism for the MoE FFN over peer-mapped symmetric memory.

Each of the ``W`` ranks keeps ``E / W`` experts and its own tokens (data parallel activations).
Dispatch and combine are not NCCL all-to-alls: the dispatch kernel stores every routed row straight
into the owning rank's slot buffer over NVLink (``moe_scatter_rows_peer``) and the combine kernel reads
the expert outputs back out of the peers' buffers (``moe_combine_peer``).  The per-expert assignment
counts travel the same way (every rank stores its ``E`` counts into row ``rank`` of a ``[W, E]`` table in
each peer's segment, double-buffered, one device barrier), and from that table every rank derives the
same slot layout; no library collective runs in the layer:

    owner(e) = e // (E / W)
    on the owner, expert e's block is padded to a multiple of 128 rows (at least 128) and holds the
    assignments ordered by (source rank, assignment id)

so every summation order (expert GEMMs, weight gradients, the k-term combine) is fixed: forward and
backward are run-to-run reproducible.

Buffer reuse is guarded by the device-side peer barrier (bounded waits; a rank that never arrives
surfaces as ``PeerTimeoutError`` from ``SymmetricMemory.check``), three per direction:

    zero recv | barrier | scatter rows to the owners | barrier | experts | publish y | barrier | combine

The reference has no MoE or expert-parallel component; the numerics oracle is the single-rank
``NativeMoEOp`` evaluated on the gathered tokens with all experts.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from rl_engine.kernels.ops.base import require_ext
from rl_engine.kernels.ops.sm100.moe import BLOCK, _RouterLogits, route_topk
from rl_engine.parallel.symmetric import SymmetricMemory


@dataclass
class EPPlan:
    dest_rank: torch.Tensor    # int32 [T*k]  owner rank of every assignment
    dest_slot: torch.Tensor    # int32 [T*k]  row in the owner's slot buffer
    token: torch.Tensor        # int32 [T*k]  source token of every assignment
    tile_group: torch.Tensor   # int32 [S/128] local expert of each tile of MY slot buffer, -1 = unused tile
    offsets: torch.Tensor      # int32 [El+1]  padded slot offsets of MY experts
    used_slots: torch.Tensor   # int64 []      slots in use on this rank (device scalar)
    top_k: int
    rows: int = 0              # ``used_slots`` on the host (a multiple of 128) once ``ExpertParallelContext.plan`` read it


def build_ep_plan(expert_idx: torch.Tensor, all_counts: torch.Tensor, rank: int, world: int, num_slots: int) -> EPPlan:
    """Slot layout shared by all ranks. ``all_counts`` int64 ``[W, E]`` = assignments per (source rank, expert)."""
    t, k = expert_idx.shape
    dev = expert_idx.device
    e = all_counts.shape[1]
    el = e // world
    total = all_counts.sum(0)                                           # [E]
    padded = torch.clamp((total + BLOCK - 1) // BLOCK, min=1) * BLOCK
    per_owner = padded.view(world, el)
    off_in_owner = (per_owner.cumsum(1) - per_owner).reshape(-1)        # [E] offset of expert e on its owner
    before_me = all_counts[:rank].sum(0) if rank else torch.zeros_like(total)
    base = off_in_owner + before_me                                     # first slot of MY assignments for e
    flat = expert_idx.reshape(-1).long()
    order = torch.argsort(flat, stable=True)
    mine = all_counts[rank]
    starts = mine.cumsum(0) - mine
    sorted_e = flat[order]
    rank_in = torch.arange(t * k, device=dev) - starts[sorted_e]
    dest_slot = torch.empty(t * k, dtype=torch.int32, device=dev)
    dest_slot[order] = (base[sorted_e] + rank_in).to(torch.int32)
    dest_rank = (flat // el).to(torch.int32)
    token = (torch.arange(t * k, device=dev) // k).to(torch.int32)
    my = per_owner[rank]
    offsets = torch.zeros(el + 1, dtype=torch.long, device=dev)
    offsets[1:] = my.cumsum(0)
    tile_start = torch.arange(num_slots // BLOCK, device=dev) * BLOCK
    tile_group = torch.searchsorted(offsets[1:].contiguous(), tile_start, right=True)
    tile_group = torch.where(tile_group >= el, torch.full_like(tile_group, -1), tile_group)  # unused tail: skipped
    return EPPlan(dest_rank, dest_slot, token, tile_group.to(torch.int32), offsets.to(torch.int32), offsets[-1], k)


class ExpertParallelContext:
    """Symmetric buffers + exchange primitives shared by every MoE layer of a model."""

    def __init__(self, hidden: int, num_experts: int, top_k: int, max_tokens: int, group=None,
                 mem: Optional[SymmetricMemory] = None, device: Optional[torch.device] = None,
                 capacity_factor: Optional[float] = None) -> None:
        import torch.distributed as dist

        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        if num_experts % self.world:
            raise ValueError(f"{num_experts} experts do not divide over {self.world} ranks")
        self.hidden, self.num_experts, self.top_k = hidden, num_experts, top_k
        self.local_experts = num_experts // self.world
        factor = float(self.world) if capacity_factor is None else float(capacity_factor)
        rows = int(factor * max_tokens * top_k) + self.local_experts * BLOCK
        self.num_slots = (rows + BLOCK - 1) // BLOCK * BLOCK
        self.worst_case = factor >= self.world
        self.max_tokens = max_tokens
        nbytes = 2 * self.num_slots * hidden * 2 + 2 * self.world * num_experts * 4 + (1 << 20)
        self.mem = mem if mem is not None else SymmetricMemory(nbytes, group=group, device=device)
        self.recv = self.mem.alloc((self.num_slots, hidden), torch.bfloat16)
        self.send = self.mem.alloc((self.num_slots, hidden), torch.bfloat16)
        # int32 counts moved as raw 32-bit words (the copy kernel does no arithmetic when source and destination
        # types match).  Two tables used alternately: a rank can be at most one exchange ahead of a peer, so the
        # table it overwrites was read by everybody before the barrier of the exchange in between.
        self._counts = [self.mem.alloc((self.world, num_experts), torch.float32) for _ in range(2)]
        self._count_turn = 0

    # -- plan ---------------------------------------------------------------------------------------
    def plan(self, expert_idx: torch.Tensor) -> EPPlan:
        if expert_idx.shape[0] > self.max_tokens:
            raise ValueError(f"{expert_idx.shape[0]} tokens exceed the context's max_tokens={self.max_tokens}")
        counts = torch.bincount(expert_idx.reshape(-1).long(), minlength=self.num_experts)
        if self.world == 1:
            all_counts = counts.unsqueeze(0)
        else:
            all_counts = self.exchange_counts(counts)
        plan = build_ep_plan(expert_idx, all_counts, self.rank, self.world, self.num_slots)
        # One host read per layer: the slot buffers are sized for the worst routing (every token of every rank to this
        # rank's experts), W times the expected load.  Knowing the rows in use lets every later kernel (zero, copies,
        # SwiGLU, the grouped GEMMs' outputs) touch only those instead of the whole buffer.
        used = int(plan.used_slots)
        if used > self.num_slots:
            raise RuntimeError(
                f"expert-parallel slot buffer overflow on rank {self.rank}: {used} > {self.num_slots}; "
                "raise capacity_factor"
            )
        plan.rows = used
        plan.tile_group = plan.tile_group[: used // BLOCK].contiguous()
        return plan

    def exchange_counts(self, counts: torch.Tensor) -> torch.Tensor:
        """``counts`` ``[E]`` (integer) of this rank -> int64 ``[W, E]`` of all ranks, through peer stores."""
        table = self._counts[self._count_turn]
        self._count_turn ^= 1
        words = counts.to(torch.int32).contiguous().view(torch.float32)
        row = self.rank * self.num_experts * 4
        require_ext().cast_broadcast(words, [p + row for p in table.ptrs], 0)
        self.mem.barrier()
        return table.local.view(torch.int32).to(torch.int64)

    # -- exchange -----------------------------------------------------------------------------------
    def dispatch(self, rows: torch.Tensor, plan: EPPlan, scale: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Send ``rows[token]`` (times ``scale``) of every assignment to its owner; returns MY received slots."""
        ext = require_ext()
        mine = self.recv.local[: plan.rows]
        mine.zero_()  # the padding rows between the experts' blocks feed the weight-gradient GEMMs: they must be zero
        self.mem.barrier()
        ext.moe_scatter_rows_peer(rows, plan.token, plan.dest_rank, plan.dest_slot, scale, self.recv.ptrs, self.hidden)
        self.mem.barrier()
        return mine.clone()

    def outbox(self, plan: EPPlan) -> torch.Tensor:
        """The rows of the send window that ``collect`` publishes: the last expert GEMM writes its output here directly
        (``grouped_gemm(..., out=...)``) instead of into a temporary that is copied afterwards.  Every reader of the
        previous contents has passed the barriers of the dispatch in between."""
        return self.send.local[: plan.rows]

    def collect(self, slots_out: torch.Tensor, plan: EPPlan) -> torch.Tensor:
        """Publish MY expert outputs and fetch, for every local assignment, its row: ``[T*k, H]``."""
        ext = require_ext()
        if slots_out.data_ptr() != self.send.local.data_ptr():
            self.send.local[: plan.rows].copy_(slots_out)
        self.mem.barrier()
        n = plan.dest_slot.numel()
        return ext.moe_combine_peer(self.send.ptrs, self.hidden, self.hidden, plan.dest_rank.view(n, 1),
                                    plan.dest_slot.view(n, 1), None)


class _EPExpertFFN(torch.autograd.Function):
    """x [T, H], weights [T, k], local W1 [El*2F, H], local W2 [El*H, F] -> out [T, H]."""

    @staticmethod
    def forward(ctx, x, weights, w1, w2, plan: EPPlan, ep: ExpertParallelContext):
        ext = require_ext()
        el = ep.local_experts
        xs = ep.dispatch(x, plan)
        h1 = ext.grouped_gemm(xs, w1, 1, plan.tile_group, el, False, False)
        act = ext.swiglu_packed_fwd(h1)
        y = ext.grouped_gemm(act, w2, 1, plan.tile_group, el, False, False, out=ep.outbox(plan))
        rows = ep.collect(y, plan)                                       # [T*k, H] in assignment order
        t, k = weights.shape
        local_slot = torch.arange(t * k, dtype=torch.int32, device=x.device).view(t, k)
        out = ext.moe_combine(rows, 0, 0, 0, local_slot, weights.detach())
        ctx.save_for_backward(xs, h1, act, rows, weights.detach(), w1, w2, local_slot)
        ctx.plan, ctx.ep = plan, ep
        return out

    @staticmethod
    def backward(ctx, dout):
        ext = require_ext()
        xs, h1, act, rows, weights, w1, w2, local_slot = ctx.saved_tensors
        plan, ep = ctx.plan, ctx.ep
        el = ep.local_experts
        dout = dout.contiguous()
        dweights = ext.moe_rowdot(dout, rows, local_slot)
        dy = ep.dispatch(dout, plan, weights.reshape(-1))
        dact = ext.grouped_gemm(dy, w2, 1, plan.tile_group, el, True, False)
        dw2 = ext.grouped_gemm(dy, act, 2, plan.offsets, el, True, False)
        dh1 = ext.swiglu_packed_bwd(h1, dact)
        dxs = ext.grouped_gemm(dh1, w1, 1, plan.tile_group, el, True, False, out=ep.outbox(plan))
        dw1 = ext.grouped_gemm(dh1, xs, 2, plan.offsets, el, True, False)
        drows = ep.collect(dxs, plan)
        dx = ext.moe_combine(drows, 0, 0, 0, local_slot, None)
        return dx, dweights, dw1, dw2, None, None


class ExpertParallelMoE:
    """``op(x, router_weight [E, H], local_gate_up [El*2F, H], local_down [El*H, F])`` -> ``[T, H]``.

    The router weight is replicated (its gradient must be summed over the ranks by the caller, like any
    data-parallel parameter); the expert weights are this rank's shard and receive complete gradients.
    """

    def __init__(self, ctx: ExpertParallelContext) -> None:
        self.ctx = ctx

    def __call__(self, x, router_weight, local_gate_up, local_down, top_k: Optional[int] = None):
        ep = self.ctx
        k = ep.top_k if top_k is None else int(top_k)
        x2 = x.reshape(-1, x.shape[-1])
        if x2.stride(1) != 1 or x2.stride(0) % 8 or x2.data_ptr() % 16:
            x2 = x2.contiguous()
        logits = _RouterLogits.apply(x2, router_weight)
        idx, weights = route_topk(logits, k)
        plan = ep.plan(idx)
        out = _EPExpertFFN.apply(x2, weights, local_gate_up, local_down, plan, ep)
        return out.reshape(x.shape)


# ---------------------------------------------------------------------------------- whole-model training
def moe_parameter_ranges(model):
    """Splits the flat parameter vector of a mixture-of-experts ``LlamaModel`` into replicated and expert parts.

    Returns ``(dense, ready_at, experts)``: ``dense`` are the ranges of the replicated parameters in flat order (the
    embedding with layer 0's attention / norms / router, then every further layer's, then final norm + LM head),
    ``ready_at[i]`` the layer whose backward completes range ``i`` (none for range 0), ``experts`` the per-layer ranges
    of the stacked expert weights (``w_gate_up`` and ``w_down`` are adjacent)."""
    off, cfg = model._offsets, model.cfg
    total = model.flat.numel()
    dense, experts, ready_at = [], [], {}
    start = 0
    for i in range(cfg.num_layers):
        e0 = off[f"l{i}.w_gate_up"]
        e1 = off[f"l{i + 1}.attn_norm"] if i + 1 < cfg.num_layers else off["final_norm"]
        dense.append((start, e0))
        if i > 0:
            ready_at[len(dense) - 1] = i
        experts.append((e0, e1))
        start = e1
    dense.append((start, total))
    ready_at[len(dense) - 1] = cfg.num_layers
    return dense, ready_at, experts


def _expert_parallel_optimizer():
    from rl_engine.parallel.data_parallel import ShardedFusedAdamW

    class ExpertParallelAdamW(ShardedFusedAdamW):
        """Replicated parameters: fused reduce-scatter + AdamW + all-gather over the ranks (state sharded 1 / W).
        Expert parameters: they exist only here and their gradients already hold every rank's tokens (the dispatch
        brought them), so they are stepped locally by the fused AdamW kernel with fp32 masters kept as 16-bit
        residuals; the loss is the mean over the ranks, hence the 1 / W on their gradients."""

        def _plan_buckets(self, model, layers_per_bucket):
            dense, ready_at, experts = moe_parameter_ranges(model)
            return dense, ready_at, experts

        def _ensure_local_state(self) -> None:
            if getattr(self, "_local", None) is not None:
                return
            dev = self.params.local.device
            self._local = []
            for lo, hi in self.local_ranges:
                n = hi - lo
                self._local.append((lo, hi, torch.zeros(n, dtype=torch.float32, device=dev),
                                    torch.zeros(n, dtype=torch.float32, device=dev),
                                    torch.zeros(n, dtype=torch.int16, device=dev) if self.master is not None else None))

        def _step_local_ranges(self) -> None:
            self._ensure_local_state()
            ext = require_ext()
            p, g = self.params.local, self.grads.local
            for lo, hi, m, v, residual in self._local:
                ext.adamw(p[lo:hi], residual, g[lo:hi], m, v, self.lr, self.betas[0], self.betas[1], self.eps,
                          self.weight_decay, self.steps + 1, float(self.grad_scale) / self.mem.world)

        def state_dict(self):
            state = super().state_dict()
            self._ensure_local_state()
            state["expert_m"] = [m for _lo, _hi, m, _v, _r in self._local]
            state["expert_v"] = [v for _lo, _hi, _m, v, _r in self._local]
            state["expert_residual"] = [r for *_x, r in self._local]
            return state

        def load_state_dict(self, state) -> None:
            super().load_state_dict(state)
            self._ensure_local_state()
            for (_lo, _hi, m, v, r), sm, sv, sr in zip(self._local, state["expert_m"], state["expert_v"],
                                                        state["expert_residual"]):
                m.copy_(sm)
                v.copy_(sv)
                if r is not None:
                    r.copy_(sr) if sr is not None else r.zero_()

    return ExpertParallelAdamW


def expert_parallel_trainer(model, *, max_tokens: int, group=None, **kw):
    """``ShardedGRPOTrainer`` for a mixture-of-experts ``LlamaModel`` built with ``expert_shard=(rank, world)``: every
    rank trains on its own completions (data parallel), every MoE layer sends its tokens to the ranks that own the routed
    experts (``ExpertParallelMoE``), and the optimiser treats replicated and expert parameters as ``ExpertParallelAdamW``
    describes.  ``max_tokens``: the largest number of packed tokens one forward pass of a rank may hold."""
    from rl_engine.parallel.data_parallel import ShardedGRPOTrainer

    cfg = model.cfg
    if not cfg.num_experts or model.expert_shard is None:
        raise ValueError("expert_parallel_trainer needs a mixture-of-experts model built with expert_shard=(rank, world)")
    optimizer = _expert_parallel_optimizer()

    class ExpertParallelGRPOTrainer(ShardedGRPOTrainer):
        optimizer_class = optimizer

    trainer = ExpertParallelGRPOTrainer(model, group=group, **kw)
    ctx = ExpertParallelContext(cfg.hidden_size, cfg.num_experts, cfg.experts_per_token, max_tokens=max_tokens,
                                group=group, device=model.flat.device)
    model.moe_op = ExpertParallelMoE(ctx)
    trainer.expert_context = ctx
    return trainer
