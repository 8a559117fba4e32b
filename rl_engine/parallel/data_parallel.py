"""Data-parallel GRPO step with optimizer state sharded over the ranks (ZeRO-1 style) and ONE fused
kernel for the whole gradient/parameter exchange of a bucket.

Every rank keeps the full bf16 parameters and gradients as flat buffers inside the symmetric heap.
The flat vector is cut into buckets at layer boundaries (``[embedding] [4 layers] ... [final norm +
LM head]``); inside a bucket rank r owns the r-th slice.  ``zero1_fused_step`` on rank r reads its
slice of every peer's gradient buffer over NVLink, sums in fixed rank order in fp32, scales by
1/world, applies AdamW on its fp32 moments and fp32 master slice and writes the updated bf16 slice
into every peer's parameter buffer.  There is no NCCL call in the step.

Overlap: the last backward pass of a step (the shared prompt's, or the only pass) visits the layers
from last to first, and once it has left a layer nothing of the step reads that layer's parameters or
adds to its gradients again.  The model reports that through ``layer_grad_hook``; the optimiser then
launches the bucket's barrier + fused kernel on a side stream (its own barrier channel) while the
backward pass continues on the main stream.  Only the first bucket (embedding + first layers) and the
closing barrier stay exposed.

The reference delegates all of this to DeepSpeed (``rl_engine/executors/deepspeed_trainer.py:
101-126,168-169``).
"""

from __future__ import annotations

import contextlib
from typing import Dict, List, Optional, Tuple

import torch

from rl_engine.kernels.ops.base import require_ext
from rl_engine.models.grpo import GRPOBatch, GRPOTrainer, _PromptPass
from rl_engine.models.config import require_untied
from rl_engine.models.llama import LlamaModel
from rl_engine.parallel.symmetric import SymmetricMemory

_SIDE_CHANNEL = 1  # barrier channel of the side stream


def layer_buckets(model: LlamaModel, layers_per_bucket: int = 4) -> Tuple[List[Tuple[int, int]], Dict[int, int]]:
    """Cuts the flat parameter vector at layer boundaries.

    Returns ``(ranges, ready_at)``: ``ranges[b] = (lo, hi)`` in elements of the flat vector, in flat order; bucket
    ``b`` is final once the backward pass has left layer ``ready_at[b]`` (``num_layers`` stands for the final norm).
    Bucket 0 (the embedding and the first layers) has no entry: it is final only when the whole backward has ended."""
    offsets = model._offsets
    n_layers = model.cfg.num_layers
    total = model.flat.numel()
    start = lambda i: offsets[f"l{i}.attn_norm"] if i < n_layers else offsets["final_norm"]
    step = max(1, int(layers_per_bucket))
    first = min(step, n_layers)
    cuts = [0] + [start(i) for i in range(first, n_layers, step)] + [start(n_layers), total]
    layer_of_cut = [0] + list(range(first, n_layers, step)) + [n_layers]
    ranges, ready_at = [], {}
    for b in range(len(cuts) - 1):
        if cuts[b + 1] > cuts[b]:
            ranges.append((cuts[b], cuts[b + 1]))
            if b > 0:
                ready_at[len(ranges) - 1] = layer_of_cut[b]
    return ranges, ready_at


class ShardedFusedAdamW:
    """AdamW whose moments and fp32 master weights exist only for this rank's slices of the buckets."""

    def __init__(self, model: LlamaModel, mem: SymmetricMemory, params, grads, lr=1e-6, betas=(0.9, 0.95), eps=1e-8,
                 weight_decay=0.0, master_weights: bool = True, layers_per_bucket: int = 4, overlap: bool = True,
                 overlap_blocks: int = 148 * 2) -> None:
        self.model, self.mem, self.params, self.grads = model, mem, params, grads
        require_untied(model.cfg, type(self).__name__)
        self.lr, self.betas, self.eps, self.weight_decay = lr, betas, eps, weight_decay
        n = model.flat.numel()
        ranges, self.ready_at, self.local_ranges = self._plan_buckets(model, layers_per_bucket)
        # the symmetric buffers are padded to a multiple of 8 elements; the pad belongs to the last bucket
        ranges[-1] = (ranges[-1][0], params.local.numel())
        self.numel = n
        self.slices: List[Tuple[int, int, int]] = []  # (lo, hi, offset into m / v / master) per bucket
        off = 0
        for lo_b, hi_b in ranges:
            size = hi_b - lo_b
            per = ((size + mem.world - 1) // mem.world + 7) // 8 * 8
            lo = min(lo_b + mem.rank * per, hi_b)
            hi = min(lo + per, hi_b)
            self.slices.append((lo, hi, off))
            off += hi - lo
        dev = params.local.device
        self.m = torch.zeros(off, dtype=torch.float32, device=dev)
        self.v = torch.zeros(off, dtype=torch.float32, device=dev)
        self.master = self._gather_local(params.local).float() if master_weights else None
        self.steps = 0
        self.grad_scale = 1.0  # extra factor on the summed gradient (1 / number of accumulated prompt groups)
        self.reduce = "mean"   # "mean": ranks hold gradients of different samples; "sum": of different tokens of one loss
        self.overlap = bool(overlap) and mem.world > 1
        self.overlap_blocks = int(overlap_blocks)
        self._side = torch.cuda.Stream(device=dev) if self.overlap else None
        self._launched: List[bool] = [False] * len(self.slices)
        self._side_used = False
        self._armed = False

    def _plan_buckets(self, model, layers_per_bucket):
        """``(ranges, ready_at, local_ranges)``: the buckets of the cross-rank exchange (see ``layer_buckets``) and the
        ranges of parameters that exist only on this rank and are stepped locally (none for a replicated model)."""
        ranges, ready_at = layer_buckets(model, layers_per_bucket)
        return ranges, ready_at, []

    def _gather_local(self, flat: torch.Tensor) -> torch.Tensor:
        return torch.cat([flat[lo:hi] for lo, hi, _ in self.slices]) if self.slices else flat[:0]

    def zero_grad(self) -> None:
        self.grads.local.zero_()

    # -- one bucket ---------------------------------------------------------------------------------------
    def _launch_bucket(self, b: int, channel: int, max_blocks: int) -> None:
        lo, hi, off = self.slices[b]
        self.mem.barrier(channel)  # every rank's gradients of this bucket are final
        n = hi - lo
        master = None if self.master is None else self.master[off : off + n]
        require_ext().zero1_fused_step(
            self.grads.ptrs, self.params.ptrs, lo, hi, self.m[off : off + n], self.v[off : off + n], master, self.lr,
            self.betas[0], self.betas[1], self.eps, self.weight_decay, self.steps + 1,
            float(self.grad_scale) / (self.mem.world if self.reduce == "mean" else 1),
            self.mem.rank, self.mem.error_word, max_blocks,
        )
        self._launched[b] = True

    # -- overlap with the last backward pass --------------------------------------------------------------
    def arm(self) -> None:
        """The pass whose forward starts now is the last one that is back-propagated in this step."""
        self._launched = [False] * len(self.slices)
        self._side_used = False
        self._armed = True

    def on_layer_done(self, layer: int) -> None:
        """Called from inside backward when it has left layer ``layer``: buckets holding only layers >= ``layer``
        are final on this rank."""
        if not (self.overlap and self._armed):
            return
        ready = [b for b, at in self.ready_at.items() if at >= layer and not self._launched[b]]
        if not ready:
            return
        main = torch.cuda.current_stream(self.m.device)
        self._side.wait_stream(main)
        self._side_used = True
        with torch.cuda.stream(self._side):
            for b in sorted(ready, reverse=True):  # the same order on every rank
                self._launch_bucket(b, _SIDE_CHANNEL, self.overlap_blocks)

    @torch.no_grad()
    def step(self) -> None:
        """Launches what the backward pass has not launched yet and waits (on the device) for all of it."""
        if not self._armed:
            self._launched = [False] * len(self.slices)
        main = torch.cuda.current_stream(self.m.device)
        for b in range(len(self.slices) - 1, -1, -1):
            if not self._launched[b]:
                self._launch_bucket(b, 0, 0)
        if self._side_used:
            main.wait_stream(self._side)
        self._step_local_ranges()
        self.steps += 1
        self._armed = False
        self._launched = [False] * len(self.slices)
        self.mem.barrier()  # every rank's parameter slices have landed everywhere

    def _step_local_ranges(self) -> None:
        """Hook for parameters that are not exchanged (see ``_plan_buckets``)."""

    # -- checkpoint ---------------------------------------------------------------------------------------
    def state_dict(self):
        """This rank's shard: tensors, ints and lists of ints only."""
        return {"m": self.m, "v": self.v, "master": self.master, "steps": self.steps, "rank": self.mem.rank,
                "world": self.mem.world, "slices": [[lo, hi] for lo, hi, _ in self.slices]}

    accepts_resharded_state = True

    @torch.no_grad()
    def _load_resharded(self, reader) -> None:
        """This rank's slices out of a checkpoint written by any number of ranks (``reader``: an
        ``OptimizerShardReader``).  Master weights come from the saved fp32 masters, else from saved bf16 residuals
        joined with the restored parameters, else from the restored parameters."""
        from rl_engine.models.grpo import join_master

        if reader.numel > self.params.local.numel():
            raise ValueError(f"the checkpoint's optimizer state covers {reader.numel} elements, this model has "
                             f"{self.params.local.numel()}")
        dev = self.m.device
        for lo, hi, off in self.slices:
            n = hi - lo
            if n <= 0:
                continue
            self.m[off : off + n].copy_(reader.read("m", lo, hi).to(dev))
            self.v[off : off + n].copy_(reader.read("v", lo, hi).to(dev))
            if self.master is None:
                continue
            param = self.params.local[lo:hi]
            if reader.has("master"):
                master = reader.read("master", lo, hi).to(dev)
                # padding past the checkpoint's end is not covered by any shard: keep the parameter there
                if hi > reader.numel:
                    master[max(0, reader.numel - lo):] = param[max(0, reader.numel - lo):].float()
            elif reader.has("master_residual") and param.dtype == torch.bfloat16:
                master = join_master(param, reader.read("master_residual", lo, hi).to(dev))
            else:
                master = param.float()
            self.master[off : off + n].copy_(master)
        self.steps = int(reader.steps)

    @torch.no_grad()
    def load_state_dict(self, state) -> None:
        """Restores a shard saved by the same rank of the same world size and bucket layout, or (given an
        ``OptimizerShardReader``) this rank's part of a checkpoint written with another world size.  Call after the
        parameters were restored; a checkpoint without master weights re-seeds them from the parameters."""
        if hasattr(state, "read"):
            self._load_resharded(state)
            return
        mine = [[lo, hi] for lo, hi, _ in self.slices]
        theirs = [list(map(int, s)) for s in state.get("slices", [])]
        if theirs != mine or int(state.get("world", self.mem.world)) != self.mem.world \
                or int(state.get("rank", self.mem.rank)) != self.mem.rank:
            raise ValueError(f"optimizer shard does not match this rank: saved slices {theirs[:2]}... of rank "
                             f"{state.get('rank')}/{state.get('world')}, expected {mine[:2]}... of rank "
                             f"{self.mem.rank}/{self.mem.world}")
        for lo, hi in mine:
            if lo % 8 or hi % 8 or hi < lo:
                raise ValueError("shard bounds must be ordered multiples of 8")
        self.m.copy_(state["m"])
        self.v.copy_(state["v"])
        self.steps = int(state["steps"])
        if self.master is not None:
            saved = state.get("master")
            self.master.copy_(self._gather_local(self.params.local).float() if saved is None else saved)


class ShardedGRPOTrainer(GRPOTrainer):
    """``GRPOTrainer`` whose parameters/gradients live in symmetric memory and whose optimizer is fused."""

    optimizer_class = ShardedFusedAdamW

    def __init__(self, model: LlamaModel, *, group=None, lr: float = 1e-6, clip_eps: float = 0.2, beta: float = 0.04,
                 adv_eps: float = 1e-6, weight_decay: float = 0.0, master_weights: bool = True,
                 micro_group="auto", overlap: bool = True, layers_per_bucket: int = 4, shard_prompt: bool = False) -> None:
        """``shard_prompt=True``: the ranks split the shared prompt's forward/backward pass between them (zig-zag context
        parallelism) instead of each running all of it.  That is only right when every rank trains on completions of
        the SAME prompt (``set_group_slice``).  Off by default: measured on the Llama-3-8B step (1 024-token prompt,
        256 completions) it is no faster on 2, 4 or 8 ranks (3 287 / 1 708 / 852 ms against 3 232 / 1 712 / 838 ms),
        because the prompt's backward pass, the last one of the step, is also the window under which the bucketed
        optimiser step runs, and a pass an eighth as long hides an eighth as much; with the prompt inside the only
        pass the whole backward hides it.  It pays when the prompt is long against the completions.
        Prompts whose length is not a multiple of ``32 * world`` run unsharded."""
        self.shard_prompt = shard_prompt
        self._group = group
        self._prompt_shards = {}
        n = model.flat.numel()
        padded = (n + 7) // 8 * 8
        itemsize = model.flat.element_size()
        self.mem = SymmetricMemory(2 * padded * itemsize + (1 << 20), group=group, device=model.flat.device)
        params = self.mem.alloc((padded,), model.flat.dtype)
        grads = self.mem.alloc((padded,), model.flat.dtype)
        params.local[:n].copy_(model.flat)
        model.rebind_storage(params.local[:n], grads.local[:n])
        self.model = model
        self.clip_eps, self.beta, self.adv_eps = clip_eps, beta, adv_eps
        self.micro_group = micro_group
        self._micro_choice = {}
        self.opt = self.optimizer_class(model, self.mem, params, grads, lr=lr, weight_decay=weight_decay,
                                        master_weights=master_weights, layers_per_bucket=layers_per_bucket,
                                        overlap=overlap)
        self._slice: Optional[slice] = None
        self.mem.barrier()

    def set_group_slice(self, sl: slice) -> None:
        """This rank trains on completions ``sl`` of the group; advantages use the whole group's rewards."""
        self._slice = sl

    def advantages(self, batch: GRPOBatch) -> torch.Tensor:
        adv = super().advantages(batch)
        return adv if self._slice is None else adv[self._slice].contiguous()

    def _prompt_sharding(self, batch: GRPOBatch):
        """``{"cp": ..., "share_row": ...}`` for a prompt of this batch's length, or ``None`` if its pass is not sharded."""
        world = self.mem.world
        on = bool(self.shard_prompt)
        n = batch.prompt_ids.numel()
        if not on or world == 1 or n % (32 * world) or not self.prompt_cacheable(batch):
            return None
        if n not in self._prompt_shards:
            from rl_engine.parallel.context_parallel import ContextParallelAttention, SharedRow

            cfg = self.model.cfg
            cp = ContextParallelAttention(n, cfg.num_kv_heads, cfg.head_dim, group=self._group,
                                          device=self.model.flat.device)
            self._prompt_shards[n] = {"cp": cp, "share_row": SharedRow(cp.mem, cfg.hidden_size, owner=0)}
        return self._prompt_shards[n]

    def force_prompt_pass(self, batch: GRPOBatch) -> bool:
        return self._prompt_sharding(batch) is not None

    def prompt_pass(self, batch: GRPOBatch):
        sharding = self._prompt_sharding(batch)
        if sharding is None:
            return super().prompt_pass(batch)
        return _PromptPass(self.model, batch.prompt_ids, **sharding)

    @contextlib.contextmanager
    def final_pass(self):
        """Wraps the forward of the pass that is back-propagated last: its layer hooks start the buckets."""
        if not self._last_group:  # more prompt groups will add to these gradients before the optimiser step
            yield
            return
        self.opt.arm()
        self.model.layer_grad_hook = self.opt.on_layer_done
        try:
            yield
        finally:
            self.model.layer_grad_hook = None

    def check(self) -> None:
        self.mem.check()
        for shard in self._prompt_shards.values():
            shard["cp"].mem.check()

    def close(self) -> None:
        """Unmaps the symmetric segments (collective: every rank calls it, with no kernel of the trainer in flight)."""
        for shard in self._prompt_shards.values():
            shard["cp"].mem.close()
        self._prompt_shards = {}
        self.mem.close()
