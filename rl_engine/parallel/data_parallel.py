"""Data-parallel GRPO step with optimizer state sharded over the ranks (ZeRO-1 style) and ONE fused
kernel for the whole gradient/parameter exchange.

Every rank keeps the full bf16 parameters and gradients as flat buffers inside the symmetric heap.
After backward, ``zero1_fused_step`` on rank r reads slice r of every peer's gradient buffer over
NVLink, sums in fixed rank order in fp32, scales by 1/world, applies AdamW on its fp32 moments (and
fp32 master slice) and writes the updated bf16 slice into every peer's parameter buffer.  Two
device-side barriers bracket the kernel.  There is no NCCL call in the step.

The reference delegates all of this to DeepSpeed (``rl_engine/executors/deepspeed_trainer.py:
101-126,168-169``).
"""

from __future__ import annotations

from typing import Optional

import torch

from rl_engine.kernels.ops.base import require_ext
from rl_engine.models.grpo import GRPOBatch, GRPOTrainer
from rl_engine.models.llama import LlamaModel
from rl_engine.parallel.symmetric import SymmetricMemory


class ShardedFusedAdamW:
    def __init__(self, model: LlamaModel, mem: SymmetricMemory, params, grads, lr=1e-6, betas=(0.9, 0.95), eps=1e-8,
                 weight_decay=0.0, master_weights: bool = True) -> None:
        self.model, self.mem, self.params, self.grads = model, mem, params, grads
        self.lr, self.betas, self.eps, self.weight_decay = lr, betas, eps, weight_decay
        n = params.local.numel()
        per = (n + mem.world - 1) // mem.world
        per = (per + 7) // 8 * 8
        self.lo = min(mem.rank * per, n)
        self.hi = min(self.lo + per, n)
        shard = self.hi - self.lo
        dev = params.local.device
        self.m = torch.zeros(shard, dtype=torch.float32, device=dev)
        self.v = torch.zeros(shard, dtype=torch.float32, device=dev)
        self.master = params.local[self.lo : self.hi].float() if master_weights else None
        self.steps = 0

    def zero_grad(self) -> None:
        self.grads.local.zero_()

    @torch.no_grad()
    def step(self) -> None:
        self.steps += 1
        self.mem.barrier()  # every rank's gradients are final
        require_ext().zero1_fused_step(
            self.grads.ptrs, self.params.ptrs, self.lo, self.hi, self.m, self.v, self.master, self.lr, self.betas[0],
            self.betas[1], self.eps, self.weight_decay, self.steps, 1.0 / self.mem.world,
        )
        self.mem.barrier()  # every rank's parameter slice has landed everywhere

    def state_dict(self):
        return {"m": self.m, "v": self.v, "master": self.master, "steps": self.steps, "lo": self.lo, "hi": self.hi}


class ShardedGRPOTrainer(GRPOTrainer):
    """``GRPOTrainer`` whose parameters/gradients live in symmetric memory and whose optimizer is fused."""

    def __init__(self, model: LlamaModel, *, group=None, lr: float = 1e-6, clip_eps: float = 0.2, beta: float = 0.04,
                 adv_eps: float = 1e-6, weight_decay: float = 0.0, master_weights: bool = True,
                 micro_group="auto") -> None:
        n = model.flat.numel()
        itemsize = model.flat.element_size()
        self.mem = SymmetricMemory(2 * n * itemsize + (1 << 20), group=group, device=model.flat.device)
        params = self.mem.alloc((n,), model.flat.dtype)
        grads = self.mem.alloc((n,), model.flat.dtype)
        params.local.copy_(model.flat)
        model.rebind_storage(params.local, grads.local)
        self.model = model
        self.clip_eps, self.beta, self.adv_eps = clip_eps, beta, adv_eps
        self.micro_group = micro_group
        self._micro_choice = {}
        self.opt = ShardedFusedAdamW(model, self.mem, params, grads, lr=lr, weight_decay=weight_decay,
                                     master_weights=master_weights)
        self._slice: Optional[slice] = None
        self.mem.barrier()

    def set_group_slice(self, sl: slice) -> None:
        """This rank trains on completions ``sl`` of the group; advantages use the whole group's rewards."""
        self._slice = sl

    def advantages(self, batch: GRPOBatch) -> torch.Tensor:
        adv = super().advantages(batch)
        return adv if self._slice is None else adv[self._slice].contiguous()

    def check(self) -> None:
        self.mem.check()
