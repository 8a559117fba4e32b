"""Training workers: consume a rollout stage result, take one policy-gradient step, publish weights.

``NativeTrainingWorker`` trains any model exposing hidden states + an LM head (the toy ``TinyPolicy``
below, a Hugging Face backbone, ...) with the registry's fused ``linear_logp`` and the reference's
clipped-ratio objective; ``GRPOTrainingWorker`` is the same contract on this build's own stack: a
``rl_engine.models.LlamaModel`` stepped by ``GRPOTrainer`` (one GPU) or ``ShardedGRPOTrainer`` (data
parallel, fused reduce-scatter + AdamW + all-gather kernel), i.e. the packed prefix-shared forward,
fused log-prob / GRPO-loss kernels and the fused optimiser.  Both publish weights through the
versioned bridge with monotonically increasing versions.

Parity: ``DeepSpeedTrainingWorker`` of the reference (``rl_engine/executors/deepspeed_trainer.py:
73-311``): ``train(rollout) -> TrainingStageResult`` with the same metric keys, ``publish_weights``,
``release_weights``, the ``Embedding -> Linear`` toy policy (``:54-70``) and ``_next_published``
version rule.  ``rl_engine.executors.deepspeed_trainer`` keeps the DeepSpeed-backed variant for users
who have DeepSpeed installed.
"""

from __future__ import annotations

import time
from dataclasses import dataclass
from typing import Any, Mapping, Optional

import torch
from torch import nn

from rl_engine.executors.bridge import WeightBridge, WeightManifestValidationError, WeightUpdateManifest, make_weight_bridge
from rl_engine.executors.training_contract import (
    RolloutBatchMixin, RolloutStageResult, TorchRLTrainingConfig, TrainingStageResult, objective_reference_logps,
)
from rl_engine.executors.hidden_states import backbone_hidden_states, extract_hidden_states, output_head  # noqa: F401
from rl_engine.testing import compute_policy_ratio, compute_reference_kl, masked_mean


class TinyPolicy(nn.Module):
    """``Embedding -> Linear`` toy policy: ``forward`` returns hidden states; ``lm_head`` is the projection."""

    def __init__(self, vocab_size: int, hidden_dim: int, *, bias: bool = True) -> None:
        super().__init__()
        self.embed = nn.Embedding(vocab_size, hidden_dim)
        self.lm_head = nn.Linear(hidden_dim, vocab_size, bias=bias)

    def forward(self, token_ids: torch.Tensor) -> torch.Tensor:
        return self.embed(token_ids)


@dataclass(frozen=True)
class NativeTrainingConfig(TorchRLTrainingConfig):
    clip_low: float = 0.8
    clip_high: float = 1.2
    kl_beta: float = 0.01
    old_logp_offset: float = 0.01
    weight_transport: str = "local-clone"
    weight_decay: float = 0.0
    # "native": this library's parameter names; "hf": the names of the Hugging Face checkpoint of the same
    # architecture (what a vLLM engine's weight loader expects), as zero-copy views of the packed parameters
    weight_names: str = "native"


def safe_token_ids(token_ids: torch.Tensor, mask: Optional[torch.Tensor]) -> torch.Tensor:
    if mask is None:
        return token_ids
    return torch.where(mask.to(torch.bool), token_ids, torch.zeros_like(token_ids))


def validate_model_input_token_ids(token_ids: torch.Tensor, *, vocab_size: int) -> None:
    if token_ids.numel() and (int(token_ids.min()) < 0 or int(token_ids.max()) >= vocab_size):
        raise ValueError(
            f"training token ids must be in [0, {vocab_size}); got [{int(token_ids.min())}, {int(token_ids.max())}]. "
            "Token ids are model inputs here: replace ignore-index / padding values (such as -100) before training; "
            "masking only protects the loss"
        )


def clipped_ratio_objective(cur: torch.Tensor, batch, cfg: "NativeTrainingConfig") -> torch.Tensor:
    """The reference worker's objective (``rl_engine/executors/deepspeed_trainer.py:160-167``) on current log-probs
    ``cur``: ratio against ``cur - old_logp_offset``, clipping to ``[clip_low, clip_high]``, KL to the payload's
    reference log-probs (or ``cur - 0.02``), masked token mean.  Shared by the native and the DeepSpeed worker."""
    old = cur.detach() - cfg.old_logp_offset
    ref = objective_reference_logps(cur, batch)
    adv = batch.advantages.float()
    ratio = compute_policy_ratio(cur, old, batch.completion_mask)
    policy = -torch.minimum(ratio * adv, torch.clamp(ratio, cfg.clip_low, cfg.clip_high) * adv)
    kl = compute_reference_kl(cur, ref, batch.completion_mask)
    return masked_mean(policy + cfg.kl_beta * kl, batch.completion_mask)


def advantage_metrics(batch) -> dict:
    active = batch.advantages.float()[batch.completion_mask]
    return {
        "active_advantage_mean_global": float(active.mean()) if active.numel() else 0.0,
        "active_advantage_std_global": float(active.std(unbiased=False)) if active.numel() else 0.0,
    }


class NativeTrainingWorker(RolloutBatchMixin):
    def __init__(self, config: Optional[NativeTrainingConfig] = None, *, model: Optional[nn.Module] = None,
                 weight_bridge: Optional[WeightBridge] = None, source_worker: str = "native-training") -> None:
        self.config = config or NativeTrainingConfig()
        self.device = torch.device(self.config.device)
        torch.manual_seed(self.config.seed)
        self.model = (model or TinyPolicy(self.config.vocab_size, self.config.hidden_dim)).to(self.device)
        if model is None:
            self.model = self.model.to(self.config.dtype)
        self.optimizer = torch.optim.AdamW(self.model.parameters(), lr=self.config.lr, weight_decay=self.config.weight_decay)
        self.bridge = weight_bridge or make_weight_bridge(self.config.weight_transport, source_worker=source_worker)
        self._published_version = -1
        from rl_engine.kernels.registry import kernel_registry

        self._linear_logp = kernel_registry.get_op("linear_logp")

    # -- one optimisation step ---------------------------------------------------------------------
    def _current_logps(self, batch) -> torch.Tensor:
        head = output_head(self.model)
        # whatever the backbone returns (tensor, ModelOutput, dict, tuple): take its final hidden states; a Hugging
        # Face causal LM is entered below its vocabulary projection
        hidden = backbone_hidden_states(self.model, batch.token_ids.long(), hidden_dim=head.weight.shape[1])
        targets = safe_token_ids(batch.token_ids.to(hidden.device), batch.completion_mask)
        logps = self._linear_logp(hidden, head.weight, targets, getattr(head, "bias", None))
        keep = batch.completion_mask.to(device=logps.device, dtype=torch.bool)
        return torch.where(keep, logps, torch.zeros_like(logps)).float()

    def train(self, rollout: RolloutStageResult) -> TrainingStageResult:
        t0 = time.perf_counter()
        cfg = self.config
        batch, payload_metrics = self._batch_from_rollout_or_synthetic(rollout)
        validate_model_input_token_ids(batch.token_ids, vocab_size=output_head(self.model).weight.shape[0])
        self.optimizer.zero_grad(set_to_none=True)
        loss = clipped_ratio_objective(self._current_logps(batch), batch, cfg)
        loss.backward()
        self.optimizer.step()
        return TrainingStageResult(
            iteration=rollout.iteration,
            consumed_weight_version=rollout.weight_version,
            published_weight_version=self._next_published_weight_version(rollout.weight_version),
            metrics={
                "loss": float(loss.detach()),
                "active_tokens": int(batch.completion_mask.sum()),
                "payload_type": type(rollout.payload).__name__,
                "training_backend": "native",
                "training_device": str(self.device),
                "current_logp_path": "linear_logp",
                "current_logp_backend": type(self._linear_logp).__name__,
                **advantage_metrics(batch),
                **payload_metrics,
            },
            started_at=t0,
            finished_at=time.perf_counter(),
        )

    def _next_published_weight_version(self, consumed: int) -> int:
        """The version the weights of this step will be published under: above the consumed one, above everything
        published, and above every version already promised to an earlier step (two steps on the same rollout version
        get two different numbers)."""
        promised = max(int(consumed), self._published_version, getattr(self, "_promised_version", -1)) + 1
        self._promised_version = promised
        return promised

    # -- weights ---------------------------------------------------------------------------------
    def publish_weights(self, weight_version: Optional[int] = None,
                        metadata: Optional[Mapping[str, Any]] = None) -> WeightUpdateManifest:
        version = self._published_version + 1 if weight_version is None else int(weight_version)
        if version <= self._published_version:
            raise WeightManifestValidationError(
                f"weight_version must increase monotonically (got {version}, latest {self._published_version})"
            )
        if not hasattr(self.model, "state_dict_views"):
            source = self.model
        elif getattr(self.config, "weight_names", "native") == "hf":
            source = self.model.state_dict_views(names="hf")
        else:
            source = self.model.state_dict_views()
        manifest = self.bridge.publish(source, weight_version=version, metadata=metadata)
        self._published_version = version
        return manifest

    def release_weights(self, update_id: str) -> None:
        self.bridge.release(update_id)

    def health_check(self) -> Mapping[str, Any]:
        return {"published_weight_version": self._published_version, "device": str(self.device)}


@dataclass(frozen=True)
class GRPOTrainingConfig(NativeTrainingConfig):
    """Objective of ``GRPOTrainer``: clip ``1 +- clip_eps``, KL weight ``beta``, group-normalised advantages."""

    clip_eps: float = 0.2
    beta: float = 0.04
    advantage_eps: float = 1e-6
    micro_group: Any = "auto"
    master_weights: bool = True


class GRPOTrainingWorker(NativeTrainingWorker):
    """The training-worker contract on the real stack.

    ``train(rollout)`` turns the rollout into prompt groups (``GRPOBatch``), takes ONE optimiser step over all of them
    with ``GRPOTrainer.step_groups`` -- packed prefix-shared forward, fused ``linear_logp`` + GRPO loss kernels, fused
    AdamW with fp32 master weights; with an initialised ``torch.distributed`` group of more than one rank and
    ``data_parallel=True`` the ``ShardedGRPOTrainer`` (fused reduce-scatter + AdamW + all-gather over NVLink) -- and
    returns the reference's ``TrainingStageResult``.  ``publish_weights`` hands ``model.state_dict_views()`` to the
    bridge, so the manifest carries checkpoint-format names and the flat buffer is not copied by the publisher.

    Accepted payloads: one mapping or a sequence of mappings with ``prompt_ids [P]``, ``completion_ids [G, L]`` and
    optionally ``rewards [G]``, ``rollout_logps`` / ``old_logps [G, L]``, ``reference_logps [G, L]``,
    ``completion_mask [G, L]`` (what ``RolloutExecutor.execute_rollout`` returns, plus scores); anything else goes
    through the reference's payload parser (vLLM-style candidates or the synthetic fallback)."""

    def __init__(self, config: Optional[GRPOTrainingConfig] = None, *, model: nn.Module,
                 weight_bridge: Optional[WeightBridge] = None, source_worker: str = "grpo-training",
                 data_parallel: Optional[bool] = None, group: Any = None) -> None:
        self.config = config or GRPOTrainingConfig()
        if not hasattr(model, "flat") or not hasattr(model, "lm_head_weight"):
            raise TypeError("GRPOTrainingWorker needs a rl_engine.models.LlamaModel (flat parameters, lm_head_weight)")
        self.model = model
        self.device = model.flat.device
        self.bridge = weight_bridge or make_weight_bridge(self.config.weight_transport, source_worker=source_worker)
        self._published_version = -1
        from rl_engine.kernels.registry import kernel_registry
        from rl_engine.models.grpo import GRPOTrainer

        self._linear_logp = kernel_registry.get_op("linear_logp")
        kw = dict(lr=self.config.lr, clip_eps=self.config.clip_eps, beta=self.config.beta,
                  adv_eps=self.config.advantage_eps, weight_decay=self.config.weight_decay,
                  master_weights=self.config.master_weights, micro_group=self.config.micro_group)
        import torch.distributed as dist

        world = dist.get_world_size(group) if dist.is_available() and dist.is_initialized() else 1
        if data_parallel is None:
            data_parallel = world > 1 and self.device.type == "cuda"
        if data_parallel:
            from rl_engine.parallel.data_parallel import ShardedGRPOTrainer

            self.trainer = ShardedGRPOTrainer(model, group=group, **kw)
            self._rank, self._world = dist.get_rank(group), world
        else:
            self.trainer = GRPOTrainer(model, **kw)
            self._rank, self._world = 0, 1
        self.optimizer = self.trainer.opt

    # -- payload -> prompt groups ------------------------------------------------------------------
    @staticmethod
    def _native_groups(payload: Any):
        items = [payload] if isinstance(payload, Mapping) else payload
        if not isinstance(items, (list, tuple)) or not items:
            return None
        if not all(isinstance(g, Mapping) and "prompt_ids" in g and "completion_ids" in g for g in items):
            return None
        return list(items)

    def _groups_from_rollout(self, rollout: RolloutStageResult):
        from rl_engine.models.grpo import GRPOBatch

        dev = self.device
        native = self._native_groups(rollout.payload)
        groups, metrics = [], {}
        if native is not None:
            for item in native:
                comp = torch.as_tensor(item["completion_ids"]).to(dev).long()
                g, l = comp.shape
                mask = item.get("completion_mask")
                mask = torch.ones(g, l, dtype=torch.bool, device=dev) if mask is None else torch.as_tensor(mask).to(dev).bool()
                rewards = item.get("rewards")
                if rewards is None:  # the reference's proxy: mean token id scaled to [0, 1)
                    rewards = comp.float().mean(dim=1) / self.model.cfg.vocab_size
                old = item.get("old_logps", item.get("rollout_logps"))
                ref = item.get("reference_logps", item.get("ref_logps"))
                groups.append((GRPOBatch(
                    prompt_ids=torch.as_tensor(item["prompt_ids"]).to(dev).long().reshape(-1), completion_ids=comp,
                    rewards=torch.as_tensor(rewards).to(dev).float(),
                    old_logps=None if old is None else torch.as_tensor(old).to(dev).float(),
                    ref_logps=None if ref is None else torch.as_tensor(ref).to(dev).float(), completion_mask=mask,
                ), old is not None, ref is not None))
            metrics = {
                "training_data_source": "rollout_payload",
                "reward_source": "payload_rewards" if all("rewards" in g for g in native) else "token_id_proxy",
                "reference_logp_source": ("payload_reference_logps" if all(r for _, _, r in groups)
                                          else "synthetic_current_offset"),
                "rollout_prompt_groups": len(groups), "rollout_sequences": sum(b.completion_ids.shape[0] for b, _, _ in groups),
                "rollout_tokens": int(sum(b.completion_mask.sum() for b, _, _ in groups)),
            }
            return groups, metrics
        batch, metrics = self._batch_from_rollout_or_synthetic(rollout)
        validate_model_input_token_ids(batch.token_ids, vocab_size=self.model.cfg.vocab_size)
        per = int(batch.metadata.get("samples_per_prompt", batch.batch_size))
        from_payload = batch.metadata.get("reference_logp_source") == "payload_reference_logps"
        for r0 in range(0, batch.batch_size, per):
            rows = slice(r0, r0 + per)
            groups.append((GRPOBatch(
                prompt_ids=batch.input_ids[r0, : batch.prompt_len].to(dev).long(),
                completion_ids=safe_token_ids(batch.token_ids[rows], batch.completion_mask[rows]).to(dev).long(),
                rewards=batch.rewards[rows].to(dev).float(), old_logps=None,
                ref_logps=batch.ref_logps[rows].to(dev).float() if from_payload else None,
                completion_mask=batch.completion_mask[rows].to(dev).bool(),
            ), False, from_payload))
        return groups, metrics

    def _fill_missing_logps(self, groups):
        """Old / reference log-probs that the rollout did not supply are the current ones minus the reference
        worker's offsets (``old_logp_offset``; 0.02 for the KL reference), computed without autograd."""
        out = []
        for batch, has_old, has_ref in groups:
            if not (has_old and has_ref):
                with torch.no_grad():
                    probe = type(batch)(batch.prompt_ids, batch.completion_ids, batch.rewards,
                                        torch.zeros_like(batch.completion_ids, dtype=torch.float32),
                                        torch.zeros_like(batch.completion_ids, dtype=torch.float32), batch.completion_mask)
                    cur = self.trainer.policy_logps(probe).float()
                if not has_old:
                    batch.old_logps = cur - self.config.old_logp_offset
                if not has_ref:
                    batch.ref_logps = cur - 0.02
            out.append(batch)
        return out

    def train(self, rollout: RolloutStageResult) -> TrainingStageResult:
        t0 = time.perf_counter()
        groups, payload_metrics = self._groups_from_rollout(rollout)
        batches = self._fill_missing_logps(groups)
        if self._world > 1:  # every rank trains on its slice of each group's completions
            batches = [self._rank_slice(b) for b in batches]
        loss = self.trainer.step_groups(batches)
        if hasattr(self.trainer, "check"):
            self.trainer.check()
        mask = torch.cat([b.completion_mask.reshape(-1) for b in batches])
        adv = torch.cat([self.trainer.advantages(b)[:, None].expand_as(b.completion_mask).reshape(-1) for b in batches])
        active = adv[mask]
        return TrainingStageResult(
            iteration=rollout.iteration,
            consumed_weight_version=rollout.weight_version,
            published_weight_version=self._next_published_weight_version(rollout.weight_version),
            metrics={
                "loss": float(loss), "active_tokens": int(mask.sum()), "payload_type": type(rollout.payload).__name__,
                "training_backend": type(self.trainer).__name__, "training_device": str(self.device),
                "current_logp_path": "linear_logp", "current_logp_backend": type(self._linear_logp).__name__,
                "optimizer_steps": int(self.trainer.opt.steps), "data_parallel_world": self._world,
                "master_weights": bool(getattr(self.trainer.opt, "has_master", self.config.master_weights)),
                "active_advantage_mean_global": float(active.mean()) if active.numel() else 0.0,
                "active_advantage_std_global": float(active.std(unbiased=False)) if active.numel() else 0.0,
                **payload_metrics,
            },
            started_at=t0, finished_at=time.perf_counter(),
        )

    def _rank_slice(self, batch):
        g = batch.completion_ids.shape[0]
        if g % self._world:
            raise ValueError(f"{g} completions per prompt do not divide over {self._world} data-parallel ranks")
        per = g // self._world
        sl = slice(self._rank * per, (self._rank + 1) * per)
        self.trainer.set_group_slice(sl)
        return batch.completions(sl.start, sl.stop)

    def save_checkpoint(self, directory: str, *, sampler: Any = None, extra: Optional[Mapping[str, Any]] = None):
        from rl_engine.executors.checkpoint import save_checkpoint

        return save_checkpoint(directory, self.model, self.trainer.opt, weight_version=max(self._published_version, 0),
                               sampler=sampler, extra=dict(extra or {}), rank=self._rank, world=self._world)

    def load_checkpoint(self, directory: str, *, sampler: Any = None):
        from rl_engine.executors.checkpoint import load_checkpoint

        state = load_checkpoint(directory, self.model, self.trainer.opt, sampler=sampler, rank=self._rank, world=self._world)
        self._published_version = int(state.get("weight_version", 0))  # the next publish continues after it
        return state
