"""Training workers: consume a rollout stage result, take one policy-gradient step, publish weights.

``NativeTrainingWorker`` is this build's trainer: any model exposing hidden states + an LM head
(the toy ``TinyPolicy`` below, or ``rl_engine.models.LlamaModel``) is trained with the registry's
fused ``linear_logp`` and the log-prob-space GRPO/PPO loss kernels and an in-tree AdamW; weights are
published through the versioned bridge with monotonically increasing versions.

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
from rl_engine.testing import compute_policy_ratio, compute_reference_kl, masked_mean


class TinyPolicy(nn.Module):
    """``Embedding -> Linear`` toy policy: ``forward`` returns hidden states; ``lm_head`` is the projection."""

    def __init__(self, vocab_size: int, hidden_dim: int) -> None:
        super().__init__()
        self.embed = nn.Embedding(vocab_size, hidden_dim)
        self.lm_head = nn.Linear(hidden_dim, vocab_size, bias=False)

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


def safe_token_ids(token_ids: torch.Tensor, mask: Optional[torch.Tensor]) -> torch.Tensor:
    if mask is None:
        return token_ids
    return torch.where(mask.to(torch.bool), token_ids, torch.zeros_like(token_ids))


def validate_model_input_token_ids(token_ids: torch.Tensor, *, vocab_size: int) -> None:
    if token_ids.numel() and (int(token_ids.min()) < 0 or int(token_ids.max()) >= vocab_size):
        raise ValueError(
            f"training token ids must be in [0, {vocab_size}); got "
            f"[{int(token_ids.min())}, {int(token_ids.max())}]"
        )


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
        head = self.model.lm_head
        hidden = self.model(batch.token_ids.long())
        targets = safe_token_ids(batch.token_ids.to(hidden.device), batch.completion_mask)
        logps = self._linear_logp(hidden, head.weight, targets, getattr(head, "bias", None))
        keep = batch.completion_mask.to(device=logps.device, dtype=torch.bool)
        return torch.where(keep, logps, torch.zeros_like(logps)).float()

    def train(self, rollout: RolloutStageResult) -> TrainingStageResult:
        t0 = time.perf_counter()
        cfg = self.config
        batch, payload_metrics = self._batch_from_rollout_or_synthetic(rollout)
        validate_model_input_token_ids(batch.token_ids, vocab_size=self.model.lm_head.weight.shape[0])
        self.optimizer.zero_grad(set_to_none=True)
        cur = self._current_logps(batch)
        old = cur.detach() - cfg.old_logp_offset
        ref = objective_reference_logps(cur, batch)
        adv = batch.advantages.float()
        ratio = compute_policy_ratio(cur, old, batch.completion_mask)
        policy = -torch.minimum(ratio * adv, torch.clamp(ratio, cfg.clip_low, cfg.clip_high) * adv)
        kl = compute_reference_kl(cur, ref, batch.completion_mask)
        loss = masked_mean(policy + cfg.kl_beta * kl, batch.completion_mask)
        loss.backward()
        self.optimizer.step()
        active = adv[batch.completion_mask]
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
                "active_advantage_mean_global": float(active.mean()) if active.numel() else 0.0,
                "active_advantage_std_global": float(active.std(unbiased=False)) if active.numel() else 0.0,
                **payload_metrics,
            },
            started_at=t0,
            finished_at=time.perf_counter(),
        )

    def _next_published_weight_version(self, consumed: int) -> int:
        return max(int(consumed), self._published_version) + 1

    # -- weights ---------------------------------------------------------------------------------
    def publish_weights(self, weight_version: Optional[int] = None,
                        metadata: Optional[Mapping[str, Any]] = None) -> WeightUpdateManifest:
        version = self._published_version + 1 if weight_version is None else int(weight_version)
        if version <= self._published_version:
            raise WeightManifestValidationError(
                f"weight_version must increase monotonically (got {version}, latest {self._published_version})"
            )
        source = self.model.state_dict_views() if hasattr(self.model, "state_dict_views") else self.model
        manifest = self.bridge.publish(source, weight_version=version, metadata=metadata)
        self._published_version = version
        return manifest

    def release_weights(self, update_id: str) -> None:
        self.bridge.release(update_id)

    def health_check(self) -> Mapping[str, Any]:
        return {"published_weight_version": self._published_version, "device": str(self.device)}
