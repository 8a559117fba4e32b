"""Rollout-side executor: versioned weight updates plus candidate generation.

Parity: ``rl_engine/executors/rollout.py:22-187`` of the reference — ``update_weights(manifest)``
imports, installs through an optional adapter, acknowledges, and on any failure rejects the update
and keeps serving the previous version; superseded updates are released; ``update_weights_via_ipc``
deliberately raises; ``generate_candidates`` goes through the lazy vLLM sampler.

``execute_rollout`` is a stub in the reference (returns a status dict).  Here, when the executor is
given a ``policy_model`` (a ``rl_engine.models.LlamaModel``), it generates completions with the
native prefix-sharing engine and the fused sampler, and returns token ids together with rollout
log-probs produced by the same ``linear_logp`` kernel the trainer uses.
"""

from __future__ import annotations

from typing import Any, Dict, Mapping, Optional

import torch

from rl_engine.executors.bridge import (
    WeightBridgeUnavailableError, WeightConsumer, WeightInstallAdapter, WeightUpdateManifest, make_weight_bridge,
)
from rl_engine.executors.vllm_sampler import VLLMSamplerConfig, VLLMSharedPrefixSampler
from rl_engine.utils.logger import logger


class RolloutExecutor:
    def __init__(self, model_config: Optional[dict] = None, *, weight_bridge: Optional[WeightConsumer] = None,
                 weight_transport: Optional[str] = None, weight_install_adapter: Optional[WeightInstallAdapter] = None,
                 policy_model: Optional[torch.nn.Module] = None) -> None:
        self.config = model_config or {}
        transport = weight_transport or str(self.config.get("weight_transport", "cuda-vmm"))
        self.bridge = weight_bridge or make_weight_bridge(transport)
        self.shared_weights: Dict[str, torch.Tensor] = {}
        self.weight_install_adapter = weight_install_adapter
        self.active_weight_version: Optional[int] = None
        self.active_weight_update_id: Optional[str] = None
        self.policy_model = policy_model
        self.logp_op = None
        self.attn_op = None
        self.sampler_config: Optional[VLLMSamplerConfig] = None
        self.sampler: Optional[VLLMSharedPrefixSampler] = None
        logger.info("Initializing RolloutExecutor with weight transport %s", transport)

    # -- weights ----------------------------------------------------------------------------------
    def update_weights(self, manifest: WeightUpdateManifest) -> Mapping[str, torch.Tensor]:
        logger.info("Importing weight update %s version=%s transport=%s", manifest.update_id, manifest.weight_version,
                    manifest.transport)
        previous = self.active_weight_update_id
        try:
            imported = dict(self.bridge.import_update(manifest))
            if self.weight_install_adapter is not None:
                self.weight_install_adapter.install(manifest, imported)
            elif self.policy_model is not None:
                self._install_into_policy(imported)
            self.bridge.acknowledge(manifest.update_id)
        except Exception as exc:
            try:
                self.bridge.reject(manifest.update_id, f"rollout weight install failed: {exc}")
            except Exception:
                logger.exception("Failed to reject weight update %s", manifest.update_id)
            raise
        self.shared_weights = imported
        self.active_weight_version = manifest.weight_version
        self.active_weight_update_id = manifest.update_id
        if previous is not None and previous != manifest.update_id:
            self.release_weight_update(previous)
        logger.info("Activated %s imported weight tensors.", len(imported))
        return self.shared_weights

    @torch.no_grad()
    def _install_into_policy(self, tensors: Mapping[str, torch.Tensor]) -> None:
        if hasattr(self.policy_model, "named_views") and "model.embed_tokens.weight" in tensors:
            # an update under Hugging Face checkpoint names (a trainer publishing for vLLM engines as well)
            from rl_engine.models.hf_interop import load_hf_state_dict

            load_hf_state_dict(self.policy_model, tensors)
            return
        views = self.policy_model.named_views() if hasattr(self.policy_model, "named_views") else dict(
            self.policy_model.named_parameters())
        missing = sorted(set(views) - set(tensors))
        if missing:
            raise KeyError(f"weight update lacks tensors for: {missing[:5]}")
        for name, dst in views.items():
            src = tensors[name]
            if tuple(src.shape) != tuple(dst.shape):
                raise ValueError(f"shape mismatch for {name}: {tuple(src.shape)} vs {tuple(dst.shape)}")
        for name, dst in views.items():
            dst.copy_(tensors[name].to(device=dst.device, dtype=dst.dtype))

    def release_weight_update(self, update_id: str) -> None:
        if self.weight_install_adapter is not None:
            self.weight_install_adapter.release(update_id)
        self.bridge.release(update_id)
        if self.active_weight_update_id == update_id:
            self.shared_weights = {}
            self.active_weight_update_id = None

    def release_weights(self) -> None:
        if self.active_weight_update_id is not None:
            self.release_weight_update(self.active_weight_update_id)

    def update_weights_via_ipc(self, ipc_handles: Mapping[str, Any]) -> Mapping[str, torch.Tensor]:
        del ipc_handles
        raise WeightBridgeUnavailableError(
            "Raw CUDA IPC handle imports are not production-ready. Publish a WeightUpdateManifest and call "
            "update_weights(...) so the bridge can validate version, tensor metadata, acknowledgement, and release lifecycle."
        )

    # -- sampling ---------------------------------------------------------------------------------
    def _prepare_kernels(self) -> None:
        if self.logp_op is None:
            from rl_engine.kernels.registry import kernel_registry

            self.logp_op = kernel_registry.get_op("logp")
            self.attn_op = kernel_registry.get_op("attn")
            logger.info("Active Kernels -> Logp: %s, Attn: %s", type(self.logp_op).__name__, type(self.attn_op).__name__)

    def _prepare_sampler(self) -> VLLMSharedPrefixSampler:
        if self.sampler is None:
            if self.sampler_config is None:
                self.sampler_config = VLLMSamplerConfig.from_model_config(self.config)
            self.sampler = VLLMSharedPrefixSampler(self.sampler_config)
            logger.info("Initialized vLLM rollout sampler (prefix_cache=%s, num_generations=%s)",
                        self.sampler_config.enable_prefix_caching, self.sampler_config.num_generations)
        return self.sampler

    def generate_candidates(self, prompts, *, num_generations: Optional[int] = None,
                            sampling_params: Optional[Mapping[str, Any]] = None) -> Dict[str, Any]:
        return self._prepare_sampler().generate(prompts, num_generations=num_generations, sampling_params=sampling_params)

    def execute_rollout(self, input_ids: torch.Tensor, *, num_generations: Optional[int] = None,
                        max_new_tokens: int = 16, **sampling: Any) -> Dict[str, Any]:
        """Generate completions for one prompt ``input_ids [P]`` with the native engine."""
        self._prepare_kernels()
        if self.policy_model is None:
            return {"status": "no_policy_model", "device": "cuda" if torch.cuda.is_available() else "cpu"}
        from rl_engine.executors.native_rollout import NativeRolloutEngine

        engine = NativeRolloutEngine(self.policy_model)
        g = int(num_generations or self.config.get("num_generations", 1))
        out = engine.generate(input_ids.reshape(-1), num_generations=g, max_new_tokens=max_new_tokens, **sampling)
        out.update(status="success", weight_version=self.active_weight_version)
        return out
