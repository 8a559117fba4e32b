"""Kernel registry: ``kernel_registry.get_op(op_type)`` returns the best operator for this process.

Parity: reference ``rl_engine/kernels/registry.py:24-253`` — enum values are dotted class paths,
per-platform priority lists, lazy import with an instance cache and a failed-backend set, a
missing *backend* module falls through to the next candidate while a broken *internal*
``rl_engine.*`` import is re-raised, and ``OpBackend["NAME"]`` lookups give a helpful error.

This build has exactly two backend families: ``SM100_*`` (hand-written sm_100a kernels from
``rl_engine._C``) and ``PYTORCH_*`` (CPU / oracle).  There is no Triton, FlashInfer, ROCm or
multi-vendor dispatch.  On a Blackwell GPU a missing extension is an error, not a silent fallback
(set ``RL_KERNEL_ALLOW_FALLBACK=1`` to permit the PyTorch path there).
"""

from __future__ import annotations

import importlib
import os
from enum import Enum, EnumMeta
from typing import Any, Dict, List, Optional, Set, Type

from rl_engine.platforms.device import device_ctx
from rl_engine.utils.logger import logger


class _BackendEnumMeta(EnumMeta):
    def __getitem__(cls, name: str):
        try:
            return super().__getitem__(name)
        except KeyError as exc:
            known = ", ".join(cls.__members__)
            raise ValueError(f"Operator '{name}' not found. Supported backends: {known}") from exc


_SM = "rl_engine.kernels.ops.sm100"
_PT = "rl_engine.kernels.ops.pytorch"


class OpBackend(Enum, metaclass=_BackendEnumMeta):
    # hand-written sm_100a kernels
    SM100_FUSED_LOGP = f"{_SM}.logp.FusedLogpSM100Op"
    SM100_LINEAR_LOGP = f"{_SM}.linear_logp.FusedLinearLogpSM100Op"
    SM100_RATIO_KL = f"{_SM}.ratio_kl.FusedRatioKLSM100Op"
    SM100_GRPO_LOSS = f"{_SM}.grpo_loss.FusedGRPOLossSM100Op"
    SM100_PPO_LOSS = f"{_SM}.policy_losses.FusedPPOLossSM100Op"
    SM100_DPO_LOSS = f"{_SM}.policy_losses.FusedDPOLossSM100Op"
    SM100_ATTN = f"{_SM}.attention.FlashAttentionSM100Op"
    SM100_PREFIX_SHARED_ATTN = f"{_SM}.attention.PrefixSharedAttentionSM100Op"
    SM100_RMS_NORM = f"{_SM}.model_ops.FusedRMSNormSM100Op"
    SM100_SILU = f"{_SM}.model_ops.FusedSiLUSM100Op"
    SM100_SWIGLU = f"{_SM}.model_ops.FusedSwiGLUSM100Op"
    SM100_ROPE = f"{_SM}.model_ops.FusedRoPESM100Op"
    SM100_EMBEDDING = f"{_SM}.model_ops.FusedEmbeddingSM100Op"
    SM100_LM_HEAD = f"{_SM}.model_ops.FusedLMHeadSM100Op"
    SM100_MOE = f"{_SM}.moe.FusedMoESM100Op"

    # PyTorch oracles (CPU path and ground truth)
    PYTORCH_NATIVE = f"{_PT}.loss.logp.NativeLogpOp"
    PYTORCH_LINEAR_LOGP = f"{_PT}.loss.linear_logp.NativeLinearLogpOp"
    PYTORCH_RATIO_KL = f"{_PT}.loss.ratio_kl.NativeRatioKLOp"
    PYTORCH_GRPO_LOSS = f"{_PT}.loss.grpo_loss.NativeGRPOLossOp"
    PYTORCH_PPO_LOSS = f"{_PT}.loss.policy_losses.NativePPOLossOp"
    PYTORCH_DPO_LOSS = f"{_PT}.loss.policy_losses.NativeDPOLossOp"
    PYTORCH_ATTN = f"{_PT}.attention.NativeAttentionOp"
    PYTORCH_PREFIX_SHARED_ATTN = f"{_PT}.attention.NativePrefixSharedAttentionOp"
    PYTORCH_NATIVE_RMS_NORM = f"{_PT}.norm.rms_norm.NativeRMSNormOp"
    PYTORCH_NATIVE_SILU = f"{_PT}.activation.swiglu.NativeSiLUOp"
    PYTORCH_NATIVE_SWIGLU = f"{_PT}.activation.swiglu.NativeSwiGLUOp"
    PYTORCH_NATIVE_ROPE = f"{_PT}.linear.rope.NativeRoPEOp"
    PYTORCH_NATIVE_EMBEDDING = f"{_PT}.linear.embedding.NativeEmbeddingOp"
    PYTORCH_NATIVE_LM_HEAD = f"{_PT}.linear.lm_head.NativeLMHeadOp"
    PYTORCH_MOE = f"{_SM}.moe.NativeMoEOp"


_B = OpBackend
_PAIRS: Dict[str, tuple] = {
    "logp": (_B.SM100_FUSED_LOGP, _B.PYTORCH_NATIVE),
    "logp_indexed": (_B.SM100_FUSED_LOGP, _B.PYTORCH_NATIVE),
    "logp_online": (_B.SM100_FUSED_LOGP, _B.PYTORCH_NATIVE),
    "logp_online_indexed": (_B.SM100_FUSED_LOGP, _B.PYTORCH_NATIVE),
    "attn": (_B.SM100_ATTN, _B.PYTORCH_ATTN),
    "prefix_shared_attn": (_B.SM100_PREFIX_SHARED_ATTN, _B.PYTORCH_PREFIX_SHARED_ATTN),
    "grpo_loss": (_B.SM100_GRPO_LOSS, _B.PYTORCH_GRPO_LOSS),
    "ppo_loss": (_B.SM100_PPO_LOSS, _B.PYTORCH_PPO_LOSS),
    "dpo_loss": (_B.SM100_DPO_LOSS, _B.PYTORCH_DPO_LOSS),
    "linear_logp": (_B.SM100_LINEAR_LOGP, _B.PYTORCH_LINEAR_LOGP),
    "ratio_kl": (_B.SM100_RATIO_KL, _B.PYTORCH_RATIO_KL),
    "rms_norm": (_B.SM100_RMS_NORM, _B.PYTORCH_NATIVE_RMS_NORM),
    "lm_head": (_B.SM100_LM_HEAD, _B.PYTORCH_NATIVE_LM_HEAD),
    "embedding": (_B.SM100_EMBEDDING, _B.PYTORCH_NATIVE_EMBEDDING),
    "silu": (_B.SM100_SILU, _B.PYTORCH_NATIVE_SILU),
    "swiglu": (_B.SM100_SWIGLU, _B.PYTORCH_NATIVE_SWIGLU),
    "rope": (_B.SM100_ROPE, _B.PYTORCH_NATIVE_ROPE),
    "moe": (_B.SM100_MOE, _B.PYTORCH_MOE),
}


class KernelRegistry:
    def __init__(self) -> None:
        self._instance_cache: Dict[str, Any] = {}
        self._failed_backends: Set[str] = set()
        self._priority_map: Dict[str, Dict[str, List[OpBackend]]] = {
            "cuda": {op: [fast, slow] for op, (fast, slow) in _PAIRS.items()},
            "cpu": {op: [slow] for op, (_fast, slow) in _PAIRS.items()},
        }
        logger.info_once("KernelRegistry initialized for %s", device_ctx.device_type)
        self._adjust_priority_for_hardware()
        self._adjust_priority_from_env()

    # -- priority shaping ------------------------------------------------------------------
    def _adjust_priority_for_hardware(self) -> None:
        """Drop the sm_100a candidates when the visible GPU is not a Blackwell part."""
        if device_ctx.device_type != "cuda":
            return
        try:
            from rl_engine.kernels.ops.base import _EXT_AVAILABLE

            if not device_ctx.is_blackwell:
                logger.warning(
                    "GPU capability %s is not sm_100; sm_100a kernels are disabled, using PyTorch operators.",
                    device_ctx.capability,
                )
                self._priority_map["cuda"] = {op: [slow] for op, (_f, slow) in _PAIRS.items()}
            elif not _EXT_AVAILABLE and os.getenv("RL_KERNEL_ALLOW_FALLBACK") != "1":
                self._strict_missing_ext = True
        except Exception as exc:  # pragma: no cover
            logger.warning("Failed to probe device capability: %s", exc)

    def _adjust_priority_from_env(self) -> None:
        """``RL_KERNEL_FORCE_BACKEND=pytorch`` forces the oracle operators (debugging aid)."""
        forced = os.getenv("RL_KERNEL_FORCE_BACKEND", "").strip().lower()
        if forced in {"pytorch", "native", "reference"}:
            self._priority_map["cuda"] = {op: [slow] for op, (_f, slow) in _PAIRS.items()}
        elif forced and forced not in {"sm100", "auto"}:
            logger.warning("Unknown RL_KERNEL_FORCE_BACKEND=%s; keeping the default priorities.", forced)

    _strict_missing_ext = False

    # -- lookup ----------------------------------------------------------------------------
    def op_types(self) -> List[str]:
        return sorted(_PAIRS)

    def get_op(self, op_type: str) -> Any:
        platform = "cuda" if device_ctx.device_type == "cuda" else "cpu"
        candidates = self._priority_map.get(platform, {}).get(op_type, [OpBackend.PYTORCH_NATIVE])
        if self._strict_missing_ext and platform == "cuda":
            raise RuntimeError(
                "rl_engine._C is not built but a Blackwell GPU is present; build it with "
                "`python setup.py build_ext --inplace` or set RL_KERNEL_ALLOW_FALLBACK=1."
            )
        for backend in candidates:
            cached = self._instance_cache.get(backend.name)
            if cached is not None:
                return cached
            if backend.name in self._failed_backends:
                continue
            op_class = self._load_backend(backend)
            if op_class is None:
                self._failed_backends.add(backend.name)
                continue
            try:
                instance = op_class()
            except Exception as exc:
                logger.error("Failed to instantiate %s: %s", backend.name, exc)
                self._failed_backends.add(backend.name)
                continue
            self._instance_cache[backend.name] = instance
            return instance
        raise RuntimeError(f"No functional backend found for {op_type} on {platform}")

    def _load_backend(self, backend: OpBackend) -> Optional[Type]:
        module_path, class_name = backend.value.rsplit(".", 1)
        try:
            return getattr(importlib.import_module(module_path), class_name)
        except (ImportError, AttributeError) as exc:
            missing = str(getattr(exc, "name", "") or "")
            backend_itself = bool(missing) and (missing == module_path or module_path.startswith(missing))
            if missing and "rl_engine" in missing and not backend_itself:
                logger.critical("Internal wrapper implementation bug in '%s': %s", module_path, exc)
                raise
            logger.warning("Backend %s unavailable: %s. Falling back...", backend.name, exc)
            return None


kernel_registry = KernelRegistry()
