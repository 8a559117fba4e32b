"""Paged-KV scoring baseline: what a generation-style engine would reserve for the same scoring job.

Parity: ``rl_engine/executors/paged_kv_baseline.py:28-413`` — really allocates
``[layers, blocks, block, kv_heads, head_dim]`` K and V tensors plus an int32 block table, runs the
model with ``use_cache=True`` and reports reserved / payload / metadata MiB next to the same scoring
outputs the stateless executor produces, so the two can be compared line by line.
"""

from __future__ import annotations

import time
from dataclasses import dataclass
from typing import Any, Dict, Optional

import torch

from rl_engine.executors.stateless_executor import (
    StatelessForwardInputs, StatelessForwardOutputs, StatelessForwardResult, TensorTreeSummary, _accepts, _logits_of,
    default_reward_adapter, extract_kv_cache_outputs, score_reference_logprobs, score_rewards, summarize_tensor_tree,
)


@dataclass(frozen=True)
class PagedKVScoringConfig:
    mode: str = "reference"
    num_layers: int = 4
    num_kv_heads: int = 8
    head_dim: int = 32
    block_size: int = 16
    kv_cache_dtype: torch.dtype = torch.float16
    kv_cache_blocks: Optional[int] = None
    use_cache: bool = True
    detach_outputs: bool = True
    return_token_scores: bool = False
    temperature: float = 1.0
    output_dtype: torch.dtype = torch.float32

    def __post_init__(self) -> None:
        if self.mode not in {"reference", "reward", "both"}:
            raise ValueError("mode must be 'reference', 'reward', or 'both'")
        for name in ("num_layers", "num_kv_heads", "head_dim", "block_size"):
            if getattr(self, name) <= 0:
                raise ValueError(f"{name} must be greater than zero")
        if self.kv_cache_blocks is not None and self.kv_cache_blocks <= 0:
            raise ValueError("kv_cache_blocks must be greater than zero")
        if not self.use_cache:
            raise ValueError("PagedKVScoringConfig.use_cache must be True")
        if self.temperature <= 0.0:
            raise ValueError("temperature must be greater than zero")


@dataclass(frozen=True)
class PagedKVCacheReservation:
    key_cache: torch.Tensor
    value_cache: torch.Tensor
    block_tables: torch.Tensor
    sequence_lengths: torch.Tensor
    blocks_per_sequence: torch.Tensor
    block_size: int
    required_blocks: int
    reserved_blocks: int
    cache_bytes: int
    metadata_bytes: int
    reserved_bytes: int = -1          # cache + metadata when not given

    def __post_init__(self) -> None:
        if self.reserved_bytes < 0:
            object.__setattr__(self, "reserved_bytes", int(self.cache_bytes) + int(self.metadata_bytes))

    @property
    def reserved_mb(self) -> float:
        return self.reserved_bytes / 1_048_576.0


def reserve_paged_kv_cache(inputs: StatelessForwardInputs, config: PagedKVScoringConfig) -> PagedKVCacheReservation:
    lengths = inputs.attention_mask.to(torch.bool).sum(dim=1)
    if bool((lengths <= 0).any()):
        raise ValueError("attention_mask must contain at least one token per sequence")
    per_seq = torch.div(lengths + config.block_size - 1, config.block_size, rounding_mode="floor")
    required = int(per_seq.sum())
    reserved = required if config.kv_cache_blocks is None else int(config.kv_cache_blocks)
    if reserved < required:
        raise ValueError(f"kv_cache_blocks={reserved} cannot fit required blocks={required}")
    device = inputs.input_ids.device
    shape = (config.num_layers, reserved, config.block_size, config.num_kv_heads, config.head_dim)
    key_cache = torch.zeros(shape, dtype=config.kv_cache_dtype, device=device)
    value_cache = torch.zeros(shape, dtype=config.kv_cache_dtype, device=device)
    max_blocks = int(per_seq.max())
    table = torch.full((inputs.input_ids.shape[0], max_blocks), -1, dtype=torch.int32, device=device)
    cursor = 0
    for row, n in enumerate(per_seq.tolist()):
        table[row, :n] = torch.arange(cursor, cursor + n, dtype=torch.int32, device=device)
        cursor += n
    nbytes = lambda t: t.numel() * t.element_size()
    return PagedKVCacheReservation(
        key_cache=key_cache, value_cache=value_cache, block_tables=table, sequence_lengths=lengths,
        blocks_per_sequence=per_seq, block_size=int(config.block_size), required_blocks=required, reserved_blocks=reserved, cache_bytes=nbytes(key_cache) + nbytes(value_cache),
        metadata_bytes=nbytes(table) + nbytes(lengths) + nbytes(per_seq),
    )


def collect_paged_kv_metrics(inputs, config, reservation, *, elapsed_seconds: float, use_cache_passed: bool,
                             model_kv_cache_summary: TensorTreeSummary, cuda_tracking: bool) -> Dict[str, Any]:
    ids = inputs.input_ids
    total = reservation.cache_bytes + model_kv_cache_summary.total_bytes
    metrics: Dict[str, Any] = {
        "baseline_kind": "generation_engine_paged_kv_reservation",
        "baseline_includes_model_kv_cache": model_kv_cache_summary.tensor_count > 0,
        "mode": config.mode,
        "batch_size": int(ids.shape[0]),
        "sequence_len": int(ids.shape[1]),
        "active_completion_tokens": int(inputs.completion_mask.to(torch.bool).sum()),
        "attention_tokens": int(reservation.sequence_lengths.sum()),
        "device": str(ids.device),
        "dtype": str(ids.dtype).replace("torch.", ""),
        "kv_cache_dtype": str(config.kv_cache_dtype).replace("torch.", ""),
        "elapsed_ms": elapsed_seconds * 1000.0,
        "use_cache": True,
        "use_cache_passed": bool(use_cache_passed),
        "detached_outputs": bool(config.detach_outputs),
        "paged_kv_layers": config.num_layers,
        "paged_kv_heads": config.num_kv_heads,
        "paged_kv_head_dim": config.head_dim,
        "paged_kv_block_size": config.block_size,
        "paged_kv_required_blocks": reservation.required_blocks,
        "paged_kv_blocks": reservation.reserved_blocks,
        "paged_kv_max_blocks_per_sequence": int(reservation.block_tables.shape[1]),
        "paged_kv_cache_reserved_mb": reservation.reserved_bytes / 1_048_576.0,
        "paged_kv_cache_payload_mb": reservation.cache_bytes / 1_048_576.0,
        "paged_kv_metadata_mb": reservation.metadata_bytes / 1_048_576.0,
        "model_kv_cache_output_present": model_kv_cache_summary.tensor_count > 0,
        "model_kv_cache_output_tensors": model_kv_cache_summary.tensor_count,
        "model_kv_cache_output_bytes": model_kv_cache_summary.total_bytes,
        "model_kv_cache_output_mb": model_kv_cache_summary.total_mb,
        "total_kv_cache_bytes": total,
        "total_kv_cache_mb": total / 1_048_576.0,
    }
    if cuda_tracking:
        metrics["peak_allocated_mb"] = torch.cuda.max_memory_allocated(ids.device) / 1_048_576.0
        metrics["peak_reserved_mb"] = torch.cuda.max_memory_reserved(ids.device) / 1_048_576.0
    return metrics


class PagedKVScoringBaseline:
    def __init__(self, model: torch.nn.Module, config: Optional[PagedKVScoringConfig] = None, *, reward_adapter=None) -> None:
        self.model = model
        self.config = config or PagedKVScoringConfig()
        self.reward_adapter = reward_adapter or default_reward_adapter

    def score(self, inputs: StatelessForwardInputs) -> StatelessForwardResult:
        cfg = self.config
        ids = inputs.input_ids
        if ids.ndim != 2 or inputs.attention_mask.shape != ids.shape or inputs.completion_mask.shape != ids.shape:
            raise ValueError("input_ids, attention_mask and completion_mask must share shape [B, S]")
        tracking = ids.device.type == "cuda" and torch.cuda.is_available()
        if tracking:
            torch.cuda.reset_peak_memory_stats(ids.device)
            torch.cuda.synchronize(ids.device)
        t0 = time.perf_counter()
        reservation = reserve_paged_kv_cache(inputs, cfg)
        with torch.no_grad():
            kwargs: Dict[str, Any] = {}
            if _accepts(self.model, "attention_mask"):
                kwargs["attention_mask"] = inputs.attention_mask
            passed = _accepts(self.model, "use_cache")
            if passed:
                kwargs["use_cache"] = True
            raw = self.model(ids, **kwargs)
            model_kv = summarize_tensor_tree(extract_kv_cache_outputs(raw))
            outputs = StatelessForwardOutputs(raw=raw, logits=_logits_of(raw), kv_cache=extract_kv_cache_outputs(raw))
            ref = rewards = tokens = None
            if cfg.mode in {"reference", "both"}:
                if outputs.logits is None:
                    raise ValueError("reference mode requires model outputs to expose logits")
                ref = score_reference_logprobs(outputs.logits, inputs, temperature=cfg.temperature, output_dtype=cfg.output_dtype)
                tokens = ref if cfg.return_token_scores else None
            if cfg.mode in {"reward", "both"}:
                rewards = score_rewards(outputs, inputs, reward_adapter=self.reward_adapter, output_dtype=cfg.output_dtype)
            if cfg.detach_outputs:
                ref, rewards, tokens = (None if t is None else t.detach() for t in (ref, rewards, tokens))
        if tracking:
            torch.cuda.synchronize(ids.device)
        metrics = collect_paged_kv_metrics(
            inputs, cfg, reservation, elapsed_seconds=time.perf_counter() - t0, use_cache_passed=passed,
            model_kv_cache_summary=model_kv, cuda_tracking=tracking,
        )
        return StatelessForwardResult(reference_logps=ref, rewards=rewards, token_scores=tokens, metrics=metrics)
