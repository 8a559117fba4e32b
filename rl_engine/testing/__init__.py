"""Reference math and synthetic RL-shaped batches used by tests, benchmarks and executors."""

from rl_engine.testing.reference_ops import (
    active_token_count, compute_policy_ratio, compute_reference_kl, masked_mean, masked_sum, selected_logprobs_reference,
    summarize_kernel_drift,
)
from rl_engine.testing.rl_batch import SyntheticRLKernelBatch, make_synthetic_rl_kernel_batch

__all__ = [
    "SyntheticRLKernelBatch", "active_token_count", "compute_policy_ratio", "compute_reference_kl",
    "make_synthetic_rl_kernel_batch", "masked_mean", "masked_sum", "selected_logprobs_reference", "summarize_kernel_drift",
]
