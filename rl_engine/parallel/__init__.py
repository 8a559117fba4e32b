"""Multi-GPU pieces: the symmetric heap (peer-mapped memory over NVLink), device-side barriers with
bounded waits, the fused reduce-scatter + AdamW + all-gather optimizer step, the in-kernel
vocab-parallel log-prob merge and the trainer -> rollout weight broadcast."""

from rl_engine.parallel.symmetric import PeerTimeoutError, SymmetricMemory

__all__ = ["PeerTimeoutError", "SymmetricMemory"]
