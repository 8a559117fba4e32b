"""CPU/PyTorch oracle for rotary position embedding (half-split / "NeoX" layout).

The reference has no RoPE operator; Llama-3 and Qwen3 both need one, so it is added here with
the same ``forward`` / ``forward_fp32`` contract as the other elementwise oracles.
``x`` is ``[..., seq, heads, head_dim]`` and ``positions`` is ``[..., seq]`` (integer).
"""

from __future__ import annotations

import torch


def rope_cos_sin(positions: torch.Tensor, head_dim: int, theta: float = 10000.0):
    half = head_dim // 2
    inv_freq = theta ** (-torch.arange(half, dtype=torch.float32, device=positions.device) / half)
    ang = positions.to(torch.float32)[..., None] * inv_freq
    return torch.cos(ang), torch.sin(ang)


class NativeRoPEOp:
    def __call__(self, x, positions, *, theta: float = 10000.0):
        return self.forward(x, positions, theta=theta)

    def forward(self, x, positions, *, theta: float = 10000.0):
        return self.forward_fp32(x, positions, theta=theta).to(x.dtype)

    def forward_fp32(self, x, positions, *, theta: float = 10000.0):
        d = x.shape[-1]
        if d % 2:
            raise ValueError(f"head_dim must be even, got {d}")
        cos, sin = rope_cos_sin(positions, d, theta)
        cos, sin = cos[..., None, :], sin[..., None, :]  # broadcast over heads
        xf = x.float()
        a, b = xf[..., : d // 2], xf[..., d // 2 :]
        return torch.cat([a * cos - b * sin, b * cos + a * sin], dim=-1)
