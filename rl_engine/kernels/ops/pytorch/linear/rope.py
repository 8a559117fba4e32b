"""CPU/PyTorch oracle for rotary position embedding (half-split / "NeoX" layout).

The reference has no RoPE operator; Llama-3 and Qwen3 both need one, so it is added here with
the same ``forward`` / ``forward_fp32`` contract as the other elementwise oracles.
``x`` is ``[..., seq, heads, head_dim]`` and ``positions`` is ``[..., seq]`` (integer).
"""

from __future__ import annotations

import torch


def scaled_inv_freq(inv_freq: torch.Tensor, scaling) -> torch.Tensor:
    """Rotary frequencies under a context-extension rule.  ``scaling`` is ``None`` or a tuple
    ``(kind, factor, low_freq_factor, high_freq_factor, original_max_positions)``:

    * ``"linear"``: every frequency divided by ``factor`` (position interpolation);
    * ``"llama3"`` (Llama-3.1 and later): wavelengths longer than ``original / low_freq_factor`` are divided by
      ``factor``, those shorter than ``original / high_freq_factor`` are kept, and the band between is blended
      linearly in ``original / wavelength``."""
    if scaling is None:
        return inv_freq
    kind, factor, low, high, original = scaling
    if kind == "linear":
        return inv_freq / float(factor)
    if kind != "llama3":
        raise ValueError(f"rope scaling {kind!r} is not supported (known: 'linear', 'llama3')")
    wavelen = 2.0 * torch.pi / inv_freq
    scaled = torch.where(wavelen > original / low, inv_freq / factor, inv_freq)
    smooth = (original / wavelen - low) / (high - low)
    blended = (1.0 - smooth) * scaled / factor + smooth * scaled
    medium = ~(wavelen < original / high) & ~(wavelen > original / low)
    return torch.where(medium, blended, scaled)


def rope_cos_sin(positions: torch.Tensor, head_dim: int, theta: float = 10000.0, scaling=None):
    half = head_dim // 2
    inv_freq = theta ** (-torch.arange(half, dtype=torch.float32, device=positions.device) / half)
    inv_freq = scaled_inv_freq(inv_freq, scaling)
    ang = positions.to(torch.float32)[..., None] * inv_freq
    return torch.cos(ang), torch.sin(ang)


class NativeRoPEOp:
    def __call__(self, x, positions, *, theta: float = 10000.0, scaling=None):
        return self.forward(x, positions, theta=theta, scaling=scaling)

    def forward(self, x, positions, *, theta: float = 10000.0, scaling=None):
        return self.forward_fp32(x, positions, theta=theta, scaling=scaling).to(x.dtype)

    def forward_fp32(self, x, positions, *, theta: float = 10000.0, scaling=None):
        d = x.shape[-1]
        if d % 2:
            raise ValueError(f"head_dim must be even, got {d}")
        cos, sin = rope_cos_sin(positions, d, theta, scaling)
        cos, sin = cos[..., None, :], sin[..., None, :]  # broadcast over heads
        xf = x.float()
        a, b = xf[..., : d // 2], xf[..., d // 2 :]
        return torch.cat([a * cos - b * sin, b * cos + a * sin], dim=-1)
