"""CPU/PyTorch oracle for rotary position embedding (half-split / "NeoX" layout).

The reference has no RoPE operator; Llama-3 and Qwen3 both need one, so it is added here with
the same ``forward`` / ``forward_fp32`` contract as the other elementwise oracles.
``x`` is ``[..., seq, heads, head_dim]`` and ``positions`` is ``[..., seq]`` (integer).
"""

from __future__ import annotations

import math

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
        raise ValueError(f"rope scaling {kind!r} is not supported (known: 'linear', 'llama3', 'yarn')")
    wavelen = 2.0 * torch.pi / inv_freq
    scaled = torch.where(wavelen > original / low, inv_freq / factor, inv_freq)
    smooth = (original / wavelen - low) / (high - low)
    blended = (1.0 - smooth) * scaled / factor + smooth * scaled
    medium = ~(wavelen < original / high) & ~(wavelen > original / low)
    return torch.where(medium, blended, scaled)


def yarn_inv_freq(head_dim: int, theta: float, factor: float, beta_fast: float, beta_slow: float, original: int, device=None):
    """YaRN ("NTK by parts"): dimensions that turn more than ``beta_fast`` times over the original context keep their
    frequency, those that turn fewer than ``beta_slow`` times are interpolated by ``factor``, a linear ramp in the
    dimension index joins the two; cos and sin are scaled by ``0.1 ln(factor) + 1``.  Returns ``(inv_freq, scale)``."""
    half = head_dim // 2

    def correction_dim(rotations: float) -> float:
        return head_dim * math.log(original / (rotations * 2.0 * math.pi)) / (2.0 * math.log(theta))

    low = max(math.floor(correction_dim(beta_fast)), 0)
    high = min(math.ceil(correction_dim(beta_slow)), head_dim - 1)
    if low == high:
        high += 0.001
    ramp = ((torch.arange(half, dtype=torch.float32, device=device) - low) / (high - low)).clamp(0.0, 1.0)
    pos_freqs = theta ** (torch.arange(half, dtype=torch.float32, device=device) / half)
    keep = 1.0 - ramp
    inv_freq = (1.0 / (factor * pos_freqs)) * (1.0 - keep) + (1.0 / pos_freqs) * keep
    return inv_freq, (1.0 if factor <= 1 else 0.1 * math.log(factor) + 1.0)


def rope_cos_sin(positions: torch.Tensor, head_dim: int, theta: float = 10000.0, scaling=None):
    """cos / sin tables ``[..., head_dim / 2]`` for integer ``positions``.  ``scaling``: ``None`` or ``(kind, factor, a, b,
    original_max_positions)`` with kind ``"linear"``, ``"llama3"`` (a, b = low / high frequency factors) or ``"yarn"``
    (a, b = beta_fast, beta_slow)."""
    half = head_dim // 2
    scale = 1.0
    if scaling is not None and scaling[0] == "yarn":
        _, factor, beta_fast, beta_slow, original = scaling
        inv_freq, scale = yarn_inv_freq(head_dim, theta, factor, beta_fast, beta_slow, original, positions.device)
    else:
        inv_freq = theta ** (-torch.arange(half, dtype=torch.float32, device=positions.device) / half)
        inv_freq = scaled_inv_freq(inv_freq, scaling)
    ang = positions.to(torch.float32)[..., None] * inv_freq
    if scale != 1.0:
        return torch.cos(ang) * scale, torch.sin(ang) * scale
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
