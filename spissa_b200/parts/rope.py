"""Rotary position encoding. ``pairing`` "half" (the default): dim i pairs with i + rotary_dim/2;
"interleaved": dim 2i pairs with dim 2i+1. Either way pair i turns by position · inv_freq_i.

angle = position · inv_freq_i with inv_freq_i = 1 / θ^(2i/rotary_dim), all in 32-bit
(crates/spissa-runtime/src/rotary.rs:454-465); the rotation itself happens in the
kernel that writes the cache (rotary.rs:98-123, :467-481).

``scaling`` of type ``llama3`` rescales the frequency table once (not in the
reference, which drops it: crates/spissa-import/src/safetensors.rs:163-175). With
λ = 2π/inv_freq: λ > n0/low ⇒ inv_freq/factor; λ < n0/high ⇒ unchanged; between,
(1−s)·inv_freq/factor + s·inv_freq with s = (n0/λ − low)/(high − low).
``linear`` divides every frequency by ``factor``.

``ramp`` (not in the reference) interpolates pair by pair: with pair(t) = dims · ln(n0 / (2π t)) / (2 ln θ) the pair
that turns t times over the original length n0, lo = max(⌊pair(fast)⌋, 0), hi = min(⌈pair(slow)⌉, dims − 1) and
r_i = clamp((i − lo) / max(hi − lo, 0.001), 0, 1), pair i turns at inv_freq_i / factor · r_i + inv_freq_i · (1 − r_i),
and cos and sin are both multiplied by the ``amplitude`` 0.1 · ln(factor) + 1. Computed in 64-bit, rounded once.
"""
from __future__ import annotations

import math

import torch

from .base import PositionEncoding
from .registry import register_part


def rotary_inv_freq(theta: float, rotary_dim: int, scaling: dict | None) -> torch.Tensor:
    """The float32 frequency table [rotary_dim/2], computed on the host in 32-bit."""
    if rotary_dim <= 0 or rotary_dim % 2:
        raise ValueError(f"rotary_dim must be a positive even number, got {rotary_dim}")
    exponent = torch.arange(0, rotary_dim, 2, dtype=torch.float32) / float(rotary_dim)
    inv_freq = 1.0 / torch.pow(torch.tensor(float(theta), dtype=torch.float32), exponent)
    if not scaling:
        return inv_freq
    kind = scaling.get("rope_type", scaling.get("type"))
    if kind in (None, "default"):
        return inv_freq
    factor = float(scaling["factor"])
    if kind == "linear":
        return inv_freq / factor
    if kind == "llama3":
        low = float(scaling["low_freq_factor"])
        high = float(scaling["high_freq_factor"])
        n0 = float(scaling["original_max_position_embeddings"])
        wavelen = 2.0 * math.pi / inv_freq
        smooth = (n0 / wavelen - low) / (high - low)
        blended = (1.0 - smooth) * inv_freq / factor + smooth * inv_freq
        out = torch.where(wavelen > n0 / low, inv_freq / factor, inv_freq)
        medium = (wavelen <= n0 / low) & (wavelen >= n0 / high)
        return torch.where(medium, blended, out).to(torch.float32)
    if kind == "ramp":
        n0, fast, slow = float(scaling["original"]), float(scaling["fast"]), float(scaling["slow"])

        def pair_of(turns: float) -> float:
            return rotary_dim * math.log(n0 / (2.0 * math.pi * turns)) / (2.0 * math.log(float(theta)))
        lo = max(math.floor(pair_of(fast)), 0)
        hi = min(math.ceil(pair_of(slow)), rotary_dim - 1)
        out = []
        for i in range(rotary_dim // 2):
            f = float(theta) ** (-2.0 * i / rotary_dim)
            r = min(1.0, max(0.0, (i - lo) / max(hi - lo, 0.001)))
            out.append(f / factor * r + f * (1.0 - r))
        return torch.tensor(out, dtype=torch.float64).to(torch.float32)
    raise ValueError(f"unsupported rope scaling type {kind!r}")


def rotary_amplitude(scaling: dict | None) -> float:
    """What multiplies cos and sin: 1, or 0.1 · ln(factor) + 1 for the ``ramp`` scaling."""
    if scaling and scaling.get("rope_type", scaling.get("type")) == "ramp":
        return 0.1 * math.log(float(scaling["factor"])) + 1.0
    return 1.0


@register_part("position", "rotary")
class RotaryEncoding(PositionEncoding):
    graph_safe = True

    def __init__(self, theta: float, rotary_dim: int, scaling: dict | None = None, prefix: str = "",
                 pairing: str = "half"):
        super().__init__(prefix)
        if pairing not in ("half", "interleaved"):
            raise ValueError(f"rotary pairing is 'half' or 'interleaved', got {pairing!r}")
        self.pairing = pairing                  # which dims form a pair; the mixer's kernel must know the layout
        self.theta = float(theta)
        self.rotary_dim = int(rotary_dim)
        self.scaling = dict(scaling) if scaling else None
        self.inv_freq_host = rotary_inv_freq(self.theta, self.rotary_dim, self.scaling)
        self.amplitude = rotary_amplitude(self.scaling)     # multiplies cos and sin (the kernel that rotates must take it)
        self.inv_freq = None

    def bind(self, tensors, rt):
        super().bind(tensors, rt)
        self.inv_freq = self.inv_freq_host.to(rt.device)

    def rotary(self):
        """(frequency table on the device, rotary_dim) for the fused rotate-and-store kernel."""
        return self.inv_freq, self.rotary_dim
