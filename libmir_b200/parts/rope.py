"""Rotary position encoding.  Half-split layout: dims i and i + r/2 of the first r dims form a pair; interleaved
layout: dims 2i and 2i + 1.

inverse frequency f_i = theta^(-2i/r) (libmir cuda/kernels/qkv_postprocess_bf16.cu:37-69), optionally
remapped by the llama3 piecewise rule (metal/src/engine/attention/rope.rs:58-96, keys
models/src/layout/decoder/rope.rs:61-95).  The table is computed once in 64-bit and held in 32-bit;
the angle position * f_i is a 32-bit product inside the kernel that applies it.

YaRN scaling (YarnScaling): with r the rotated dims, pair i turns original * f_i / (2 pi) times over `original`
positions; the pair index at which a pair turns t times is d(t) = r ln(original / (2 pi t)) / (2 ln theta).  Between
lo = max(floor(d(fast)), 0) and hi = min(ceil(d(slow)), r - 1) a ramp clamp((i - lo) / max(hi - lo, 0.001), 0, 1)
blends f_i (ramp 0) into f_i / factor (ramp 1), and cos and sin are multiplied by 0.1 ln(factor) + 1 (`magnitude`).
"""

from __future__ import annotations

import math

import torch

from ..config.spec import YarnScaling
from .base import Position


def yarn_magnitude(scaling) -> float:
    """What cos and sin are multiplied by: 1 unless the scaling is YaRN's."""
    return 0.1 * math.log(scaling.factor) + 1.0 if isinstance(scaling, YarnScaling) else 1.0


def inverse_frequencies(rotary_dim: int, theta: float, scaling=None) -> torch.Tensor:
    index = torch.arange(0, rotary_dim, 2, dtype=torch.float64)
    inverse = torch.pow(torch.tensor(theta, dtype=torch.float64), -index / rotary_dim)
    if isinstance(scaling, YarnScaling):
        at = lambda turns: rotary_dim * math.log(scaling.original / (2.0 * math.pi * turns)) / (2.0 * math.log(theta))
        low = max(math.floor(at(scaling.fast)), 0)
        high = min(math.ceil(at(scaling.slow)), rotary_dim - 1)
        ramp = ((torch.arange(rotary_dim // 2, dtype=torch.float64) - low) / max(high - low, 0.001)).clamp(0, 1)
        inverse = inverse / scaling.factor * ramp + inverse * (1.0 - ramp)
    elif scaling is not None:
        wavelength = 2.0 * math.pi / inverse
        ratio = scaling.original_max_position_embeddings / wavelength
        smooth = ((ratio - scaling.low_freq_factor) / (scaling.high_freq_factor - scaling.low_freq_factor)).clamp(0, 1)
        inverse = (inverse / scaling.factor) * (1.0 - smooth) + inverse * smooth
    return inverse.to(torch.float32)


class Rotary(Position):
    """Owned by a mixer; `table` is what its kernel multiplies positions with."""

    graph_safe = True

    def __init__(self, spec, env):
        super().__init__(spec, env)
        if spec.rotary_dim % 2 or not 0 <= spec.rotary_dim <= spec.head_dim:
            raise ValueError(f"rotary_dim {spec.rotary_dim} must be even and at most head_dim {spec.head_dim}")
        if spec.layout not in ("half", "interleaved"):
            raise ValueError(f"unknown rotary layout {spec.layout!r}")
        self.rotary_dim = spec.rotary_dim
        self.table = inverse_frequencies(spec.rotary_dim, spec.theta, spec.scaling).to(env.device)
        self.interleaved = spec.layout == "interleaved"
        self.magnitude = yarn_magnitude(spec.scaling)

    def rotation(self):
        """The table for kernels that apply the half-split rotation with cos and sin as they are; None for the other
        layout or a magnitude, which only kernels that take `interleaved` and `magnitude` apply."""
        if self.interleaved or self.magnitude != 1.0:
            return None
        return self.table, self.rotary_dim
