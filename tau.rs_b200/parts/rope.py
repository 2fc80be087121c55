"""Rotate-half rotary position encoding: the tables.

crates/models/src/components/rope.rs:91-108: `inv_freq = 1f32 / (theta^(i/rot) as f32)`
for even `i` (the power in 64-bit), angle = position (32-bit) times `inv_freq` in 32-bit,
tables of its cosine and sine kept in 32-bit.  The rotation itself pairs element `j`
with `j + rot/2` (crates/cuda-kernels/src/kernels/decode_attention.cu:50-62) and runs
inside the attention part's prepare kernel, which reads these tables; elements beyond
`rotary_dim` pass through (rope.rs:141-153).
"""
from __future__ import annotations

import torch

from .base import Part
from .registry import register_position


_TABLES = {}


@register_position("rope_half")
class RotaryTables(Part):
    def __init__(self, spec, device):
        if spec.rotary_dim % 2 != 0 or spec.rotary_dim <= 0:
            raise ValueError(f"rotary_dim must be a positive even number, found {spec.rotary_dim}")
        self.spec = spec
        self.cos = self.sin = None
        self.device = device

    def finalize_weights(self):
        spec = self.spec
        key = (spec, str(self.device))
        if key in _TABLES:          # layers with the same encoding share one pair of tables
            self.cos, self.sin = _TABLES[key]
            return
        power = torch.tensor(
            [float(spec.theta) ** (index / spec.rotary_dim) for index in range(0, spec.rotary_dim, 2)],
            dtype=torch.float64,
        ).to(torch.float32)
        inverse = torch.ones_like(power) / power
        positions = torch.arange(spec.max_positions, dtype=torch.float32)
        angles = positions[:, None] * inverse[None, :]
        self.cos = torch.cos(angles).contiguous().to(self.device)
        self.sin = torch.sin(angles).contiguous().to(self.device)
        _TABLES[key] = (self.cos, self.sin)


@register_position("rope_pairs")
class PairRotation(Part):
    """Rotation of neighbouring pairs: element `2i` with `2i + 1`, by the angle `position * theta^(-2i / rotary_dim)`.

    Holds the frequencies alone (`inv_freq`, float32 `[rotary_dim / 2]`, the power taken in 64-bit and rounded once); the
    kernels that rotate multiply them by the position and take sine and cosine in 32-bit themselves, so no table over
    positions exists and no position is too large for one."""

    def __init__(self, spec, device):
        if spec.rotary_dim % 2 != 0 or spec.rotary_dim <= 0:
            raise ValueError(f"rotary_dim must be a positive even number, found {spec.rotary_dim}")
        self.spec, self.device = spec, device
        self.inv_freq = None

    def finalize_weights(self):
        spec = self.spec
        values = [float(spec.theta) ** (-2.0 * index / spec.rotary_dim) for index in range(spec.rotary_dim // 2)]
        self.inv_freq = torch.tensor(values, dtype=torch.float64).to(torch.float32).to(self.device)


@register_position("rope_half_scaled")
class ScaledHalfRotation(Part):
    """Rotation of element `i` with element `i + rotary_dim / 2`, with frequencies that may be blended between the plain ones and
    ones slowed down by a factor (`ScaledRotationSpec` states the rule), and a factor on sine and cosine.

    Holds the frequencies (`frequency`, float32 `[rotary_dim / 2]`, computed in 64-bit and rounded once) and `magnitude`; the
    kernels that rotate multiply the frequencies by the position and take sine and cosine in 32-bit themselves, so no table over
    positions exists."""

    def __init__(self, spec, device):
        if spec.rotary_dim % 2 != 0 or spec.rotary_dim <= 0:
            raise ValueError(f"rotary_dim must be a positive even number, found {spec.rotary_dim}")
        self.spec, self.device = spec, device
        self.frequency = None
        self.magnitude = 1.0

    def values(self):
        """The frequencies as Python floats, and the magnitude."""
        import math

        spec = self.spec
        dims = spec.rotary_dim
        plain = [float(spec.theta) ** (-2.0 * index / dims) for index in range(dims // 2)]
        if spec.factor is None:
            return plain, 1.0

        def index_of(turns):
            return dims * math.log(spec.original / (2.0 * math.pi * turns)) / (2.0 * math.log(spec.theta))

        low = max(math.floor(index_of(spec.fast)), 0)
        high = min(math.ceil(index_of(spec.slow)), dims - 1)
        blended = []
        for index, frequency in enumerate(plain):
            ramp = min(max((index - low) / max(high - low, 0.001), 0.0), 1.0)
            blended.append(frequency / spec.factor * ramp + frequency * (1.0 - ramp))
        return blended, 0.1 * math.log(spec.factor) + 1.0

    def finalize_weights(self):
        values, self.magnitude = self.values()
        self.frequency = torch.tensor(values, dtype=torch.float64).to(torch.float32).to(self.device)
