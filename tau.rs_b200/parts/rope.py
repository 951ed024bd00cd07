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
