"""SwiGLU feed-forward: `down(silu(gate(x)) * up(x))`, no biases.

crates/models/src/components/mlp.rs:99-122,177-191; gate and up are one stacked product
followed by one fused activation kernel (crates/models/src/components/mlp/
projection.rs:123-143; crates/cuda-kernels/src/kernels/silu_and_mul.cu:51-76:
`out[r, c] = silu(in[r, c]) * in[r, I + c]`, in 32-bit with one rounding).
"""
from __future__ import annotations

import torch

from ..csrc import kernels
from .base import FeedForward
from .linear import StackedLinear
from .registry import register_feed_forward


@register_feed_forward("swiglu")
class SwiGLU(FeedForward):
    def __init__(self, spec, prefix: str, dtype, device):
        self.spec = spec
        # Where the gated product exists (bfloat16, aligned sizes) gate and up rows are interleaved for it and the
        # activation is its epilogue; otherwise the two are stacked and the activation is a kernel of its own.
        self.fused = kernels.gated_fits(spec.hidden, spec.intermediate, dtype)
        self.gate_up = StackedLinear(
            [(f"{prefix}.gate_proj", spec.intermediate), (f"{prefix}.up_proj", spec.intermediate)],
            spec.hidden, False, dtype, device, interleave=kernels.GATE_GROUP if self.fused else 0,
        )
        self.down = StackedLinear([(f"{prefix}.down_proj", spec.hidden)], spec.intermediate, False, dtype, device)

    def tensor_specs(self):
        return {**self.gate_up.tensor_specs(), **self.down.tensor_specs()}

    def assign(self, name, tensor):
        part = self.gate_up if name in self.gate_up.tensor_specs() else self.down
        part.assign(name, tensor)

    def finalize_weights(self):
        self.gate_up.finalize_weights()
        self.down.finalize_weights()

    def forward(self, hidden, step):
        if self.fused:
            return self.down.forward(self.gate_up.forward_gated(hidden))
        stacked = self.gate_up.forward(hidden)
        activated = torch.empty((hidden.shape[0], self.spec.intermediate), dtype=hidden.dtype, device=hidden.device)
        kernels.silu_mul(stacked, activated)
        return self.down.forward(activated)
