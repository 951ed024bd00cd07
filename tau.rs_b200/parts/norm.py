"""RMSNorm: `x * rsqrt(mean(x^2) + eps) * w`, statistic in 32-bit, one rounding.

crates/models/src/components/rms_norm.rs:205-210 and :147-150; the in-tree norm scales
by `1 + w`, this part by `w`.  The fused form first rounds `residual + branch` to the
storage dtype and normalises that (rms_norm.rs:39-74;
crates/cuda-kernels/src/kernels/centered_rms_norm.cu:267-308).
"""
from __future__ import annotations

import torch

from ..csrc import kernels
from ..weights.tensor_spec import TensorSpec
from .base import Norm
from .registry import register_norm


@register_norm("rms_norm")
class RMSNorm(Norm):
    def __init__(self, spec, name: str, dtype, device):
        self.spec, self.name = spec, name
        self.weight = None

    def tensor_specs(self):
        return {self.name: TensorSpec((self.spec.width,), role="vector", init="ones")}

    def assign(self, name, tensor):
        if name != self.name:
            raise KeyError(name)
        self.weight = tensor

    def forward(self, values, rows=None, branch=None):
        count = values.shape[0] if rows is None else rows.shape[0]
        out = torch.empty((count, self.spec.width), dtype=values.dtype, device=values.device)
        kernels.rms_norm(values, self.weight, self.spec.eps, out, rows, branch)
        return out

    def add_forward(self, branch, residual):
        out = torch.empty_like(residual)
        kernels.add_rms_norm(branch, residual, self.weight, self.spec.eps, out)
        return out
