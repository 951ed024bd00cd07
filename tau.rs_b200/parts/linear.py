"""`y = x W^T + b` with `W` stored `[out, in]`, several named weights stacked into one.

crates/cuda-kernels/src/kernels/linear_bf16_fp32.cuh:31-33 (the row-major `[N, K]`
weight is the transposed operand as it lies); crates/models/src/components/mlp/
projection.rs:45-68 (gate and up stacked into one `[2I, H]` weight when the model is
built, so that one product serves both).
"""
from __future__ import annotations

from typing import Optional, Sequence, Tuple

import torch

from ..csrc import kernels
from ..weights.tensor_spec import TensorSpec
from .base import Part


class StackedLinear(Part):
    """One product for several checkpoint tensors that share their input.

    `pieces` lists `(name prefix, out features)`; the tensors `<prefix>.weight` (and
    `<prefix>.bias` if `bias`) are stacked along the output axis in that order.
    """

    def __init__(self, pieces: Sequence[Tuple[str, int]], in_features: int, bias: bool, dtype, device, interleave: int = 0):
        """`interleave` > 0 (two pieces of equal size, no bias): rows are stored in groups of `interleave` rows of the
        first piece followed by the matching rows of the second, which is what a gated product reads."""
        self.interleave = interleave
        self.pieces = list(pieces)
        self.in_features = in_features
        self.out_features = sum(width for _, width in self.pieces)
        self.has_bias = bias
        self.dtype, self.device = dtype, device
        self._parts = {}
        self.weight: Optional[torch.Tensor] = None
        self.bias: Optional[torch.Tensor] = None

    def tensor_specs(self):
        specs = {}
        for prefix, width in self.pieces:
            specs[f"{prefix}.weight"] = TensorSpec((width, self.in_features), role="matrix")
            if self.has_bias:
                specs[f"{prefix}.bias"] = TensorSpec((width,), role="vector")
        return specs

    def assign(self, name, tensor):
        if name not in self.tensor_specs():
            raise KeyError(name)
        self._parts[name] = tensor

    def finalize_weights(self):
        weights = [self._parts.pop(f"{prefix}.weight") for prefix, _ in self.pieces]
        if self.interleave:
            first, second = weights
            group, width = self.interleave, first.shape[1]
            self.weight = torch.stack([first.view(-1, group, width), second.view(-1, group, width)], dim=1).reshape(-1, width).contiguous()
        else:
            self.weight = weights[0] if len(weights) == 1 else torch.cat(weights, dim=0).contiguous()
        del weights
        if self.has_bias:
            biases = [self._parts.pop(f"{prefix}.bias") for prefix, _ in self.pieces]
            self.bias = biases[0] if len(biases) == 1 else torch.cat(biases, dim=0).contiguous()

    def forward_gated(self, values):
        """`silu(first piece) * second piece`, for a stack built with `interleave`."""
        out = torch.empty((values.shape[0], self.out_features // 2), dtype=values.dtype, device=values.device)
        kernels.linear_gated(values, self.weight, out)
        return out

    def forward(self, values, out_dtype=None, rows: Optional[int] = None):
        """`rows` limits the product to the first `rows` output features (a prefix of the stack)."""
        weight, bias = self.weight, self.bias
        if rows is not None and rows != self.out_features:
            weight = weight[:rows]
            bias = bias[:rows] if bias is not None else None
        out = torch.empty((values.shape[0], weight.shape[0]), dtype=out_dtype or values.dtype, device=values.device)
        kernels.linear(values, weight, bias, out)
        return out
