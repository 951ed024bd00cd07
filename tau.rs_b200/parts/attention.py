"""Grouped-query softmax attention over the cache, with optional per-head q/k norm and rotation.

Order of operations as in crates/models/src/components/gated_attention.rs:337-372,402:
project; view as heads; normalise each query and key head over `head_dim` (values
untouched); rotate queries and keys at their positions; store keys and values in the
cache; attend over everything the cache holds for the sequence up to each query's own
position (`key <= query position`, crates/models/src/qwen3_5_common/model.rs:154); project
with `o_proj`.  Query head `h` reads KV head `h // (n_heads / n_kv_heads)`
(crates/cuda-kernels/src/kernels/decode_attention.cu:192).  One bias flag covers q, k, v
and o (gated_attention.rs:273-296).  The three input projections are one stacked
product; norm, rotation and the cache write are one kernel
(decode_attention.cu:120-181 does the same for one token).
"""
from __future__ import annotations

import torch

from ..csrc import kernels
from .base import CacheNeed, Mixer
from .linear import StackedLinear
from .registry import build, register_mixer


@register_mixer("attention")
class Attention(Mixer):
    def __init__(self, spec, prefix: str, dtype, device):
        if spec.n_heads % spec.n_kv_heads != 0:
            raise ValueError(f"n_heads ({spec.n_heads}) must be a multiple of n_kv_heads ({spec.n_kv_heads})")
        if spec.head_dim % 16 != 0 or not 16 <= spec.head_dim <= 256:
            raise ValueError(f"head_dim must be a multiple of 16 between 16 and 256, found {spec.head_dim}")
        self.spec, self.prefix = spec, prefix
        q_width, kv_width = spec.n_heads * spec.head_dim, spec.n_kv_heads * spec.head_dim
        self.q_width, self.kv_width = q_width, kv_width
        self.qkv = StackedLinear(
            [(f"{prefix}.q_proj", q_width), (f"{prefix}.k_proj", kv_width), (f"{prefix}.v_proj", kv_width)],
            spec.hidden, spec.bias, dtype, device,
        )
        self.out = StackedLinear([(f"{prefix}.o_proj", spec.hidden)], q_width, spec.bias, dtype, device)
        self.q_norm = self.k_norm = None
        if spec.qk_norm is not None:
            if spec.qk_norm.width != spec.head_dim:
                raise ValueError("the q/k norm runs over head_dim")
            # The prepare and decode kernels compute this norm themselves, from its weight and eps: `x * rsqrt(mean(x^2) + eps) * w`.
            # A norm part of another kind (a centred weight, a bias) would be computed wrongly without a word, so it is refused.
            if spec.qk_norm.kind != "rms_norm":
                raise ValueError(f"the attention kernels compute the q/k norm as rms_norm; a q/k norm of kind {spec.qk_norm.kind!r} is not served")
            self.q_norm = build("norm", spec.qk_norm, name=f"{prefix}.q_norm.weight", dtype=dtype, device=device)
            self.k_norm = build("norm", spec.qk_norm, name=f"{prefix}.k_norm.weight", dtype=dtype, device=device)
        self.position = None
        if spec.position is not None:
            if spec.position.rotary_dim > spec.head_dim:
                raise ValueError("rotary_dim exceeds head_dim")
            self.position = build("position", spec.position, device=device)
        self._children = [part for part in (self.qkv, self.out, self.q_norm, self.k_norm, self.position) if part is not None]

    def cache_need(self):
        return CacheNeed("kv", n_kv_heads=self.spec.n_kv_heads, head_dim=self.spec.head_dim, window=self.spec.window)

    def decode_blocks(self) -> int:
        """Blocks that the decode kernel launches per sequence and context split."""
        group = self.spec.n_heads // self.spec.n_kv_heads
        heads_per_pass = 8 if group >= 8 else 4 if group > 2 else group
        return self.spec.n_kv_heads * -(-group // heads_per_pass)

    def tensor_specs(self):
        specs = {}
        for part in self._children:
            specs.update(part.tensor_specs())
        return specs

    def assign(self, name, tensor):
        for part in self._children:
            if name in part.tensor_specs():
                return part.assign(name, tensor)
        raise KeyError(name)

    def finalize_weights(self):
        for part in self._children:
            part.finalize_weights()

    def forward(self, hidden, step, cache, writes_cache: bool):
        spec = self.spec
        # A run that only reads another run's keys and values needs its queries alone.
        projected = self.qkv.forward(hidden, rows=None if writes_cache else self.q_width)
        context = torch.empty((hidden.shape[0], self.q_width), dtype=hidden.dtype, device=hidden.device)
        pages = step.page_rows[cache.group]
        prepare = (
            None if self.q_norm is None else self.q_norm.weight,
            None if self.k_norm is None else self.k_norm.weight,
            0.0 if spec.qk_norm is None else spec.qk_norm.eps,
            None if self.position is None else self.position.cos,
            None if self.position is None else self.position.sin,
            0 if self.position is None else spec.position.rotary_dim,
        )
        # One token per sequence in bfloat16: norm, rotation, cache write and attention are one kernel.
        if kernels.attention_decode_fused(projected, cache.keys, cache.values, context, step, pages, writes_cache, *prepare,
                                          spec.n_heads, spec.n_kv_heads, spec.head_dim, spec.softmax_scale, spec.window or 0):
            return self.out.forward(context)
        queries = torch.empty_like(context)
        kernels.attention_prepare(projected, queries, cache.keys, cache.values, writes_cache, *prepare,
                                  step.positions, step.token_seq, pages, spec.n_heads, spec.n_kv_heads, spec.head_dim)
        kernels.attention(queries, cache.keys, cache.values, context, step, pages, spec.n_heads, spec.n_kv_heads, spec.head_dim,
                          spec.softmax_scale, spec.window or 0)
        return self.out.forward(context)
