"""Pre-norm block: `r = x + mixer(norm(x))`, `out = r + feed_forward(norm(r))`.

crates/models/src/qwen3_5_common/decoder.rs:96-117.  The hidden state travels as
`(residual, branch)` with `x = residual + branch`, so each sum is rounded to the storage
dtype and normalised by one fused kernel (crates/models/src/components/rms_norm.rs:39-74).
Weight names: `<prefix>.input_layernorm`, `<prefix>.self_attn`,
`<prefix>.post_attention_layernorm`, `<prefix>.mlp` (decoder.rs:52,296,302).
"""
from __future__ import annotations

from .base import Block
from .registry import build, register_block


@register_block("pre_norm")
class PreNormBlock(Block):
    mixer_name = "self_attn"
    feed_forward_name = "mlp"
    mixer_norm_name = "input_layernorm"
    feed_forward_norm_name = "post_attention_layernorm"

    def __init__(self, spec, dtype, device):
        self.spec = spec
        prefix = spec.prefix
        self.mixer_norm = build("norm", spec.mixer_norm, name=f"{prefix}.{self.mixer_norm_name}.weight", dtype=dtype, device=device)
        self.mixer = build("mixer", spec.mixer, prefix=f"{prefix}.{self.mixer_name}", dtype=dtype, device=device)
        self.feed_forward_norm = build(
            "norm", spec.feed_forward_norm, name=f"{prefix}.{self.feed_forward_norm_name}.weight", dtype=dtype, device=device
        )
        self.feed_forward = build(
            "feed_forward", spec.feed_forward, prefix=f"{prefix}.{self.feed_forward_name}", dtype=dtype, device=device
        )
        self._children = (self.mixer_norm, self.mixer, self.feed_forward_norm, self.feed_forward)
        self.capturable = all(getattr(part, "capturable", True) for part in self._children)

    def cache_need(self):
        return self.mixer.cache_need()

    def decode_blocks(self):
        return self.mixer.decode_blocks()

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

    def bytes_read_per_step(self, dtype) -> int:
        return sum(part.bytes_read_per_step(dtype) for part in self._children)

    def forward(self, residual, branch, step, cache, writes_cache: bool):
        if branch is None:
            normalized = self.mixer_norm.forward(residual)
        else:
            normalized = self.mixer_norm.add_forward(branch, residual)
        mixed = self.mixer.forward(normalized, step, cache, writes_cache)
        normalized = self.feed_forward_norm.add_forward(mixed, residual)
        return residual, self.feed_forward.forward(normalized, step)
