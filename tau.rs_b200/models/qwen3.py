"""Dense Qwen3 as a list of blocks: the only place that knows this architecture.

Every layer is a pre-norm block (crates/models/src/qwen3_5_common/decoder.rs:96-117)
of grouped-query attention with per-head q/k RMSNorm and full-width rotate-half RoPE
(crates/models/src/loader.rs:185-187; analogue crates/models/src/components/
gated_attention.rs:337-372) and a SwiGLU feed-forward (crates/models/src/components/
mlp.rs:99-122).  Tensor names follow the checkpoint's own
(`model.layers.{i}.self_attn.q_proj.weight`, ...; naming scheme as in
crates/models/src/qwen3_5_common/tensors.rs:21-45).  The softmax scale `d^-1/2` is the
one constant that config.json does not carry (gated_attention.rs:458).
"""
from __future__ import annotations

from ..config.qwen3 import ARCHITECTURE, MODEL_TYPE, Qwen3Config
from ..config.registry import register_architecture
from ..config.specs import (AttentionSpec, BlockSpec, ModelSpec, NormSpec, PositionSpec, ScheduleEntry, SwiGLUSpec)


def build_qwen3_spec(config: Qwen3Config) -> ModelSpec:
    layer_norm = NormSpec(width=config.hidden_size, eps=config.rms_norm_eps)
    attention = AttentionSpec(
        hidden=config.hidden_size,
        n_heads=config.num_attention_heads,
        n_kv_heads=config.num_key_value_heads,
        head_dim=config.head_dim,
        bias=config.attention_bias,
        softmax_scale=config.head_dim ** -0.5,
        qk_norm=NormSpec(width=config.head_dim, eps=config.rms_norm_eps),
        position=PositionSpec(
            rotary_dim=config.head_dim, theta=config.rope_theta, max_positions=config.max_position_embeddings
        ),
        window=None,
    )
    feed_forward = SwiGLUSpec(hidden=config.hidden_size, intermediate=config.intermediate_size)
    blocks = tuple(
        BlockSpec(
            prefix=f"model.layers.{index}",
            mixer=attention,
            feed_forward=feed_forward,
            mixer_norm=layer_norm,
            feed_forward_norm=layer_norm,
        )
        for index in range(config.num_hidden_layers)
    )
    schedule = tuple(
        ScheduleEntry(layer=index, cache_group="attention", cache_layer=index, writes_cache=True)
        for index in range(config.num_hidden_layers)
    )
    return ModelSpec(
        architecture=ARCHITECTURE,
        vocab_size=config.vocab_size,
        hidden=config.hidden_size,
        max_positions=config.max_position_embeddings,
        embedding_name="model.embed_tokens.weight",
        blocks=blocks,
        schedule=schedule,
        final_norm=layer_norm,
        final_norm_name="model.norm.weight",
        head_name="lm_head.weight",
        tie_head=config.tie_word_embeddings,
        declared_dtype=config.declared_dtype,
    )


register_architecture(ARCHITECTURE, MODEL_TYPE, Qwen3Config.from_json, build_qwen3_spec)
