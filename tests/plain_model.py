"""Plain, slow implementation of the dense Qwen3 decoder: whole sequences, no cache.

One function for each part, written from the reference's formulas; nothing here is
imported from the engine package, and the engine imports nothing from here.  It runs
on the CPU in float32 (or float64).  tau.rs does not hold the dense Qwen3 layer math
itself (crates/models/src/qwen3.rs:8-10 re-exports an external crate that is not part
of the tree, and there is no Rust toolchain to build it), so this file rests on the
formulas: the in-tree components that tau.rs wrote for its other families show how
each kind of operation is computed, and the deviations for dense Qwen3 (plain norm
weight instead of `1 + w`, full rotary width, no output gate) are stated beside each
function.

`round_to` emulates a storage dtype: every tensor that the engine would store in
bfloat16 is rounded there and computed on in float32 afterwards, so that a bfloat16
engine can be compared with a tolerance that does not have to absorb the roundings.
"""
from __future__ import annotations

import json
import math
import os
import struct
from dataclasses import dataclass
from typing import Callable, Dict, List, Optional, Sequence

import numpy as np
import torch


# --------------------------------------------------------------------------- config
@dataclass
class PlainConfig:
    """The config.json keys of crates/models/src/qwen3.rs:136-156, as plain fields."""

    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    attention_bias: bool
    rms_norm_eps: float
    rope_theta: float
    max_position_embeddings: int
    tie_word_embeddings: bool


def read_plain_config(folder: str) -> PlainConfig:
    with open(os.path.join(folder, "config.json")) as handle:
        raw = json.load(handle)
    heads = raw["num_attention_heads"]
    return PlainConfig(
        vocab_size=raw["vocab_size"],
        hidden_size=raw["hidden_size"],
        intermediate_size=raw["intermediate_size"],
        num_hidden_layers=raw["num_hidden_layers"],
        num_attention_heads=heads,
        num_key_value_heads=raw.get("num_key_value_heads", heads),
        head_dim=raw.get("head_dim", raw["hidden_size"] // heads),
        attention_bias=raw.get("attention_bias", False),
        rms_norm_eps=raw["rms_norm_eps"],
        rope_theta=raw["rope_theta"],
        max_position_embeddings=raw["max_position_embeddings"],
        tie_word_embeddings=raw.get("tie_word_embeddings", False),
    )


# --------------------------------------------------------------------------- weights
_NUMPY_OF = {"F32": np.float32, "F64": np.float64, "I32": np.int32, "I64": np.int64}


def read_plain_weights(folder: str) -> Dict[str, torch.Tensor]:
    """Reads every tensor of every *.safetensors file of a folder as float32.

    The file format is the one crates/models/src/safetensors.rs:107-184 maps: eight
    bytes of little-endian header length, a JSON header with dtype, shape and byte
    offsets for each name, then the raw bytes.  Written here by hand, with numpy.
    """
    tensors: Dict[str, torch.Tensor] = {}
    for entry in sorted(os.listdir(folder)):
        if not entry.endswith(".safetensors"):
            continue
        with open(os.path.join(folder, entry), "rb") as handle:
            blob = handle.read()
        (header_bytes,) = struct.unpack("<Q", blob[:8])
        header = json.loads(blob[8 : 8 + header_bytes])
        body = blob[8 + header_bytes :]
        for name, meta in header.items():
            if name == "__metadata__":
                continue
            begin, end = meta["data_offsets"]
            raw = body[begin:end]
            if meta["dtype"] == "BF16":
                halves = np.frombuffer(raw, dtype=np.uint16).astype(np.uint32) << 16
                values = halves.view(np.float32)
            else:
                values = np.frombuffer(raw, dtype=_NUMPY_OF[meta["dtype"]]).astype(np.float32)
            tensors[name] = torch.from_numpy(values.copy()).reshape(meta["shape"])
    return tensors


Rounding = Callable[[torch.Tensor], torch.Tensor]


def no_rounding(values: torch.Tensor) -> torch.Tensor:
    return values


def bfloat16_rounding(values: torch.Tensor) -> torch.Tensor:
    return values.to(torch.bfloat16).to(values.dtype)


# --------------------------------------------------------------------------- parts
def embedding(table: torch.Tensor, tokens: Sequence[int]) -> torch.Tensor:
    """`h_t = E[token_t, :]`, no scale.

    crates/models/src/qwen3_5_common/model.rs:228 (embedding lookup before the layers);
    crates/cuda-kernels/src/kernels/decode_attention.cu:25 (kind 0 copies one row).
    """
    return table[torch.tensor(list(tokens), dtype=torch.long)]


def rms_norm(values: torch.Tensor, weight: torch.Tensor, eps: float, round_to: Rounding) -> torch.Tensor:
    """`x * rsqrt(mean(x^2) + eps) * w`, statistic and scaling in the wide type, one rounding.

    crates/models/src/components/rms_norm.rs:205-210 (upcast, mean of squares over the
    last axis, `1/sqrt(var + eps)`, multiply) and :147-150 (weight applied in the wide
    type, then cast back).  The in-tree norm scales by `1 + w`; dense Qwen3 scales by
    `w` itself.
    """
    variance = values.pow(2).mean(dim=-1, keepdim=True)
    return round_to(values * torch.rsqrt(variance + eps) * weight)


def linear(values: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], round_to: Rounding) -> torch.Tensor:
    """`y = x W^T + b` with `W` stored `[out, in]`.

    crates/cuda-kernels/src/kernels/linear_bf16_fp32.cuh:31-33 (row-major `[N, K]`
    weight used as the transposed operand); crates/models/src/components/
    gated_attention.rs:273-296 (one bias flag for all attention projections).
    """
    out = values @ weight.t()
    if bias is not None:
        out = out + bias
    return round_to(out)


def rope_tables(head_dim: int, theta: float, positions: int) -> tuple[torch.Tensor, torch.Tensor]:
    """cos and sin of `p * theta^(-2j/d)` for `j < d/2`, in 32-bit.

    crates/models/src/components/rope.rs:91-108: the inverse frequency is
    `1f32 / (theta.powf(i / d) as f32)` for even `i` (the power in 64-bit, its result
    and everything after it in 32-bit), the angle is the 32-bit product of the position
    and the inverse frequency, and the tables are its cosine and sine.  Dense Qwen3
    rotates the whole head (`rotary_dim == head_dim`, rope.rs:141-143).
    """
    inverse = torch.tensor(
        [np.float32(1.0) / np.float32(float(theta) ** (index / head_dim)) for index in range(0, head_dim, 2)],
        dtype=torch.float32,
    )
    angles = torch.arange(positions, dtype=torch.float32)[:, None] * inverse[None, :]
    return torch.cos(angles), torch.sin(angles)


def apply_rope(heads: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, round_to: Rounding) -> torch.Tensor:
    """Rotate-half: element `j` pairs with `j + d/2`.  `heads` is `[T, n, d]`, tables `[T, d/2]`.

    `y_j = x_j cos - x_{j+d/2} sin`, `y_{j+d/2} = x_{j+d/2} cos + x_j sin`
    (crates/cuda-kernels/src/kernels/decode_attention.cu:50-62 pairs `j` with
    `j + half`; :164-167 rotates in 32-bit and rounds once).
    """
    half = heads.shape[-1] // 2
    first, second = heads[..., :half], heads[..., half:]
    cos = cos[:, None, :].to(heads.dtype)
    sin = sin[:, None, :].to(heads.dtype)
    return round_to(torch.cat([first * cos - second * sin, second * cos + first * sin], dim=-1))


def causal_attention(query: torch.Tensor, key: torch.Tensor, value: torch.Tensor, round_to: Rounding) -> torch.Tensor:
    """Grouped-query causal softmax attention of one whole sequence.

    `query` `[T, nq, d]`, `key`/`value` `[T, nkv, d]`.  Query head `h` reads KV head
    `h // (nq / nkv)` (consecutive grouping: decode_attention.cu:192,
    gated_attention.rs:451).  Scores are `q.k * d^-1/2` (gated_attention.rs:458-462),
    keys after the query's own position are masked (qwen3_5_common/model.rs:154,
    `key <= query + offset`), the softmax is taken in the wide type
    (gated_attention.rs:466-468), the context is `P V` (:469-473) and is rounded once.
    """
    tokens, heads, width = query.shape
    group = heads // key.shape[1]
    scale = 1.0 / math.sqrt(width)
    mask = torch.ones(tokens, tokens, dtype=torch.bool).tril()
    context = torch.empty_like(query)
    for head in range(heads):
        scores = (query[:, head, :] @ key[:, head // group, :].t()) * scale
        scores = scores.masked_fill(~mask, float("-inf"))
        weights = torch.softmax(scores, dim=-1)
        context[:, head, :] = weights @ value[:, head // group, :]
    return round_to(context)


def attention_mixer(hidden: torch.Tensor, weights: Dict[str, torch.Tensor], prefix: str, config: PlainConfig,
                    cos: torch.Tensor, sin: torch.Tensor, round_to: Rounding) -> torch.Tensor:
    """Projections, per-head q/k norm, rotation, attention, output projection.

    Order as in crates/models/src/components/gated_attention.rs:337-372: project, view
    as heads, normalise each query and key head over `head_dim` before the rotation,
    leave values untouched, rotate q and k, attend, project with `o_proj` (:402).
    Dense Qwen3 has neither the doubled query projection nor the sigmoid gate of that
    component (crates/models/src/loader.rs:185-187 names what it does have: explicit
    head dimensions and per-head q/k normalisation).
    """
    tokens = hidden.shape[0]
    heads, groups, width = config.num_attention_heads, config.num_key_value_heads, config.head_dim

    def bias(name: str) -> Optional[torch.Tensor]:
        return weights[f"{prefix}.{name}.bias"] if config.attention_bias else None

    query = linear(hidden, weights[f"{prefix}.q_proj.weight"], bias("q_proj"), round_to).view(tokens, heads, width)
    key = linear(hidden, weights[f"{prefix}.k_proj.weight"], bias("k_proj"), round_to).view(tokens, groups, width)
    value = linear(hidden, weights[f"{prefix}.v_proj.weight"], bias("v_proj"), round_to).view(tokens, groups, width)
    query = rms_norm(query, weights[f"{prefix}.q_norm.weight"], config.rms_norm_eps, round_to)
    key = rms_norm(key, weights[f"{prefix}.k_norm.weight"], config.rms_norm_eps, round_to)
    query = apply_rope(query, cos[:tokens], sin[:tokens], round_to)
    key = apply_rope(key, cos[:tokens], sin[:tokens], round_to)
    context = causal_attention(query, key, value, round_to).reshape(tokens, heads * width)
    return linear(context, weights[f"{prefix}.o_proj.weight"], bias("o_proj"), round_to)


def swiglu(hidden: torch.Tensor, weights: Dict[str, torch.Tensor], prefix: str, round_to: Rounding) -> torch.Tensor:
    """`down(silu(gate(x)) * up(x))`, no biases.

    crates/models/src/components/mlp.rs:99-122 (the three bias-free projections),
    :177-191 (`silu(gate) * up`, then `down`); crates/cuda-kernels/src/kernels/
    silu_and_mul.cu:71-74 (`g / (1 + exp(-g)) * u` in 32-bit, one rounding).
    """
    gate = linear(hidden, weights[f"{prefix}.gate_proj.weight"], None, round_to)
    up = linear(hidden, weights[f"{prefix}.up_proj.weight"], None, round_to)
    activated = round_to(gate / (1.0 + torch.exp(-gate)) * up)
    return linear(activated, weights[f"{prefix}.down_proj.weight"], None, round_to)


def decoder_block(hidden: torch.Tensor, weights: Dict[str, torch.Tensor], prefix: str, config: PlainConfig,
                  cos: torch.Tensor, sin: torch.Tensor, round_to: Rounding) -> torch.Tensor:
    """Pre-norm block: `r = x + mixer(norm(x))`, `out = r + ff(norm(r))`.

    crates/models/src/qwen3_5_common/decoder.rs:96-117; the residual sum is rounded to
    the storage type before the second norm reads it (crates/models/src/components/
    rms_norm.rs:39-74, crates/cuda-kernels/src/kernels/centered_rms_norm.cu:267-274).
    """
    normalized = rms_norm(hidden, weights[f"{prefix}.input_layernorm.weight"], config.rms_norm_eps, round_to)
    branch = attention_mixer(normalized, weights, f"{prefix}.self_attn", config, cos, sin, round_to)
    residual = round_to(hidden + branch)
    normalized = rms_norm(residual, weights[f"{prefix}.post_attention_layernorm.weight"], config.rms_norm_eps, round_to)
    return round_to(residual + swiglu(normalized, weights, f"{prefix}.mlp", round_to))


def forward_logits(config: PlainConfig, weights: Dict[str, torch.Tensor], tokens: Sequence[int],
                   round_to: Rounding = no_rounding, rows: Optional[Sequence[int]] = None) -> torch.Tensor:
    """Logits `[T, V]` at every position of one sequence (or at the positions `rows` only: the head is the one part
    whose cost a caller may want to bound when the vocabulary is large).

    Embedding, the blocks in order, the final norm and the head
    (crates/models/src/qwen3_5_common/model.rs:168-195); the head is `lm_head.weight`,
    or the embedding table when `tie_word_embeddings` (model.rs:295-299).  The logits
    stay in the wide type.
    """
    cos, sin = rope_tables(config.head_dim, config.rope_theta, config.max_position_embeddings)
    hidden = embedding(weights["model.embed_tokens.weight"], tokens)
    for layer in range(config.num_hidden_layers):
        hidden = decoder_block(hidden, weights, f"model.layers.{layer}", config, cos, sin, round_to)
    if rows is not None:
        hidden = hidden[torch.tensor(list(rows), dtype=torch.long)]
    hidden = rms_norm(hidden, weights["model.norm.weight"], config.rms_norm_eps, round_to)
    head = weights["model.embed_tokens.weight"] if config.tie_word_embeddings else weights["lm_head.weight"]
    return hidden @ head.t()


# --------------------------------------------------------------------------- selection
def greedy_token(logits: Sequence[float]) -> int:
    """Greatest logit by the total order of 32-bit floats; NaN never wins; last index wins ties.

    crates/engine/src/generation.rs:81-95 (`filter(!is_nan)`, `max_by(total_cmp)`, which
    keeps the last of equal elements; an error if nothing is left).
    """
    values = np.asarray(logits, dtype=np.float32)
    bits = values.view(np.uint32).astype(np.uint64)
    is_nan = (bits & 0x7FFFFFFF) > 0x7F800000
    keys = np.where(bits & 0x80000000, bits ^ 0xFFFFFFFF, bits ^ 0x80000000)
    best = -1
    best_key = -1
    for index in range(len(values)):
        if is_nan[index]:
            continue
        if int(keys[index]) >= best_key:
            best, best_key = index, int(keys[index])
    if best < 0:
        raise ValueError("model logits are all NaN")
    return best


def greedy_generate(config: PlainConfig, weights: Dict[str, torch.Tensor], prompt: Sequence[int], max_new_tokens: int,
                    stop_tokens: Sequence[int] = (), round_to: Rounding = no_rounding) -> List[int]:
    """Whole-sequence recomputation for each new token.

    crates/engine/src/model_engine/generation.rs:60-116: the token chosen after the
    prompt counts toward the limit; a stop token is neither returned nor fed back
    (:280-285); generation ends at the limit (:165-219).
    """
    tokens = list(prompt)
    produced: List[int] = []
    while len(produced) < max_new_tokens:
        logits = forward_logits(config, weights, tokens, round_to, rows=[len(tokens) - 1])[0]
        token = greedy_token(logits.numpy())
        if token in stop_tokens:
            break
        produced.append(token)
        tokens.append(token)
    return produced
