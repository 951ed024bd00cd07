"""Descriptions of parts: what a layer is made of, as data.

A model is a list of block descriptions and a schedule.  Each description names the
kind of part (looked up in `tau_rs_b200.parts.registry`) and carries every size and
constant that the part needs, so no part reads a model-wide configuration and none
knows which architecture it serves.  tau.rs expresses the same idea with one enum per
layer (crates/models/src/qwen3_5_common/decoder.rs:22-25,59-78: each layer owns either
kind of token mixer and its own state).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional, Tuple


@dataclass(frozen=True)
class NormSpec:
    width: int
    eps: float
    kind: str = "rms_norm"


@dataclass(frozen=True)
class PositionSpec:
    """Rotary position encoding of the first `rotary_dim` elements of each head."""

    rotary_dim: int
    theta: float
    max_positions: int
    kind: str = "rope_half"


@dataclass(frozen=True)
class AttentionSpec:
    hidden: int
    n_heads: int
    n_kv_heads: int
    head_dim: int
    bias: bool
    softmax_scale: float
    qk_norm: Optional[NormSpec] = None
    position: Optional[PositionSpec] = None
    window: Optional[int] = None
    kind: str = "attention"


@dataclass(frozen=True)
class SwiGLUSpec:
    hidden: int
    intermediate: int
    kind: str = "swiglu"


@dataclass(frozen=True)
class BlockSpec:
    """One layer: its weight-name prefix, its two parts and the norm before each."""

    prefix: str
    mixer: object
    feed_forward: object
    mixer_norm: NormSpec
    feed_forward_norm: NormSpec
    kind: str = "pre_norm"


@dataclass(frozen=True)
class ScheduleEntry:
    """One run of a layer.

    `layer` indexes the model's blocks (a block may be named by several entries and
    then runs several times with the same weights).  `cache_group` and `cache_layer`
    say where the mixer keeps what it remembers; two entries with the same pair share
    that storage, and an entry with `writes_cache=False` only reads what another entry
    wrote earlier in the same step.
    """

    layer: int
    cache_group: Optional[str] = None
    cache_layer: int = 0
    writes_cache: bool = True


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    vocab_size: int
    hidden: int
    max_positions: int
    embedding_name: str
    blocks: Tuple[BlockSpec, ...]
    schedule: Tuple[ScheduleEntry, ...]
    final_norm: NormSpec
    final_norm_name: str
    head_name: str
    tie_head: bool
    declared_dtype: Optional[str] = None
    extra: dict = field(default_factory=dict, compare=False)
    # A position encoding that acts on the embedded tokens before the first block (learned or absolute positions): a spec of
    # the "position" family whose part offers `add_to(hidden, step)`.  None for encodings that act inside the mixers.
    input_position: Optional[object] = None
