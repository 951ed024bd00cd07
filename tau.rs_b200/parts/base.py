"""Interfaces of the parts.

A part owns its weights (declared by name through `tensor_specs`, received through
`assign`) and a `forward`.  Activations are packed: row `i` of every activation tensor
belongs to token `i` of the step, whichever sequence it is from; `StepContext` says
which sequence and which position each row has.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Optional, Tuple

import torch

from ..weights.tensor_spec import TensorSpec


@dataclass(frozen=True)
class CacheNeed:
    """What a mixer wants the cache to keep for it, per cache layer.

    `kind == "kv"`: keys and values of `n_kv_heads` heads of `head_dim` elements for
    every position (or for the last `window` positions).  `kind == "state"`: one
    tensor of `state_shape` and `state_dtype` for each sequence, zero when the sequence
    starts, whatever its length.
    """

    kind: str
    n_kv_heads: int = 0
    head_dim: int = 0
    window: Optional[int] = None
    state_shape: Tuple[int, ...] = ()
    state_dtype: torch.dtype = torch.float32


class Part:
    def tensor_specs(self) -> Dict[str, TensorSpec]:
        return {}

    def assign(self, name: str, tensor: torch.Tensor) -> None:
        raise KeyError(name)

    def finalize_weights(self) -> None:
        pass

    def bytes_read_per_step(self, dtype) -> int:
        """Bytes of this part's weights that one step reads: every tensor once, unless the part knows better (a feed-forward
        that routes each token to a few of its experts reads only those).  The roofline of a decode step is built on it."""
        from ..weights.loader import device_dtype

        total = 0
        for spec in self.tensor_specs().values():
            count = 1
            for extent in spec.shape:
                count *= extent
            total += count * torch.empty((), dtype=device_dtype(spec, dtype)).element_size()
        return total


class Mixer(Part):
    """Mixes information between the tokens of a sequence.

    `forward(hidden, step, cache, writes_cache)` takes `[tokens, hidden]` and returns
    the same shape.  `cache` is the view of this run's cache layer (`KVLayerView` or
    `StateLayerView`), or None if `cache_need()` is None.
    """

    # False: a decode step through this mixer cannot be captured in a CUDA graph (its `forward` reads device values on the
    # host, say); an engine whose model has such a part runs its decode steps launch by launch.
    capturable = True

    def cache_need(self) -> Optional[CacheNeed]:
        return None

    def decode_blocks(self) -> Optional[int]:
        """Blocks that the mixer's decode kernel launches per sequence and context split, where the mixer splits the
        context of a decode step at all (None: it does not).  The number of splits is chosen so that all blocks of a step
        are resident at once, and it is part of a captured graph's key."""
        return None

    def forward(self, hidden, step, cache, writes_cache: bool):
        raise NotImplementedError


class FeedForward(Part):
    """`forward(hidden, step)`: `[tokens, hidden] -> [tokens, hidden]`, token by token."""

    capturable = True   # as for a mixer

    def forward(self, hidden, step):
        raise NotImplementedError


class Norm(Part):
    """`forward(x, rows=None, branch=None)` normalises rows (optionally only the rows listed,
    optionally of `x + branch` rounded to the storage dtype); `x` is left as it is.

    `add_forward(branch, residual)` rounds `residual + branch` into `residual` and
    returns its normalisation, as one fused operation.
    """

    def forward(self, values, rows=None, branch=None):
        raise NotImplementedError

    def add_forward(self, branch, residual):
        raise NotImplementedError


class Block(Part):
    """Arrangement of a mixer and a feed-forward around the residual stream.

    The residual stream travels as a pair `(residual, branch)` whose sum is the hidden
    state, so that the sum can be fused with the next norm wherever that is.
    `forward(residual, branch, step, cache, writes_cache) -> (residual, branch)`.
    """

    capturable = True   # False if a part of the block is not

    def cache_need(self) -> Optional[CacheNeed]:
        return None

    def decode_blocks(self) -> Optional[int]:
        """The mixer's answer (see `Mixer.decode_blocks`)."""
        return None

    def forward(self, residual, branch, step, cache, writes_cache: bool):
        raise NotImplementedError
