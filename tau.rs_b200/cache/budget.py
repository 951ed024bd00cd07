"""Whether a cache of the asked size fits the device: pure arithmetic, the device is asked by the caller.

crates/engine/src/model_engine/kv_budget.rs:17-56 derives a token capacity from a snapshot of free memory taken
after the weights are loaded, keeps headroom for activations and allocator slack, and refuses with a named error
when nothing fits.  Here the capacity is the caller's (`max_tokens`), so the same arithmetic answers the other
question: does what was asked for fit, and if not, how much would.  The reference keeps the larger of 2 GiB and a
quarter of the memory free; a quarter of 180 GB would turn away the largest shape this library is measured on
(65 GB of weights beside 69 GB of cache), so the share kept here is a thirty-second.
"""
from __future__ import annotations

from typing import Dict, Optional, Tuple

from ..config.errors import ModelLoadError

PAGE_TOKENS = 64
_ELEMENT_BYTES = {"float32": 4, "bfloat16": 2, "torch.float32": 4, "torch.bfloat16": 2}


class CacheDoesNotFit(ModelLoadError):
    """The cache that was asked for does not fit the device's free memory."""

    def __init__(self, needed_bytes: int, free_bytes: int, headroom_bytes: int, fitting_tokens: int, asked_tokens: int):
        self.needed_bytes, self.free_bytes, self.headroom_bytes = needed_bytes, free_bytes, headroom_bytes
        self.fitting_tokens, self.asked_tokens = fitting_tokens, asked_tokens
        super().__init__(
            f"a cache of {asked_tokens} tokens needs {needed_bytes} bytes; {free_bytes} bytes are free on the device, of which "
            f"{headroom_bytes} are kept for activations; a cache of at most {fitting_tokens} tokens fits")


def headroom(total_bytes: int) -> int:
    return max(2 << 30, total_bytes // 32)


def kv_bytes_per_token(groups: Dict[str, Tuple[object, int]], element_bytes: int) -> int:
    """Bytes that one cached position takes over all kv groups (keys and values of every cache layer)."""
    total = 0
    for need, layers in groups.values():
        if need.kind == "kv":
            total += 2 * layers * need.n_kv_heads * need.head_dim * element_bytes
    return total


def state_bytes_per_slot(groups: Dict[str, Tuple[object, int]]) -> int:
    import torch

    total = 0
    for need, layers in groups.values():
        if need.kind == "state":
            count = layers
            for extent in need.state_shape:
                count *= extent
            total += count * torch.empty((), dtype=need.state_dtype).element_size()
    return total


def check_fits(groups: Dict[str, Tuple[object, int]], max_tokens: int, n_slots: int, element_bytes: int, free_bytes: int,
               total_bytes: int, headroom_bytes: Optional[int] = None) -> int:
    """Returns the bytes the cache takes, or raises `CacheDoesNotFit`.  `max_tokens` is rounded up to whole pages."""
    if free_bytes > total_bytes or free_bytes < 0:
        raise ValueError("invalid memory snapshot")
    pages = -(-max_tokens // PAGE_TOKENS)
    per_token = kv_bytes_per_token(groups, element_bytes)
    needed = pages * PAGE_TOKENS * per_token + n_slots * state_bytes_per_slot(groups)
    kept = headroom(total_bytes) if headroom_bytes is None else headroom_bytes
    if needed + kept > free_bytes:
        room = max(0, free_bytes - kept - n_slots * state_bytes_per_slot(groups))
        fitting = (room // (per_token * PAGE_TOKENS)) * PAGE_TOKENS if per_token else 0
        raise CacheDoesNotFit(needed, free_bytes, kept, fitting, max_tokens)
    return needed
