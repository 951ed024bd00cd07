"""The cache: a slot for each live sequence, storage for each group of layers.

tau.rs keeps, per attention layer, keys and values `[batch, kv_heads, capacity, d]` with a
live length, appends only at `offset == len`, and resets by setting the length to zero
without clearing (crates/models/src/components/gated_attention/kv_cache.rs:12-24,
85-111,177-222,249-255: stale tail values are never read).  Its layers with a recurrent
mixer keep state of fixed size beside that (crates/models/src/qwen3_5_common/
decoder.rs:22-25,59-78).  Here the batch axis becomes slots that sequences take and give
back, and the capacity axis becomes pages of `PAGE_TOKENS` positions that a sequence
takes as it grows, so that the cache is sized by the tokens that live sequences hold
together and not by the longest of them times their number.

A group is a set of cache layers with the same need (`CacheNeed`): a `kv` group has one
pool of pages for keys and one for values, `[cache layers, pages, kv heads, PAGE_TOKENS,
head_dim]`, and on the host a page table `[slots, pages per sequence]`; a page number
means the same page in every layer of the group.  Each step carries the table rows of
its own sequences to the device with its other metadata, so the device never holds a row
of a sequence that has ended.  A `state` group has `[cache layers, slots, *shape]`
and is zeroed for a slot when a sequence takes it.  Pages are not cleared: a position is
written before anything reads it, and nothing reads beyond a sequence's length.

A group whose need has a `window` gives a sequence's pages back as they fall out of the
window: the next query, at position `length`, sees keys from `length - window + 1` on, so
pages that lie wholly before that are returned when the length is published and their
table entries are cleared.  Work already put on the stream may still read them; whoever
takes them next writes them in work that is put on the stream later.  Such a sequence
holds about `window / 64 + 2` pages however long it grows.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Tuple

import numpy as np
import torch

from ..parts.base import CacheNeed
from .allocator import CacheFull, FreeList

PAGE_TOKENS = 64


def pages_for(tokens: int) -> int:
    return (tokens + PAGE_TOKENS - 1) // PAGE_TOKENS


@dataclass
class KVLayerView:
    keys: torch.Tensor        # [pages, kv_heads, PAGE_TOKENS, head_dim]
    values: torch.Tensor
    group: str                # key of the step's page rows (`StepContext.page_rows[group]`)
    window: Optional[int]


@dataclass
class StateLayerView:
    state: torch.Tensor       # [slots, *shape]


class _KVGroup:
    def __init__(self, need: CacheNeed, layers: int, pages: int, slots: int, pages_per_sequence: int, dtype, device):
        self.need, self.layers = need, layers
        shape = (layers, pages, need.n_kv_heads, PAGE_TOKENS, need.head_dim)
        self.keys = torch.empty(shape, dtype=dtype, device=device)
        self.values = torch.empty(shape, dtype=dtype, device=device)
        self.pool = FreeList(pages, "cache page")
        self.table = np.zeros((slots, pages_per_sequence), dtype=np.int32)
        self.held: Dict[int, List[int]] = {}          # the pages a sequence holds, oldest first
        self.released: Dict[int, int] = {}            # how many older pages it has given back already (a window's doing)

    def tokens_read(self, length: int) -> int:
        return min(length, self.need.window) if self.need.window else length

    def bytes_per_token(self) -> int:
        return 2 * self.layers * self.need.n_kv_heads * self.need.head_dim * self.keys.element_size()


class _StateGroup:
    def __init__(self, need: CacheNeed, layers: int, slots: int, device):
        self.need, self.layers = need, layers
        self.state = torch.zeros((layers, slots, *need.state_shape), dtype=need.state_dtype, device=device)


class SequenceCache:
    """`groups`: name -> (`CacheNeed`, number of cache layers), as `DecoderModel.cache_groups()` gives it.

    `max_tokens` is the most tokens that live sequences may hold together, each
    sequence's count rounded up to a multiple of `PAGE_TOKENS`.
    """

    def __init__(self, groups: Dict[str, Tuple[CacheNeed, int]], max_tokens: int, max_sequence_tokens: int,
                 dtype: torch.dtype, device, max_slots: Optional[int] = None):
        if max_tokens <= 0:
            raise ValueError("the cache must hold at least one token")
        self.device, self.dtype = device, dtype
        self.n_pages = pages_for(max_tokens)
        # A sequence cannot hold more pages than there are, unless every kv group lets old pages go (a window) or the model
        # keeps no keys and values at all (state of fixed size only).
        kv_needs = [need for need, _ in groups.values() if need.kind == "kv"]
        bounded = all(need.window for need in kv_needs)
        self.widest_window = max((need.window for need in kv_needs), default=0) if bounded else None
        self.pages_per_sequence = pages_for(max_sequence_tokens) if bounded else min(self.n_pages, pages_for(max_sequence_tokens))
        self.max_sequence_tokens = min(max_sequence_tokens, self.pages_per_sequence * PAGE_TOKENS)
        self.n_slots = min(self.n_pages, max_slots) if max_slots else self.n_pages
        self.slots = FreeList(self.n_slots, "sequence slot")
        self.lengths: Dict[int, int] = {}
        self.kv: Dict[str, _KVGroup] = {}
        self.states: Dict[str, _StateGroup] = {}
        for name, (need, layers) in groups.items():
            if need.kind == "kv":
                self.kv[name] = _KVGroup(need, layers, self.n_pages, self.n_slots, self.pages_per_sequence, dtype, device)
            elif need.kind == "state":
                self.states[name] = _StateGroup(need, layers, self.n_slots, device)
            else:
                raise ValueError(f"cache group {name!r}: unknown kind {need.kind!r}")

    # ---- sequences ---------------------------------------------------------------
    def open(self) -> int:
        """Takes a slot for a new, empty sequence."""
        (slot,) = self.slots.take(1)
        self.lengths[slot] = 0
        for group in self.kv.values():
            group.held[slot] = []
            group.released[slot] = 0
        for group in self.states.values():
            group.state[:, slot].zero_()
        return slot

    def close(self, slot: int) -> None:
        """Gives back the slot and every page the sequence held."""
        self._require_open(slot)
        for group in self.kv.values():
            group.pool.give_back(group.held.pop(slot))
            del group.released[slot]
        del self.lengths[slot]
        self.slots.give_back([slot])

    def length(self, slot: int) -> int:
        self._require_open(slot)
        return self.lengths[slot]

    def pages_needed(self, slot: int, new_length: int) -> int:
        """Pages that `reserve(slot, new_length)` would take from each kv group."""
        self._require_open(slot)
        wanted = pages_for(new_length)
        return max((max(0, wanted - group.released[slot] - len(group.held[slot])) for group in self.kv.values()), default=0)

    def reserve(self, slot: int, new_length: int) -> None:
        """Makes room for the sequence to grow to `new_length` positions."""
        self._require_open(slot)
        if new_length > self.max_sequence_tokens:
            raise CacheFull(f"a sequence of {new_length} tokens exceeds the limit of {self.max_sequence_tokens}")
        for group in self.kv.values():
            held = group.held[slot]
            begin = group.released[slot] + len(held)
            extra = pages_for(new_length) - begin
            if extra <= 0:
                continue
            taken = group.pool.take(extra)
            held.extend(taken)
            group.table[slot, begin : begin + extra] = taken

    def advance(self, slot: int, new_length: int) -> None:
        """Publishes the new length once the step that wrote the positions is issued."""
        if new_length < self.lengths[slot]:
            raise ValueError("a sequence cannot shrink")
        self.lengths[slot] = new_length
        for group in self.kv.values():
            if not group.need.window:
                continue
            # The next query sits at position `new_length` and sees keys from `new_length - window + 1` on.
            keep_from = max(0, new_length - group.need.window + 1) // PAGE_TOKENS
            gone = keep_from - group.released[slot]
            if gone > 0:
                held = group.held[slot]
                group.pool.give_back(held[:gone])
                del held[:gone]
                group.table[slot, group.released[slot] : keep_from] = 0
                group.released[slot] = keep_from

    def page_rows(self, group: str, slots, pages: int) -> np.ndarray:
        """Page numbers `[len(slots), pages]` of the given sequences (host memory)."""
        return self.kv[group].table[np.asarray(slots, dtype=np.int64), :pages]

    def _require_open(self, slot: int) -> None:
        if not self.slots.is_out(slot):
            raise ValueError(f"sequence slot {slot} is not in use")

    # ---- views and accounting ----------------------------------------------------
    def layer_view(self, group: str, layer: int):
        if group in self.kv:
            entry = self.kv[group]
            return KVLayerView(entry.keys[layer], entry.values[layer], group, entry.need.window)
        return StateLayerView(self.states[group].state[layer])

    def free_tokens(self) -> int:
        pools = [group.pool.available for group in self.kv.values()]
        return (min(pools) if pools else self.n_pages) * PAGE_TOKENS

    def bytes_per_token(self) -> int:
        return sum(group.bytes_per_token() for group in self.kv.values())

    def live_bytes(self) -> int:
        """Bytes of keys and values that a step over all live sequences reads."""
        return sum(group.tokens_read(length) * group.bytes_per_token() for length in self.lengths.values() for group in self.kv.values())

    def check(self) -> None:
        """No slot or page lost, held twice or shared between sequences."""
        self.slots.check()
        if set(self.lengths) != {slot for slot in range(self.n_slots) if self.slots.is_out(slot)}:
            raise AssertionError("lengths and slots disagree")
        for group in self.kv.values():
            group.pool.check()
            held = [page for pages in group.held.values() for page in pages]
            if len(held) != len(set(held)):
                raise AssertionError("a cache page is held by two sequences")
            if len(held) != group.pool.in_use:
                raise AssertionError("a cache page is in use but belongs to no sequence")
            for slot, pages in group.held.items():
                if self.lengths[slot] > (group.released[slot] + len(pages)) * PAGE_TOKENS:
                    raise AssertionError("a sequence is longer than the pages it holds")
                if group.released[slot] and not group.need.window:
                    raise AssertionError("a group without a window gave pages back early")
                if group.need.window and group.released[slot] * PAGE_TOKENS > max(0, self.lengths[slot] - group.need.window + 1):
                    raise AssertionError("a page inside the window was given back")
