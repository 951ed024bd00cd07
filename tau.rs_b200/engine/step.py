"""The step function: a batch of sequences, each with its next tokens, through the model once.

The reference's contract per request is `forward(input [1, T], offset) -> logits` with
`offset == cache length` (crates/models/src/interface.rs:24-28; crates/models/src/
components/gated_attention/kv_cache.rs:85-111), a prompt first and then one token per call
(crates/engine/src/model_engine/generation.rs:120-161,165-219).  Here one call takes
many sequences with runs of unequal length: a first step carries whole prompts packed
along one token axis, later steps carry one token each (or any mixture; a run continues
where the sequence's cache ends).  Only the tokens given are computed, everything
earlier is read from the cache, and logits come back only for the places asked for.
Every check happens before anything is changed, so a refused step leaves the cache as it was.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

from ..cache.allocator import CacheFull
from ..cache.sequence_cache import PAGE_TOKENS, SequenceCache, pages_for
from .batch import StepContext, StepEntry, StepLayout, fill_step, step_views
from .staging import PinnedRing


class StepError(ValueError):
    """The step's entries do not fit the sequences they name."""


MAX_DECODE_SPLITS = 64   # decode attention merges at most this many blocks of a context (the kernel takes up to 2 * head_dim)


class Engine:
    """A model, its cache and the step function over both."""

    def __init__(self, model, max_tokens: int, max_sequence_tokens: Optional[int] = None, max_slots: Optional[int] = None,
                 headroom_bytes: Optional[int] = None):
        """`max_tokens` sizes the cache: the most tokens that live sequences hold together, each rounded up to 64.
        On a CUDA device a cache that does not fit the free memory (less `headroom_bytes` for activations; default: the
        larger of 2 GiB and 1/32 of the device) is refused with `CacheDoesNotFit` before anything is allocated."""
        self.model = model
        self.device = torch.device(model.device)
        limit = model.spec.max_positions
        if max_sequence_tokens is not None:
            limit = min(limit, max_sequence_tokens)
        if self.device.type == "cuda":
            from ..cache.budget import check_fits

            free_bytes, total_bytes = torch.cuda.mem_get_info(self.device)
            free_bytes += torch.cuda.memory_reserved(self.device) - torch.cuda.memory_allocated(self.device)   # what torch holds unused
            pages = -(-max_tokens // PAGE_TOKENS)
            check_fits(model.cache_groups(), max_tokens, min(pages, max_slots) if max_slots else pages,
                       torch.empty((), dtype=model.dtype).element_size(), free_bytes, total_bytes, headroom_bytes)
        self.cache = SequenceCache(model.cache_groups(), max_tokens, limit, model.dtype, self.device, max_slots)
        self._ring: Optional[PinnedRing] = None
        self._graphs: Dict = {}
        self._graph_stream = None
        self._weight_bytes = None
        self._graph_pool = None
        self._split_choice: Dict = {}
        self.last_step_ints = 0     # size of the last step's metadata (int32 words copied to the device)
        # Decode steps replay a captured graph unless a part of the model says that it cannot be captured.
        self.use_graphs = self.device.type == "cuda" and all(getattr(block, "capturable", True) for block in model.blocks)
        # Context tokens per block of decode attention (`--attention-block-size`, crates/server/src/args.rs: "context tokens
        # per prepared decode attention tile"); None: chosen from the batch and the context by `DecoderModel.decode_splits`.
        self.attention_block_size: Optional[int] = None

    def decode_splits(self, n_seqs: int, max_len: int) -> int:
        """Blocks that the context of a decode step is cut into for attention."""
        if self.attention_block_size:
            bucket = 1 << max(0, (max_len - 1).bit_length())   # as the graphs are keyed: a power of two of positions
            return max(1, min(-(-bucket // self.attention_block_size), MAX_DECODE_SPLITS))
        return self.model.decode_splits(n_seqs, max_len)

    def ring(self, ints: int) -> PinnedRing:
        """The pinned staging ring, grown if a step needs more room."""
        if self._ring is None or self._ring.capacity < ints:
            self._ring = PinnedRing(max(ints * 2, 1 << 16))
        return self._ring

    # ---- sequences ---------------------------------------------------------------
    def open_sequence(self) -> int:
        return self.cache.open()

    def close_sequence(self, slot: int) -> None:
        self.cache.close(slot)

    def sequence_length(self, slot: int) -> int:
        return self.cache.length(slot)

    @property
    def capacity_tokens(self) -> int:
        """Tokens the whole cache holds (whole pages)."""
        return self.cache.n_pages * PAGE_TOKENS

    @property
    def max_sequence_tokens(self) -> int:
        return self.cache.max_sequence_tokens

    def peak_cache_tokens(self, prompt_tokens: int, total_tokens: int, chunk: Optional[int] = None) -> int:
        """The most cache positions that a request holds at any one time if its prompt enters in runs of at most `chunk`
        tokens and it grows to `total_tokens`: all of them, unless every group of keys and values has a window (then the
        widest window, one run and the slack of whole pages) or the model keeps none at all."""
        if not self.cache.kv:
            return 0
        if self.cache.widest_window is None:
            return total_tokens
        run = min(prompt_tokens, chunk) if chunk else prompt_tokens
        return min(total_tokens, self.cache.widest_window + run + 3 * PAGE_TOKENS)

    def bytes_read_by_a_decode_step(self) -> int:
        """Every weight once, and the cached keys and values of the live sequences: what a decode step of all of them reads."""
        if self._weight_bytes is None:
            self._weight_bytes = self.model.weight_bytes()
        return self._weight_bytes + self.cache.live_bytes()

    # ---- the step ----------------------------------------------------------------
    accepts_device_tokens = True   # `step(entries, device_tokens=...)`

    def _validate(self, entries: Sequence[StepEntry]) -> List[int]:
        if not entries:
            raise StepError("a step needs at least one sequence")
        seen = set()
        starts = []
        pages_wanted = 0
        vocab = self.model.spec.vocab_size
        for entry in entries:
            if entry.slot in seen:
                raise StepError(f"sequence slot {entry.slot} appears twice in one step")
            seen.add(entry.slot)
            try:
                start = self.cache.length(entry.slot)
            except ValueError as error:
                raise StepError(str(error)) from None
            count = len(entry.tokens)
            if count == 0:
                raise StepError(f"sequence slot {entry.slot} brings no token")
            low, high = min(entry.tokens), max(entry.tokens)
            if low < 0 or high >= vocab:
                raise StepError(f"token id {low if low < 0 else high} lies outside the vocabulary of {vocab}")
            for place in entry.want:
                if not 0 <= place < count:
                    raise StepError(f"wanted place {place} lies outside the {count} tokens of the step")
            if start + count > self.cache.max_sequence_tokens:
                raise CacheFull(
                    f"sequence slot {entry.slot} would reach {start + count} tokens; the limit is {self.cache.max_sequence_tokens}"
                )
            pages_wanted += self.cache.pages_needed(entry.slot, start + count)
            starts.append(start)
        if pages_wanted * PAGE_TOKENS > self.cache.free_tokens():
            raise CacheFull(
                f"the step needs {pages_wanted} more cache pages of {PAGE_TOKENS} tokens, "
                f"{self.cache.free_tokens() // PAGE_TOKENS} are free"
            )
        return starts

    def _context(self, entries: Sequence[StepEntry], starts: Sequence[int], page_stride: Optional[int] = None,
                 buffer: Optional[torch.Tensor] = None) -> StepContext:
        n_tokens = sum(len(entry.tokens) for entry in entries)
        n_wanted = sum(len(entry.want) for entry in entries)
        max_new = max(len(entry.tokens) for entry in entries)
        max_len = max(start + len(entry.tokens) for entry, start in zip(entries, starts))
        stride = page_stride if page_stride is not None else pages_for(max_len)
        layout = StepLayout(n_tokens, len(entries), n_wanted, {group: stride for group in self.cache.kv})
        self.last_step_ints = layout.total
        if buffer is None:
            buffer = torch.empty(layout.total, dtype=torch.int32, device=self.device)
        if self.device.type == "cuda":
            ring = self.ring(layout.total)
            staged, ticket = ring.acquire(layout.total)
            fill_step(layout, staged, entries, starts, self.cache)
            ring.upload(ticket, layout.total, buffer)
        else:
            staged = np.zeros(layout.total, dtype=np.int32)
            fill_step(layout, staged, entries, starts, self.cache)
            buffer.copy_(torch.from_numpy(staged))
        return step_views(layout, buffer, max_new, max_len, all(len(entry.tokens) == 1 for entry in entries))

    def step(self, entries: Sequence[StepEntry], device_tokens: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
        """Runs the entries' tokens; returns 32-bit logits `[wanted places, vocab]` in the order of the
        entries and of their `want`, or None if nothing is wanted.

        How long the logits stay valid: a step in which every entry brings one token and wants it (a decode step)
        returns a buffer that belongs to the captured graph of that batch size; the next decode step of the same batch
        size writes its logits into the same buffer.  Use them (select, copy to the host) or `clone()` them before
        that step.  Every other step returns a tensor of its own.

        `device_tokens` (int32, one per entry, on the engine's device) replaces the token ids of a step in which every
        entry brings one token: the ids are taken on the device, in stream order, so a step can be started before the
        host has seen what the step before it chose.  An id outside the vocabulary embeds as zeros."""
        starts = self._validate(entries)
        if device_tokens is not None and (any(len(entry.tokens) != 1 for entry in entries) or device_tokens.numel() != len(entries)
                                          or device_tokens.dtype != torch.int32 or device_tokens.device != self.device):
            raise StepError("device tokens need one int32 id per entry on the engine's device, and one token per entry")
        for entry, start in zip(entries, starts):
            self.cache.reserve(entry.slot, start + len(entry.tokens))
        single = all(len(entry.tokens) == 1 and tuple(entry.want) == (0,) for entry in entries)
        if single and self.use_graphs:
            from .graph import run_decode_graph
            logits = run_decode_graph(self, entries, starts, device_tokens)
        else:
            context = self._context(entries, starts)
            if device_tokens is not None:
                context.token_ids.copy_(device_tokens)
            if context.all_single and self.attention_block_size:
                context.decode_splits = self.decode_splits(len(entries), max(starts) + 1)
            logits = self.model.forward(context, self.cache)
        for entry, start in zip(entries, starts):
            self.cache.advance(entry.slot, start + len(entry.tokens))
        return logits
