"""What one step runs, on the host and as device metadata.

The reference forwards `input [1, T]` at one `offset` (crates/models/src/
interface.rs:24-28) and keeps `[token, position]` in device memory so that one captured
graph serves every decode step (crates/models/src/components/cuda/decode.rs:489-513).
Here a step is a batch of sequences, each with its own run of new tokens; the tokens are
packed along one axis, and the same metadata, for every token and sequence, travels to
the device as one int32 buffer.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Sequence

import numpy as np
import torch



@dataclass
class StepEntry:
    """The next tokens of one sequence, and the places among them whose logits are wanted."""

    slot: int
    tokens: Sequence[int]
    want: Sequence[int] = ()


def _aligned(count: int) -> int:
    return (count + 3) // 4 * 4


@dataclass
class StepLayout:
    """Offsets (in ints) of each array inside the step's metadata buffer."""

    n_tokens: int
    n_seqs: int
    n_wanted: int
    page_stride: Dict[str, int]
    offsets: Dict[str, int] = field(default_factory=dict)
    total: int = 0

    def __post_init__(self):
        cursor = 0
        for name, count in (
            ("token_ids", self.n_tokens), ("positions", self.n_tokens), ("token_seq", self.n_tokens),
            ("want_rows", self.n_wanted), ("cu_seqlens", self.n_seqs + 1), ("seq_slot", self.n_seqs),
            ("seq_start", self.n_seqs), ("seq_len", self.n_seqs),
        ):
            self.offsets[name] = cursor
            cursor += _aligned(count)
        for group, stride in self.page_stride.items():
            self.offsets["pages:" + group] = cursor
            cursor += _aligned(self.n_seqs * stride)
        self.total = cursor


@dataclass
class StepContext:
    """Device views of a step's metadata (all int32), with the host facts kernels are launched by."""

    n_tokens: int
    n_seqs: int
    n_wanted: int
    token_ids: torch.Tensor      # [n_tokens]
    positions: torch.Tensor      # [n_tokens] absolute position of each token in its sequence
    token_seq: torch.Tensor      # [n_tokens] index of the token's sequence within this step
    want_rows: torch.Tensor      # [n_wanted] packed rows whose logits are wanted
    cu_seqlens: torch.Tensor     # [n_seqs + 1] first packed row of each sequence
    seq_slot: torch.Tensor       # [n_seqs] cache slot of each sequence
    seq_start: torch.Tensor      # [n_seqs] positions the cache held before this step
    seq_len: torch.Tensor        # [n_seqs] positions it holds after this step
    page_rows: Dict[str, torch.Tensor]   # group -> [n_seqs, stride] page numbers
    max_new: int                 # longest run of new tokens
    max_len: int                 # longest sequence after the step
    all_single: bool             # every sequence brings exactly one token
    decode_splits: int = 0       # context splits of decode attention, fixed by a captured graph (0: chosen per step)


def fill_step(layout: StepLayout, out: np.ndarray, entries: Sequence[StepEntry], starts: Sequence[int], cache) -> None:
    """Writes the metadata of `entries` into `out` (int32, `layout.total` long)."""
    off = layout.offsets
    cursor = 0
    wanted = 0
    cu = out[off["cu_seqlens"] : off["cu_seqlens"] + layout.n_seqs + 1]
    for index, (entry, start) in enumerate(zip(entries, starts)):
        count = len(entry.tokens)
        cu[index] = cursor
        out[off["token_ids"] + cursor : off["token_ids"] + cursor + count] = entry.tokens
        out[off["positions"] + cursor : off["positions"] + cursor + count] = np.arange(start, start + count, dtype=np.int32)
        out[off["token_seq"] + cursor : off["token_seq"] + cursor + count] = index
        for place in entry.want:
            out[off["want_rows"] + wanted] = cursor + place
            wanted += 1
        out[off["seq_slot"] + index] = entry.slot
        out[off["seq_start"] + index] = start
        out[off["seq_len"] + index] = start + count
        cursor += count
    cu[layout.n_seqs] = cursor
    slots = [entry.slot for entry in entries]
    for group, stride in layout.page_stride.items():
        begin = off["pages:" + group]
        out[begin : begin + layout.n_seqs * stride] = cache.page_rows(group, slots, stride).reshape(-1)


def step_views(layout: StepLayout, buffer: torch.Tensor, max_new: int, max_len: int, all_single: bool) -> StepContext:
    off = layout.offsets

    def view(name, count):
        return buffer[off[name] : off[name] + count]

    pages = {
        group: buffer[off["pages:" + group] : off["pages:" + group] + layout.n_seqs * stride].view(layout.n_seqs, stride)
        for group, stride in layout.page_stride.items()
    }
    return StepContext(
        n_tokens=layout.n_tokens, n_seqs=layout.n_seqs, n_wanted=layout.n_wanted,
        token_ids=view("token_ids", layout.n_tokens), positions=view("positions", layout.n_tokens),
        token_seq=view("token_seq", layout.n_tokens), want_rows=view("want_rows", layout.n_wanted),
        cu_seqlens=view("cu_seqlens", layout.n_seqs + 1), seq_slot=view("seq_slot", layout.n_seqs),
        seq_start=view("seq_start", layout.n_seqs), seq_len=view("seq_len", layout.n_seqs),
        page_rows=pages, max_new=max_new, max_len=max_len, all_single=all_single,
    )
