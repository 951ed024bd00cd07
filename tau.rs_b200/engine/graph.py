"""One captured CUDA graph per decode batch size.

crates/models/src/qwen3_5_common/model/graph.rs:33-51,162-225: a warm-up run, then a
capture of the whole forward over fixed buffers, then per step only a metadata write and
a replay.  A decode step here has a fixed shape for a given number of sequences (one token
and one wanted place each); everything that changes between steps (tokens, positions,
page rows, lengths) lies in the metadata buffer at a fixed address, and kernels take no
host value that depends on the sequences' lengths except the number of context splits,
which is part of the graph's key.
"""
from __future__ import annotations

from typing import Sequence

import numpy as np
import torch

from ..csrc import kernels
from .batch import StepEntry, StepLayout, step_views


class _DecodeGraph:
    """A captured decode step for one number of sequences and one number of context splits.

    The layout of the metadata buffer, its device views and the parts of it that never change (row numbers,
    token-to-sequence map, run bounds) are made once; a step fills in tokens, positions, slots, lengths and page rows.
    """

    def __init__(self, engine, n_seqs: int, splits: int):
        self.stride = engine.cache.pages_per_sequence
        self.layout = StepLayout(n_seqs, n_seqs, n_seqs, {group: self.stride for group in engine.cache.kv})
        self.buffer = torch.zeros(self.layout.total, dtype=torch.int32, device=engine.device)
        self.context = step_views(self.layout, self.buffer, 1, 1, True)
        self.context.decode_splits = splits
        self.graph = None
        self.logits = None
        self.splits = splits
        self.launches = 0
        off = self.layout.offsets
        self.constant = np.zeros(self.layout.total, dtype=np.int32)
        counting = np.arange(n_seqs + 1, dtype=np.int32)
        self.constant[off["token_seq"] : off["token_seq"] + n_seqs] = counting[:n_seqs]
        self.constant[off["want_rows"] : off["want_rows"] + n_seqs] = counting[:n_seqs]
        self.constant[off["cu_seqlens"] : off["cu_seqlens"] + n_seqs + 1] = counting

    def fill(self, staged: np.ndarray, entries, starts, cache) -> None:
        n, off = self.layout.n_seqs, self.layout.offsets
        staged[:] = self.constant
        slots = [entry.slot for entry in entries]
        staged[off["token_ids"] : off["token_ids"] + n] = [entry.tokens[0] for entry in entries]
        staged[off["positions"] : off["positions"] + n] = starts
        staged[off["seq_slot"] : off["seq_slot"] + n] = slots
        staged[off["seq_start"] : off["seq_start"] + n] = starts
        staged[off["seq_len"] : off["seq_len"] + n] = staged[off["seq_start"] : off["seq_start"] + n] + 1
        for group, stride in self.layout.page_stride.items():
            begin = off["pages:" + group]
            staged[begin : begin + n * stride] = cache.page_rows(group, slots, stride).reshape(-1)


def run_decode_graph(engine, entries: Sequence[StepEntry], starts: Sequence[int], device_tokens=None):
    max_len = max(starts) + 1
    bucket = (len(entries), max(0, (max_len - 1).bit_length()))
    splits = engine._split_choice.get(bucket)
    if splits is None:
        splits = engine._split_choice[bucket] = engine.decode_splits(len(entries), max_len)
    key = (len(entries), splits)
    state = engine._graphs.get(key)
    if state is None:
        state = engine._graphs[key] = _DecodeGraph(engine, len(entries), splits)
    engine.last_step_ints = state.layout.total
    staged, ticket = engine.ring(state.layout.total).acquire(state.layout.total)
    state.fill(staged, entries, starts, engine.cache)
    engine.ring(state.layout.total).upload(ticket, state.layout.total, state.buffer)
    context = state.context
    if device_tokens is not None:   # after the upload, in stream order: the ids that an earlier kernel chose
        context.token_ids.copy_(device_tokens)
    context.max_len = max_len
    if state.graph is None:
        # Warm-up outside capture: compiles and loads every kernel, sizes torch's pools.
        stream = torch.cuda.Stream()
        stream.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(stream):
            engine.model.forward(context, engine.cache)
        torch.cuda.current_stream().wait_stream(stream)
        graph = torch.cuda.CUDAGraph()
        before = kernels.launch_count()
        with torch.cuda.graph(graph):
            state.logits = engine.model.forward(context, engine.cache)
        state.launches = kernels.launch_count() - before
        state.graph = graph
    state.graph.replay()
    kernels.count_replay(state.launches)
    return state.logits
