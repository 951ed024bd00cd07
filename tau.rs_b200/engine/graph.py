"""One captured CUDA graph per decode batch size.

crates/models/src/qwen3_5_common/model/graph.rs:33-51,162-225: a warm-up run, then a
capture of the whole forward over fixed buffers, then per step only a metadata write and
a replay.  A decode step here has a fixed shape for a given number of sequences (one token
and one wanted place each); everything that changes between steps (tokens, positions,
page rows, lengths) lies in the metadata buffer at a fixed address, and kernels take no
host value that depends on the sequences' lengths except the number of context splits,
which is part of the graph's key.

All graphs of an engine are captured into one memory pool and warmed up on one side stream, and the
least recently used ones are dropped beyond `MAX_GRAPHS`, so a batch that shrinks request by request
does not leave a private pool of activations and logits behind for every size it went through.
A mixer that updates per-sequence state in place would see its state advanced twice, by the warm-up
run and by the first replay; the state of the step's sequences is therefore put back after the
warm-up (the reference snapshots such state around its warm-up the same way, model/graph.rs:183-211).
"""
from __future__ import annotations

from typing import Sequence

import numpy as np
import torch

from ..csrc import kernels
from .batch import StepEntry, StepLayout, step_views

MAX_GRAPHS = 96   # per engine; a graph of a Qwen3-8B step holds a few MB of activations and its logits


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
    state = engine._graphs.pop(key, None)
    if state is None:
        state = _DecodeGraph(engine, len(entries), splits)
        while len(engine._graphs) >= MAX_GRAPHS:
            engine._graphs.pop(next(iter(engine._graphs)))     # the least recently used: a dict keeps its order
    engine._graphs[key] = state                                 # (re-)inserted as the most recent
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
        if engine._graph_stream is None:
            engine._graph_stream = torch.cuda.Stream()
            engine._graph_pool = torch.cuda.graph_pool_handle()
        stream = engine._graph_stream
        slots = [entry.slot for entry in entries]
        kept = {name: group.state[:, slots].clone() for name, group in engine.cache.states.items()}
        stream.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(stream):
            engine.model.forward(context, engine.cache)
        torch.cuda.current_stream().wait_stream(stream)
        for name, group in engine.cache.states.items():        # the warm-up advanced the state; the replay below is the step
            group.state[:, slots] = kept[name]
        graph = torch.cuda.CUDAGraph()
        before = kernels.launch_count()
        with torch.cuda.graph(graph, pool=engine._graph_pool, stream=stream):
            state.logits = engine.model.forward(context, engine.cache)
        state.launches = kernels.launch_count() - before
        state.graph = graph
    state.graph.replay()
    kernels.count_replay(state.launches)
    return state.logits
