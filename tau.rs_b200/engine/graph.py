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

import torch

from ..csrc import kernels
from .batch import StepEntry, StepLayout


class _DecodeGraph:
    def __init__(self, engine, n_seqs: int, splits: int):
        self.stride = engine.cache.pages_per_sequence
        layout = StepLayout(n_seqs, n_seqs, n_seqs, {group: self.stride for group in engine.cache.kv})
        self.buffer = torch.zeros(layout.total, dtype=torch.int32, device=engine.device)
        self.graph = None
        self.logits = None
        self.splits = splits
        self.launches = 0


def run_decode_graph(engine, entries: Sequence[StepEntry], starts: Sequence[int]):
    max_len = max(start + 1 for start in starts)
    splits = engine.model.decode_splits(len(entries), max_len)
    key = (len(entries), splits)
    state = engine._graphs.get(key)
    if state is None:
        state = engine._graphs[key] = _DecodeGraph(engine, len(entries), splits)
    context = engine._context(entries, starts, page_stride=state.stride, buffer=state.buffer)
    context.decode_splits = splits
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
