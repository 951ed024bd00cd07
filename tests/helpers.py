"""Shared by the tests: building engines on tiny folders, replaying requests in several cuttings."""
from __future__ import annotations

from typing import Dict, List, Sequence

import numpy as np
import torch

import plain_model
from tau_rs_b200 import Engine, StepEntry, load_model


def random_prompts(vocab: int, lengths: Sequence[int], seed: int) -> List[List[int]]:
    rng = np.random.default_rng(seed)
    return [rng.integers(0, vocab, size=length).tolist() for length in lengths]


def plain_logits(folder: str, tokens: Sequence[int], bf16: bool = False) -> torch.Tensor:
    config = plain_model.read_plain_config(folder)
    weights = plain_model.read_plain_weights(folder)
    if bf16:
        weights = {name: plain_model.bfloat16_rounding(value) if value.dim() > 1 else value for name, value in weights.items()}
    rounding = plain_model.bfloat16_rounding if bf16 else plain_model.no_rounding
    return plain_model.forward_logits(config, weights, tokens, rounding)


def engine_for(folder: str, dtype: str, device, max_tokens: int = 4096) -> Engine:
    device = torch.device(device) if isinstance(device, str) and device != "gpu" else device
    return Engine(load_model(folder, dtype, device), max_tokens)


def run_whole(engine: Engine, tokens: Sequence[int]) -> torch.Tensor:
    """One request alone, all tokens in one step, logits everywhere."""
    slot = engine.open_sequence()
    try:
        logits = engine.step([StepEntry(slot, list(tokens), list(range(len(tokens))))])
        return logits.float().cpu().clone()
    finally:
        engine.close_sequence(slot)


def run_tail_stepwise(engine: Engine, tokens: Sequence[int], tail: int) -> torch.Tensor:
    """The prefix in one step, the last `tail` tokens one by one; logits of the tail."""
    tail = min(tail, len(tokens) - 1)
    slot = engine.open_sequence()
    rows = []
    try:
        prefix = list(tokens[: len(tokens) - tail])
        engine.step([StepEntry(slot, prefix, [])])
        for token in tokens[len(tokens) - tail :]:
            rows.append(engine.step([StepEntry(slot, [token], [0])]).float().cpu().clone())
        return torch.cat(rows, dim=0)
    finally:
        engine.close_sequence(slot)


def run_batched(engine: Engine, requests: Sequence[Sequence[int]], prompt_lengths: Sequence[int]) -> List[torch.Tensor]:
    """Requests start together: prompts of the given lengths in one step, then one token each until each
    request's tokens run out; a request that ends gives its slot back at once.  Returns for each request
    the logits at its last prompt token and at every later token."""
    slots = [engine.open_sequence() for _ in requests]
    live = list(range(len(requests)))
    out: List[List[torch.Tensor]] = [[] for _ in requests]
    try:
        entries = [StepEntry(slots[i], list(requests[i][: prompt_lengths[i]]), [prompt_lengths[i] - 1]) for i in live]
        logits = engine.step(entries).float().cpu()
        for row, i in enumerate(live):
            out[i].append(logits[row].clone())
        cursor = {i: prompt_lengths[i] for i in live}
        while True:
            for i in list(live):
                if cursor[i] >= len(requests[i]):
                    engine.close_sequence(slots[i])
                    live.remove(i)
            if not live:
                break
            entries = [StepEntry(slots[i], [requests[i][cursor[i]]], [0]) for i in live]
            logits = engine.step(entries).float().cpu()
            for row, i in enumerate(live):
                out[i].append(logits[row].clone())
                cursor[i] += 1
        return [torch.stack(rows) for rows in out]
    finally:
        for i in live:
            engine.close_sequence(slots[i])


def relative_error(found: torch.Tensor, wanted: torch.Tensor) -> float:
    """Largest absolute difference over the largest absolute wanted value."""
    return float((found.double() - wanted.double()).abs().max() / wanted.double().abs().max())
