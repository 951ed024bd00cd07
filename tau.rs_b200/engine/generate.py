"""The generation loop above the step function.

Per request the reference resets, reserves `prompt + max_new`, prefills, decodes and
resets again, on every exit path (crates/engine/src/model_engine/generation.rs:33-56,
60-116).  The token chosen after the prompt counts toward the limit (:97-101); a stop token
is neither returned nor fed back (:280-285); a request ends with `length` iff it produced
`max_new` tokens, else `stop` (crates/engine/src/model_engine.rs:243-247); `max_new == 0`
returns at once without touching the model (:152-159); an empty prompt is an error
(:187-192); `prompt + max_new` must fit the context (crates/engine/src/model_engine/
kv_budget.rs:126-134).  Here the unit is a batch: requests that start together with
unequal prompts, prefilled in one packed step (or in chunks of it), decoded one token each
per step; a request that ends gives its slot back at once and the rest go on; when there
are more requests than fit, batches run one after another on the same cache.

The loop needs only `open_sequence`, `close_sequence`, `step` and the two limits of a
backend, and a `select` function, so its decisions can be tested with fakes.

Where the backend takes token ids from the device (`accepts_device_tokens`) and `select`
comes in two halves (`launch`, `collect`), decoding runs one step ahead of the host: step
t + 1 is started with the ids that step t chose, straight from the device, and only then
does the host wait for step t's ids, look for stop tokens and book the results.  A request
that turns out to have stopped at step t has had one more token computed, which is dropped
with its slot; a request whose limit the token of step t reaches is left out of step t + 1
beforehand.  The tokens are the same either way.
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field
from typing import Callable, List, Optional, Sequence

from ..cache.sequence_cache import PAGE_TOKENS, pages_for
from ..config.errors import AllLogitsNaN
from .batch import StepEntry


@dataclass
class GenerationResult:
    tokens: List[int]
    finish_reason: str        # "stop" or "length"
    prompt_tokens: int


@dataclass
class GenerationMetrics:
    """Counters in the reference's sense (crates/metrics/src/serving.rs:35-54,84-93): the decode
    rate is decoded tokens over the summed time of decode steps; the token that prefill produces
    and stop tokens are not decoded tokens.

    With `log_interval_s` and `sink`, a record with `status: "running"` goes to `sink` at a token boundary whenever
    that many seconds have passed since the last one (serving.rs:56-58,92-95,160-165: every 5 s there, no thread of
    its own); `interval_decode_tokens_per_second` is the rate of the decode work since the record before (:46-47).

    Beyond the reference's fields: where the backend says how many bytes a decode step has to read (every weight once and
    the cache of the live requests), `decode_gb_per_second` is that over the decode time, and with `peak_gb_per_second`
    (the device's measured copy bandwidth) `fraction_of_roofline` is their ratio."""

    prompt_tokens: int = 0
    generated_tokens: int = 0
    decode_tokens: int = 0
    prefill_ms: float = 0.0
    decode_ms: float = 0.0
    prefill_steps: int = 0
    decode_steps: int = 0
    batches: int = 0
    decode_bytes: int = 0
    peak_gb_per_second: Optional[float] = None
    log_interval_s: Optional[float] = None
    sink: Optional[Callable[[dict], None]] = None
    _started: float = field(default_factory=time.perf_counter, repr=False)
    _last_reported: float = field(default_factory=time.perf_counter, repr=False)
    _last_decode_tokens: int = field(default=0, repr=False)
    _last_decode_ms: float = field(default=0.0, repr=False)

    def report(self, status: str, now: Optional[float] = None) -> dict:
        """The counters as one record; advances the interval's baseline."""
        now = time.perf_counter() if now is None else now
        tokens, span = self.decode_tokens - self._last_decode_tokens, self.decode_ms - self._last_decode_ms
        record = dict(self.as_dict(), status=status, elapsed_ms=round((now - self._started) * 1e3, 3),
                      interval_decode_tokens_per_second=round(tokens / (span / 1e3), 2) if tokens > 0 and span > 0 else None)
        self._last_reported, self._last_decode_tokens, self._last_decode_ms = now, self.decode_tokens, self.decode_ms
        return record

    def tick(self, now: Optional[float] = None) -> None:
        """Called at token boundaries of decoding: sends a progress record if one is due."""
        if self.log_interval_s is None or self.sink is None:
            return
        now = time.perf_counter() if now is None else now
        if now - self._last_reported >= self.log_interval_s:
            self.sink(self.report("running", now))

    @property
    def decode_tokens_per_second(self) -> float:
        return self.decode_tokens / (self.decode_ms / 1e3) if self.decode_ms > 0 else 0.0

    @property
    def decode_gb_per_second(self) -> Optional[float]:
        return self.decode_bytes / (self.decode_ms * 1e6) if self.decode_bytes and self.decode_ms > 0 else None

    @property
    def prefill_tokens_per_second(self) -> float:
        return self.prompt_tokens / (self.prefill_ms / 1e3) if self.prefill_ms > 0 else 0.0

    def as_dict(self) -> dict:
        return {
            "prompt_tokens": self.prompt_tokens, "generated_tokens": self.generated_tokens,
            "decode_tokens": self.decode_tokens, "prefill_ms": round(self.prefill_ms, 3),
            "decode_ms": round(self.decode_ms, 3),
            "decode_tokens_per_second": round(self.decode_tokens_per_second, 2),
            "prefill_tokens_per_second": round(self.prefill_tokens_per_second, 2),
            "prefill_steps": self.prefill_steps, "decode_steps": self.decode_steps, "batches": self.batches,
            "decode_gb_per_second": self.decode_gb_per_second and round(self.decode_gb_per_second, 1),
            "fraction_of_roofline": (round(self.decode_gb_per_second / self.peak_gb_per_second, 4)
                                     if self.decode_gb_per_second and self.peak_gb_per_second else None),
        }


def plan_batches(needs: Sequence[int], max_batch: int, capacity_tokens: int) -> List[List[int]]:
    """Splits request numbers `0..n` into consecutive batches.

    `needs[i]` is the most tokens request `i` can come to hold at one time.  A batch has at most
    `max_batch` requests and its needs, each rounded up to whole pages, fit the cache.
    """
    batches: List[List[int]] = []
    current: List[int] = []
    used = 0
    for index, need in enumerate(needs):
        rounded = pages_for(need) * PAGE_TOKENS
        if rounded > capacity_tokens:
            raise ValueError(f"request {index} needs {rounded} cache tokens, the cache holds {capacity_tokens}")
        if current and (len(current) >= max_batch or used + rounded > capacity_tokens):
            batches.append(current)
            current, used = [], 0
        current.append(index)
        used += rounded
    if current:
        batches.append(current)
    return batches


@dataclass(eq=False)     # a request in flight is itself, whatever it holds
class _Live:
    request: int
    slot: int
    prompt: Sequence[int]
    limit: int
    fed: int = 0
    produced: List[int] = field(default_factory=list)


def generate_tokens(backend, prompts: Sequence[Sequence[int]], max_new_tokens, select: Callable, stop_tokens=(),
                    max_batch: int = 64, prefill_chunk_tokens: Optional[int] = None,
                    metrics: Optional[GenerationMetrics] = None) -> List[GenerationResult]:
    """Generates for every prompt; results keep the order of the prompts.

    `max_new_tokens` is one limit or one per prompt.  `select(logits, request_ids,
    token_indices) -> tokens` chooses one token per logits row.  `backend` offers
    `open_sequence()`, `close_sequence(slot)`, `step(entries)`, `capacity_tokens` and
    `max_sequence_tokens`.
    """
    limits = list(max_new_tokens) if isinstance(max_new_tokens, (list, tuple)) else [max_new_tokens] * len(prompts)
    if len(limits) != len(prompts):
        raise ValueError("one output limit per prompt is needed")
    if prefill_chunk_tokens is not None and prefill_chunk_tokens <= 0:
        raise ValueError("prefill chunk size must be positive")
    if max_batch <= 0:
        raise ValueError("the batch size must be positive")
    stop = frozenset(stop_tokens)
    metrics = metrics if metrics is not None else GenerationMetrics()
    for index, (prompt, limit) in enumerate(zip(prompts, limits)):
        if limit < 0:
            raise ValueError(f"request {index}: the output limit must not be negative")
        if limit > 0 and len(prompt) == 0:
            raise ValueError(f"request {index}: the prompt is empty")
        if limit > 0 and len(prompt) + limit > backend.max_sequence_tokens:
            raise ValueError(
                f"request {index}: prompt ({len(prompt)}) plus output limit ({limit}) exceeds the "
                f"context of {backend.max_sequence_tokens} tokens"
            )
    results: List[Optional[GenerationResult]] = [None] * len(prompts)
    active = []
    for index, (prompt, limit) in enumerate(zip(prompts, limits)):
        if limit == 0:
            results[index] = GenerationResult([], "length", len(prompt))
        else:
            active.append(index)
    # What a request holds in the cache at most: its whole length, unless the backend knows better (windows let pages go).
    peak = getattr(backend, "peak_cache_tokens", None)
    needs = [len(prompts[index]) + limits[index] if peak is None
             else peak(len(prompts[index]), len(prompts[index]) + limits[index], prefill_chunk_tokens) for index in active]
    for batch in plan_batches(needs, max_batch, backend.capacity_tokens):
        metrics.batches += 1
        _run_batch(backend, [active[position] for position in batch], prompts, limits, select, stop,
                   prefill_chunk_tokens, metrics, results)
    return results


def _run_batch(backend, requests, prompts, limits, select, stop, chunk, metrics, results) -> None:
    live: List[_Live] = []
    try:
        for request in requests:
            live.append(_Live(request, backend.open_sequence(), prompts[request], limits[request]))

        def finish(item: _Live, reason: str) -> None:
            results[item.request] = GenerationResult(item.produced, reason, len(item.prompt))
            backend.close_sequence(item.slot)
            live.remove(item)

        def accept(item: _Live, token: int) -> None:
            if token < 0:   # the selector found only NaN in this request's row
                raise AllLogitsNaN(f"request {item.request}: model logits are all NaN")
            if token in stop:
                finish(item, "stop")
                return
            item.produced.append(token)
            metrics.generated_tokens += 1
            if len(item.produced) == item.limit:
                finish(item, "length")

        # Prefill: the prompts packed along one axis, in chunks of at most `chunk` tokens.
        first_tokens = {}
        started = time.perf_counter()
        while any(item.fed < len(item.prompt) for item in live):
            budget = chunk if chunk is not None else sum(len(item.prompt) for item in live)
            entries, owners = [], []
            for item in live:
                remaining = len(item.prompt) - item.fed
                if remaining == 0 or budget == 0:
                    continue
                count = min(remaining, budget)
                ends = item.fed + count == len(item.prompt)
                entries.append(StepEntry(item.slot, item.prompt[item.fed : item.fed + count], [count - 1] if ends else []))
                if ends:
                    owners.append(item)
                item.fed += count
                budget -= count
            logits = backend.step(entries)
            metrics.prefill_steps += 1
            if owners:
                tokens = select(logits, [item.request for item in owners], [0] * len(owners))
                for item, token in zip(owners, tokens):
                    first_tokens[item.request] = token
        metrics.prefill_ms += (time.perf_counter() - started) * 1e3
        metrics.prompt_tokens += sum(len(item.prompt) for item in live)
        for item in list(live):
            accept(item, first_tokens[item.request])

        # Decode: one token for every request that is still going.
        step_bytes = getattr(backend, "bytes_read_by_a_decode_step", lambda: 0)
        launch, collect = getattr(select, "launch", None), getattr(select, "collect", None)
        if launch is not None and collect is not None and getattr(backend, "accepts_device_tokens", False):
            _decode_ahead(backend, live, launch, collect, stop, accept, metrics, step_bytes)
        while live:
            started = time.perf_counter()
            entries = [StepEntry(item.slot, [item.produced[-1]], [0]) for item in live]
            logits = backend.step(entries)
            tokens = select(logits, [item.request for item in live], [len(item.produced) for item in live])
            metrics.decode_ms += (time.perf_counter() - started) * 1e3
            metrics.decode_steps += 1
            metrics.decode_bytes += step_bytes()
            for item, token in zip(list(live), tokens):
                if token not in stop:
                    metrics.decode_tokens += 1
                accept(item, token)
            metrics.tick()
    finally:
        for item in list(live):
            backend.close_sequence(item.slot)


def _decode_ahead(backend, live, launch, collect, stop, accept, metrics, step_bytes=lambda: 0) -> None:
    """The decode loop, one step ahead of the host; returns with `live` empty."""
    if not live:
        return
    started = time.perf_counter()
    # The first step takes its tokens from the host (the prefill chose them).
    items = list(live)
    logits = backend.step([StepEntry(item.slot, [item.produced[-1]], [0]) for item in items])
    pending = launch(logits, [item.request for item in items], [len(item.produced) for item in items])
    metrics.decode_steps += 1
    metrics.decode_bytes += step_bytes()
    while True:
        # Who goes on after the token that is on its way?  Not those whose limit it reaches; the others do, unless it
        # turns out to be a stop token, which is known only after their next step has been started.
        # (A request of `items` that stopped at the step before is still in `items`, for its row, but no longer in `live`.)
        rows = [row for row, item in enumerate(items) if item in live and len(item.produced) + 1 < item.limit]
        following = None
        if rows:
            next_items = [items[row] for row in rows]
            tokens_on_device = pending.tokens if len(rows) == len(items) else _take(pending.tokens, rows)
            logits = backend.step([StepEntry(item.slot, [0], [0]) for item in next_items], device_tokens=tokens_on_device)
            following = launch(logits, [item.request for item in next_items], [len(item.produced) + 1 for item in next_items])
            metrics.decode_steps += 1
            metrics.decode_bytes += step_bytes()
        tokens = collect(pending)
        for item, token in zip(items, tokens):
            if item not in live:      # stopped one step ago; this token was computed for nothing
                continue
            if token not in stop:
                metrics.decode_tokens += 1
            accept(item, token)
        now = time.perf_counter()
        metrics.decode_ms += (now - started) * 1e3
        started = now
        if following is None:
            break
        metrics.tick(now)
        items, pending = next_items, following


def _take(tokens, rows):
    """The entries `rows` (ascending) of the ids that a step chose, where they are: a device tensor, or a fake's list."""
    if isinstance(tokens, list):
        return [tokens[row] for row in rows]
    if rows == list(range(rows[0], rows[-1] + 1)):
        return tokens[rows[0] : rows[-1] + 1]
    import torch

    if tokens.device.type != "cuda":
        return tokens.index_select(0, torch.tensor(rows, dtype=torch.int64, device=tokens.device))
    # The row numbers go up from page-locked memory without waiting (a copy from ordinary memory would make the host wait
    # for the stream, and with it for the step that runs ahead).  A place is used again eight calls later.
    ring = _row_rings.setdefault(tokens.device, [[], 0])
    if len(ring[0]) < 8 or ring[0][0].numel() < len(rows):
        ring[0] = [torch.empty(max(256, 2 * len(rows)), dtype=torch.int64).pin_memory() for _ in range(8)]
    host = ring[0][ring[1] % 8]
    ring[1] += 1
    host.numpy()[: len(rows)] = rows
    return tokens.index_select(0, host[: len(rows)].to(tokens.device, non_blocking=True))


_row_rings = {}   # device -> [page-locked buffers, calls so far]
