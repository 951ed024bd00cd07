"""Choosing the next token from 32-bit logits, on the device.

Greedy: the greatest logit by the total order of 32-bit floats, NaN never chosen, the
highest token id among equals, an error if every logit is NaN
(crates/engine/src/generation.rs:81-95; crates/cuda-kernels/src/kernels/
greedy_argmax.cu:19-31).  The reference samples with nothing else (its request parser
takes no temperature, crates/server/src/chat_completions_handler/request.rs:27-110).
Temperature sampling is this library's own: `argmax(logit / T + g)` with Gumbel noise
`g = -log(-log u)` from a counter-based generator keyed by the seed, the request's number
and the index of the token within the request, so a request's tokens do not depend on
what else is in its batch.  `T == 0` means greedy.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Sequence

import torch

from ..config.errors import AllLogitsNaN
from ..csrc import kernels


@dataclass(frozen=True)
class SamplingParams:
    temperature: float = 0.0
    seed: int = 0

    def __post_init__(self):
        if not self.temperature >= 0.0:
            raise ValueError("temperature must be zero (greedy) or positive")


NO_TOKEN = -1   # what `collect` gives for a row with nothing to choose from


class Pending:
    """Tokens that have been chosen on the device and are on their way to the host."""

    def __init__(self, result: torch.Tensor, host: torch.Tensor, done):
        self.result = result          # [2, rows] on the device: token ids, and whether the row had a number to choose from
        self.host = host              # the same, on the host (pinned), valid once `done` has passed
        self.done = done              # an event, or None where the copy was synchronous

    @property
    def tokens(self) -> torch.Tensor:
        """The chosen ids on the device, for a step that starts before the host has seen them."""
        return self.result[0]


class Sampler:
    """`select` chooses and waits; `launch` and `collect` are its two halves, so that a caller can put more work
    on the device between them: the host waits for the event behind the copy of the tokens, not for the stream."""

    def __init__(self, params: SamplingParams = SamplingParams()):
        self.params = params
        self._pinned = {}
        self._key_rings = {}
        self._next = 0

    def launch(self, logits: torch.Tensor, request_ids: Sequence[int], token_indices: Sequence[int]) -> Pending:
        rows = logits.shape[0]
        result = torch.empty((2, rows), dtype=torch.int32, device=logits.device)
        if self.params.temperature == 0.0:
            kernels.argmax(logits, result[0], result[1])
        else:
            keys = self._upload(logits.device, request_ids, token_indices)
            kernels.sample_gumbel(logits, result[0], result[1], 1.0 / self.params.temperature, self.params.seed, keys[0], keys[1])
        if logits.device.type != "cuda":
            return Pending(result, result, None)
        if (rows, logits.device) not in self._pinned:
            self._pinned[(rows, logits.device)] = [torch.empty((2, rows), dtype=torch.int32).pin_memory() for _ in range(4)]
        ring = self._pinned[(rows, logits.device)]
        host = ring[self._next % len(ring)]
        self._next += 1
        # A kernel stores the tokens into page-locked host memory (a copy by the copy engine in this stream held the next
        # step up by 80 us) and an event marks it: work put on the stream afterwards (the next step) does not hold up the
        # host's wait for these tokens.
        kernels.store_words_host(result, host)
        done = torch.cuda.Event()
        done.record()
        return Pending(result, host, done)

    def _upload(self, device, request_ids: Sequence[int], token_indices: Sequence[int]) -> torch.Tensor:
        """The rows' request numbers and token indices on the device, `[2, rows]`.  From page-locked memory and without
        waiting: a copy from ordinary memory would make the host wait for the stream, and with it for the step that the
        generation loop has just put there to run while the host works."""
        rows = len(request_ids)
        if device.type != "cuda":
            return torch.tensor([list(request_ids), list(token_indices)], dtype=torch.int32, device=device)
        if (rows, device) not in self._key_rings:   # a place is used again four launches later: the copy out of it is long over
            self._key_rings[(rows, device)] = [torch.empty((2, rows), dtype=torch.int32).pin_memory() for _ in range(4)]
        ring = self._key_rings[(rows, device)]
        host = ring[self._next % len(ring)]
        view = host.numpy()
        view[0, :] = request_ids
        view[1, :] = token_indices
        return host.to(device, non_blocking=True)

    def collect(self, pending: Pending) -> List[int]:
        """Blocks until the tokens of `pending` are on the host.  A row that held only NaN gives `NO_TOKEN`: whether that
        is an error is for the caller to say, who knows whether the row's request is still going."""
        if pending.done is not None:
            pending.done.synchronize()
        tokens, valid = pending.host.tolist()
        return [token if ok else NO_TOKEN for token, ok in zip(tokens, valid)]

    def select(self, logits: torch.Tensor, request_ids: Sequence[int], token_indices: Sequence[int]) -> List[int]:
        """One token for each row of `logits` `[rows, vocab]`; blocks until the tokens are on the host."""
        tokens = self.collect(self.launch(logits, request_ids, token_indices))
        if NO_TOKEN in tokens:
            raise AllLogitsNaN("model logits are all NaN")
        return tokens

    __call__ = select
