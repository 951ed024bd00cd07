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

from ..csrc import kernels


@dataclass(frozen=True)
class SamplingParams:
    temperature: float = 0.0
    seed: int = 0

    def __post_init__(self):
        if not self.temperature >= 0.0:
            raise ValueError("temperature must be zero (greedy) or positive")


class AllLogitsNaN(RuntimeError):
    pass


class Sampler:
    def __init__(self, params: SamplingParams = SamplingParams()):
        self.params = params

    def select(self, logits: torch.Tensor, request_ids: Sequence[int], token_indices: Sequence[int]) -> List[int]:
        """One token for each row of `logits` `[rows, vocab]`; blocks until the tokens are on the host."""
        rows = logits.shape[0]
        result = torch.empty((2, rows), dtype=torch.int32, device=logits.device)
        if self.params.temperature == 0.0:
            kernels.argmax(logits, result[0], result[1])
        else:
            keys = torch.tensor([list(request_ids), list(token_indices)], dtype=torch.int32).to(logits.device)
            kernels.sample_gumbel(logits, result[0], result[1], 1.0 / self.params.temperature, self.params.seed, keys[0], keys[1])
        tokens, valid = result.cpu().tolist()
        if not all(valid):
            raise AllLogitsNaN("model logits are all NaN")
        return tokens
