"""Generation settings of a model folder: stop tokens and the default output limit.

crates/models/src/generation_config.rs:31-63: `generation_config.json` wins; without
it the same two fields are taken from `config.json`; `eos_token_id` is one integer or
a list and must name at least one token; `max_new_tokens` defaults to 16 and must be
positive.  This library works on token ids and lets the caller pass the stop set, so a
folder without stop tokens is allowed here and yields an empty set.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass
from typing import Tuple

from .errors import InvalidConfig

DEFAULT_MAX_NEW_TOKENS = 16


@dataclass(frozen=True)
class GenerationConfig:
    eos_token_ids: Tuple[int, ...] = ()
    max_new_tokens: int = DEFAULT_MAX_NEW_TOKENS

    def is_eos_token(self, token: int) -> bool:
        return token in self.eos_token_ids


def _token_list(value, source: str) -> Tuple[int, ...]:
    items = value if isinstance(value, list) else [value]
    for item in items:
        if isinstance(item, bool) or not isinstance(item, int) or item < 0 or item > 0xFFFFFFFF:
            raise InvalidConfig(f"{source}: eos_token_id must be a non-negative 32-bit integer or a list of them")
    return tuple(items)


def load_generation_config(folder: str) -> GenerationConfig:
    path = os.path.join(folder, "generation_config.json")
    source = "generation_config.json"
    if not os.path.exists(path):
        path, source = os.path.join(folder, "config.json"), "config.json"
    try:
        with open(path) as handle:
            raw = json.load(handle)
    except (OSError, ValueError) as error:
        raise InvalidConfig(f"{source}: {error}") from error
    eos = raw.get("eos_token_id")
    eos_ids = _token_list(eos, source) if eos is not None else ()
    limit = raw.get("max_new_tokens")
    if limit is None:
        limit = DEFAULT_MAX_NEW_TOKENS
    if isinstance(limit, bool) or not isinstance(limit, int) or limit <= 0:
        raise InvalidConfig(f"{source}: max_new_tokens must be greater than zero")
    return GenerationConfig(eos_ids, limit)
