"""One registry from the architecture's name to its model.

crates/models/src/loader.rs:160-260 dispatches on `(architectures[0], model_type)` and
names both in the error for an unknown pair (:257-259).  Here an architecture is two
functions: one that turns config.json into a typed configuration and one that turns
that configuration into a `ModelSpec` (the list of blocks and the schedule); the
model itself is always built from the spec by `tau_rs_b200.parts.model.DecoderModel`.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Dict

from .errors import InvalidConfig
from .metadata import metadata_from_json
from .specs import ModelSpec


@dataclass(frozen=True)
class Architecture:
    name: str
    model_type: str
    parse_config: Callable[[dict], object]
    build_spec: Callable[[object], ModelSpec]


_ARCHITECTURES: Dict[str, Architecture] = {}


def register_architecture(name: str, model_type: str, parse_config, build_spec) -> Architecture:
    entry = Architecture(name, model_type, parse_config, build_spec)
    _ARCHITECTURES[name] = entry
    return entry


def unregister_architecture(name: str) -> None:
    _ARCHITECTURES.pop(name, None)


def registered_architectures():
    return sorted(_ARCHITECTURES)


def architecture_for(raw_config: dict) -> Architecture:
    metadata = metadata_from_json(raw_config)
    entry = _ARCHITECTURES.get(metadata.architecture)
    if entry is None or entry.model_type != metadata.model_type:
        known = ", ".join(f"{a.name}/{a.model_type}" for a in _ARCHITECTURES.values()) or "none"
        raise InvalidConfig(
            f"unsupported model {metadata.architecture}/{metadata.model_type}; registered: {known}"
        )
    return entry


def spec_from_config_json(raw_config: dict) -> ModelSpec:
    entry = architecture_for(raw_config)
    return entry.build_spec(entry.parse_config(raw_config))
