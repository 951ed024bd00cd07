"""The part of config.json that every architecture shares: who it is and how it is stored.

crates/models/src/metadata.rs:23-75: `architectures[0]` and `model_type` are required
and form the dispatch key; the storage dtype is spelled `torch_dtype` or `dtype`, and
two spellings that disagree are rejected (:78-89).  crates/models/src/dtype.rs:54-62:
bfloat16 may run only if the folder declares it, 32-bit always.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass
from typing import Optional, Tuple

from .errors import InvalidConfig, InvalidModelDir, MissingFile, UnsupportedDType

RUN_DTYPES = ("float32", "bfloat16")
_DTYPE_ALIASES = {
    "f32": "float32", "fp32": "float32", "float32": "float32", "float": "float32",
    "bf16": "bfloat16", "bfloat16": "bfloat16",
}


def canonical_dtype(name: str) -> str:
    try:
        return _DTYPE_ALIASES[name.lower()]
    except KeyError:
        raise UnsupportedDType(f"unsupported dtype {name!r}; choose one of f32, float32, bf16, bfloat16") from None


@dataclass(frozen=True)
class ModelMetadata:
    architecture: str
    model_type: str
    declared_dtype: Optional[str]

    @property
    def supported_dtypes(self) -> Tuple[str, ...]:
        if self.declared_dtype in ("bfloat16", "bf16"):
            return ("float32", "bfloat16")
        return ("float32",)


def read_config_json(folder: str) -> dict:
    if not os.path.isdir(folder):
        raise InvalidModelDir(f"model folder {folder!r} is not a directory")
    path = os.path.join(folder, "config.json")
    if not os.path.isfile(path):
        raise MissingFile(f"{path} is missing")
    try:
        with open(path) as handle:
            raw = json.load(handle)
    except ValueError as error:
        raise InvalidConfig(f"{path}: {error}") from error
    if not isinstance(raw, dict):
        raise InvalidConfig(f"{path}: the top level must be an object")
    return raw


def metadata_from_json(raw: dict) -> ModelMetadata:
    architectures = raw.get("architectures")
    if not isinstance(architectures, list) or not architectures or not isinstance(architectures[0], str):
        raise InvalidConfig("config.json must name the model class in architectures[0]")
    model_type = raw.get("model_type")
    if not isinstance(model_type, str):
        raise InvalidConfig("config.json must include model_type")
    torch_dtype, dtype = raw.get("torch_dtype"), raw.get("dtype")
    for value in (torch_dtype, dtype):
        if value is not None and not isinstance(value, str):
            raise InvalidConfig("config.json: torch_dtype/dtype must be a string")
    if torch_dtype is not None and dtype is not None and torch_dtype != dtype:
        raise InvalidConfig(f"config.json declares torch_dtype={torch_dtype!r} but dtype={dtype!r}")
    return ModelMetadata(architectures[0], model_type, torch_dtype if torch_dtype is not None else dtype)


def validate_run_dtype(metadata: ModelMetadata, requested: str) -> str:
    requested = canonical_dtype(requested)
    if requested not in metadata.supported_dtypes:
        raise UnsupportedDType(
            f"{metadata.architecture} folder declares dtype {metadata.declared_dtype!r}; "
            f"{requested} needs a folder that declares bfloat16 (float32 always runs)"
        )
    return requested
