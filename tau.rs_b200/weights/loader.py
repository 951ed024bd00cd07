"""Weights by tensor name, with one error for everything that does not fit.

crates/models/src/tensor_contract.rs:68-142 checks names, shapes and storage dtypes of
a required list against all headers before anything is allocated; that check is applied
here to every architecture, and a tensor that the model does not ask for is an error
too.  crates/models/src/qwen3.rs:67-75 converts each stored tensor to the run's dtype
on the way to the device; here matrices are converted so, and vectors are kept in
32-bit (see `TensorSpec`).
"""
from __future__ import annotations

import sys
from typing import Dict

import torch

from ..config.errors import WeightError
from .safetensors_io import SafetensorsFolder
from .tensor_spec import TensorSpec

_FLOAT_STORAGE = ("BF16", "F16", "F32", "F64")
_INT_STORAGE = ("I32", "I64", "U8")


def device_dtype(spec: TensorSpec, run_dtype: torch.dtype) -> torch.dtype:
    if spec.role == "matrix":
        return run_dtype
    if spec.role == "vector":
        return torch.float32
    if spec.role == "table":
        return torch.int32
    raise ValueError(f"unknown tensor role {spec.role!r}")


def check_contract(wanted: Dict[str, TensorSpec], ignored, found: SafetensorsFolder):
    """Returns the names to read (with fallbacks resolved) or raises `WeightError`."""
    missing, wrong_shape, wrong_dtype = [], [], []
    source_of: Dict[str, str] = {}
    used = set()
    for name, spec in wanted.items():
        source = name
        if name not in found.tensors:
            if spec.fallback is not None and spec.fallback in found.tensors:
                print(f"note: {name} is absent; using {spec.fallback} in its place", file=sys.stderr)
                source = spec.fallback
            else:
                missing.append(name)
                continue
        info = found.tensors[source]
        used.add(source)
        if tuple(info.shape) != tuple(spec.shape):
            wrong_shape.append((name, info.shape, spec.shape))
        allowed = _INT_STORAGE if spec.role == "table" else _FLOAT_STORAGE
        if info.dtype not in allowed:
            wrong_dtype.append((name, info.dtype))
        source_of[name] = source
    unexpected = [name for name in found.tensors if name not in used and name not in ignored]
    if missing or unexpected or wrong_shape or wrong_dtype:
        raise WeightError(missing, unexpected, wrong_shape, wrong_dtype)
    return source_of


def load_weights(model, folder: str, run_dtype: torch.dtype, device) -> None:
    """Reads every tensor that `model` asks for and hands it over by name."""
    found = SafetensorsFolder(folder)
    wanted = model.tensor_specs()
    source_of = check_contract(wanted, model.ignored_tensors(), found)
    for name, spec in wanted.items():
        stored = found.read(source_of[name])
        model.assign(name, stored.to(device=device, dtype=device_dtype(spec, run_dtype)).contiguous())
    found.close()
    model.finalize_weights()
