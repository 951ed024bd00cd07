"""Random weights: a model folder (config.json, model.safetensors) from a configuration and a seed.

Each tensor has a generator of its own, keyed by the seed and the tensor's name, so a
tensor's values do not depend on which other tensors exist or on their order.
Matrices, embeddings and biases are N(0, 0.02); norm weights are `1 + N(0, jitter)`
with the jitter chosen by the caller (0 leaves them at one).
"""
from __future__ import annotations

import hashlib
import json
import os
from typing import Dict, Iterator, Tuple

import torch

from ..config.registry import architecture_for
from .safetensors_io import write_safetensors
from .tensor_spec import TensorSpec

_STORAGE = {"bfloat16": torch.bfloat16, "float32": torch.float32}


def _generator(seed: int, name: str, device) -> torch.Generator:
    digest = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    generator = torch.Generator(device=device)
    generator.manual_seed(int.from_bytes(digest[:8], "little") & 0x7FFFFFFFFFFFFFFF)
    return generator


def random_tensor(name: str, spec: TensorSpec, seed: int, norm_jitter: float, device="cpu") -> torch.Tensor:
    """One tensor in float32 (int32 for tables)."""
    generator = _generator(seed, name, device)
    if spec.role == "table":
        return torch.zeros(spec.shape, dtype=torch.int32, device=device)
    values = torch.randn(spec.shape, generator=generator, dtype=torch.float32, device=device)
    if spec.init == "ones":
        jitter = spec.jitter if spec.jitter else norm_jitter
        return 1.0 + values * jitter
    return values * spec.std


def random_tensors(specs: Dict[str, TensorSpec], seed: int, norm_jitter: float, device="cpu") -> Iterator[Tuple[str, torch.Tensor, TensorSpec]]:
    for name, spec in specs.items():
        yield name, random_tensor(name, spec, seed, norm_jitter, device), spec


def write_random_model(folder: str, config_json: dict, seed: int, norm_jitter: float = 0.0,
                       storage: str = "bfloat16", model_specs: Dict[str, TensorSpec] = None) -> None:
    """Writes `config.json` and `model.safetensors` for the architecture that `config_json` names.

    `storage` is the dtype of the stored matrices and vectors; `torch_dtype` of the
    written config.json is set to it, which is what later allows a bfloat16 run.
    """
    from ..parts.model import DecoderModel  # late: parts import weights

    os.makedirs(folder, exist_ok=True)
    config_json = dict(config_json)
    config_json.pop("dtype", None)
    config_json["torch_dtype"] = storage
    if model_specs is None:
        entry = architecture_for(config_json)
        spec = entry.build_spec(entry.parse_config(config_json))
        model_specs = DecoderModel.tensor_specs_of(spec)
    dtype = _STORAGE[storage]

    def stored():
        for name, tensor, spec in random_tensors(model_specs, seed, norm_jitter):
            yield name, tensor if spec.role == "table" else tensor.to(dtype)

    write_safetensors(os.path.join(folder, "model.safetensors"), stored())
    with open(os.path.join(folder, "config.json"), "w") as handle:
        json.dump(config_json, handle, indent=1)
