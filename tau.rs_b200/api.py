"""The Python entry point: a model folder to an engine, prompts of token ids to generated token ids.

Loading follows crates/models/src/loader.rs:135-261 (read config.json, dispatch on the
architecture, check the dtype against what the folder declares, read the generation
settings and every safetensors file, build the model; the context window is
`max_position_embeddings`, :199) and crates/server/src/device.rs:48-58, dtype.rs:31-45
(the device must be a CUDA GPU; `auto` dtype is bfloat16 there if the folder declares it).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Sequence

import torch

from . import models  # noqa: F401  (registers the architectures)
from .config.errors import UnsupportedDType
from .config.generation import GenerationConfig, load_generation_config
from .config.metadata import canonical_dtype, metadata_from_json, read_config_json, validate_run_dtype
from .config.registry import architecture_for
from .engine.generate import GenerationMetrics, GenerationResult, generate_tokens
from .engine.step import Engine
from .parts.model import DecoderModel
from .sampling.sampler import Sampler, SamplingParams
from .weights.loader import device_dtype, load_weights
from .weights.random_init import random_tensors

_TORCH_DTYPE = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def resolve_device(device: str = "gpu") -> torch.device:
    """`gpu` (or `auto`, `cuda`, `cuda:0`) is CUDA GPU 0; there is no CPU path."""
    if device in ("cpu",):
        raise UnsupportedDType("this library runs on a CUDA GPU only; --device cpu is not available")
    if not torch.cuda.is_available():
        raise RuntimeError("no CUDA GPU is available")
    return torch.device("cuda:0" if device in ("gpu", "auto", "cuda") else device)


def resolve_dtype(requested: str, declared: Optional[str]) -> str:
    if requested == "auto":
        return "bfloat16" if declared in ("bfloat16", "bf16") else "float32"
    return canonical_dtype(requested)


def load_model(folder: str, dtype: str = "auto", device="gpu", enforce_declared_dtype: bool = True) -> DecoderModel:
    """Builds the model that the folder's config.json names and reads its weights.

    With `enforce_declared_dtype` a bfloat16 run needs a folder that declares bfloat16, as
    the reference demands; without it any folder runs in either dtype.
    """
    raw = read_config_json(folder)
    metadata = metadata_from_json(raw)
    entry = architecture_for(raw)
    run_dtype = resolve_dtype(dtype, metadata.declared_dtype)
    if enforce_declared_dtype:
        run_dtype = validate_run_dtype(metadata, run_dtype)
    spec = entry.build_spec(entry.parse_config(raw))
    target = device if isinstance(device, torch.device) else resolve_device(device)
    model = DecoderModel(spec, _TORCH_DTYPE[run_dtype], target)
    load_weights(model, folder, _TORCH_DTYPE[run_dtype], target)
    model.generation_config = load_generation_config(folder)
    return model


def random_model(config_json: dict, seed: int = 0, dtype: str = "bfloat16", device="gpu", norm_jitter: float = 0.0) -> DecoderModel:
    """A model of the architecture that `config_json` names with random weights drawn on the device (no files).

    The values are those that `write_random_model` writes for the same seed, tensor by tensor: a bfloat16 model here
    equals a folder written with `storage="bfloat16"`, a float32 model one written with `storage="float32"`."""
    entry = architecture_for(config_json)
    spec = entry.build_spec(entry.parse_config(config_json))
    target = device if isinstance(device, torch.device) else resolve_device(device)
    run_dtype = _TORCH_DTYPE[canonical_dtype(dtype)]
    model = DecoderModel(spec, run_dtype, target)
    # Every tensor is drawn in the run's dtype, as a folder of that storage holds it; vectors are then widened to 32-bit.
    for name, tensor, tensor_spec in random_tensors(model.tensor_specs(), seed, norm_jitter, device=target, dtype_of=lambda _: run_dtype):
        model.assign(name, tensor.to(device_dtype(tensor_spec, run_dtype)))
    model.finalize_weights()
    model.generation_config = GenerationConfig()
    return model


def load_engine(folder: str, dtype: str = "auto", device="gpu", max_tokens: int = 8192,
                max_sequence_tokens: Optional[int] = None, enforce_declared_dtype: bool = True) -> Engine:
    """`max_tokens`: the most tokens that live sequences hold together (each rounded up to 64); it sizes the cache."""
    return Engine(load_model(folder, dtype, device, enforce_declared_dtype), max_tokens, max_sequence_tokens)


@dataclass
class GenerateOutput:
    results: List[GenerationResult]
    metrics: GenerationMetrics

    def __iter__(self):
        return iter(self.results)

    def __getitem__(self, index):
        return self.results[index]

    def __len__(self):
        return len(self.results)


def generate(model, prompts: Sequence[Sequence[int]], max_new_tokens=None, temperature: float = 0.0, seed: int = 0,
             stop_tokens: Optional[Sequence[int]] = None, dtype: str = "auto", device="gpu", max_tokens: Optional[int] = None,
             max_batch: int = 64, prefill_chunk_tokens: Optional[int] = 8192, metrics: Optional[GenerationMetrics] = None) -> GenerateOutput:
    """Generates token ids for prompts of token ids.

    `model` is a model folder, a `DecoderModel` or an `Engine`.  `max_new_tokens` defaults to
    the folder's generation settings (16 if it has none) and `stop_tokens` to its
    `eos_token_id`.  `temperature == 0` is greedy.  Results keep the prompts' order.  `metrics` may bring a
    `GenerationMetrics` of the caller's (with a `sink` and a `log_interval_s`, say, to watch the decode rate while it runs).
    """
    if isinstance(model, Engine):
        engine = model
    else:
        loaded = load_model(model, dtype, device) if isinstance(model, str) else model
        limit = max_new_tokens if max_new_tokens is not None else loaded.generation_config.max_new_tokens
        limits = list(limit) if isinstance(limit, (list, tuple)) else [limit] * len(prompts)
        if max_tokens is None:
            needs = sorted((-(-(len(p) + l) // 64) * 64 for p, l in zip(prompts, limits)), reverse=True)
            max_tokens = max(sum(needs[:max_batch]), 64)
        engine = Engine(loaded, max_tokens)
    settings = getattr(engine.model, "generation_config", GenerationConfig())
    if max_new_tokens is None:
        max_new_tokens = settings.max_new_tokens
    if stop_tokens is None:
        stop_tokens = settings.eos_token_ids
    sampler = Sampler(SamplingParams(temperature=temperature, seed=seed))
    metrics = metrics if metrics is not None else GenerationMetrics()
    results = generate_tokens(engine, prompts, max_new_tokens, sampler, stop_tokens, max_batch,
                              prefill_chunk_tokens, metrics)
    return GenerateOutput(results, metrics)
