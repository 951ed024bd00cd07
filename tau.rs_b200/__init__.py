"""A small generation library for dense Qwen3 on one B200: tokens in, next tokens out.

Import name `tau_rs_b200`.  Entry points: `generate`, `load_engine`, `load_model`,
`random_model`, `Engine`/`StepEntry` (the step function), `write_random_model`.
"""
from . import models  # noqa: F401
from .api import GenerateOutput, generate, load_engine, load_model, random_model
from .config import (GenerationConfig, InvalidConfig, ModelLoadError, Qwen3Config, UnsupportedDType, WeightError,
                     register_architecture)
from .engine import Engine, GenerationMetrics, GenerationResult, StepEntry, StepError, generate_tokens
from .cache import CacheDoesNotFit, CacheFull, SequenceCache
from .parts import DecoderModel
from .sampling import Sampler, SamplingParams
from .weights import write_random_model

__all__ = [
    "CacheDoesNotFit", "CacheFull", "DecoderModel", "Engine", "GenerateOutput", "GenerationConfig", "GenerationMetrics", "GenerationResult",
    "InvalidConfig", "ModelLoadError", "Qwen3Config", "Sampler", "SamplingParams", "SequenceCache", "StepEntry", "StepError",
    "UnsupportedDType", "WeightError", "generate", "generate_tokens", "load_engine", "load_model", "random_model",
    "register_architecture", "write_random_model",
]
