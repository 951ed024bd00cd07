from .errors import (InvalidConfig, InvalidModelDir, MissingFile, ModelLoadError, UnsupportedDType, WeightError)
from .generation import DEFAULT_MAX_NEW_TOKENS, GenerationConfig, load_generation_config
from .metadata import (ModelMetadata, canonical_dtype, metadata_from_json, read_config_json, validate_run_dtype)
from .qwen3 import Qwen3Config
from .registry import (Architecture, architecture_for, register_architecture, registered_architectures,
                       spec_from_config_json, unregister_architecture)
from .specs import (AttentionSpec, BlockSpec, ModelSpec, NormSpec, PositionSpec, ScheduleEntry, SwiGLUSpec)
