from .batch import StepContext, StepEntry
from .generate import GenerationMetrics, GenerationResult, generate_tokens, plan_batches
from .step import Engine, StepError
