"""The step function and the generation loop above it."""

from .engine import Engine, StepContext, StepEntry
from .generate import GenerationResult, GenerationStats, generate, plan_batches

__all__ = ["Engine", "StepContext", "StepEntry", "GenerationResult", "GenerationStats", "generate", "plan_batches"]
