"""Step function, generation loop and the engine that owns model and cache."""
from .context import SequenceStep, StepContext, build_context
from .engine import Engine, parse_dtype
from .generate import (EmptyBatch, EmptyPrompt, GenerateError, Generation, PromptTooLong,
                       generate, is_stopped, plan_batch)
from .model import Model, expected_tensors

__all__ = ["SequenceStep", "StepContext", "build_context", "Engine", "parse_dtype", "EmptyBatch",
           "EmptyPrompt", "GenerateError", "Generation", "PromptTooLong", "generate", "is_stopped",
           "plan_batch", "Model", "expected_tensors"]
