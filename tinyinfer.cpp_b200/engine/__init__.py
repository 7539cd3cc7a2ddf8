"""The step function and what stands on it."""
from .batch import StepBatch, StepEntry, build_step_batch
from .engine import Engine, parse_dtype

__all__ = ["Engine", "StepBatch", "StepEntry", "build_step_batch", "parse_dtype"]
