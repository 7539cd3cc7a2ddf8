"""The step function and what stands on it."""
from .batch import StepBatch, StepEntry, build_step_batch
from .engine import Engine, parse_dtype
from .generate import Generation, LLM, RunStats
from .scheduler import Request, Scheduled, Scheduler

__all__ = ["Engine", "Generation", "LLM", "Request", "RunStats", "Scheduled", "Scheduler",
           "StepBatch", "StepEntry", "build_step_batch", "parse_dtype"]
