"""The step function, the scheduler above it and the entry point."""
from .engine import Engine, StepEntry, StepError, StepStats, parse_dtype

__all__ = ["Engine", "StepEntry", "StepError", "StepStats", "parse_dtype"]
