"""The engine: step function, scheduler, generation."""
from .engine import Engine, EngineOptions, StepEntry, StepError

__all__ = ["Engine", "EngineOptions", "StepEntry", "StepError"]
