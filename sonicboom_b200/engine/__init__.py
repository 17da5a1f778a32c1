"""The step function, the engine that owns model and cache, and the generation loop."""
from .engine import Engine
from .step import StepEntry, StepError, StepPlan, step

__all__ = ["Engine", "StepEntry", "StepError", "StepPlan", "step"]
