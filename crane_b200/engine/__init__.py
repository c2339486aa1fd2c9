"""The step function, the scheduler and the engine loop above them."""
from .step import ModelRunner, StepContext, StepEntry

__all__ = ["ModelRunner", "StepContext", "StepEntry"]
