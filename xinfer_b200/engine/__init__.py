"""The engine: the step function (runner), the scheduler above it and the generation loop."""
from .runner import ModelRunner, StepError, StepInput

__all__ = ["ModelRunner", "StepError", "StepInput"]
