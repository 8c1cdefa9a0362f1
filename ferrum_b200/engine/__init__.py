from .batch import StepContext, StepEntry
from .runner import ModelRunner

__all__ = ["StepContext", "StepEntry", "ModelRunner"]
