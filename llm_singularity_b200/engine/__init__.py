"""Engine: the step function, the scheduler above it and the entry point."""
from .batch import StepContext, StepEntry
from .runner import ModelRunner, OutOfPages

__all__ = ["StepContext", "StepEntry", "ModelRunner", "OutOfPages"]
