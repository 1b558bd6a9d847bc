"""The engine: model construction, the step function, and generation above it."""
from .model import Model, expected_tensors, parse_dtype
from .step import Engine, StepEntry, StepError
from .workspace import Workspace

__all__ = ["Model", "expected_tensors", "parse_dtype", "Engine", "StepEntry", "StepError",
           "Workspace"]
