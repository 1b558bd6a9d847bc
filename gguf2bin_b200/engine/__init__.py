"""The engine: model construction, the step function, and generation above it."""
from .model import Model, expected_tensors, parse_dtype
from .step import Engine, StepEntry, StepError
from .generate import Generation, GenerationError, decide, generate, plan_batch
from .backend import EngineBackend
from .decode import DecodeSession
from .workspace import Workspace

__all__ = ["Model", "expected_tensors", "parse_dtype", "Engine", "StepEntry", "StepError",
           "Workspace", "Generation", "GenerationError", "decide", "generate", "plan_batch", "EngineBackend", "DecodeSession"]
