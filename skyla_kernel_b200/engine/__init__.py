"""Model assembly, the step function and the generation loop."""
from .batch import StepContext, StepItem, Workspace
from .engine import Engine, EngineError
from .generate import Finished, Request, generate, plan_batches
from .model import DecoderModel, declared_tensors

__all__ = ["StepContext", "StepItem", "Workspace", "Engine", "EngineError", "Finished", "Request",
           "generate", "plan_batches", "DecoderModel", "declared_tensors"]
