from .batch import StepBatch, StepEntry
from .engine import Engine, parse_dtype
from .model import Model, tensor_needs_of_spec

__all__ = ["StepBatch", "StepEntry", "Engine", "parse_dtype", "Model", "tensor_needs_of_spec"]
