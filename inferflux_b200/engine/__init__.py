from .batch import StepEntry, StepContext
from .model import Model
from .runner import StepRunner, torch_dtype

__all__ = ["StepEntry", "StepContext", "Model", "StepRunner", "torch_dtype"]
