from .batch import StepEntry, StepContext
from .model import Model
from .runner import StepRunner, torch_dtype
from .scheduler import Scheduler, Request, Phase, StepPlan, CacheView
from .engine import Engine, GenerationResult

__all__ = ["StepEntry", "StepContext", "Model", "StepRunner", "torch_dtype", "Scheduler", "Request",
           "Phase", "StepPlan", "CacheView", "Engine", "GenerationResult"]
