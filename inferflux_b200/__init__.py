"""inferflux_b200: a small, whole inference engine for one NVIDIA B200.

From a model folder (``config.json`` + ``model.safetensors``) to next-token
logits and generated tokens: typed configuration and architecture registry,
weights bound by name, layers assembled from parts, a paged key/value cache
with state slots, one step function over mixed batches, a scheduler, sampling,
hand-written sm_100a kernels, a true float32 path, and trace replay.
"""
__version__ = "0.1.0"

from .config import EngineConfig, Qwen2Config, load_config  # noqa: E402
from .sampling import SamplingParams  # noqa: E402
from .engine import Engine, GenerationResult, StepEntry  # noqa: E402

__all__ = ["Engine", "EngineConfig", "GenerationResult", "Qwen2Config", "SamplingParams", "StepEntry",
           "load_config"]
