from .safetensors_io import SafetensorsFile, SafetensorsError, write_safetensors, open_model_files
from .loader import WeightSpec, WeightsError, load_weights, MATRIX, VECTOR, TABLE, IGNORED

__all__ = ["SafetensorsFile", "SafetensorsError", "write_safetensors", "open_model_files",
           "WeightSpec", "WeightsError", "load_weights", "MATRIX", "VECTOR", "TABLE", "IGNORED"]
