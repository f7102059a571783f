from .loader import TensorSpec, WeightError, WeightStore, open_model_weights
from .random_init import RandomWeightStore, write_random_model
from .safetensors_io import SafetensorsError, read_safetensors, write_safetensors

__all__ = ["TensorSpec", "WeightError", "WeightStore", "open_model_weights", "RandomWeightStore",
           "write_random_model", "SafetensorsError", "read_safetensors", "write_safetensors"]
