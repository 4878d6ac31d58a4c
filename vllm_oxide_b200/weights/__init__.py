from .safetensors_io import SafetensorsFile, write_safetensors
from .loader import TensorSpec, WeightSet, load_safetensors_weights, weights_from_tensors, check_against_manifest
from .random_init import random_tensors, write_random_model

__all__ = ["SafetensorsFile", "write_safetensors", "TensorSpec", "WeightSet", "load_safetensors_weights",
           "weights_from_tensors", "check_against_manifest", "random_tensors", "write_random_model"]
