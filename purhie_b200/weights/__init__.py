"""Weights: safetensors by tensor name, one error for all misfits, seeded random models."""
from .loader import MATRIX, TABLE, VECTOR, TensorSpec, WeightError, check_folder, device_dtype, load_tensors
from .random_init import expected_tensors, random_tensor, random_tensors, tensor_seed, write_random_model
from .safetensors_io import SafetensorsError, SafetensorsFile, SafetensorsFolder, write_safetensors

__all__ = [
    "MATRIX", "TABLE", "VECTOR", "TensorSpec", "WeightError", "check_folder", "device_dtype", "load_tensors",
    "expected_tensors", "random_tensor", "random_tensors", "tensor_seed", "write_random_model",
    "SafetensorsError", "SafetensorsFile", "SafetensorsFolder", "write_safetensors",
]
