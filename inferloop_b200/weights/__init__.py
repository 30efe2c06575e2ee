from .decl import WeightDecl
from .loader import WeightError, load_weights, resolve_prefix, target_dtype
from .random_init import random_tensor, random_weights, tensor_seed, write_random_model
from .safetensors_io import SafetensorsError, SafetensorsFile, TensorSource, write_safetensors

__all__ = [
    "WeightDecl", "WeightError", "load_weights", "resolve_prefix", "target_dtype",
    "random_tensor", "random_weights", "tensor_seed", "write_random_model",
    "SafetensorsError", "SafetensorsFile", "TensorSource", "write_safetensors",
]
