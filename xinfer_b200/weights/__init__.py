"""Weights: safetensors by tensor name, strict checking, and the random-weights mode."""
from .loader import UnexpectedWeightsWarning, WeightError, WeightSpec, WeightStore
from .random_init import RandomWeightStore, draw, write_random_model
from .safetensors_io import SafetensorsError, SafetensorsFile, find_weight_files, write_safetensors

__all__ = ["UnexpectedWeightsWarning", "WeightError", "WeightSpec", "WeightStore", "draw", "write_random_model", "RandomWeightStore",
           "SafetensorsError", "SafetensorsFile", "find_weight_files", "write_safetensors"]
