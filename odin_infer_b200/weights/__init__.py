"""Weights: safetensors by tensor name, one clear error, random-weights mode."""
from .loader import WeightError, check_folder, load_weights
from .random_init import model_param_specs, random_weights, write_random_model
from .safetensors_io import ModelFiles, SafetensorsError, SafetensorsFile, write_safetensors

__all__ = ["ModelFiles", "SafetensorsError", "SafetensorsFile", "WeightError", "check_folder", "load_weights",
           "model_param_specs", "random_weights", "write_random_model", "write_safetensors"]
