"""Weights: the safetensors container, the checked loader and the random-weights mode."""
from .safetensors_io import Checkpoint, SafetensorsFile, SafetensorsError, write_safetensors
from .loader import ParamSpec, UnusedWeightsWarning, WeightError, check, convert, load_into, load_folder
from .random_init import random_tensor, random_tensors, write_random_model

__all__ = ["Checkpoint", "SafetensorsFile", "SafetensorsError", "write_safetensors", "ParamSpec", "UnusedWeightsWarning", "WeightError",
           "check", "convert", "load_into", "load_folder", "random_tensor", "random_tensors", "write_random_model"]
