"""Weights: safetensors reading and writing, name binding, and the random-weights mode."""
from .binding import ParamSpec, Stacked, Tied
from .loader import load_parameters, open_model_weights
from .random_init import random_tensors, write_random_model
from .safetensors_io import SafetensorsFile, WeightsError, write_safetensors

__all__ = ["ParamSpec", "Stacked", "Tied", "load_parameters", "open_model_weights", "random_tensors",
           "write_random_model", "SafetensorsFile", "WeightsError", "write_safetensors"]
