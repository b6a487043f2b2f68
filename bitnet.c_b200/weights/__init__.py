"""Weights: the safetensors container, loading by tensor name, and seeded random models."""
from .safetensors_io import SafetensorsError, SafetensorsFile, write_safetensors
from .loader import WeightsError, load_weights
from .random_init import random_parameters, random_tensor, standard_normal, standard_normal_on, write_random_model

__all__ = ["SafetensorsError", "SafetensorsFile", "write_safetensors", "WeightsError", "load_weights",
           "random_parameters", "random_tensor", "standard_normal", "standard_normal_on", "write_random_model"]
