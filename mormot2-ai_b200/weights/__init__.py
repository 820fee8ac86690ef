"""Weights: safetensors files, binding by name, random initialisation."""
from .binding import bind_tensors, check_names, convert
from .random_init import random_tensors, write_random_model
from .safetensors_file import SafeTensorsFile, SafeTensorsFolder, write_safetensors

__all__ = ["bind_tensors", "check_names", "convert", "random_tensors", "write_random_model",
           "SafeTensorsFile", "SafeTensorsFolder", "write_safetensors"]
