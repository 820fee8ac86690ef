"""mormot2-ai_b200: a small B200-native model library with generation of its own for the
Qwen3 dense decoder: everything between a request's token ids and its next token, on one GPU.

    from mormot2_ai_b200 import Engine, Entry, Qwen3Config, write_random_model
"""
from . import parts  # registers the built-in parts
from .config import (ModelSpec, PartSpec, Qwen3Config, Run, LayerSpec, architectures,
                     config_of_folder, register_architecture)
from .errors import CacheError, ConfigError, InferError, KernelError, WeightsError
from .weights import SafeTensorsFolder, write_random_model, write_safetensors
from .engine import DecoderModel, Engine, Entry, Runtime
from .sampling import Sampling, sampling_from_config
from .client import LlmClient

__all__ = ["ModelSpec", "PartSpec", "Qwen3Config", "Run", "LayerSpec", "architectures",
           "config_of_folder", "register_architecture", "CacheError", "ConfigError",
           "InferError", "KernelError", "WeightsError", "SafeTensorsFolder",
           "write_random_model", "write_safetensors", "DecoderModel", "Engine", "Entry",
           "Runtime", "Sampling", "sampling_from_config", "LlmClient"]
