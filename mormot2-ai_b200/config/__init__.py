"""Typed configurations, the model as data (``ModelSpec``) and the architecture registry."""
from .spec import LayerSpec, ModelSpec, PartSpec, Run
from .qwen3 import Qwen3Config
from .registry import (architectures, config_of_folder, family_of, read_config_json,
                       register_architecture)

register_architecture(Qwen3Config, Qwen3Config.ARCHITECTURE, Qwen3Config.MODEL_TYPE)

__all__ = ["LayerSpec", "ModelSpec", "PartSpec", "Run", "Qwen3Config", "architectures",
           "config_of_folder", "family_of", "read_config_json", "register_architecture"]
