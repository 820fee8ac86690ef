"""Choosing the next token: settings (``Sampling``) and the device sampler."""
from .settings import Sampling, sampling_from_config
from .device import DeviceSampler

__all__ = ["Sampling", "sampling_from_config", "DeviceSampler"]
