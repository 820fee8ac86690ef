"""The engine: model from parts, step function, generation loop."""
from .engine import DTYPES, Engine, Entry
from .model import DecoderModel
from .runtime import Runtime

__all__ = ["DTYPES", "Engine", "Entry", "DecoderModel", "Runtime"]
