"""The description of a model as data: which parts make up each layer, with which sizes and
constants, and in which order the layers run.

A model family (``config/qwen3.py``) turns its config.json into a ``ModelSpec``; the engine
builds parts from it through the part registries (``parts/__init__.py``) and knows nothing of
the family. The reference keeps the same split: ``TDecoderConfig`` plus one
``TDecoderLayerSpec`` per layer (``decoder.pas:132-225``) selected by the family unit
(``model.qwen3.pas:231-313``).

Every spec is ``kind`` + ``params``: ``kind`` is a key of a part registry, ``params`` are the
sizes and constants of that part. No size stands in code.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, Optional, Tuple


@dataclass(frozen=True)
class PartSpec:
    """One part: a registry key and its parameters."""
    kind: str
    params: Dict[str, Any] = field(default_factory=dict)

    def get(self, name: str, default: Any = None) -> Any:
        return self.params.get(name, default)


@dataclass(frozen=True)
class LayerSpec:
    """One layer: the arrangement (``block``) and the parts that it arranges.

    ``prefix`` is the tensor-name prefix of the layer in the model folder
    (``model.layers.3.``); part tensor names are relative to it.
    """
    block: PartSpec
    mixer: PartSpec
    feed_forward: PartSpec
    norms: Dict[str, PartSpec]
    prefix: str


@dataclass(frozen=True)
class Run:
    """One entry of the order in which layers run.

    ``layer`` indexes ``ModelSpec.layers`` and may occur in several entries. ``cache_line`` is
    the line of the cache that the mixer of this run uses (``None``: the mixer keeps nothing).
    ``writes_cache`` is false for a run whose mixer reads a line that an earlier run wrote
    (keys and values shared between layers).
    """
    layer: int
    cache_line: Optional[int] = None
    writes_cache: bool = True


@dataclass(frozen=True)
class ModelSpec:
    """A whole decoder: embedding, layers, their order, final norm and head."""
    architecture: str
    vocab_size: int
    hidden_size: int
    max_positions: int
    embedding: PartSpec            # params: name
    positions: Dict[str, PartSpec]  # named position encodings that mixers refer to
    layers: Tuple[LayerSpec, ...]
    schedule: Tuple[Run, ...]
    final_norm: PartSpec           # params: name, eps, size
    head: PartSpec                 # params: name, tied

    def cache_lines(self) -> int:
        lines = [r.cache_line for r in self.schedule if r.cache_line is not None]
        return (max(lines) + 1) if lines else 0
