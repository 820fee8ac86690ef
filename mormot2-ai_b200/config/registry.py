"""One registry from an architecture's name to its model family.

A family is a configuration class with ``from_dict(doc, source)``, ``to_dict()`` and
``to_model_spec()``. The name looked up is ``architectures[0]`` of config.json, else its
``model_type`` (the reference registers classes by ``model_type`` and the first registered
wins: ``decoder.pas:3434-3456``; it names the unknown value in its error, ``:3480-3482``).
"""
from __future__ import annotations

import json
import os
from typing import Any, Dict, List

from ..errors import ConfigError

_BY_ARCHITECTURE: Dict[str, Any] = {}
_BY_MODEL_TYPE: Dict[str, Any] = {}


def register_architecture(family: Any, architecture: str, model_type: str = "") -> None:
    """Adds a family; the first registration of a name wins."""
    _BY_ARCHITECTURE.setdefault(architecture, family)
    if model_type:
        _BY_MODEL_TYPE.setdefault(model_type, family)


def architectures() -> List[str]:
    return sorted(_BY_ARCHITECTURE)


def family_of(doc: Dict[str, Any], source: str = "config") -> Any:
    """The family that a config.json names."""
    if not isinstance(doc, dict):
        raise ConfigError(f"{source} is no JSON object")
    names = doc.get("architectures")
    if isinstance(names, list) and names:
        if names[0] in _BY_ARCHITECTURE:
            return _BY_ARCHITECTURE[names[0]]
        if doc.get("model_type") not in _BY_MODEL_TYPE:
            raise ConfigError(
                f"{source}: architecture \"{names[0]}\" is not known "
                f"(known: {', '.join(architectures())})")
    model_type = doc.get("model_type")
    if model_type in _BY_MODEL_TYPE:
        return _BY_MODEL_TYPE[model_type]
    raise ConfigError(
        f"{source}: model_type \"{model_type}\" is not known "
        f"(known: {', '.join(sorted(_BY_MODEL_TYPE))})")


def read_config_json(folder: str) -> Dict[str, Any]:
    path = os.path.join(folder, "config.json") if os.path.isdir(folder) else folder
    try:
        with open(path, "r", encoding="utf-8") as f:
            return json.load(f)
    except (OSError, ValueError) as e:
        raise ConfigError(f"cannot read {path}: {e}") from None


def config_of_folder(folder: str) -> Any:
    """The typed configuration of a model folder, of the class its config.json names."""
    path = os.path.join(folder, "config.json")
    doc = read_config_json(folder)
    return family_of(doc, path).from_dict(doc, path)
