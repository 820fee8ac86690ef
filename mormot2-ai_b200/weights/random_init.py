"""Random weights from a configuration and a seed: a model folder (config.json,
model.safetensors) for tests and traces, or tensors made on the device for benchmarks of
large shapes.

Matrices and tables are N(0, std), norm weights 1 + N(0, norm_std), drawn in float32 from one
seeded generator in the order of the tensor names and then rounded to the stored type (the
reference's fixture tool draws 0.08·randn and 1 + 0.25·randn and rounds to BF16:
``tools/infer-ref/make_reference_qwen3.py:837-844`` of the reference project).
"""
from __future__ import annotations

import json
import os
from typing import Dict, Iterable

import torch

from ..parts.base import TensorNeed
from .safetensors_file import write_safetensors


def random_tensors(needs: Iterable[TensorNeed], seed: int, std: float = 0.02,
                   norm_std: float = 0.1, dtype: torch.dtype = torch.bfloat16,
                   device: str = "cpu") -> Dict[str, torch.Tensor]:
    gen = torch.Generator(device=device)
    gen.manual_seed(seed)
    out: Dict[str, torch.Tensor] = {}
    for n in sorted((n for n in needs if not n.optional), key=lambda n: n.name):
        if device == "cpu":
            t = torch.randn(n.shape, generator=gen, dtype=torch.float32)
        else:
            # drawn in the stored type on the device: a large model never exists in float32
            t = torch.empty(n.shape, dtype=dtype, device=device).normal_(0.0, 1.0, generator=gen)
        if n.role == "vector":
            t = t.mul_(norm_std).add_(1.0)
        else:
            t = t.mul_(std)
        out[n.name] = t.to(dtype)
    return out


def write_random_model(folder: str, config, seed: int, std: float = 0.02,
                       norm_std: float = 0.1, dtype: torch.dtype = torch.bfloat16) -> str:
    """Writes ``config.json`` and ``model.safetensors`` of a randomly initialised model of the
    configuration's architecture into ``folder`` and returns it."""
    from ..engine.model import DecoderModel
    os.makedirs(folder, exist_ok=True)
    needs = DecoderModel(config.to_model_spec()).tensors()
    tensors = random_tensors(needs, seed, std, norm_std, dtype)
    doc = config.to_dict()
    doc["torch_dtype"] = str(dtype).replace("torch.", "")
    with open(os.path.join(folder, "config.json"), "w", encoding="utf-8") as f:
        json.dump(doc, f, indent=1)
    write_safetensors(os.path.join(folder, "model.safetensors"), tensors)
    return folder
