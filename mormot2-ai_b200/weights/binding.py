"""Binding the tensors of a model folder to what the model's parts need, by name.

Every problem of a folder is found before anything is loaded and reported in ONE error:
missing tensors, unexpected tensors, wrong shapes, unsupported types. The reference checks
the same things one at a time (``decoder.pas:1919-1958`` shape and type,
``model.qwen3.pas:615-617`` "N tensors in the file, M understood").

Types: bfloat16 stays bfloat16 (widened exactly to float32 on the 32-bit path), a tensor
stored in float32 stays float32, integer tables become int32; float16 is refused as the
reference refuses it (``decoder.pas:1950-1957``).
"""
from __future__ import annotations

from typing import Dict, Iterable

import torch

from ..errors import WeightsError
from ..parts.base import TensorNeed

_INTEGERS = (torch.int64, torch.int32, torch.int16, torch.int8, torch.uint8)


def check_names(needs: Iterable[TensorNeed], source) -> None:
    """Raises one ``WeightsError`` that lists everything wrong with the folder."""
    needs = list(needs)
    by_name = {n.name: n for n in needs}
    have = set(source.names())
    missing = sorted(n.name for n in needs if not n.optional and n.name not in have)
    unexpected = sorted(have - set(by_name))
    shapes, types = [], []
    for n in needs:
        if n.name in have:
            if tuple(source.shape(n.name)) != tuple(n.shape):
                shapes.append(f"{n.name} is shaped {list(source.shape(n.name))}, "
                              f"expected {list(n.shape)}")
            dt = source.dtype(n.name)
            if dt not in (torch.float32, torch.bfloat16) + _INTEGERS:
                types.append(f"{n.name} is {str(dt).replace('torch.', '')}, not supported here")
    if missing or unexpected or shapes or types:
        lines = [f"the tensors of {getattr(source, 'folder', 'the model')} do not match the model:"]
        if missing:
            lines.append(f"  missing ({len(missing)}): " + ", ".join(missing))
        if unexpected:
            lines.append(f"  unexpected ({len(unexpected)}): " + ", ".join(unexpected))
        if shapes:
            lines.append(f"  wrong shape ({len(shapes)}): " + "; ".join(shapes))
        if types:
            lines.append(f"  wrong type ({len(types)}): " + "; ".join(types))
        raise WeightsError("\n".join(lines))


def convert(t: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    """The tensor as the engine keeps it for activations of ``dtype``."""
    if t.dtype in _INTEGERS:
        return t.to(torch.int32)
    if dtype == torch.float32:
        return t.to(torch.float32)  # exact for bfloat16
    return t  # bfloat16 stays, float32 stays


def bind_tensors(needs: Iterable[TensorNeed], source, dtype: torch.dtype,
                 device: torch.device) -> Dict[str, torch.Tensor]:
    """Checks the folder against the needs, then loads every bound tensor onto the device."""
    needs = list(needs)
    check_names(needs, source)
    out: Dict[str, torch.Tensor] = {}
    for n in needs:
        if n.name not in source:
            continue
        t = source.tensor(n.name)
        if n.must_equal is not None:
            other = source.tensor(n.must_equal)
            same = (t.dtype == other.dtype and t.shape == other.shape
                    and torch.equal(t.view(torch.uint8) if t.dtype != torch.bfloat16
                                    else t.view(torch.int16),
                                    other.view(torch.uint8) if other.dtype != torch.bfloat16
                                    else other.view(torch.int16)))
            if not same:
                raise WeightsError(f"{n.name} is stored and differs from {n.must_equal}, "
                                   "which it is tied to")
            continue
        out[n.name] = convert(t, dtype).to(device)
    return out
