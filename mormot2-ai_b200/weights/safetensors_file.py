"""Reading and writing safetensors files: one file, or the files of a
``model.safetensors.index.json``.

The checks follow the reference's ``TSafeTensorsFile.Parse``
(``loader.safetensors.pas:355-494``): header length, JSON object with unique keys, known
dtype, shape product equal to the byte range, ranges inside the file, non-overlapping, without
gaps or trailing bytes; and ``CreateFromIndex`` (``:181-284``): the index and the files name
exactly the same tensors. Tensors are returned as views of the mapped file (no copy).
"""
from __future__ import annotations

import json
import os
import struct
from typing import Dict, List, Mapping, Tuple

import numpy as np
import torch

from ..errors import WeightsError

MAX_HEADER = 100 * 1000 * 1000  # loader.safetensors.pas: a header above 100 MB is refused

# safetensors dtype -> (numpy storage dtype, torch dtype)
_DTYPES = {
    "F64": (np.float64, torch.float64), "F32": (np.float32, torch.float32),
    "F16": (np.float16, torch.float16), "BF16": (np.uint16, torch.bfloat16),
    "I64": (np.int64, torch.int64), "I32": (np.int32, torch.int32),
    "I16": (np.int16, torch.int16), "I8": (np.int8, torch.int8),
    "U8": (np.uint8, torch.uint8), "BOOL": (np.bool_, torch.bool),
}
_NAMES = {v[1]: k for k, v in _DTYPES.items()}


def _unique_object(pairs):
    seen = {}
    for k, v in pairs:
        if k in seen:
            raise WeightsError(f"the key \"{k}\" occurs twice")
        seen[k] = v
    return seen


class SafeTensorsFile:
    """The tensors of one safetensors file, by name."""

    def __init__(self, path: str):
        self.path = path
        try:
            size = os.path.getsize(path)
            with open(path, "rb") as f:
                head = f.read(8)
                if len(head) != 8:
                    raise WeightsError(f"{path}: no header length")
                (n,) = struct.unpack("<Q", head)
                if n <= 0 or n > MAX_HEADER or 8 + n > size:
                    raise WeightsError(f"{path}: a header of {n} bytes in a file of {size}")
                raw = f.read(n)
        except OSError as e:
            raise WeightsError(f"cannot read {path}: {e}") from None
        try:
            header = json.loads(raw.decode("utf-8"), object_pairs_hook=_unique_object)
        except (ValueError, WeightsError) as e:
            raise WeightsError(f"{path}: the header is no valid JSON object: {e}") from None
        if not isinstance(header, dict):
            raise WeightsError(f"{path}: the header is no JSON object")
        self.metadata = header.pop("__metadata__", None)
        self._base = 8 + n
        data = size - self._base
        self._entries: Dict[str, Tuple[str, Tuple[int, ...], int, int]] = {}
        spans = []
        for name, e in header.items():
            if not isinstance(e, dict) or not {"dtype", "shape", "data_offsets"} <= set(e):
                raise WeightsError(f"{path}: {name} has no dtype, shape and data_offsets")
            dtype, shape, off = e["dtype"], e["shape"], e["data_offsets"]
            if dtype not in _DTYPES:
                raise WeightsError(f"{path}: {name} is {dtype}, not supported here")
            if (not isinstance(shape, list)
                    or any(isinstance(d, bool) or not isinstance(d, int) or d < 0 for d in shape)):
                raise WeightsError(f"{path}: {name} is shaped {shape}")
            if (not isinstance(off, list) or len(off) != 2
                    or any(isinstance(o, bool) or not isinstance(o, int) for o in off)):
                raise WeightsError(f"{path}: {name} has the data_offsets {off}")
            begin, end = off
            count = 1
            for d in shape:
                count *= d
            itemsize = np.dtype(_DTYPES[dtype][0]).itemsize
            if not (0 <= begin <= end <= data) or end - begin != count * itemsize:
                raise WeightsError(
                    f"{path}: {name} {dtype}{shape} needs {count * itemsize} bytes, "
                    f"its range is [{begin}, {end}) of {data}")
            if begin % itemsize:
                raise WeightsError(f"{path}: {name} starts at the odd offset {begin}")
            self._entries[name] = (dtype, tuple(shape), begin, end)
            spans.append((begin, end, name))
        spans.sort()
        at = 0
        for begin, end, name in spans:
            if begin != at:
                raise WeightsError(
                    f"{path}: {name} starts at {begin}, the tensor before it ends at {at}")
            at = end
        if at != data:
            raise WeightsError(f"{path}: {data - at} bytes after the last tensor")
        self._map = np.memmap(path, dtype=np.uint8, mode="r") if data > 0 else None

    def names(self) -> List[str]:
        return sorted(self._entries)

    def __contains__(self, name: str) -> bool:
        return name in self._entries

    def shape(self, name: str) -> Tuple[int, ...]:
        return self._entries[name][1]

    def dtype(self, name: str) -> torch.dtype:
        return _DTYPES[self._entries[name][0]][1]

    def tensor(self, name: str) -> torch.Tensor:
        """The tensor as stored (a read-only view of the mapped file)."""
        if name not in self._entries:
            raise WeightsError(f"{self.path}: no tensor {name}")
        dtype, shape, begin, end = self._entries[name]
        np_dtype, torch_dtype = _DTYPES[dtype]
        if end == begin:
            return torch.empty(shape, dtype=torch_dtype)
        raw = self._map[self._base + begin:self._base + end]
        arr = raw.view(np_dtype).reshape(shape)
        # torch has no read-only tensors: the view is never written by this library
        import warnings
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")
            t = torch.from_numpy(arr)
        return t.view(torch_dtype) if dtype == "BF16" else t


class SafeTensorsFolder:
    """The tensors of a model folder: ``model.safetensors``, else the files that
    ``model.safetensors.index.json`` names (``loader.safetensors.pas:133-143``)."""

    def __init__(self, folder: str):
        self.folder = folder
        single = os.path.join(folder, "model.safetensors")
        index = os.path.join(folder, "model.safetensors.index.json")
        self._where: Dict[str, SafeTensorsFile] = {}
        if os.path.isfile(single):
            f = SafeTensorsFile(single)
            for n in f.names():
                self._where[n] = f
            return
        if not os.path.isfile(index):
            raise WeightsError(f"{folder}: no model.safetensors and no model.safetensors.index.json")
        try:
            with open(index, "r", encoding="utf-8") as fh:
                doc = json.load(fh, object_pairs_hook=_unique_object)
            weight_map = doc["weight_map"]
            assert isinstance(weight_map, dict)
        except (OSError, ValueError, KeyError, AssertionError, WeightsError) as e:
            raise WeightsError(f"{index}: no valid weight_map: {e}") from None
        files: Dict[str, SafeTensorsFile] = {}
        for name, fname in weight_map.items():
            if not isinstance(fname, str) or os.path.basename(fname) != fname:
                raise WeightsError(f"{index}: {name} is in the file {fname!r}")
            if fname not in files:
                files[fname] = SafeTensorsFile(os.path.join(folder, fname))
            if name not in files[fname]:
                raise WeightsError(f"{index}: {name} is not in {fname}")
            self._where[name] = files[fname]
        for fname, f in files.items():
            for n in f.names():
                if weight_map.get(n) != fname:
                    raise WeightsError(f"{index}: {fname} holds {n}, the index does not say so")

    def names(self) -> List[str]:
        return sorted(self._where)

    def __contains__(self, name: str) -> bool:
        return name in self._where

    def shape(self, name: str) -> Tuple[int, ...]:
        return self._where[name].shape(name)

    def dtype(self, name: str) -> torch.dtype:
        return self._where[name].dtype(name)

    def tensor(self, name: str) -> torch.Tensor:
        if name not in self._where:
            raise WeightsError(f"{self.folder}: no tensor {name}")
        return self._where[name].tensor(name)


def write_safetensors(path: str, tensors: Mapping[str, torch.Tensor]) -> None:
    """Writes tensors (CPU, contiguous) as one safetensors file, in name order, without gaps."""
    header = {}
    at = 0
    order = sorted(tensors)
    for name in order:
        t = tensors[name]
        if t.dtype not in _NAMES:
            raise WeightsError(f"{name} is {t.dtype}, not supported here")
        size = t.numel() * t.element_size()
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape),
                        "data_offsets": [at, at + size]}
        at += size
    raw = json.dumps(header, separators=(",", ":")).encode("utf-8")
    raw += b" " * (-len(raw) % 8)  # the data starts on an 8-byte boundary
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(raw)))
        f.write(raw)
        for name in order:
            t = tensors[name].detach().cpu().contiguous()
            if t.dtype == torch.bfloat16:
                t = t.view(torch.int16)
            if t.numel():
                f.write(t.numpy().tobytes())
