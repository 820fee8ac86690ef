"""Guard bands around the device buffers that kernels write: a stand-in for a memory checker
where none can be run. A buffer made through ``Guards.alloc`` lies between two bands of a
fixed pattern; ``Guards.damaged()`` names the buffers whose bands no longer hold it, that is
the buffers that some kernel wrote before or beyond. The bands cost 2 x 4 KiB a buffer and
nothing at run time; the engine makes them when it is built with ``guard=True``.
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

import torch

BAND_BYTES = 4096
PATTERN = 0x5A


class Guards:
    def __init__(self):
        self.bands: List[Tuple[str, torch.Tensor, torch.Tensor]] = []

    def alloc(self, name: str, shape: Sequence[int], dtype: torch.dtype, device,
              fill: Optional[float] = 0.0) -> torch.Tensor:
        """A tensor of ``shape`` between two bands (``fill`` None: left as it is)."""
        n = 1
        for d in shape:
            n *= int(d)
        size = torch.empty((), dtype=dtype).element_size()
        raw = torch.empty(2 * BAND_BYTES + n * size, dtype=torch.uint8, device=device)
        front, back = raw[:BAND_BYTES], raw[BAND_BYTES + n * size:]
        front.fill_(PATTERN)
        back.fill_(PATTERN)
        body = raw[BAND_BYTES:BAND_BYTES + n * size].view(dtype).view(*shape)
        if fill is not None:
            body.fill_(fill)
        self.bands.append((name, front, back))
        return body

    def damaged(self) -> List[str]:
        """The buffers with a changed band, as "name (before)" / "name (behind)"."""
        out = []
        for name, front, back in self.bands:
            if int((front != PATTERN).sum()):
                out.append(f"{name} (before)")
            if int((back != PATTERN).sum()):
                out.append(f"{name} (behind)")
        return out


def alloc(guards: Optional[Guards], name: str, shape: Sequence[int], dtype: torch.dtype, device,
          fill: Optional[float] = 0.0) -> torch.Tensor:
    """Through the guards if there are any, else a plain tensor."""
    if guards is not None:
        return guards.alloc(name, shape, dtype, device, fill)
    if fill is None:
        return torch.empty(tuple(shape), dtype=dtype, device=device)
    return torch.full(tuple(shape), fill, dtype=dtype, device=device)
