"""Position encodings. A mixer asks its encoding for the inverse frequencies and for how many
values of a head rotate; the angle of a position is formed in the kernel as the float32
product inv_freq[i] · pos.

``rope_half`` is the rotary encoding in the rotate-half pairing (i, i + rot_dim/2) with
inv_freq[i] = 1 / f32(theta ^ f32(2i / rot_dim)), each step rounded to float32 as the
reference does (``decoder.pas:1733-1736``; angles ``:2539-2561``). ``none`` rotates nothing.
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import numpy as np
import torch

from ..errors import ConfigError
from .base import POSITIONS, Part


def rope_inverse_frequencies(theta: float, rot_dim: int) -> np.ndarray:
    out = np.empty(rot_dim // 2, dtype=np.float32)
    for i in range(rot_dim // 2):
        exponent = np.float32((2 * i) / rot_dim)
        power = np.float32(math.exp(math.log(theta) * float(exponent)))
        out[i] = np.float32(1.0 / float(power))
    return out


class RopeHalf(Part):
    capturable = True

    def __init__(self, spec, prefix: str = ""):
        super().__init__(spec, prefix)
        self.theta = float(spec.params["theta"])
        self.rot_dim = int(spec.params["rot_dim"])
        if self.rot_dim <= 0 or self.rot_dim % 2:
            raise ConfigError(f"a rotary encoding over {self.rot_dim} values of a head")
        self.inv_freq: Optional[torch.Tensor] = None

    def bind(self, weights, rt) -> None:
        self.inv_freq = torch.from_numpy(
            rope_inverse_frequencies(self.theta, self.rot_dim)).to(rt.device)

    def frequencies(self) -> Tuple[Optional[torch.Tensor], int]:
        return self.inv_freq, self.rot_dim


class NoPosition(Part):
    capturable = True

    def frequencies(self) -> Tuple[Optional[torch.Tensor], int]:
        return None, 0


POSITIONS.register("rope_half", RopeHalf)
POSITIONS.register("none", NoPosition)
