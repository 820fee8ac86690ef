"""How a layer's parts are arranged around the residual stream.

``prenorm_residual``: x += mixer(norm_mixer(x)); x += feed_forward(norm_ff(x)), the residual
x in float32 throughout (``decoder.pas:2625-2702``, ``:2880-2899`` of the reference).
"""
from __future__ import annotations

from .base import BLOCKS, Part


class PreNormResidualBlock(Part):
    capturable = True

    def __init__(self, spec, prefix: str = "", mixer=None, feed_forward=None, norms=None):
        super().__init__(spec, prefix)
        self.mixer, self.feed_forward, self.norms = mixer, feed_forward, norms

    def forward(self, x, step, line, state, writes_cache: bool) -> None:
        h = self.norms["mixer"].forward(x)
        self.mixer.forward(h, x, step, line, state, writes_cache)
        h = self.norms["feed_forward"].forward(x)
        self.feed_forward.forward(h, x, step)


BLOCKS.register("prenorm_residual", PreNormResidualBlock)
