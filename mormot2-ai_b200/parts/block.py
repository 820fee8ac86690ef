"""How a layer's parts are arranged around the residual stream.

``prenorm_residual``: x += mixer(norm_mixer(x)); x += feed_forward(norm_ff(x)), the residual
x in float32 throughout (``decoder.pas:2625-2702``, ``:2880-2899`` of the reference).

A mixer or feed-forward may hand its output back as ``Pending`` split sums instead of adding
it into x; the norm that reads x next adds them (one kernel does the sum, the residual add
and the norm). A block that takes part in this says ``accepts_pending = True``, takes the
sums that the block before left in ``pending`` and returns its own.
"""
from __future__ import annotations

from .base import BLOCKS, Part


class PreNormResidualBlock(Part):
    capturable = True

    def __init__(self, spec, prefix: str = "", mixer=None, feed_forward=None, norms=None):
        super().__init__(spec, prefix)
        self.mixer, self.feed_forward, self.norms = mixer, feed_forward, norms

    accepts_pending = True

    def forward(self, x, step, line, state, writes_cache: bool, pending=None):
        h = self._norm("mixer", x, pending)
        pending = self.mixer.forward(h, x, step, line, state, writes_cache)
        h = self._norm("feed_forward", x, pending)
        return self.feed_forward.forward(h, x, step)

    def _norm(self, which, x, pending):
        norm = self.norms[which]
        if pending is None:
            return norm.forward(x)
        if getattr(norm, "accepts_pending", False):
            return norm.forward(x, pending=pending)
        settle(x, pending)             # a norm that knows nothing of pending sums
        return norm.forward(x)


def settle(x, pending) -> None:
    """Adds pending split sums into the residual x."""
    from .. import kernels as K
    K.add_partials(x, pending.partial)


BLOCKS.register("prenorm_residual", PreNormResidualBlock)
