"""SwiGLU feed-forward: x += (silu(h·Wgᵀ) · (h·Wuᵀ)) · Wdᵀ, no bias
(``decoder.pas:2865-2899``, ``backend.cpu.pas:1827-1833`` of the reference). Gate and up are
one product whose epilogue applies the activation: their rows are laid out alternately (gate
of output 0, up of output 0, gate of output 1, ...), a pure re-layout done once at load."""
from __future__ import annotations

from typing import Dict, List

import torch

from .base import FEED_FORWARDS, Part, TensorNeed
from .linear import Linear


class SwiGluFfn(Part):
    capturable = True

    def __init__(self, spec, prefix: str = ""):
        super().__init__(spec, prefix)
        p = spec.params
        self.hidden = int(p["hidden_size"])
        self.inter = int(p["intermediate_size"])
        self.names = {k: prefix + v for k, v in p["names"].items()}

    def tensors(self) -> List[TensorNeed]:
        n = self.names
        return [TensorNeed(n["gate"], (self.inter, self.hidden)),
                TensorNeed(n["up"], (self.inter, self.hidden)),
                TensorNeed(n["down"], (self.hidden, self.inter))]

    def bind(self, weights: Dict[str, torch.Tensor], rt) -> None:
        n = self.names
        g, u = weights[n["gate"]], weights[n["up"]]
        if g.dtype != u.dtype:
            g, u = g.float(), u.float()
        pairs = torch.stack([g, u], dim=1).reshape(2 * self.inter, self.hidden)
        self.gate_up = Linear(pairs, rt, swiglu=True)
        if getattr(rt, "consume_weights", False):   # the originals go once they are interleaved
            del g, u
            weights.pop(n["gate"], None)
            weights.pop(n["up"], None)
        self.down = Linear(weights[n["down"]], rt)

    def forward(self, h, x, step):
        """Adds the feed-forward's output into x, or returns it as ``Pending`` split sums for
        the next norm to add."""
        from .linear import Pending
        act = self.gate_up(h)
        out = self.down(act, add_into=x, defer=True)
        return out if isinstance(out, Pending) else None


FEED_FORWARDS.register("swiglu", SwiGluFfn)
