"""What a part is, and the registries that the configuration chooses parts from.

A part is built from a ``PartSpec`` (sizes and constants as parameters) and knows nothing of
the model it sits in. It names the tensors it binds (``tensors``), what it keeps per sequence
(``cache_need``, ``state_need``), takes its weights (``bind``) and computes (``forward``).
The kinds are registry keys, so a test or a user adds a mixer, feed-forward, norm, position
encoding or block arrangement with ``register_*`` and a spec that names it; no file of the
library changes. The reference makes the same choice per layer through
``TDecoderLayerSpec`` (``decoder.pas:132-154``).

Interfaces (``rt`` is the ``Runtime``: device, activation dtype, kernels; ``step`` is the
``StepContext`` of ``engine/batch.py``: which token belongs to which sequence, at which
position, in which slot):

- Norm:      ``forward(x_f32[T, size], rows=None) -> h[R, size]`` in the activation dtype. A
             norm with ``accepts_pending = True`` also takes ``pending=`` (split sums of the
             product before, which it adds into x first).
- Position:  ``frequencies() -> (inv_freq_f32[rot_dim/2] on the device, rot_dim)``.
- Mixer:     ``forward(h[T, hidden], x_f32[T, hidden], step, line, state, writes_cache)``:
             adds its output to the residual ``x`` in place and returns None. ``line`` is the
             view of its cache line (``cache/storage.py``), ``state`` its per-sequence state
             ``[slots, *shape]`` or None. (A built-in part may instead return its output as
             ``Pending`` split sums, ``parts/linear.py``, which the next norm adds into x.)
- FeedForward: ``forward(h[T, hidden], x_f32[T, hidden], step)``: adds into ``x``, returns None
             (or ``Pending``, as above).
- Block:     ``forward(x_f32, step, line, state, writes_cache)``: arranges norms, mixer and
             feed-forward around the residual stream. A block with ``accepts_pending = True``
             also takes ``pending=`` (sums that the block before left) and returns its own.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Dict, List, Optional, Tuple

from ..config.spec import PartSpec
from ..errors import ConfigError


@dataclass(frozen=True)
class TensorNeed:
    """A tensor that a part binds: its name in the model folder, its shape and its role
    (``matrix``: a projection, drawn N(0, std) by the random-weights mode; ``vector``: a norm
    weight, drawn 1 + N(0, norm_std); ``table``: an embedding, drawn like a matrix).
    ``optional``: may be absent; ``must_equal``: if present it must hold the same bytes as the
    tensor of that name (a tied head's stored copy, ``model.qwen3.pas:555-567`` of the
    reference)."""
    name: str
    shape: Tuple[int, ...]
    role: str = "matrix"
    optional: bool = False
    must_equal: Optional[str] = None


@dataclass(frozen=True)
class CacheNeed:
    """Keys and values that a mixer keeps for every token: ``kv_heads`` x ``head_dim`` each;
    ``window`` > 0: only the last ``window`` positions are ever read."""
    kv_heads: int
    head_dim: int
    window: int = 0


@dataclass(frozen=True)
class StateNeed:
    """State of fixed size that a mixer keeps for every sequence: ``shape`` values of
    ``dtype`` (a torch type by name) per slot, every one ``init`` when a sequence starts."""
    shape: Tuple[int, ...]
    dtype: str = "float32"
    init: float = 0.0


class Part:
    """Base of every part. ``spec.params`` hold its sizes and constants.

    ``capturable``: the part's ``forward`` only launches kernels on the current stream, reads
    nothing back to the host and takes no decision from the contents of a step, so that a decode
    pass through it can be captured once as a CUDA graph and replayed. A part that does not say
    so keeps the engine from using graphs."""
    capturable = False

    def __init__(self, spec: PartSpec, prefix: str = ""):
        self.spec = spec
        self.prefix = prefix

    def tensors(self) -> List[TensorNeed]:
        return []

    def bind(self, weights: Dict[str, Any], rt: Any) -> None:
        """Takes the bound tensors (already on the device, by full name)."""

    def cache_need(self) -> Optional[CacheNeed]:
        return None

    def state_need(self) -> Optional[StateNeed]:
        return None


class Registry:
    def __init__(self, what: str):
        self.what = what
        self._kinds: Dict[str, Callable[..., Part]] = {}

    def register(self, kind: str, factory: Callable[..., Part]) -> None:
        self._kinds[kind] = factory

    def build(self, spec: PartSpec, *args: Any, **kwargs: Any) -> Part:
        if spec.kind not in self._kinds:
            raise ConfigError(
                f"no {self.what} \"{spec.kind}\" is registered (known: {', '.join(sorted(self._kinds))})")
        return self._kinds[spec.kind](spec, *args, **kwargs)

    def kinds(self) -> List[str]:
        return sorted(self._kinds)


MIXERS = Registry("mixer")
FEED_FORWARDS = Registry("feed-forward")
NORMS = Registry("norm")
POSITIONS = Registry("position encoding")
BLOCKS = Registry("block arrangement")
EMBEDDINGS = Registry("embedding")
HEADS = Registry("head")


def register_mixer(kind, factory):
    MIXERS.register(kind, factory)


def register_feed_forward(kind, factory):
    FEED_FORWARDS.register(kind, factory)


def register_norm(kind, factory):
    NORMS.register(kind, factory)


def register_position(kind, factory):
    POSITIONS.register(kind, factory)


def register_block(kind, factory):
    BLOCKS.register(kind, factory)
