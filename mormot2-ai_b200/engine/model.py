"""A decoder built from a ``ModelSpec``: embedding, layers of parts, the order in which they
run, final norm and head. It knows no architecture; the family made the spec.

``forward`` runs one pass over the tokens of a ``StepContext`` from the cache and returns the
float32 logits of the wanted rows (``decoder.pas:3245-3369`` of the reference: embed, the
layers, the final norm over the rows whose logits are wanted, the head).
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..config.spec import ModelSpec
from ..errors import ConfigError
from ..parts import BLOCKS, EMBEDDINGS, FEED_FORWARDS, HEADS, MIXERS, NORMS, POSITIONS
from ..parts.base import CacheNeed, StateNeed, TensorNeed
from ..parts.block import settle


class Layer:
    def __init__(self, spec, positions):
        self.spec = spec
        p = spec.prefix
        self.mixer = MIXERS.build(spec.mixer, p, positions=positions)
        self.feed_forward = FEED_FORWARDS.build(spec.feed_forward, p)
        self.norms = {k: NORMS.build(v, p) for k, v in spec.norms.items()}
        self.block = BLOCKS.build(spec.block, p, mixer=self.mixer,
                                  feed_forward=self.feed_forward, norms=self.norms)

    def parts(self):
        return [self.mixer, self.feed_forward] + list(self.norms.values())


class DecoderModel:
    def __init__(self, spec: ModelSpec):
        self.spec = spec
        self.positions = {k: POSITIONS.build(v) for k, v in spec.positions.items()}
        self.embedding = EMBEDDINGS.build(spec.embedding)
        self.layers = [Layer(l, self.positions) for l in spec.layers]
        self.final_norm = NORMS.build(spec.final_norm)
        self.head = HEADS.build(spec.head)
        for i, run in enumerate(spec.schedule):
            if not 0 <= run.layer < len(self.layers):
                raise ConfigError(f"entry {i} of the order names layer {run.layer} of "
                                  f"{len(self.layers)}")
        self._check_lines()

    # ---------------------------------------------------------------- what the model needs
    def parts(self):
        out = [self.embedding, self.final_norm, self.head] + list(self.positions.values())
        for l in self.layers:
            out += l.parts()
        return out

    def capturable(self) -> bool:
        """Whether a decode pass may be captured as a CUDA graph: every part must allow it."""
        blocks = [l.block for l in self.layers]
        return all(getattr(p, "capturable", False) for p in self.parts() + blocks)

    def tensors(self) -> List[TensorNeed]:
        seen: Dict[str, TensorNeed] = {}
        for part in self.parts():
            for need in part.tensors():
                if need.name in seen and seen[need.name].shape != need.shape:
                    raise ConfigError(f"{need.name} is bound with two shapes")
                if need.name not in seen or not need.optional:
                    seen[need.name] = need
        return list(seen.values())

    def _check_lines(self) -> None:
        """Every cache line is written by exactly one entry of the order, before it is read,
        by a mixer whose needs the readers share."""
        self.line_needs: Dict[int, CacheNeed] = {}
        self.state_needs: Dict[int, StateNeed] = {}
        for i, run in enumerate(self.spec.schedule):
            mixer = self.layers[run.layer].mixer
            need, state = mixer.cache_need(), mixer.state_need()
            if need is None and state is None:
                continue
            if run.cache_line is None:
                raise ConfigError(f"entry {i} of the order runs a mixer that keeps keys, "
                                  "values or state but names no cache line")
            line = run.cache_line
            if run.writes_cache:
                if line in self.line_needs or line in self.state_needs:
                    raise ConfigError(f"cache line {line} is written by two entries of the order")
                if need is not None:
                    self.line_needs[line] = need
                if state is not None:
                    self.state_needs[line] = state
            else:
                if need is None or line not in self.line_needs:
                    raise ConfigError(f"entry {i} of the order reads cache line {line} "
                                      "before any entry wrote it")
                have = self.line_needs[line]
                if (have.kv_heads, have.head_dim) != (need.kv_heads, need.head_dim):
                    raise ConfigError(f"entry {i} of the order reads cache line {line} with "
                                      "other head sizes than it was written with")

    # ---------------------------------------------------------------- weights
    def bind(self, weights: Dict[str, torch.Tensor], rt) -> None:
        self.rt = rt
        for part in self.parts():
            part.bind(weights, rt)

    # ---------------------------------------------------------------- one pass
    def forward(self, step, cache, on_state=None) -> Optional[torch.Tensor]:
        """``cache``: the ``CacheStorage``. ``on_state(name, x)``: called with the residual
        after the embedding and after every entry of the order (for tests)."""
        x = torch.empty((step.T, self.spec.hidden_size), dtype=torch.float32,
                        device=self.rt.device)
        self.embedding.forward(step.tok_ids, x)
        if on_state:
            on_state("embed", x)
        pending = None      # split sums of the last product, not yet added into x
        for i, run in enumerate(self.spec.schedule):
            line = cache.lines.get(run.cache_line) if run.cache_line is not None else None
            state = cache.states.get(run.cache_line) if run.cache_line is not None else None
            block = self.layers[run.layer].block
            if getattr(block, "accepts_pending", False):
                pending = block.forward(x, step, line, state, run.writes_cache, pending=pending)
            else:
                if pending is not None:
                    settle(x, pending)
                pending = None
                block.forward(x, step, line, state, run.writes_cache)
            if on_state:
                if pending is not None:
                    settle(x, pending)
                    pending = None
                on_state(f"run{i:02d}", x)
        if pending is not None:
            settle(x, pending)
        if step.n_want == 0:
            return None
        h = self.final_norm.forward(x, rows=step.want_rows, n_rows=step.n_want)
        return self.head.forward(h)
