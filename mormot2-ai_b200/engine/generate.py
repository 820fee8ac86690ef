"""The generation loop above the step function: batches of unequal prompts that start
together, stop tokens, sequences that end earlier (their slot is given back at once), and as
many batches one after another as there are requests.

Per sequence the loop is the reference's ``NativeDecode`` (``llm.native.pas:2133-2187``):
the prompt in one step, then ``pick; stop or cap? else feed the token``; an empty prompt or a
cap <= 0 is refused (``:2147-2154``); the cap shrinks to ``limit - len(prompt) + 1``
(``:2155-2157``: token n is fed only when another one follows); the stop token is part of the
result and is not fed back (``:2176-2178``). Batching is this library's own.

The loop decides on the host and computes nothing: it drives a *stepper* (``open``, ``close``,
``pick``), which in the product is the engine with the device sampler.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Set, Tuple

from ..cache.pages import pages_for
from ..errors import InferError


@dataclass
class Request:
    prompt: List[int]
    max_new: int
    stop: Set[int] = field(default_factory=set)
    seed: int = 0


@dataclass
class Outcome:
    tokens: List[int]
    stopped: bool      # ended on a stop token (else on its cap)


def checked(requests: Sequence[Request], limit: int) -> List[Request]:
    """The requests with their caps cut to the context; refuses what the reference refuses."""
    out = []
    for i, r in enumerate(requests):
        if not r.prompt:
            raise InferError(f"request {i}: empty prompt")
        if len(r.prompt) > limit:
            raise InferError(f"request {i}: a prompt of {len(r.prompt)} tokens exceeds the "
                             f"context of {limit}")
        if r.max_new <= 0:
            raise InferError(f"request {i}: {r.max_new} new tokens")
        out.append(Request(list(r.prompt), min(r.max_new, limit - len(r.prompt) + 1),
                           set(r.stop), r.seed))
    return out


def plan_batches(requests: Sequence[Request], max_batch: int, total_pages: int) -> List[List[int]]:
    """Which requests run together: in order, as many as ``max_batch`` slots and the cache's
    pages allow (a sequence may come to hold len(prompt) + max_new - 1 positions)."""
    batches: List[List[int]] = []
    cur: List[int] = []
    pages = 0
    for i, r in enumerate(requests):
        need = pages_for(len(r.prompt) + r.max_new - 1)
        if need > total_pages:
            raise InferError(f"request {i} needs {need} pages of the cache, which has {total_pages}")
        if cur and (len(cur) >= max_batch or pages + need > total_pages):
            batches.append(cur)
            cur, pages = [], 0
        cur.append(i)
        pages += need
    if cur:
        batches.append(cur)
    return batches


def generate(stepper, requests: Sequence[Request]) -> List[Outcome]:
    """Runs every request to its end and returns the new tokens of each, in request order."""
    reqs = checked(requests, stepper.context_limit())
    results: List[Optional[Outcome]] = [None] * len(reqs)
    for batch in plan_batches(reqs, stepper.max_batch(), stepper.total_pages()):
        live: Dict[int, int] = {}          # request index -> slot
        new: Dict[int, List[int]] = {i: [] for i in batch}
        try:
            for i in batch:
                live[i] = stepper.open(reqs[i].seed)
            feed = {i: reqs[i].prompt for i in batch}
            while live:
                order = [i for i in batch if i in live]
                picked = stepper.pick([(live[i], feed[i]) for i in order])
                feed = {}
                for i, token in zip(order, picked):
                    token = int(token)
                    new[i].append(token)
                    stopped = token in reqs[i].stop
                    if stopped or len(new[i]) >= reqs[i].max_new:
                        results[i] = Outcome(new[i], stopped)
                        stepper.close(live.pop(i))   # the slot is free for a later batch
                    else:
                        feed[i] = [token]
        finally:
            for slot in live.values():   # an error: nothing stays held
                stepper.close(slot)
    return results  # type: ignore[return-value]


class EngineStepper:
    """The engine and the device sampler as the stepper of ``generate``."""

    def __init__(self, engine, sampling, vocab_limit: Optional[int] = None,
                 max_batch: Optional[int] = None):
        from ..sampling.device import DeviceSampler
        import torch
        self.engine, self.sampling, self.vocab_limit = engine, sampling, vocab_limit
        self._max_batch = min(max_batch or engine.max_slots, engine.max_slots)
        self.sampler = DeviceSampler(engine.rt.device, engine.max_slots, engine.vocab_size)
        self._torch = torch
        self.h2d_bytes = 0
        self.d2h_bytes = 0

    def context_limit(self) -> int:
        return self.engine.max_context

    def max_batch(self) -> int:
        return self._max_batch

    def total_pages(self) -> int:
        return min(p.n_pages for p in self.engine.plans) if self.engine.plans else 1 << 30

    def open(self, seed: int) -> int:
        slot = self.engine.open()
        self.sampler.start(slot, seed)
        return slot

    def close(self, slot: int) -> None:
        self.engine.close(slot)

    def pick(self, entries: List[Tuple[int, List[int]]]) -> List[int]:
        from .engine import Entry
        logits = self.engine.step([Entry(slot, tokens) for slot, tokens in entries])
        if self.engine.last_passes == 1:
            ctx_slots = self.engine.last_slots  # int32 [B] on the device, in entry order
        else:
            ctx_slots = self._torch.tensor([slot for slot, _ in entries],
                                           dtype=self._torch.int32, device=logits.device)
        rt = self.engine.rt
        rows = logits.shape[0]
        box = rt.token_box(rows)
        tokens = self.sampler.pick(logits, ctx_slots, self.sampling, self.vocab_limit, out=box)
        self.h2d_bytes += self.engine.last_h2d_bytes
        if box is None:
            host = tokens.cpu()
            rt.check_cheap()
            self.d2h_bytes += host.numel() * 4
            return host.tolist()
        self.d2h_bytes += (rows + 1) * 4
        return rt.read_tokens(rows)
