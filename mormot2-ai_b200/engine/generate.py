"""The generation loop above the step function: batches of unequal prompts that start
together, stop tokens, sequences that end earlier (their slot is given back at once), and as
many batches one after another as there are requests.

Per sequence the loop is the reference's ``NativeDecode`` (``llm.native.pas:2133-2187``):
the prompt in one step, then ``pick; stop or cap? else feed the token``; an empty prompt or a
cap <= 0 is refused (``:2147-2154``); the cap shrinks to ``limit - len(prompt) + 1``
(``:2155-2157``: token n is fed only when another one follows); the stop token is part of the
result and is not fed back (``:2176-2178``). Batching is this library's own.

The loop decides on the host and computes nothing: it drives a *stepper*, which in the
product is the engine with the device sampler. ``stepper.prefill`` runs the prompts of a batch
in one step and returns each sequence's first pick. ``stepper.decode`` opens a *run* over the
sequences that go on: ``run.launch()`` queues a step in which every sequence is fed its last
pick (on the device), ``run.read()`` returns the picks of the oldest unread step. The loop
keeps one step queued behind the one it reads, so the device does not wait for the host; what
it learns a step late (a stop token) ends the run: the steps already queued still count for
the sequences that go on, which then form the next run. Caps are known beforehand, so a run
is never launched beyond the step in which its first sequence reaches its cap.
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


def pages_needed(pools: Sequence[Tuple[int, int]], positions: int) -> List[int]:
    """The pages of every pool that a sequence of ``positions`` positions holds.
    ``pools[g] = (pages of the pool, ring)``: a windowed group keeps a ring of ``ring`` pages
    per sequence however long it grows (0: every page is kept)."""
    n = pages_for(positions)
    return [min(n, ring) if ring else n for _, ring in pools]


def plan_batches(requests: Sequence[Request], max_batch: int,
                 pools: Sequence[Tuple[int, int]]) -> List[List[int]]:
    """Which requests run together: in order, as many as ``max_batch`` slots and the pages of
    every pool allow (a sequence may come to hold len(prompt) + max_new - 1 positions; in a
    windowed group never more than its ring)."""
    batches: List[List[int]] = []
    cur: List[int] = []
    used = [0] * len(pools)
    for i, r in enumerate(requests):
        need = pages_needed(pools, len(r.prompt) + r.max_new - 1)
        for g, (have, _) in enumerate(pools):
            if need[g] > have:
                raise InferError(f"request {i} needs {need[g]} pages of the cache, "
                                 f"which has {have}")
        if cur and (len(cur) >= max_batch
                    or any(u + n > have for u, n, (have, _) in zip(used, need, pools))):
            batches.append(cur)
            cur, used = [], [0] * len(pools)
        cur.append(i)
        used = [u + n for u, n in zip(used, need)]
    if cur:
        batches.append(cur)
    return batches


AHEAD = 2      # steps launched before the oldest of them is read


def generate(stepper, requests: Sequence[Request]) -> List[Outcome]:
    """Runs every request to its end and returns the new tokens of each, in request order."""
    reqs = checked(requests, stepper.context_limit())
    results: List[Optional[Outcome]] = [None] * len(reqs)
    for batch in plan_batches(reqs, stepper.max_batch(), stepper.pools()):
        live: Dict[int, int] = {}          # request index -> slot
        new: Dict[int, List[int]] = {i: [] for i in batch}

        def take(i: int, token: int) -> bool:
            """Books a pick of request i; True if it was its last."""
            new[i].append(token)
            stopped = token in reqs[i].stop
            if stopped or len(new[i]) >= reqs[i].max_new:
                results[i] = Outcome(new[i], stopped)
                return True
            return False

        run = None
        try:
            for i in batch:
                live[i] = stepper.open(reqs[i].seed)
            picks = stepper.prefill([(live[i], reqs[i].prompt) for i in batch])
            for i, token in zip(list(batch), picks):
                if take(i, int(token)):
                    stepper.close(live.pop(i))       # the slot is free for a later batch
            while live:
                members = [i for i in batch if i in live]
                left = [reqs[i].max_new - len(new[i]) for i in members]   # picks still allowed
                run = stepper.decode([(live[i], new[i][-1], n) for i, n in zip(members, left)])
                horizon = min(left)        # the step in which the first cap is reached
                launched = n_read = 0
                kept = [0] * len(members)
                done = [False] * len(members)
                while not any(done):
                    while launched < horizon and launched - n_read < AHEAD:
                        run.launch()
                        launched += 1
                    tokens = run.read()
                    n_read += 1
                    for m, i in enumerate(members):
                        kept[m] += 1
                        done[m] = take(i, int(tokens[m]))
                while n_read < launched:
                    # launched before the host knew that a sequence had ended: these steps
                    # still count for the sequences that go on
                    tokens = run.read()
                    n_read += 1
                    for m, i in enumerate(members):
                        if not done[m]:
                            kept[m] += 1
                            done[m] = take(i, int(tokens[m]))
                run.finish(kept)
                run = None
                for m, i in enumerate(members):
                    if done[m]:
                        stepper.close(live.pop(i))
        finally:
            if run is not None:          # an error: nothing stays held
                run.abandon()
            for slot in live.values():
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
        self.decode_steps = 0

    def context_limit(self) -> int:
        return self.engine.max_context

    def max_batch(self) -> int:
        return self._max_batch

    def pools(self) -> List[Tuple[int, int]]:
        return [(p.n_pages, p.ring_pages) for p in self.engine.plans]

    def open(self, seed: int) -> int:
        slot = self.engine.open()
        self.sampler.start(slot, seed)
        return slot

    def close(self, slot: int) -> None:
        self.engine.close(slot)

    def prefill(self, entries: List[Tuple[int, List[int]]]) -> List[int]:
        """The prompts in one step; each sequence's first pick, read on the host."""
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
            rt.check()
            self.d2h_bytes += host.numel() * 4
            return host.tolist()
        self.d2h_bytes += (rows + 1) * 4
        return rt.read_tokens(rows)

    def decode(self, members: List[Tuple[int, int, int]]):
        """A decode run over ``members = [(slot, last pick, steps it may still take)]``."""
        run = self.engine.decode_run([m[0] for m in members], [m[1] for m in members],
                                     [m[2] for m in members], self.sampler, self.sampling,
                                     self.vocab_limit)
        self.h2d_bytes += self.engine.last_h2d_bytes
        return _CountedRun(run, self)


class _CountedRun:
    """A decode run that books the bytes it brings to the host."""

    def __init__(self, run, stepper):
        self.run, self.stepper = run, stepper
        self.launch, self.finish, self.abandon = run.launch, run.finish, run.abandon

    def read(self) -> List[int]:
        got = self.run.read()
        self.stepper.d2h_bytes += 4 * (1 + len(got))
        self.stepper.decode_steps += 1
        return got
