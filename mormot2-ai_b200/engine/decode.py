"""A decode run: a fixed set of sequences decoded step after step without the host in the way.

A step of the run is the engine's decode pass (replayed as a CUDA graph), the sampler's pick
and a small kernel that makes the picks the next step's token ids and moves every position on
by one: ids and positions stay in device memory. After every step the picks (and the word
that kernels set when a bounded wait of theirs ran out) are copied to pinned host memory
asynchronously; the host reads them a step late, while the next step is already running, so
the GPU never waits for Python. The reference decodes one sequence with a host round trip
per token (``NativeDecode``, ``llm.native.pas:2171-2180``) and replays its decode step as a
graph (``TQwen3Cuda.Chunk``, ``model.qwen3.cuda.pas:1442-1449``); the run is this library's
own.

What the host learns a step late it cannot undo: a sequence whose stop token was picked in
step j has been fed that token in step j + 1 if that step was launched before the host read
step j. That is harmless: its keys lie beyond the length that ``finish`` commits for it and
are written over or given back with the slot; the picks of the other sequences do not depend
on it. Only fixed-size state cannot be taken back: a slot that keeps fewer steps than were
launched has its state marked as not matching its length.
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import torch

from .. import kernels as K
from ..errors import InferError


class DecodeRun:
    """Made by ``Engine.decode_run``. ``launch()`` queues one step; ``read()`` returns the
    picks of the oldest step not read yet (waits for it); ``finish(kept)`` commits lengths and
    ends the run. At most ``DEPTH`` launched steps may be unread. A run opened with
    ``history`` keeps every step's picks in a device tensor instead (``history[step]``) and is
    not read step by step: the caller looks at the picks, and at ``Runtime.check``, when it
    likes."""

    DEPTH = 4

    def __init__(self, engine, ctx, slots: List[int], tokens: List[int], max_steps: int,
                 sampler, sampling, vocab_limit: Optional[int], history: bool,
                 order: Optional[List[int]] = None):
        # ``order[j]``: which of ``slots`` row j of ``ctx`` (and of every step's picks) is
        self.engine, self.ctx, self.slots = engine, ctx, slots
        self.order = None if order is None or order == sorted(order) else list(order)
        self.first_tokens = tokens
        self.max_steps = max_steps
        self.sampler, self.sampling, self.vocab_limit = sampler, sampling, vocab_limit
        self.launched = 0
        self.n_read = 0
        self.past = [engine.book.length[s] for s in slots]
        self.picks: List[List[int]] = []        # what the host has read, step by step
        rt = engine.rt
        self.box = rt.token_box(ctx.B)
        if self.box is None:
            raise InferError(f"a decode run of {ctx.B} sequences")
        self.history = (torch.empty((max_steps, ctx.B), dtype=torch.int32, device=rt.device)
                        if history else None)
        self.d2h_bytes = 0

    # ------------------------------------------------------------------ stepping
    def launch(self) -> None:
        if self.launched >= self.max_steps:
            raise InferError(f"the decode run was opened for {self.max_steps} steps")
        if self.history is None and self.launched - self.n_read >= self.DEPTH:
            raise InferError(f"{self.DEPTH} launched steps are unread: read one first")
        eng, ctx, rt = self.engine, self.ctx, self.engine.rt
        ctx.max_len = max(self.past) + self.launched + 1   # the positions moved on on the device
        logits = eng._forward(ctx)
        self.sampler.pick(logits, ctx.seq_slot, self.sampling, self.vocab_limit, out=self.box)
        K.advance_decode(ctx.tok_ids, ctx.tok_pos, self.box,
                         self.history[self.launched] if self.history is not None else None)
        if self.history is None:
            rt.post_mail(self.launched % self.DEPTH, ctx.B)
        eng.passes += 1
        self.launched += 1

    def read(self) -> List[int]:
        """The picks of the oldest unread step, in the order of the run's slots. Raises
        ``KernelError`` if a kernel of that step (or before) gave up a wait."""
        if self.history is not None:
            raise InferError("a run that keeps its picks on the device is not read step by step")
        if self.n_read >= self.launched:
            raise InferError("no launched step is unread")
        got = self.engine.rt.take_mail(self.n_read % self.DEPTH, self.ctx.B)
        if self.order is not None:
            rows, got = got, [0] * len(got)
            for j, i in enumerate(self.order):
                got[i] = rows[j]
        self.d2h_bytes += 4 * (1 + self.ctx.B)
        self.n_read += 1
        self.picks.append(got)
        return got

    def picks_on_device(self) -> torch.Tensor:
        """The picks of a run opened with ``history``: ``[steps, sequences]`` in the order of
        the run's slots (int32, on the device)."""
        if self.history is None:
            raise InferError("the run was not opened with history")
        if self.order is None:
            return self.history
        back = [0] * len(self.order)
        for j, i in enumerate(self.order):
            back[i] = j
        return self.history.index_select(
            1, torch.tensor(back, dtype=torch.int64, device=self.history.device))

    # ------------------------------------------------------------------ ending
    def finish(self, kept: Optional[Sequence[int]] = None) -> None:
        """Ends the run. ``kept[i]``: how many of the launched steps count for sequence i
        (default: all of them): its length grows by that many positions."""
        eng = self.engine
        kept = [self.launched] * len(self.slots) if kept is None else list(kept)
        if len(kept) != len(self.slots) or any(not 0 <= k <= self.launched for k in kept):
            raise InferError(f"finish: {kept} of {self.launched} launched steps")
        for i, (slot, k) in enumerate(zip(self.slots, kept)):
            eng.book.commit(slot, self.past[i] + k)
            fed = [self.first_tokens[i]] + [p[i] for p in self.picks[:max(0, k - 1)]]
            fed += [-1] * (k - len(fed))          # picks that the host never read
            eng.ids[slot].extend(fed[:k])
            if eng.has_state and k != self.launched:
                eng.state_ok[slot] = False
        eng.run = None

    def abandon(self) -> None:
        """Ends the run after an error: nothing of it counts. Waits for what was launched."""
        eng = self.engine
        try:
            torch.cuda.synchronize(eng.rt.device)
        finally:
            if eng.has_state and self.launched:
                for slot in self.slots:
                    eng.state_ok[slot] = False
            eng.run = None
