"""One pass of the model over a batch: which tokens, of which sequences, at which positions.

The tokens of all sequences are packed one after another (no padding); per token the index of
its sequence and its position, per sequence its slot, its first packed row and how many
positions it held before. Parts and kernels read only this. All index arrays live in one
device buffer that is filled by one copy from pinned host memory.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Sequence, Tuple

import numpy as np
import torch

from ..errors import InferError


# A pass whose longest sequence has at least this many positions may be planned differently by
# the kernels (a decode attention that deals a long sequence out over more CTAs): the engine
# keeps a captured graph of its own for such passes.
LONG_CONTEXT = 24576


@dataclass
class StepContext:
    T: int                      # tokens in this pass
    B: int                      # sequences in this pass
    tok_ids: torch.Tensor       # int32 [T]
    tok_seq: torch.Tensor       # int32 [T] index of the token's sequence in this pass
    tok_pos: torch.Tensor       # int32 [T] absolute position
    tok_slot: torch.Tensor      # int32 [T] the cache slot of the token's sequence
    seq_slot: torch.Tensor      # int32 [B]
    seq_start: torch.Tensor     # int32 [B + 1] first packed row of each sequence
    seq_past: torch.Tensor      # int32 [B] positions held before this pass
    want_rows: torch.Tensor     # int32 [n_want] packed rows whose logits are wanted
    n_want: int
    max_new: int                # most new tokens of one sequence
    max_len: int                # longest sequence after this pass
    decode: bool                # every sequence brings exactly one token
    # host copies, for parts that plan launches from them
    host_new: List[int]
    host_past: List[int]
    host_slots: List[int]

    @property
    def long(self) -> bool:
        return self.max_len >= LONG_CONTEXT


class StepBuffers:
    """Pinned host and device index buffers, reused by every pass."""

    def __init__(self, max_tokens: int, max_seqs: int, device: torch.device, guards=None):
        self.max_tokens, self.max_seqs = max_tokens, max_seqs
        self.size = 5 * max_tokens + 3 * max_seqs + 1
        self.host = torch.zeros(self.size, dtype=torch.int32).pin_memory()
        self.host_np = self.host.numpy()      # the same pinned memory, for vectorised filling
        from ..cache.guards import alloc
        self.dev = alloc(guards, "step index arrays", (self.size,), torch.int32, device)
        self.copied = torch.cuda.Event()
        self.in_flight = False
        self.views = {}

    def fill(self, seqs: Sequence[Tuple[int, int, Sequence[int], Sequence[int]]]) -> StepContext:
        """``seqs = [(slot, past, tokens, want)]``; ``want`` are places among ``tokens``."""
        B = len(seqs)
        T = sum(len(s[2]) for s in seqs)
        n_want = sum(len(s[3]) for s in seqs)
        if not (0 < T <= self.max_tokens and B <= self.max_seqs and n_want <= self.max_tokens):
            raise InferError(f"a pass of {T} tokens, {B} sequences and {n_want} wanted rows; the "
                             f"buffers take {self.max_tokens} tokens and {self.max_seqs} sequences")
        if self.in_flight:
            self.copied.synchronize()  # the last copy must have read the host buffer
        o_ids, o_seq, o_pos, o_tslot = 0, T, 2 * T, 3 * T
        o_slot, o_start, o_past, o_want = 4 * T, 4 * T + B, 4 * T + 2 * B + 1, 4 * T + 3 * B + 1
        n_new = [len(s[2]) for s in seqs]
        total = 4 * T + 3 * B + 1 + n_want
        if T <= 64:
            # a decode step or a few tokens: plain lists are quicker than array slices
            ids: List[int] = []
            seq: List[int] = []
            pos: List[int] = []
            tslot: List[int] = []
            starts = [0]
            wants: List[int] = []
            for b, (slot, past, tokens, want) in enumerate(seqs):
                n = n_new[b]
                ids.extend(int(t) for t in tokens)
                seq.extend([b] * n)
                pos.extend(range(past, past + n))
                tslot.extend([slot] * n)
                wants.extend(starts[-1] + w for w in want)
                starts.append(starts[-1] + n)
            self.host_np[:total] = (ids + seq + pos + tslot + [s[0] for s in seqs] + starts
                                    + [s[1] for s in seqs] + wants)
        else:
            starts = np.zeros(B + 1, dtype=np.int64)
            np.cumsum(n_new, out=starts[1:])
            flat = self.host_np[:total]
            at = 0
            for b, (slot, past, tokens, want) in enumerate(seqs):
                n, lo = n_new[b], int(starts[b])
                flat[o_ids + lo:o_ids + lo + n] = tokens
                flat[o_seq + lo:o_seq + lo + n] = b
                flat[o_pos + lo:o_pos + lo + n] = np.arange(past, past + n, dtype=np.int32)
                flat[o_tslot + lo:o_tslot + lo + n] = slot
                flat[o_slot + b] = slot
                flat[o_past + b] = past
                if len(want):
                    flat[o_want + at:o_want + at + len(want)] = np.asarray(want, dtype=np.int64) + lo
                    at += len(want)
            flat[o_start:o_start + B + 1] = starts
        self.dev[:total].copy_(self.host[:total], non_blocking=True)
        self.copied.record()
        self.in_flight = True
        # the device views depend on the counts only: made once per shape of step
        views = self.views.get((T, B, n_want))
        if views is None:
            d = self.dev
            views = (d[o_ids:o_ids + T], d[o_seq:o_seq + T], d[o_pos:o_pos + T],
                     d[o_tslot:o_tslot + T], d[o_slot:o_slot + B], d[o_start:o_start + B + 1],
                     d[o_past:o_past + B], d[o_want:o_want + n_want])
            if len(self.views) < 4096:
                self.views[(T, B, n_want)] = views
        return StepContext(
            T=T, B=B, tok_ids=views[0], tok_seq=views[1], tok_pos=views[2], tok_slot=views[3],
            seq_slot=views[4], seq_start=views[5], seq_past=views[6], want_rows=views[7],
            n_want=n_want, max_new=max(n_new),
            max_len=max(s[1] + len(s[2]) for s in seqs), decode=max(n_new) == 1,
            host_new=n_new, host_past=[s[1] for s in seqs], host_slots=[s[0] for s in seqs])
