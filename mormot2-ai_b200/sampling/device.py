"""Sampling on the device: one splitmix64 state per slot, arg-max, temperature draws and the
top-k / top-p / min-p filters as kernels (``csrc/sampling.cu``). Only the chosen token ids
come back to the host."""
from __future__ import annotations

from typing import Optional

import torch

from .. import kernels as K
from .settings import Sampling


class DeviceSampler:
    def __init__(self, device: torch.device, max_slots: int, vocab_size: int):
        self.device, self.vocab_size, self.max_slots = device, vocab_size, max_slots
        self.states = torch.zeros(max_slots, dtype=torch.int64, device=device)
        self.argmax_scratch = torch.empty(max_slots * (vocab_size // 2048 + 1), dtype=torch.int64,
                                          device=device)
        self.scratch: Optional[torch.Tensor] = None
        self.scratch_stride = 1
        while self.scratch_stride < vocab_size:
            self.scratch_stride *= 2

    def start(self, slot: int, seed: int) -> None:
        """Seeds the stream of the sequence in ``slot``."""
        s = seed & 0xFFFFFFFFFFFFFFFF
        self.states[slot] = s - (1 << 64) if s >= 1 << 63 else s

    def pick(self, logits: torch.Tensor, slots: torch.Tensor, sampling: Sampling,
             vocab_limit: Optional[int] = None,
             out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """One token per row of ``logits`` [rows, vocab]; ``slots`` int32 [rows] on the device
        names each row's stream. ``vocab_limit``: only the ids below it are candidates (rows of
        a padded embedding that no tokenizer id stands for are never drawn,
        ``llm.native.pas:2159-2162`` of the reference). ``out``: int32 [rows] on the device to
        write into (else a new tensor)."""
        rows = logits.shape[0]
        if vocab_limit is not None and vocab_limit < logits.shape[1]:
            logits = logits[:, :vocab_limit]
        if out is None:
            out = torch.empty(rows, dtype=torch.int32, device=logits.device)
        if sampling.greedy:
            K.argmax(logits, out, self.argmax_scratch if rows <= self.max_slots else None)
        elif not sampling.filtered:
            K.sample(logits, sampling.temperature, slots, self.states, out)
        else:
            if self.scratch is None or self.scratch.shape[0] < rows:
                self.scratch = torch.empty((max(rows, 8), self.scratch_stride), dtype=torch.int64,
                                           device=self.device)
            K.sample_filtered(logits, sampling, slots, self.states, self.scratch, out)
        return out
