"""The engine: a model on the device, its cache, and ONE step function.

``step(entries)`` runs a batch of sequences that start together with unequal lengths: their
prompts in one step, then one token each. It runs only the tokens it is given, packed as one
batch, from the cache that earlier steps left, and returns the float32 logits at the wanted
places. The reference's ``Forward`` does this for one sequence (``decoder.pas:768-781``,
``:3245-3369``): tokens are checked before the cache changes (``:3253-3298``) and a
sequence's length advances only after all layers ran (``:3343-3348``); batching, slots and
pages are this library's own.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from .. import kernels as K
from ..cache.pages import PAGE, CacheBook, pages_for, plan_groups
from ..cache.storage import CacheStorage
from ..config.registry import config_of_folder
from ..csrc import build
from ..errors import CacheError, InferError
from ..weights.binding import bind_tensors
from ..weights.safetensors_file import SafeTensorsFolder
from .batch import StepBuffers, StepContext
from .model import DecoderModel
from .runtime import Runtime

DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16,
          "float32": torch.float32, "fp32": torch.float32, "f32": torch.float32}


@dataclass
class Entry:
    """The next tokens of one sequence in a step: its slot, the tokens, and the places among
    these tokens whose logits are wanted (None: the last one)."""
    slot: int
    tokens: Sequence[int]
    want: Optional[Sequence[int]] = None


@dataclass
class _DecodeGraph:
    graph: "torch.cuda.CUDAGraph"
    logits: torch.Tensor
    launches: int


class Engine:
    def __init__(self, config, weights: Dict[str, torch.Tensor], rt: Runtime,
                 max_tokens: int = 4096, max_context: Optional[int] = None,
                 max_slots: Optional[int] = None, prefill_chunk: int = 1024,
                 max_step_tokens: int = 16384, model: Optional[DecoderModel] = None):
        """``weights``: tensors by name, already on the device and of the kept types.
        ``max_tokens``: the most tokens that live sequences hold together, each sequence's
        count rounded up to a multiple of 64; it sizes the cache. ``max_context``: the most
        positions of one sequence. ``prefill_chunk``: the most new tokens of one sequence in
        one pass of the model (longer prompts run as several passes with equal results)."""
        self.config = config
        self.rt = rt
        self.model = model or DecoderModel(config.to_model_spec())
        spec = self.model.spec
        self.vocab_size = spec.vocab_size
        max_tokens = pages_for(max_tokens) * PAGE
        self.max_context = min(max_context or spec.max_positions, spec.max_positions, max_tokens)
        self.max_slots = max_slots or max(1, min(max_tokens // PAGE, 1024))
        self.prefill_chunk = max(1, prefill_chunk)
        self.max_step_tokens = max(max_step_tokens, self.max_slots)
        build.compile_libraries(rt.libraries())
        self.model.bind(weights, rt)
        needs = {line: (n.kv_heads, n.head_dim, n.window)
                 for line, n in self.model.line_needs.items()}
        self.plans = plan_groups(needs, max_tokens, self.max_context, self.max_slots,
                                 self.prefill_chunk)
        self.book = CacheBook(self.plans, self.max_slots, self.max_context)
        self.cache = CacheStorage(self.plans, self.max_slots, rt.dtype, rt.device,
                                  {l: s.shape for l, s in self.model.state_needs.items()})
        self.buffers = StepBuffers(self.max_step_tokens, self.max_slots, rt.device)
        self.on_state: Optional[Callable[[str, torch.Tensor], None]] = None
        self.passes = 0  # passes of the model so far (a step of long prompts takes several)
        self.last_slots: Optional[torch.Tensor] = None   # slots of the last step, on the device
        # decode passes are replayed as CUDA graphs, one per (sequences, wanted rows)
        self.use_graphs = self.model.capturable()
        self.graphs: Dict[Tuple[int, int], "_DecodeGraph"] = {}
        self.last_h2d_bytes = 0                          # index bytes copied for the last step

    # ------------------------------------------------------------------ making one
    @classmethod
    def from_folder(cls, folder: str, dtype: str = "bfloat16", device: str = "cuda:0",
                    **kwargs) -> "Engine":
        """Loads a model folder; the model class is the one its config.json names."""
        if dtype not in DTYPES:
            raise InferError(f"dtype \"{dtype}\" is not bfloat16 or float32")
        config = config_of_folder(folder)
        rt = Runtime(DTYPES[dtype], device, kwargs.pop("fast_kernels", True))
        model = DecoderModel(config.to_model_spec())
        weights = bind_tensors(model.tensors(), SafeTensorsFolder(folder), rt.dtype, rt.device)
        return cls(config, weights, rt, model=model, **kwargs)

    @classmethod
    def from_random(cls, config, seed: int, dtype: str = "bfloat16", device: str = "cuda:0",
                    std: float = 0.02, norm_std: float = 0.1, **kwargs) -> "Engine":
        """Random weights drawn on the device (for shapes too large to write to a folder)."""
        from ..weights.random_init import random_tensors
        rt = Runtime(DTYPES[dtype], device, kwargs.pop("fast_kernels", True))
        model = DecoderModel(config.to_model_spec())
        weights = random_tensors(model.tensors(), seed, std, norm_std, rt.dtype, device)
        return cls(config, weights, rt, model=model, **kwargs)

    # ------------------------------------------------------------------ sequences
    def open(self) -> int:
        """A slot for a new sequence (its fixed-size state zeroed)."""
        slot = self.book.open()
        self.cache.reset_state(slot)
        return slot

    def close(self, slot: int) -> None:
        """Gives the slot and its pages back; later sequences use them again."""
        self.book.close(slot)

    def length(self, slot: int) -> int:
        self.book.check_open(slot)
        return self.book.length[slot]

    # ------------------------------------------------------------------ the step
    def step(self, entries: Sequence[Entry]) -> Optional[torch.Tensor]:
        """Appends each entry's tokens to its sequence and returns the logits
        ``[wanted, vocab]`` (float32, on the device) in the order of the entries and of their
        ``want``; None when nothing is wanted. Nothing changes if an entry is refused."""
        if not entries:
            raise InferError("a step without entries")
        seen = set()
        plan: List[Tuple[int, int, List[int], List[int]]] = []
        for e in entries:
            self.book.check_open(e.slot)
            if e.slot in seen:
                raise InferError(f"slot {e.slot} occurs twice in one step")
            seen.add(e.slot)
            if len(e.tokens) == 1:                      # a decode step: no arrays for one token
                tokens = [int(e.tokens[0])]
                if not 0 <= tokens[0] < self.vocab_size:
                    raise InferError(f"slot {e.slot}: token {tokens[0]} is outside the "
                                     f"vocabulary of {self.vocab_size}")
            else:
                tokens = np.asarray(e.tokens, dtype=np.int64).reshape(-1)
                if tokens.size == 0:
                    raise InferError(f"slot {e.slot}: a step of 0 tokens")
                bad = (tokens < 0) | (tokens >= self.vocab_size)
                if bad.any():
                    raise InferError(f"slot {e.slot}: token {int(tokens[bad][0])} is outside "
                                     f"the vocabulary of {self.vocab_size}")
            want = [len(tokens) - 1] if e.want is None else [int(w) for w in e.want]
            if any(not 0 <= w < len(tokens) for w in want):
                raise InferError(f"slot {e.slot}: wanted places {want} among {len(tokens)} tokens")
            past = self.book.length[e.slot]
            if past + len(tokens) > self.max_context:
                raise CacheError(f"slot {e.slot}: {past} + {len(tokens)} positions exceed the "
                                 f"context of {self.max_context}")
            plan.append((e.slot, past, tokens, want))
        new_pages = self.book.reserve([(s, p + len(t)) for s, p, t, _ in plan])
        self.cache.map_pages(new_pages)

        n_want = sum(len(w) for _, _, _, w in plan)
        passes = self._passes(plan)
        out = None
        if n_want and len(passes) > 1:
            out = torch.empty((n_want, self.vocab_size), dtype=torch.float32, device=self.rt.device)
        self.last_h2d_bytes = 0
        self.last_passes = len(passes)
        for seqs, dest in passes:
            ctx = self.buffers.fill(seqs)
            self.last_h2d_bytes += 4 * (4 * ctx.T + 3 * ctx.B + 1 + ctx.n_want)
            self.last_slots = ctx.seq_slot
            logits = self._forward(ctx)
            self.passes += 1
            if logits is not None:
                if out is None and len(passes) == 1:
                    out = logits
                else:
                    out.index_copy_(0, torch.tensor(dest, dtype=torch.long, device=out.device),
                                    logits)
        for slot, past, tokens, _ in plan:
            self.book.commit(slot, past + len(tokens))
        return out

    # ------------------------------------------------------------------ one pass
    def _forward(self, ctx: StepContext) -> Optional[torch.Tensor]:
        """One pass of the model. A decode pass (one token per sequence) is captured as a CUDA
        graph the first time its shape occurs and replayed from then on: the index arrays, the
        page tables and the cache are read from fixed device addresses, so only their contents
        change between replays. The logits of a replayed pass live in the graph's own buffer
        and are overwritten by the next replay of the same shape."""
        if not (self.use_graphs and ctx.decode and self.on_state is None):
            return self.model.forward(ctx, self.cache, self.on_state)
        key = (ctx.B, ctx.n_want)
        g = self.graphs.get(key)
        if g is None:
            out = self.model.forward(ctx, self.cache)     # this step's result, computed eagerly
            self.graphs[key] = self._capture(ctx)         # the same launches, for later steps
            return out
        g.graph.replay()
        K.Launches.count += g.launches
        return g.logits

    def _capture(self, ctx: StepContext) -> "_DecodeGraph":
        graph = torch.cuda.CUDAGraph()
        before = K.Launches.count
        with torch.cuda.graph(graph):
            logits = self.model.forward(ctx, self.cache)
        launches = K.Launches.count - before
        K.Launches.count = before                         # capturing launched nothing
        return _DecodeGraph(graph, logits, launches)

    def decode_steps(self, slots: Sequence[int], tokens: Sequence[int], n_steps: int, sampler,
                     sampling, vocab_limit: Optional[int] = None) -> torch.Tensor:
        """``n_steps`` decode steps of the sequences in ``slots`` without a host round trip:
        ``tokens`` are fed first, then each step feeds what the sampler chose in the step before
        (the token ids and positions move on in device memory). Returns the chosen tokens
        ``[n_steps, sequences]`` (int32, on the device); the last row is not fed. No stop
        token is looked at: the caller cuts the rows."""
        if len(set(slots)) != len(slots) or len(tokens) != len(slots) or n_steps <= 0:
            raise InferError("decode_steps: one token for each of distinct slots, n_steps > 0")
        seqs = []
        for slot, t in zip(slots, tokens):
            self.book.check_open(slot)
            if not 0 <= int(t) < self.vocab_size:
                raise InferError(f"slot {slot}: token {t} is outside the vocabulary")
            past = self.book.length[slot]
            if past + n_steps > self.max_context:
                raise CacheError(f"slot {slot}: {past} + {n_steps} positions exceed the "
                                 f"context of {self.max_context}")
            seqs.append((slot, past, [int(t)], [0]))
        self.cache.map_pages(self.book.reserve([(s, p + n_steps) for s, p, _, _ in seqs]))
        ctx = self.buffers.fill(seqs)
        self.last_slots, self.last_passes = ctx.seq_slot, 1
        history = torch.empty((n_steps, ctx.B), dtype=torch.int32, device=self.rt.device)
        for i in range(n_steps):
            logits = self._forward(ctx)
            chosen = sampler.pick(logits, ctx.seq_slot, sampling, vocab_limit)
            K.advance_decode(ctx.tok_ids, ctx.tok_pos, chosen, history[i])
            self.passes += 1
        for slot, past, _, _ in seqs:
            self.book.commit(slot, past + n_steps)
        return history

    def _passes(self, plan):
        """Cuts a step into passes of at most ``prefill_chunk`` new tokens per sequence and
        ``max_step_tokens`` in all. Returns ``[(seqs, dest)]``: ``seqs`` as
        ``StepBuffers.fill`` takes them, ``dest`` the output rows of the pass's wanted logits."""
        if (max(len(p[2]) for p in plan) <= self.prefill_chunk
                and sum(len(p[2]) for p in plan) <= self.max_step_tokens):
            # everything fits one pass (every decode step does): the plan is the pass, and its
            # wanted rows come out in the order of the entries already
            return [(plan, list(range(sum(len(p[3]) for p in plan))))]
        # output rows in the order of the entries and of their want
        row_of: List[Dict[int, List[int]]] = []
        at = 0
        for _, _, tokens, want in plan:
            d: Dict[int, List[int]] = {}
            for w in want:
                d.setdefault(w, []).append(at)
                at += 1
            row_of.append(d)
        done = [0] * len(plan)
        passes = []
        while any(done[i] < len(plan[i][2]) for i in range(len(plan))):
            budget = self.max_step_tokens
            seqs, dest = [], []
            for i, (slot, past, tokens, want) in enumerate(plan):
                left = len(tokens) - done[i]
                if left <= 0 or budget <= 0:
                    continue
                n = min(left, self.prefill_chunk, budget)
                lo, hi = done[i], done[i] + n
                w_here, d_here = [], []
                for w in sorted(w for w in row_of[i] if lo <= w < hi):
                    for r in row_of[i][w]:
                        w_here.append(w - lo)
                        d_here.append(r)
                seqs.append((slot, past + lo, tokens[lo:hi], w_here))
                dest.extend(d_here)
                done[i] = hi
                budget -= n
            passes.append((seqs, dest))
        return passes
