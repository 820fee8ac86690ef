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

from collections import OrderedDict
from dataclasses import dataclass
from typing import Callable, Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from .. import kernels as K
from ..cache.guards import Guards
from ..cache.pages import PAGE, CacheBook, pages_for, plan_groups
from ..cache.storage import CacheStorage
from ..config.registry import config_of_folder
from ..csrc import build
from ..errors import CacheError, InferError
from ..weights.binding import bind_tensors
from ..weights.safetensors_file import SafeTensorsFolder
from .batch import StepBuffers, StepContext
from .decode import DecodeRun
from .model import DecoderModel
from .runtime import Runtime

MAX_GRAPHS = 24      # decode graphs kept (one per batch size and wanted rows), oldest use first out

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
                                  self.model.state_needs, rt.guards)
        # whether a slot's fixed-size state holds exactly the slot's length (the reference's
        # fStateOk, decoder.pas:436, :3301, :3348); only models with such state look at it
        self.has_state = bool(self.model.state_needs)
        self.state_ok = [True] * self.max_slots
        # the token at every position of a slot, for prefix reuse (the reference's fIds,
        # decoder.pas:412-421, Common :1264-1273)
        self.ids: List[List[int]] = [[] for _ in range(self.max_slots)]
        self.run: Optional[DecodeRun] = None             # the decode run that is open, if any
        self.buffers = StepBuffers(self.max_step_tokens, self.max_slots, rt.device, rt.guards)
        self.on_state: Optional[Callable[[str, torch.Tensor], None]] = None
        self.passes = 0  # passes of the model so far (a step of long prompts takes several)
        self.last_slots: Optional[torch.Tensor] = None   # slots of the last step, on the device
        # decode passes are replayed as CUDA graphs, one per (sequences, wanted rows)
        self.use_graphs = self.model.capturable()
        self.graphs: "OrderedDict[Tuple[int, int], _DecodeGraph]" = OrderedDict()
        self.graph_pool = None                           # one memory pool for all of them
        self.last_h2d_bytes = 0                          # index bytes copied for the last step

    # ------------------------------------------------------------------ making one
    @classmethod
    def from_folder(cls, folder: str, dtype: str = "bfloat16", device: str = "cuda:0",
                    **kwargs) -> "Engine":
        """Loads a model folder; the model class is the one its config.json names."""
        if dtype not in DTYPES:
            raise InferError(f"dtype \"{dtype}\" is not bfloat16 or float32")
        config = config_of_folder(folder)
        rt = Runtime(DTYPES[dtype], device, kwargs.pop("fast_kernels", True),
                     Guards() if kwargs.pop("guard", False) else None)
        model = DecoderModel(config.to_model_spec())
        weights = bind_tensors(model.tensors(), SafeTensorsFolder(folder), rt.dtype, rt.device)
        rt.consume_weights = True
        return cls(config, weights, rt, model=model, **kwargs)

    @classmethod
    def from_random(cls, config, seed: int, dtype: str = "bfloat16", device: str = "cuda:0",
                    std: float = 0.02, norm_std: float = 0.1, **kwargs) -> "Engine":
        """Random weights drawn on the device (for shapes too large to write to a folder)."""
        from ..weights.random_init import random_tensors
        rt = Runtime(DTYPES[dtype], device, kwargs.pop("fast_kernels", True),
                     Guards() if kwargs.pop("guard", False) else None)
        model = DecoderModel(config.to_model_spec())
        weights = random_tensors(model.tensors(), seed, std, norm_std, rt.dtype, device)
        rt.consume_weights = True
        return cls(config, weights, rt, model=model, **kwargs)

    # ------------------------------------------------------------------ sequences
    def open(self) -> int:
        """A slot for a new sequence (its fixed-size state at its initial value)."""
        slot = self.book.open()
        self.cache.reset_state(slot)
        self.state_ok[slot] = True
        self.ids[slot] = []
        return slot

    def close(self, slot: int) -> None:
        """Gives the slot and its pages back; later sequences use them again."""
        if self.run is not None and slot in self.run.slots:
            raise InferError(f"slot {slot} is part of the open decode run: finish it first")
        self.book.close(slot)
        self.ids[slot] = []

    def truncate(self, slot: int, length: int) -> None:
        """Shortens the slot's sequence to its first ``length`` positions; the next step goes
        on from there, and its logits are those of a fresh pass over the kept tokens and the
        new ones. Whole pages beyond ``length`` go back to the pool. Refused when a sliding
        window's ring no longer holds the keys before ``length``, and, for a model with
        fixed-size state, for every length but 0 and the present one (such state cannot go
        back). ``TDecoderContext.Truncate`` of the reference (``decoder.pas:996-1018``)."""
        if self.run is not None and slot in self.run.slots:
            raise InferError(f"slot {slot} is part of the open decode run: finish it first")
        self.book.check_open(slot)
        now = self.book.length[slot]
        if self.has_state and length not in (0, now) and 0 <= length <= now:
            raise CacheError(f"slot {slot}: truncate({length}): the fixed-size state of a "
                             f"sequence of {now} tokens cannot go back there")
        if self.has_state and length == now and not self.state_ok[slot]:
            raise CacheError(f"slot {slot}: its fixed-size state does not hold its {now} "
                             "tokens any more; only truncate(0) is left")
        self.book.truncate(slot, length)
        del self.ids[slot][length:]
        if length == 0:
            self.cache.reset_state(slot)
            self.state_ok[slot] = True

    def common(self, slot: int, tokens: Sequence[int]) -> int:
        """How many of the slot's first tokens equal the first of ``tokens``
        (``TDecoderContext.Common``, ``decoder.pas:1264-1273``)."""
        self.book.check_open(slot)
        held = self.ids[slot]
        n = 0
        while n < len(held) and n < len(tokens) and held[n] == int(tokens[n]):
            n += 1
        return n

    def reuse(self, slot: int, tokens: Sequence[int]) -> int:
        """Keeps of the slot what a new request of ``tokens`` can use again and returns that
        many positions: the common prefix, but never the whole request, whose last token must
        still be fed to give logits (``TDecoderModel.Reuse``, ``decoder.pas:3371-3388``).
        When that prefix cannot be cut to (a window's ring, fixed-size state) nothing is
        kept."""
        n = min(self.common(slot, tokens), max(0, len(tokens) - 1))
        try:
            self.truncate(slot, n)
        except CacheError:
            n = 0
            self.truncate(slot, 0)
        return n

    def length(self, slot: int) -> int:
        self.book.check_open(slot)
        return self.book.length[slot]

    def faults(self) -> List[str]:
        """Checks that stand in for a memory checker, for tests and debugging (they read the
        device): buffers whose guard bands a kernel damaged (engines made with ``guard=True``)
        and page tables that differ from the bookkeeping. Empty when all is well."""
        torch.cuda.synchronize(self.rt.device)
        found = self.rt.guards.damaged() if self.rt.guards is not None else []
        return found + self.cache.table_faults(self.book)

    def stats(self) -> Dict[str, object]:
        """Counters and sizes for logs: passes of the model and kernel launches so far, the
        bytes of the cache's pools and of everything this process holds on the device, slots
        and pages in use per group of cache lines, decode graphs kept."""
        return {
            "passes": self.passes,
            "kernel_launches": K.Launches.count,
            "cache_bytes": self.cache.bytes(),
            "device_bytes": int(torch.cuda.memory_allocated(self.rt.device)),
            "slots_open": self.max_slots - self.book.slots.free,
            "slots": self.max_slots,
            "pages_held": [self.book.held_pages(g) for g in range(len(self.plans))],
            "pages": [p.n_pages for p in self.plans],
            "decode_graphs": len(self.graphs),
        }

    # ------------------------------------------------------------------ the step
    def step(self, entries: Sequence[Entry]) -> Optional[torch.Tensor]:
        """Appends each entry's tokens to its sequence and returns the logits
        ``[wanted, vocab]`` (float32, on the device) in the order of the entries and of their
        ``want``; None when nothing is wanted. Nothing changes if an entry is refused, and a
        step that fails between its passes leaves lengths and fixed-size state as it found
        them. The logits of a decode step lie in memory that the next decode step writes
        again: copy them if they are to outlive it."""
        if not entries:
            raise InferError("a step without entries")
        if self.run is not None:
            raise InferError("a decode run is open: finish it before another step")
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
            if self.has_state and not self.state_ok[e.slot]:
                raise CacheError(f"slot {e.slot}: its fixed-size state does not hold its "
                                 f"{past} tokens (a step failed, or a decode run fed it "
                                 "further than it kept): truncate it to 0 or close it")
            plan.append((e.slot, past, tokens, want))
        if len(plan) > self.max_slots:
            raise InferError(f"a step of {len(plan)} sequences; the engine has "
                             f"{self.max_slots} slots")
        n_want = sum(len(w) for _, _, _, w in plan)
        passes = self._passes(plan)
        for seqs, _ in passes:
            if sum(len(s[3]) for s in seqs) > self.max_step_tokens:
                raise InferError(f"a pass of the step wants more than {self.max_step_tokens} "
                                 "rows of logits (max_step_tokens)")
        new_pages = self.book.reserve([(s, p + len(t)) for s, p, t, _ in plan])
        self.cache.map_pages(new_pages)

        out = None
        if n_want and len(passes) > 1:
            out = torch.empty((n_want, self.vocab_size), dtype=torch.float32, device=self.rt.device)
        self.last_h2d_bytes = 0
        self.last_passes = len(passes)
        touched = None
        if self.has_state:
            touched = torch.tensor([p[0] for p in plan], dtype=torch.long, device=self.rt.device)
            self.cache.save_states(touched)
        try:
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
                        out.index_copy_(0, torch.tensor(dest, dtype=torch.long,
                                                        device=out.device), logits)
        except BaseException:
            # lengths were not committed; keys written beyond them are never read; the state
            # goes back to what the step found
            if touched is not None:
                self.cache.restore_states(touched)
            raise
        for slot, past, tokens, _ in plan:
            self.book.commit(slot, past + len(tokens))
            self.ids[slot].extend(tokens.tolist() if isinstance(tokens, np.ndarray) else tokens)
        return out

    def timed_step(self, entries: Sequence[Entry]):
        """``step`` with its kernels run one by one and timed by class: returns the logits, the
        milliseconds of each class (products, attention, norms, rotary, embedding, ...) and
        of the whole step. Graphs are off for it and every kernel waits for the one before, so
        the sum is larger than the step of the product path; the shares say where time goes
        (the reference's ``llm-bench`` prints the same, ``demos/infer/llm-bench.lpr:499-527``)."""
        graphs, self.use_graphs = self.use_graphs, False
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        try:
            with K.Timing() as timing:
                e0.record()
                logits = self.step(entries)
                e1.record()
        finally:
            self.use_graphs = graphs
        shares = timing.shares(e0, e1)
        return logits, shares, e0.elapsed_time(e1)

    # ------------------------------------------------------------------ one pass
    def _forward(self, ctx: StepContext) -> Optional[torch.Tensor]:
        """One pass of the model. A decode pass (one token per sequence) is captured as a CUDA
        graph the first time its shape occurs and replayed from then on: the index arrays, the
        page tables and the cache are read from fixed device addresses, so only their contents
        change between replays. The logits of a replayed pass live in the graph's own buffer
        and are overwritten by the next replay of the same shape."""
        if not (self.use_graphs and ctx.decode and self.on_state is None):
            return self.model.forward(ctx, self.cache, self.on_state)
        key = (ctx.B, ctx.n_want, ctx.long)
        g = self.graphs.get(key)
        if g is None:
            out = self.model.forward(ctx, self.cache)     # this step's result, computed eagerly
            while len(self.graphs) >= MAX_GRAPHS:         # the graph used longest ago goes
                self.graphs.popitem(last=False)
            self.graphs[key] = self._capture(ctx)         # the same launches, for later steps
            return out
        self.graphs.move_to_end(key)
        g.graph.replay()
        K.Launches.count += g.launches
        return g.logits

    def _capture(self, ctx: StepContext) -> "_DecodeGraph":
        """Captures a decode pass. All graphs allocate from one memory pool: one graph runs
        at a time and each is complete in itself (its inputs are the index buffers, the page
        tables and the cache, which lie outside the pool), so the activations of one may lie
        where those of another lay."""
        graph = torch.cuda.CUDAGraph()
        if self.graph_pool is None:
            self.graph_pool = torch.cuda.graph_pool_handle()
        before = K.Launches.count
        with torch.cuda.graph(graph, pool=self.graph_pool):
            logits = self.model.forward(ctx, self.cache)
        launches = K.Launches.count - before
        K.Launches.count = before                         # capturing launched nothing
        return _DecodeGraph(graph, logits, launches)

    # ------------------------------------------------------------------ decoding on the device
    def decode_run(self, slots: Sequence[int], tokens: Sequence[int], steps: Sequence[int],
                   sampler, sampling, vocab_limit: Optional[int] = None,
                   history: bool = False) -> DecodeRun:
        """Opens a decode run (``engine/decode.py``): the sequences in ``slots`` are fed
        ``tokens`` in its first step and from then on what the sampler chose for them in the
        step before, in device memory. ``steps[i]``: the most steps sequence i takes part in;
        its pages up to there are reserved now (all or nothing), and the run goes no further
        than the smallest of them. Until the run is finished no other step may be made."""
        if self.run is not None:
            raise InferError("a decode run is open already")
        if (len(set(slots)) != len(slots) or len(tokens) != len(slots)
                or len(steps) != len(slots) or not slots):
            raise InferError("a decode run: one token and one step count for each of "
                             "distinct slots")
        if len(slots) > self.max_slots:
            raise InferError(f"a decode run of {len(slots)} sequences; the engine has "
                             f"{self.max_slots} slots")
        seqs = []
        for slot, t, n in zip(slots, tokens, steps):
            self.book.check_open(slot)
            if not 0 <= int(t) < self.vocab_size:
                raise InferError(f"slot {slot}: token {t} is outside the vocabulary of "
                                 f"{self.vocab_size}")
            past = self.book.length[slot]
            if n <= 0 or past + n > self.max_context:
                raise CacheError(f"slot {slot}: {past} + {n} positions exceed the "
                                 f"context of {self.max_context}")
            if self.has_state and not self.state_ok[slot]:
                raise CacheError(f"slot {slot}: its fixed-size state does not hold its "
                                 f"{past} tokens: truncate it to 0 or close it")
            seqs.append((slot, past, [int(t)], [0]))
        self.cache.map_pages(self.book.reserve(
            [(s, p + n) for (s, p, _, _), n in zip(seqs, steps)]))
        # Inside the run the longest sequence comes first: the attention's CTAs start in the
        # order of the rows, and the long ones must not be the last to start. The order holds
        # for the whole run, since every sequence grows by one position a step.
        order = sorted(range(len(seqs)), key=lambda i: -seqs[i][1])
        ctx = self.buffers.fill([seqs[i] for i in order])
        self.last_h2d_bytes = 4 * (4 * ctx.T + 3 * ctx.B + 1 + ctx.n_want)
        self.last_slots, self.last_passes = ctx.seq_slot, 1
        self.run = DecodeRun(self, ctx, list(slots), [int(t) for t in tokens], min(steps),
                             sampler, sampling, vocab_limit, history, order)
        return self.run

    def decode_steps(self, slots: Sequence[int], tokens: Sequence[int], n_steps: int, sampler,
                     sampling, vocab_limit: Optional[int] = None) -> torch.Tensor:
        """``n_steps`` steps of a decode run without looking at what was chosen in between.
        Returns the chosen tokens ``[n_steps, sequences]`` (int32, on the device); the last
        row is not fed. No stop token is looked at: the caller cuts the rows."""
        if n_steps <= 0:
            raise InferError("decode_steps: n_steps > 0")
        run = self.decode_run(slots, tokens, [n_steps] * len(slots), sampler, sampling,
                              vocab_limit, history=True)
        try:
            for _ in range(n_steps):
                run.launch()
        except BaseException:
            run.abandon()
            raise
        run.finish()
        return run.picks_on_device()[:n_steps]

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
