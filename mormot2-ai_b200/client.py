"""The Python entry point: a model folder in, token ids out — the role of the reference's
``TNativeLlmClient`` (``llm.native.pas:560-662``) without text (tokenizers and chat templates
are not part of this library: prompts and answers are token ids).

    client = LlmClient("model-folder", dtype="bfloat16")
    answers = client.generate([[5, 17, 3], [9, 2]], max_tokens=32, temperature=0.7, seed=1)

Names follow the reference: ``sampling`` (its ``Sampling`` defaults, read from
generation_config.json as ``InferSamplingFromConfig`` does), ``max_tokens`` (``MaxTokens``),
``max_context`` (``MaxContext``); per call ``temperature`` >= 0 overrides the default and
``top_p``, ``top_k``, ``min_p``, ``seed`` are the request's extras (``NativeSampling``,
``llm.native.pas:2063-2128``: a random seed when none is given).
"""
from __future__ import annotations

import os
import random
from dataclasses import replace
from typing import Iterable, List, Optional, Sequence

from .config.registry import read_config_json
from .engine.engine import Engine
from .engine.generate import EngineStepper, Outcome, Request, generate
from .errors import InferError
from .sampling.settings import Sampling, sampling_from_config


def _stop_ids(folder: str) -> List[int]:
    """eos_token_id of generation_config.json, else of config.json (an id or a list)."""
    for name in ("generation_config.json", "config.json"):
        path = os.path.join(folder, name)
        if os.path.isfile(path):
            eos = read_config_json(path).get("eos_token_id")
            if isinstance(eos, int) and not isinstance(eos, bool):
                return [eos]
            if isinstance(eos, list) and eos:
                return [int(e) for e in eos]
    return []


class LlmClient:
    def __init__(self, folder: Optional[str] = None, dtype: str = "bfloat16",
                 device: str = "cuda:0", max_context: Optional[int] = None,
                 max_tokens: int = 256, max_batch: int = 64, cache_tokens: Optional[int] = None,
                 engine: Optional[Engine] = None, **engine_options):
        """``folder``: config.json and model.safetensors (or an index and its files).
        ``max_tokens``: the default cap of new tokens per request. ``max_context``: the most
        positions of one sequence (default: the model's). ``cache_tokens``: the tokens the
        cache holds over all live sequences (default: ``max_batch`` sequences of
        ``max_context``, at most 1 Mi)."""
        if engine is None:
            if folder is None:
                raise InferError("LlmClient: a model folder or an engine")
            from .config.registry import config_of_folder
            limit = config_of_folder(folder).max_position_embeddings
            ctx = min(max_context or limit, limit)
            total = cache_tokens or min(max_batch * ctx, 1 << 20)
            engine = Engine.from_folder(folder, dtype=dtype, device=device, max_tokens=total,
                                        max_context=ctx, max_slots=max_batch, **engine_options)
        self.engine = engine
        self.folder = folder
        self.sampling = sampling_from_config(folder) if folder else Sampling()
        self.stop = _stop_ids(folder) if folder else []
        self.max_tokens = max_tokens
        self.max_batch = min(max_batch, engine.max_slots)
        self.vocab_limit: Optional[int] = None   # ids at or above it are never drawn

    @property
    def max_context(self) -> int:
        return self.engine.max_context

    def generate(self, prompts: Sequence[Sequence[int]], max_tokens: Optional[int] = None,
                 temperature: float = -1.0, top_k: Optional[int] = None,
                 top_p: Optional[float] = None, min_p: Optional[float] = None,
                 seed: Optional[int] = None, stop: Optional[Iterable[int]] = None,
                 details: bool = False):
        """New token ids of every prompt (the stop token included when one ended it). Sequence
        i draws from the stream of ``seed + i``. ``details``: ``Outcome`` objects instead."""
        s = self.sampling
        s = replace(s, temperature=temperature if temperature >= 0 else s.temperature,
                    top_k=s.top_k if top_k is None else top_k,
                    top_p=s.top_p if top_p is None else top_p,
                    min_p=s.min_p if min_p is None else min_p)
        base = random.getrandbits(63) if seed is None else seed
        stops = set(self.stop if stop is None else stop)
        cap = self.max_tokens if max_tokens is None else max_tokens
        requests = [Request(list(p), cap, stops, base + i) for i, p in enumerate(prompts)]
        self.stepper = EngineStepper(self.engine, s, self.vocab_limit, self.max_batch)
        outcomes = generate(self.stepper, requests)
        return outcomes if details else [o.tokens for o in outcomes]

    def greedy(self, prompt: Sequence[int], max_new: int, stop: Iterable[int] = ()) -> List[int]:
        """Greedy decoding of one prompt (``TDecoderModel.Greedy``, ``decoder.pas:3390-3426``)."""
        return self.generate([prompt], max_tokens=max_new, temperature=0.0, stop=stop)[0]
