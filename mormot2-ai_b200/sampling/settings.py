"""How the next token is chosen: the reference's ``TInferSampling`` (``sampler.pas:47-59``)
with its ranges (``:208-220``), its greedy default (``:160-164``) and the defaults of a
Hugging Face generation_config.json (``:167-203``)."""
from __future__ import annotations

import json
import math
import os
from dataclasses import dataclass, replace

from ..errors import InferError


@dataclass(frozen=True)
class Sampling:
    """``temperature`` <= 0: greedy, else the logits are divided by it; ``top_k`` > 0: only the
    k highest logits (and those tied with the k-th) stay; ``top_p`` < 1: only the most probable
    tokens reaching that share of the mass top-k kept; ``min_p`` > 0: only tokens at least that
    share as probable as the best; ``seed``: of the splitmix64 stream, one draw per token."""
    temperature: float = 0.0
    top_k: int = 0
    top_p: float = 1.0
    min_p: float = 0.0
    seed: int = 0

    def __post_init__(self):
        vals = (self.temperature, self.top_p, self.min_p)
        if (any(isinstance(v, bool) or not isinstance(v, (int, float)) for v in vals)
                or any(math.isnan(v) or math.isinf(v) for v in vals)
                or isinstance(self.top_k, bool) or not isinstance(self.top_k, int)
                or self.top_k < 0 or self.top_p <= 0 or self.top_p > 1
                or self.min_p < 0 or self.min_p >= 1):
            raise InferError(f"sampling: temperature {self.temperature}, top_k {self.top_k}, "
                             f"top_p {self.top_p}, min_p {self.min_p}")

    @property
    def greedy(self) -> bool:
        # a temperature this close to 0 is greedy (sampler.pas:305-312)
        return self.temperature < 1e-30

    @property
    def filtered(self) -> bool:
        return self.top_k > 0 or self.top_p < 1 or self.min_p > 0

    def with_seed(self, seed: int) -> "Sampling":
        return replace(self, seed=seed)


def sampling_from_config(path: str) -> Sampling:
    """The defaults of a generation_config.json: greedy when the file is missing or says
    ``do_sample`` false; else ``temperature`` 1, ``top_k`` 50, ``top_p`` 1, ``min_p`` 0 unless
    given; the seed stays 0 for the caller to set."""
    if os.path.isdir(path):
        path = os.path.join(path, "generation_config.json")
    if not os.path.isfile(path):
        return Sampling()
    try:
        with open(path, "r", encoding="utf-8") as f:
            doc = json.load(f)
    except (OSError, ValueError) as e:
        raise InferError(f"{path} is no JSON object: {e}") from None
    if not isinstance(doc, dict):
        raise InferError(f"{path} is no JSON object")
    if not doc.get("do_sample"):
        return Sampling()

    def num(name: str, default: float) -> float:
        v = doc.get(name)
        if v is None:
            return default
        if isinstance(v, bool) or not isinstance(v, (int, float)) or math.isnan(v) or math.isinf(v):
            raise InferError(f"{name} is no number in {path}")
        return float(v)

    k = num("top_k", 50)
    if k < 0 or k > 2 ** 31 - 1 or k != int(k):
        raise InferError(f"top_k {k} in {path}")
    return Sampling(temperature=num("temperature", 1.0), top_k=int(k), top_p=num("top_p", 1.0),
                    min_p=num("min_p", 0.0))
