"""The command line, in the manner of the reference's demos: positional arguments first
(``llm-bench [model folder] [prompt tokens=200] [new tokens=32] [...]``,
``demos/infer/llm-bench.lpr:8-19``; ``llm-quickstart <model folder> [question] [...]``,
``demos/llm/llm-quickstart.lpr:5-7``), the sampler's settings under the reference's names
(``temperature``, ``top_k``, ``top_p``, ``min_p``, ``seed``; ``sampler.pas:47-59``). Prompts
and answers are token ids: tokenizers are not part of this library.

    python -m mormot2_ai_b200 llm-bench <folder> [prompt tokens=200] [new tokens=32] [bf16|f32]
    python -m mormot2_ai_b200 llm-quickstart <folder> [ids "5,17,3;9,2"] [bf16|f32] [options]
    python -m mormot2_ai_b200 random-model <out folder> <config.json> [seed=0]
"""
from __future__ import annotations

import argparse
import json
import sys
import time
from typing import List

import torch


def _dtype(word: str) -> str:
    table = {"bf16": "bfloat16", "bfloat16": "bfloat16", "f32": "float32", "fp32": "float32",
             "float32": "float32"}
    if word not in table:
        raise SystemExit(f"weights: bf16 or f32, not {word}")
    return table[word]


def llm_bench(argv: List[str]) -> int:
    """Feeds a prompt of a given length in one pass (prefill), then generates tokens one by
    one through the cache (decode), greedy, and reports tokens/s of both."""
    ap = argparse.ArgumentParser(prog="llm-bench", description=llm_bench.__doc__)
    ap.add_argument("folder")
    ap.add_argument("prompt_tokens", nargs="?", type=int, default=200)
    ap.add_argument("new_tokens", nargs="?", type=int, default=32)
    ap.add_argument("weights", nargs="?", default="bf16", help="bf16 (default) | f32")
    ap.add_argument("--batch", type=int, default=1, help="sequences decoded together")
    ap.add_argument("--shares", action="store_true",
                    help="also time the kernels of one prefill and of the decode steps by class "
                         "(products, attention, norms, rotary, ...), run one by one")
    a = ap.parse_args(argv)
    if a.prompt_tokens < 1 or a.new_tokens < 1:
        print("prompt tokens and new tokens: at least 1 each")
        return 1
    from .engine.engine import Engine, Entry
    from .sampling.device import DeviceSampler
    from .sampling.settings import Sampling
    t0 = time.time()
    total = a.batch * (a.prompt_tokens + a.new_tokens + 64)
    eng = Engine.from_folder(a.folder, dtype=_dtype(a.weights), max_tokens=total,
                             max_slots=a.batch)
    c = eng.config
    st = eng.stats()
    print(f"loaded in {int((time.time() - t0) * 1000)} ms: {c.num_hidden_layers} layers, "
          f"hidden {c.hidden_size}, vocab {c.vocab_size}, weights {a.weights}; on the device "
          f"{st['device_bytes'] / 2**20:.0f} MiB, of which cache {st['cache_bytes'] / 2**20:.0f} MiB "
          f"({st['slots']} slots, {sum(st['pages'])} pages of 64 positions)")
    gen = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, c.vocab_size, (a.prompt_tokens,), generator=gen).tolist()
               for _ in range(a.batch)]
    sampler = DeviceSampler(eng.rt.device, eng.max_slots, eng.vocab_size)
    slots = [eng.open() for _ in prompts]
    greedy = Sampling()
    torch.cuda.synchronize()
    t0 = time.time()
    logits = eng.step([Entry(s, p) for s, p in zip(slots, prompts)])
    ids = sampler.pick(logits, eng.last_slots, greedy).tolist()
    t1 = time.time()
    if a.new_tokens > 1:
        # the picks are fed back on the device; the host reads them when the last is chosen
        eng.decode_steps(slots, ids, a.new_tokens - 1, sampler, greedy).cpu()
    t2 = time.time()
    eng.rt.check()
    print(f"prefill: {a.batch * a.prompt_tokens} tokens in {int((t1 - t0) * 1000)} ms = "
          f"{a.batch * a.prompt_tokens / (t1 - t0):.0f} tokens/s")
    if a.new_tokens > 1:
        print(f"decode: {a.batch * (a.new_tokens - 1)} tokens in {int((t2 - t1) * 1000)} ms = "
              f"{a.batch * (a.new_tokens - 1) / (t2 - t1):.1f} tokens/s")
    st = eng.stats()
    print(f"passes of the model: {st['passes']}, kernel launches: {st['kernel_launches']}, "
          f"decode graphs: {st['decode_graphs']}, pages held: {sum(st['pages_held'])}")
    if a.shares:
        for s in slots:
            eng.truncate(s, 0)
        logits, shares, total = eng.timed_step([Entry(s, p) for s, p in zip(slots, prompts)])
        _print_shares("prefill", shares, total)
        ids = sampler.pick(logits, eng.last_slots, greedy).tolist()
        sums, whole = {}, 0.0
        n = min(a.new_tokens, 16)
        for _ in range(n):
            logits, shares, total = eng.timed_step([Entry(s, [t]) for s, t in zip(slots, ids)])
            ids = sampler.pick(logits, eng.last_slots, greedy).tolist()
            whole += total
            for k, v in shares.items():
                sums[k] = sums.get(k, 0.0) + v
        _print_shares(f"decode, mean of {n} steps", {k: v / n for k, v in sums.items()}, whole / n)
    return 0


def _print_shares(what: str, shares: dict, total: float) -> None:
    """Where the time of a step goes, by class of kernel, largest first."""
    in_kernels = sum(shares.values())
    print(f"{what}: {total * 1000:.0f} us, {in_kernels * 1000:.0f} us in kernels run one by one")
    for name, ms in sorted(shares.items(), key=lambda kv: -kv[1]):
        print(f"  {name:<10} {ms * 1000:9.1f} us {100 * ms / max(in_kernels, 1e-9):5.1f} %")


def llm_quickstart(argv: List[str]) -> int:
    """Loads a model folder and continues the given prompts (token ids)."""
    ap = argparse.ArgumentParser(prog="llm-quickstart", description=llm_quickstart.__doc__)
    ap.add_argument("folder")
    ap.add_argument("ids", nargs="?", default="1,2,3",
                    help="prompts as token ids: \"5,17,3;9,2\" (';' between prompts)")
    ap.add_argument("weights", nargs="?", default="bf16", help="bf16 (default) | f32")
    ap.add_argument("--max-tokens", type=int, default=32, help="new tokens per prompt at most")
    ap.add_argument("--max-context", type=int, default=None)
    ap.add_argument("--temperature", type=float, default=-1.0,
                    help=">= 0 overrides generation_config.json; 0 is greedy")
    ap.add_argument("--top-k", type=int, default=None)
    ap.add_argument("--top-p", type=float, default=None)
    ap.add_argument("--min-p", type=float, default=None)
    ap.add_argument("--seed", type=int, default=None)
    ap.add_argument("--stop", type=int, action="append", default=None,
                    help="a stop token id (repeatable); default: the model's eos_token_id")
    a = ap.parse_args(argv)
    from .client import LlmClient
    prompts = [[int(t) for t in part.split(",") if t.strip()] for part in a.ids.split(";")]
    client = LlmClient(a.folder, dtype=_dtype(a.weights), max_context=a.max_context,
                       max_batch=max(1, len(prompts)))
    out = client.generate(prompts, max_tokens=a.max_tokens, temperature=a.temperature,
                          top_k=a.top_k, top_p=a.top_p, min_p=a.min_p, seed=a.seed, stop=a.stop)
    for tokens in out:
        print(",".join(str(t) for t in tokens))
    return 0


def random_model(argv: List[str]) -> int:
    """Writes a model folder (config.json, model.safetensors) with random weights."""
    ap = argparse.ArgumentParser(prog="random-model", description=random_model.__doc__)
    ap.add_argument("out")
    ap.add_argument("config", help="a config.json of a registered architecture")
    ap.add_argument("seed", nargs="?", type=int, default=0)
    ap.add_argument("--std", type=float, default=0.02)
    ap.add_argument("--norm-std", type=float, default=0.1)
    ap.add_argument("--dtype", default="bf16")
    a = ap.parse_args(argv)
    from .config.registry import family_of, read_config_json
    from .weights.random_init import write_random_model
    doc = read_config_json(a.config)
    config = family_of(doc, a.config).from_dict(doc, a.config)
    dtype = torch.bfloat16 if _dtype(a.dtype) == "bfloat16" else torch.float32
    write_random_model(a.out, config, a.seed, a.std, a.norm_std, dtype)
    print(f"wrote {a.out}")
    return 0


COMMANDS = {"llm-bench": llm_bench, "llm-quickstart": llm_quickstart, "random-model": random_model}


def main(argv: List[str] = None) -> int:
    argv = sys.argv[1:] if argv is None else argv
    if not argv or argv[0] not in COMMANDS:
        print(__doc__)
        return 0 if argv and argv[0] in ("-h", "--help") else 1
    return COMMANDS[argv[0]](argv[1:])


if __name__ == "__main__":
    sys.exit(main())
