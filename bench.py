"""Measures decoding and prefill of the Qwen3-8B shape with random weights on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

A step is one decode step of a batch of 8 sequences whose context reaches 4,096 at the end of
the timed steps. ``value`` is decoded tokens a second with the steps running back to back on
the device (token ids and positions move on in device memory); ``e2e`` is the same through
the generation loop of the Python entry point, host token ids in and out: the prompts are
copied in from pinned host memory, every step's picks are read back into pinned memory (with
the kernels' error word) and looked at for stops and caps; a step's input ids are the step
before's picks, which the engine keeps on the device, so in a steady batch no id travels back
(``h2d_bytes_per_step`` counts what was copied: the index arrays whenever a run of steps is
opened). Both go through ``Engine.decode_run``. One JSON line is printed.

Beside the headline: ``prefill`` (2,048 tokens), ``points`` (tokens/s of decode at batch 1
and 64, of prefills of 8,192 and 16,384 tokens, of the Qwen3-0.6B shape with 64 unequal
prompts, and of the Qwen3-32B shape) with ``points_detail`` (each point's ms, bytes or flops,
fraction of the measured peak and its own clock samples).
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

CONTEXT = 4096
BATCH = 8
PREFILL_TOKENS = 2048
# Untimed decode steps between a batch's prefill and its warm-up steps, on the device-timed
# and on the end-to-end path alike: the prefill of a whole batch holds the GPU at its power
# cap, and for some tens of milliseconds afterwards a decode step runs up to a quarter slower
# while the clocks come back (measured: 4.95 ms falling to 3.88 ms over 30 steps).
SETTLE = 40
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    out = dict(FALLBACK_PEAKS, source="fallback")
    if os.path.isfile(path):
        try:
            doc = json.load(open(path))
            out["hbm_gbs"] = float(doc["hbm_gbs"])
            out["bf16_tflops"] = float(doc["bf16_tflops"])
            out["source"] = "measured"
        except (ValueError, KeyError, TypeError):
            pass
    return out


class Clocks:
    """Samples nvidia-smi's SM clock and throttle reasons while a region runs."""
    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")
    NAMES = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]

    def __init__(self):
        self.samples, self.proc = [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}",
                 "--format=csv,noheader,nounits", "-lms", "200"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.samples.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
        sm = sorted(int(s[0]) for s in self.samples if s and s[0].isdigit())
        mx = [int(s[1]) for s in self.samples if len(s) > 1 and s[1].isdigit()]
        reasons = sorted({n for s in self.samples if len(s) >= 6
                          for n, v in zip(self.NAMES, s[2:6]) if v == "Active"})
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(sm)}


def model_config(layers):
    from mormot2_ai_b200 import Qwen3Config
    return Qwen3Config(vocab_size=151936, hidden_size=4096, num_hidden_layers=layers,
                       num_attention_heads=32, num_key_value_heads=8, head_dim=128,
                       intermediate_size=12288, max_position_embeddings=40960,
                       rms_norm_eps=1e-6, rope_theta=1e6, tie_word_embeddings=False)


def shape_config(name):
    """The other model shapes of the measurement (random weights, never loaded from disk)."""
    from mormot2_ai_b200 import Qwen3Config
    if name == "0.6B":
        return Qwen3Config(vocab_size=151936, hidden_size=1024, num_hidden_layers=28,
                           num_attention_heads=16, num_key_value_heads=8, head_dim=128,
                           intermediate_size=3072, max_position_embeddings=40960,
                           rms_norm_eps=1e-6, rope_theta=1e6, tie_word_embeddings=True)
    return Qwen3Config(vocab_size=151936, hidden_size=5120, num_hidden_layers=64,
                       num_attention_heads=64, num_key_value_heads=8, head_dim=128,
                       intermediate_size=25600, max_position_embeddings=40960,
                       rms_norm_eps=1e-6, rope_theta=1e6, tie_word_embeddings=False)


def step_bytes(cfg, batch, tokens_held, itemsize=2):
    """What a decode step has to read: every weight it uses once (the embedding table only
    through its looked-up rows) and the keys and values of the live sequences."""
    h, i, v = cfg.hidden_size, cfg.intermediate_size, cfg.vocab_size
    per_layer = ((cfg.q_width + 2 * cfg.kv_width) * h + h * cfg.q_width + 3 * h * i
                 + 2 * h + 2 * cfg.head_dim)
    weights = (cfg.num_hidden_layers * per_layer + h + v * h + batch * h) * itemsize
    # tokens_held: the summed lengths of the batch's sequences
    cache = tokens_held * cfg.num_hidden_layers * 2 * cfg.kv_width * itemsize
    return weights + cache


def prefill_flops(cfg, n, lens=None):
    """Of one prompt of n tokens, or of prompts of ``lens`` tokens in one step."""
    h, i, v = cfg.hidden_size, cfg.intermediate_size, cfg.vocab_size
    lens = [n] if lens is None else lens
    total = sum(lens)
    per_layer = 2 * total * ((cfg.q_width + 2 * cfg.kv_width) * h + h * cfg.q_width + 3 * h * i)
    attention = sum(4 * cfg.q_width * m * (m + 1) / 2 for m in lens)
    return cfg.num_hidden_layers * (per_layer + attention) + 2 * v * h * len(lens)


def timed_decode(torch, eng, sampler, sampling, lens, steps, warmup, rng_seed):
    """Prefills prompts of ``lens`` tokens, decodes ``warmup`` steps, then times ``steps``
    steps on the device. Returns the time (ms), the summed lengths of the sequences in the
    middle of the timed steps, and the launches of the timed steps."""
    from mormot2_ai_b200 import Entry
    from mormot2_ai_b200 import kernels as K
    gen = torch.Generator().manual_seed(rng_seed)
    slots = [eng.open() for _ in lens]
    for s in slots:
        sampler.start(s, s)
    # prompts of different content, prefilled a few sequences at a time
    firsts, b0 = [], 0
    while b0 < len(lens):
        b1, tokens = b0, 0
        while b1 < len(lens) and (b1 == b0 or tokens + lens[b1] <= eng.max_step_tokens):
            tokens += lens[b1]
            b1 += 1
        prompts = [torch.randint(0, eng.vocab_size, (n,), generator=gen).tolist()
                   for n in lens[b0:b1]]
        logits = eng.step([Entry(s, p) for s, p in zip(slots[b0:b1], prompts)])
        firsts += sampler.pick(logits, eng.last_slots, sampling).tolist()
        b0 = b1
    hist = eng.decode_steps(slots, firsts, SETTLE + warmup, sampler, sampling)
    nxt = hist[-1].tolist()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    before = K.Launches.count
    e0.record()
    eng.decode_steps(slots, nxt, steps, sampler, sampling)
    e1.record()
    torch.cuda.synchronize()
    launches = K.Launches.count - before
    ms = e0.elapsed_time(e1)
    eng.rt.check()
    for s in slots:
        eng.close(s)
    return ms, sum(lens) + len(lens) * (SETTLE + warmup + steps / 2.0), launches


def timed_e2e(torch, eng, batch, steps, warmup, rng_seed):
    """The same decoding through the entry point's loop: the generation loop with a stepper
    that times the last `steps` decode steps on the device (events around them)."""
    from mormot2_ai_b200.engine.generate import EngineStepper, Request, generate
    from mormot2_ai_b200.sampling import Sampling

    class TimedStepper(EngineStepper):
        """Times the decode steps after the warm-up ones: an event before the launch of the
        first of them, another after the host has read the last one's tokens (the requests'
        caps end the run there, so nothing else is queued in between)."""

        def __init__(self, *a, **k):
            super().__init__(*a, **k)
            self.launches = self.reads = 0
            self.e0 = torch.cuda.Event(enable_timing=True)
            self.e1 = torch.cuda.Event(enable_timing=True)

        def decode(self, members):
            run = super().decode(members)
            launch, read = run.launch, run.read

            def timed_launch():
                if self.launches == SETTLE + warmup:
                    self.h2d_bytes = self.d2h_bytes = 0
                    self.e0.record()
                launch()
                self.launches += 1

            def timed_read():
                got = read()
                self.reads += 1
                if self.reads == SETTLE + warmup + steps:
                    self.e1.record()
                return got

            run.launch, run.read = timed_launch, timed_read
            return run

    prompt_len = CONTEXT - steps - warmup - SETTLE
    gen = torch.Generator().manual_seed(rng_seed)
    prompts = [torch.randint(0, eng.vocab_size, (prompt_len,), generator=gen).tolist()
               for _ in range(batch)]
    stepper = TimedStepper(eng, Sampling(), None, batch)
    generate(stepper, [Request(p, SETTLE + warmup + steps + 1, set(), i)
                       for i, p in enumerate(prompts)])
    torch.cuda.synchronize()
    ms = stepper.e0.elapsed_time(stepper.e1)
    return ms, stepper.h2d_bytes / steps, stepper.d2h_bytes / steps


def timed_prefill(torch, eng, lens, repeats=3):
    """One step over prompts of ``lens`` tokens (best of ``repeats`` after a warm-up run)."""
    from mormot2_ai_b200 import Entry
    gen = torch.Generator().manual_seed(7)
    best = None
    for r in range(repeats + 1):
        prompts = [torch.randint(0, eng.vocab_size, (n,), generator=gen).tolist() for n in lens]
        slots = [eng.open() for _ in lens]
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        eng.step([Entry(s, p) for s, p in zip(slots, prompts)])
        e1.record()
        torch.cuda.synchronize()
        for s in slots:
            eng.close(s)
        if r > 0:          # the first run warms up
            ms = e0.elapsed_time(e1)
            best = ms if best is None else min(best, ms)
    eng.rt.check()
    return best


class Points:
    """The extra measurements: tokens/s under ``points``, the rest under ``points_detail``."""

    def __init__(self, pk):
        self.pk, self.values, self.detail = pk, {}, {}

    def decode(self, name, cfg, ms, steps, batch, tokens_held, clocks):
        per_step = ms / steps
        gbs = step_bytes(cfg, batch, tokens_held) / (per_step / 1e3) / 1e9
        self.values[name] = round(batch * steps / (ms / 1e3), 1)
        self.detail[name] = {"ms_per_step": round(per_step, 4), "steps": steps, "batch": batch,
                             "gb_per_step": round(step_bytes(cfg, batch, tokens_held) / 1e9, 3),
                             "gbs": round(gbs, 1), "frac_hbm": round(gbs / self.pk["hbm_gbs"], 4),
                             "clocks": clocks}

    def prefill(self, name, cfg, ms, lens, clocks, passes=1):
        flops = prefill_flops(cfg, 0, lens)
        self.values[name] = round(sum(lens) / (ms / 1e3), 1)
        self.detail[name] = {"ms": round(ms, 3), "tokens": sum(lens), "prompts": len(lens),
                             "tflop": round(flops / 1e12, 2), "passes": passes,
                             "frac_bf16": round(flops / (ms / 1e3) / (self.pk["bf16_tflops"] * 1e12), 4),
                             "clocks": clocks}


def clocked(fn, *args, **kw):
    clocks = Clocks()
    clocks.start()
    try:
        out = fn(*args, **kw)
    finally:
        record = clocks.stop()
    return out, record


def other_shapes(torch, a, pts):
    """The Qwen3-0.6B shape with 64 prompts of unequal lengths (one prefill step, then 256
    decode steps), the 8B shape decoding at a context of 32,768 (batch 1 and 8), and the
    Qwen3-32B shape (prefill of 2,048 tokens, decode at batch 1 and 8 toward a context of
    4,096). Each engine is made, measured and dropped."""
    from mormot2_ai_b200 import Engine
    from mormot2_ai_b200.sampling import DeviceSampler, Sampling
    greedy = Sampling()
    # -- 0.6B, ragged
    cfg = shape_config("0.6B")
    lens = torch.randint(16, 2049, (64,), generator=torch.Generator().manual_seed(3)).tolist()
    steps, warm = 256, max(a.warmup, 3)
    room = sum(-(-(n + steps + warm + SETTLE + 1) // 64) * 64 for n in lens)
    eng = Engine.from_random(cfg, seed=3, std=0.02, max_tokens=room, max_context=2048 + 512,
                             max_slots=64, prefill_chunk=2048, max_step_tokens=sum(lens))
    sampler = DeviceSampler(eng.rt.device, eng.max_slots, eng.vocab_size)
    ms, rec = clocked(timed_prefill, torch, eng, lens)
    pts.prefill("ragged_0p6b_prefill", cfg, ms, lens, rec)
    (ms, held, _), rec = clocked(timed_decode, torch, eng, sampler, greedy, lens, steps, warm, 30)
    pts.decode("ragged_0p6b_decode", cfg, ms, steps, 64, held, rec)
    pts.detail["ragged_0p6b_decode"]["prompt_lens"] = f"uniform 16..2048, seed 3, sum {sum(lens)}"
    del eng, sampler
    torch.cuda.empty_cache()
    # -- the 8B shape at a context of 32,768: the cache, not the weights, is most of a step
    cfg = model_config(36)
    long_context = 32768
    eng = Engine.from_random(cfg, seed=2, std=0.02, max_tokens=8 * long_context,
                             max_context=long_context, max_slots=8, prefill_chunk=4096,
                             max_step_tokens=8192)
    sampler = DeviceSampler(eng.rt.device, eng.max_slots, eng.vocab_size)
    steps = min(a.steps, 32)
    for b in (1, 8):
        lens = [long_context - steps - warm - SETTLE] * b
        (ms, held, _), rec = clocked(timed_decode, torch, eng, sampler, greedy, lens, steps, warm,
                                     50 + b)
        pts.decode(f"decode_b{b}_ctx{long_context}", cfg, ms, steps, b, held, rec)
    del eng, sampler
    torch.cuda.empty_cache()
    # -- 32B
    cfg = shape_config("32B")
    eng = Engine.from_random(cfg, seed=4, std=0.02, max_tokens=8 * CONTEXT, max_context=CONTEXT,
                             max_slots=8, prefill_chunk=2048, max_step_tokens=8192)
    sampler = DeviceSampler(eng.rt.device, eng.max_slots, eng.vocab_size)
    ms, rec = clocked(timed_prefill, torch, eng, [PREFILL_TOKENS], repeats=2)
    pts.prefill("qwen3_32b_prefill", cfg, ms, [PREFILL_TOKENS], rec)
    steps = min(a.steps, 64)
    for b in (1, 8):
        lens = [CONTEXT - steps - warm - SETTLE] * b
        (ms, held, _), rec = clocked(timed_decode, torch, eng, sampler, greedy, lens, steps, warm,
                                     40 + b)
        pts.decode(f"qwen3_32b_decode_b{b}", cfg, ms, steps, b, held, rec)
    del eng, sampler
    torch.cuda.empty_cache()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=36, help="fewer layers than the 36 of the shape "
                    "(named in config); the layer sizes stay")
    ap.add_argument("--skip-points", action="store_true", help="only the headline: no prefill, "
                    "no other batch sizes, no other shapes")
    ap.add_argument("--skip-shapes", action="store_true", help="not the 0.6B and 32B shapes")
    ap.add_argument("--batches", default="1,64", help="batch sizes of the extra decode points")
    ap.add_argument("--long-prefills", default="8192,16384",
                    help="token counts of the long prefill points (one sequence each)")
    ap.add_argument("--only-prefill", type=int, nargs="?", const=PREFILL_TOKENS, default=0,
                    help="only a prefill of this many tokens (for profiles; prints a short line)")
    a = ap.parse_args()
    if a.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "the reference is Free Pascal / Delphi source without a Python package; "
                          "no Pascal compiler and no mORMot 2 sources are in this image"}))
        return 0
    if a.gpus != 1:
        print(f"bench.py measures one GPU: --gpus {a.gpus} is not supported "
              "(this library has no multi-GPU path)")
        return 2
    a.warmup = max(a.warmup, 3)
    if a.steps < 1 or a.steps + a.warmup + SETTLE > CONTEXT - 64:
        print(f"bench.py: --steps + --warmup must leave a prompt of at least 64 tokens in the "
              f"context of {CONTEXT}")
        return 2
    import torch
    from mormot2_ai_b200 import Engine
    from mormot2_ai_b200.sampling import DeviceSampler, Sampling

    pk = peaks()
    cfg = model_config(a.layers)
    longs = [] if (a.skip_points or a.only_prefill) else [int(v) for v in a.long_prefills.split(",") if v]
    max_batch = BATCH if (a.skip_points or a.only_prefill) else 64
    context = max([CONTEXT, a.only_prefill] + longs)
    eng = Engine.from_random(cfg, seed=2, std=0.02, max_tokens=max(max_batch * CONTEXT, context),
                             max_context=context, max_slots=max_batch, prefill_chunk=4096,
                             max_step_tokens=8192)
    sampler = DeviceSampler(eng.rt.device, eng.max_slots, eng.vocab_size)
    greedy = Sampling()
    if a.only_prefill:
        pms = timed_prefill(torch, eng, [a.only_prefill], repeats=1)
        print(json.dumps({"prefill_ms": round(pms, 3), "tokens": a.only_prefill,
                          "layers": a.layers}))
        return 0
    pts = Points(pk)
    # the prefills first, as the bursts that they are in service (and as the burst peak is
    # measured); the decode runs after them hold the GPU at its power cap for seconds
    pms = prefill_clocks = None
    if not a.skip_points:
        pms, prefill_clocks = clocked(timed_prefill, torch, eng, [PREFILL_TOKENS])
        for n in longs:
            ms, rec = clocked(timed_prefill, torch, eng, [n], repeats=2)
            pts.prefill(f"prefill_{n}", cfg, ms, [n], rec, passes=-(-n // eng.prefill_chunk))
    lens = [CONTEXT - a.steps - a.warmup - SETTLE] * BATCH
    (ms, held, launches), clock_record = clocked(timed_decode, torch, eng, sampler, greedy, lens,
                                                 a.steps, a.warmup, 1)
    value = BATCH * a.steps / (ms / 1e3)
    achieved = step_bytes(cfg, BATCH, held) / (ms / a.steps / 1e3) / 1e9
    e2e_ms, h2d, d2h = timed_e2e(torch, eng, BATCH, a.steps, a.warmup, 2)
    out = {
        "metric": "Qwen3-8B decode tokens/s at batch 8, context 4096 (random BF16 weights)",
        "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": a.steps,
        "warmup": a.warmup, "ms_per_step": round(ms / a.steps, 4), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "impl": "ours",
        "config": {
            "model": "Qwen3-8B shape, random weights N(0,0.02) seed 2", "global_batch": BATCH,
            "seq_len": CONTEXT, "parallelism": "none (1 GPU)", "layers": a.layers,
            "layers_of_shape": 36, "hidden": cfg.hidden_size, "heads": cfg.num_attention_heads,
            "kv_heads": cfg.num_key_value_heads, "head_dim": cfg.head_dim,
            "intermediate": cfg.intermediate_size, "vocab": cfg.vocab_size,
            "rope_theta": cfg.rope_theta, "rms_norm_eps": cfg.rms_norm_eps, "tied_head": False,
            "prompt_tokens": CONTEXT - a.steps - a.warmup - SETTLE, "settle_steps": SETTLE,
            "prefill_tokens": PREFILL_TOKENS,
            "l2": "a step reads its weights (>15 GB), far larger than L2",
            "peaks": pk["source"],
        },
        "e2e": {"value": round(BATCH * a.steps / (e2e_ms / 1e3), 1), "unit": "tokens/s",
                "h2d_bytes_per_step": round(h2d, 1), "d2h_bytes_per_step": round(d2h, 1),
                "inputs": "a step's ids are the step before's picks and stay on the device; "
                          "prompts and index arrays come from pinned host memory"},
        "gpu_launches": launches,
        "clocks": clock_record,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"],
                     "unit": "GB/s", "frac": round(achieved / pk["hbm_gbs"], 4)},
    }
    if not a.skip_points:
        flops = prefill_flops(cfg, PREFILL_TOKENS)
        out["prefill"] = {"value": round(PREFILL_TOKENS / (pms / 1e3), 1), "tokens": PREFILL_TOKENS,
                          "ms": round(pms, 3),
                          "frac": round(flops / (pms / 1e3) / (pk["bf16_tflops"] * 1e12), 4),
                          "timing": "best of 3 after 1 warm-up, before the decode runs",
                          "clocks": prefill_clocks}
        for b in [int(v) for v in a.batches.split(',') if v]:
            steps = min(a.steps, 128)
            lens = [CONTEXT - steps - a.warmup - SETTLE] * b
            (bms, held, _), rec = clocked(timed_decode, torch, eng, sampler, greedy, lens, steps,
                                          a.warmup, 10 + b)
            pts.decode(f"decode_b{b}", cfg, bms, steps, b, held, rec)
        # the same batches (and the headline's) at shorter contexts: the weights' share of a step
        # grows as the cache's shrinks
        for ctx in (512, 2304):
            for b in sorted(set([BATCH] + [int(v) for v in a.batches.split(',') if v])):
                steps = min(a.steps, 64)
                lens = [ctx - steps - a.warmup - SETTLE] * b
                (bms, held, _), rec = clocked(timed_decode, torch, eng, sampler, greedy, lens,
                                              steps, a.warmup, 100 + b + ctx)
                pts.decode(f"decode_b{b}_ctx{ctx}", cfg, bms, steps, b, held, rec)
        e1_ms, _, _ = timed_e2e(torch, eng, 1, min(a.steps, 128), a.warmup, 3)
        pts.values["e2e_b1"] = round(min(a.steps, 128) / (e1_ms / 1e3), 1)
        del eng, sampler
        torch.cuda.empty_cache()
        if not a.skip_shapes and a.layers == 36:
            other_shapes(torch, a, pts)
        out["points"] = pts.values
        out["points_detail"] = pts.detail
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
