"""Measures decoding and prefill of the Qwen3-8B shape with random weights on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

A step is one decode step of a batch of 8 sequences whose context reaches 4,096 at the end of
the timed steps. ``value`` is decoded tokens a second with the steps running back to back on
the device (token ids and positions move on in device memory); ``e2e`` is the same through
the Python entry point's loop: every step copies its token ids from pinned host memory to the
device and reads the chosen tokens back. One JSON line is printed.
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


def step_bytes(cfg, batch, context, itemsize=2):
    """What a decode step has to read: every weight it uses once (the embedding table only
    through its looked-up rows) and the keys and values of the live sequences."""
    h, i, v = cfg.hidden_size, cfg.intermediate_size, cfg.vocab_size
    per_layer = ((cfg.q_width + 2 * cfg.kv_width) * h + h * cfg.q_width + 3 * h * i
                 + 2 * h + 2 * cfg.head_dim)
    weights = (cfg.num_hidden_layers * per_layer + h + v * h + batch * h) * itemsize
    cache = batch * context * cfg.num_hidden_layers * 2 * cfg.kv_width * itemsize
    return weights + cache


def prefill_flops(cfg, n):
    h, i, v = cfg.hidden_size, cfg.intermediate_size, cfg.vocab_size
    per_layer = 2 * n * ((cfg.q_width + 2 * cfg.kv_width) * h + h * cfg.q_width + 3 * h * i)
    attention = 4 * cfg.q_width * n * (n + 1) / 2
    return cfg.num_hidden_layers * (per_layer + attention) + 2 * v * h


def timed_decode(torch, eng, sampler, sampling, batch, steps, warmup, rng_seed):
    """Prefills `batch` prompts so that warm-up and timed steps end at CONTEXT; returns the
    device time of the timed steps (ms) and the mean context during them."""
    from mormot2_ai_b200 import Entry
    from mormot2_ai_b200 import kernels as K
    prompt_len = CONTEXT - steps - warmup
    gen = torch.Generator().manual_seed(rng_seed)
    slots = [eng.open() for _ in range(batch)]
    for s in slots:
        sampler.start(s, s)
    # prompts of different content; prefilled a few sequences at a time
    firsts = []
    for b0 in range(0, batch, 4):
        part = slots[b0:b0 + 4]
        prompts = [torch.randint(0, eng.vocab_size, (prompt_len,), generator=gen).tolist()
                   for _ in part]
        logits = eng.step([Entry(s, p) for s, p in zip(part, prompts)])
        firsts += sampler.pick(logits, eng.last_slots, sampling).tolist()
    hist = eng.decode_steps(slots, firsts, warmup, sampler, sampling)
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
    return ms, CONTEXT - steps / 2.0, launches


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
            self.wall = [0.0, 0.0]

        def decode(self, members):
            run = super().decode(members)
            launch, read = run.launch, run.read

            def timed_launch():
                if self.launches == warmup:
                    self.h2d_bytes = self.d2h_bytes = 0
                    self.e0.record()
                    self.wall[0] = time.perf_counter()
                launch()
                self.launches += 1

            def timed_read():
                got = read()
                self.reads += 1
                if self.reads == warmup + steps:
                    self.e1.record()
                    self.wall[1] = time.perf_counter()
                return got

            run.launch, run.read = timed_launch, timed_read
            return run

    prompt_len = CONTEXT - steps - warmup
    gen = torch.Generator().manual_seed(rng_seed)
    prompts = [torch.randint(0, eng.vocab_size, (prompt_len,), generator=gen).tolist()
               for _ in range(batch)]
    stepper = TimedStepper(eng, Sampling(), None, batch)
    generate(stepper, [Request(p, warmup + steps + 1, set(), i) for i, p in enumerate(prompts)])
    torch.cuda.synchronize()
    ms = stepper.e0.elapsed_time(stepper.e1)
    wall_ms = (stepper.wall[1] - stepper.wall[0]) * 1e3
    return ms, stepper.h2d_bytes / steps, stepper.d2h_bytes / steps, wall_ms


def timed_prefill(torch, eng, tokens, repeats=3):
    from mormot2_ai_b200 import Entry
    gen = torch.Generator().manual_seed(7)
    best = None
    for r in range(repeats + 1):
        ids = torch.randint(0, eng.vocab_size, (tokens,), generator=gen).tolist()
        slot = eng.open()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        eng.step([Entry(slot, ids)])
        e1.record()
        torch.cuda.synchronize()
        eng.close(slot)
        if r > 0:          # the first run warms up
            ms = e0.elapsed_time(e1)
            best = ms if best is None else min(best, ms)
    eng.rt.check()
    return best


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=36, help="fewer layers than the 36 of the shape "
                    "(named in config); the layer sizes stay")
    ap.add_argument("--skip-points", action="store_true", help="no batch 1 / 64 / prefill runs")
    ap.add_argument("--batches", default="1,64", help="batch sizes of the extra decode points")
    ap.add_argument("--only-prefill", action="store_true",
                    help="only the 2,048-token prefill (for profiles; prints its own short line)")
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
    if a.steps < 1 or a.steps + a.warmup > CONTEXT - 64:
        print(f"bench.py: --steps + --warmup must leave a prompt of at least 64 tokens in the "
              f"context of {CONTEXT}")
        return 2
    import torch
    from mormot2_ai_b200 import Engine
    from mormot2_ai_b200.sampling import DeviceSampler, Sampling

    pk = peaks()
    cfg = model_config(a.layers)
    max_batch = BATCH if (a.skip_points or a.only_prefill) else 64
    eng = Engine.from_random(cfg, seed=2, std=0.02, max_tokens=max_batch * CONTEXT,
                             max_context=CONTEXT, max_slots=max_batch, prefill_chunk=2048,
                             max_step_tokens=8192)
    sampler = DeviceSampler(eng.rt.device, eng.max_slots, eng.vocab_size)
    greedy = Sampling()
    if a.only_prefill:
        pms = timed_prefill(torch, eng, PREFILL_TOKENS, repeats=1)
        print(json.dumps({"prefill_ms": round(pms, 3), "layers": a.layers}))
        return 0
    # the prefill first, as the burst that it is in service (and as the burst peak is measured);
    # the decode runs after it hold the GPU at its power cap for seconds
    pms = None if a.skip_points else timed_prefill(torch, eng, PREFILL_TOKENS)
    clocks = Clocks()
    clocks.start()
    ms, mean_ctx, launches = timed_decode(torch, eng, sampler, greedy, BATCH, a.steps, a.warmup, 1)
    clock_record = clocks.stop()
    value = BATCH * a.steps / (ms / 1e3)
    achieved = step_bytes(cfg, BATCH, mean_ctx) / (ms / a.steps / 1e3) / 1e9
    e2e_ms, h2d, d2h, e2e_wall = timed_e2e(torch, eng, BATCH, a.steps, a.warmup, 2)
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
            "prompt_tokens": CONTEXT - a.steps - a.warmup, "prefill_tokens": PREFILL_TOKENS,
            "l2": "a step reads its weights (>15 GB), far larger than L2",
            "peaks": pk["source"],
            "prefill_timing": "best of 3 after 1 warm-up, before the decode runs",
        },
        "e2e": {"value": round(BATCH * a.steps / (e2e_ms / 1e3), 1), "unit": "tokens/s",
                "h2d_bytes_per_step": round(h2d, 1), "d2h_bytes_per_step": round(d2h, 1)},
        "gpu_launches": launches,
        "clocks": clock_record,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"],
                     "unit": "GB/s", "frac": round(achieved / pk["hbm_gbs"], 4)},
    }
    if not a.skip_points:
        flops = prefill_flops(cfg, PREFILL_TOKENS)
        out["prefill"] = {"value": round(PREFILL_TOKENS / (pms / 1e3), 1), "tokens": PREFILL_TOKENS,
                          "ms": round(pms, 3),
                          "frac": round(flops / (pms / 1e3) / (pk["bf16_tflops"] * 1e12), 4)}
        points = {}
        for b in [int(v) for v in a.batches.split(',') if v]:
            steps = min(a.steps, 128)
            bms, _, _ = timed_decode(torch, eng, sampler, greedy, b, steps, a.warmup, 10 + b)
            points[f"decode_b{b}"] = round(b * steps / (bms / 1e3), 1)
        out["points"] = points
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
