"""Decoding on the device (``Engine.decode_run``, the path of the generation loop and of
``bench.py``): many steps across page boundaries at batch 1, 8 and 64 with unequal lengths,
greedy and seeded temperature sampling, every pick compared with the plain implementation;
steps read a step late; sequences that keep fewer steps than were launched; and the same
kernels at the sizes of a real model, batch 64, against the engine's own 32-bit path."""
import copy

import numpy as np
import pytest
import torch

from mormot2_ai_b200 import CacheError, Engine, Entry, InferError, Sampling
from mormot2_ai_b200.sampling import DeviceSampler
from tests.conftest import close

pytestmark = pytest.mark.gpu
DTYPES = ["float32", "bfloat16"]
STEPS = 72
# how near a tie must be for another pick than the plain implementation's to be right: the
# top-2 margin of the plain logits (greedy), the distance of the draw from the edge of the
# picked token's share of the distribution (sampling)
NEAR = {"float32": 1e-4, "bfloat16": 2e-2}


def prompts_of(tiny, batch):
    limit = tiny.config.max_position_embeddings
    rng = np.random.default_rng(17 + batch)
    # unequal lengths on both sides of the page boundary at 64, the longest as long as fits
    lens = rng.integers(1, max(2, min(70, limit - STEPS - 1)), batch).tolist()
    lens[0] = limit - STEPS - 1
    return [tiny.tokens(n, seed=3000 + 7 * i + batch) for i, n in enumerate(lens)]


def check_picks(tiny, dtype, prompt, picks, temperature, seed):
    """``picks``: the first from the prompt's last logits, then one per decode step. The
    plain implementation is fed the engine's own tokens, so every pick is judged alone."""
    ids = list(prompt) + picks[:-1]
    logits = tiny.reference(ids)[len(prompt) - 1:]
    assert len(logits) == len(picks)
    sampler = tiny.plain.PlainSampler(temperature=temperature, seed=seed)
    for i, (row, got) in enumerate(zip(logits, picks)):
        if temperature <= 0:
            order = np.argsort(-row, kind="stable")
            if got != int(order[0]):
                assert row[order[0]] - row[got] < NEAR[dtype], (i, got, int(order[0]))
            continue
        u = copy.copy(sampler).next_double()
        want = sampler.next(row)
        if got != want:
            p = np.exp((row.astype(np.float64) - row.max()) / temperature)
            cdf = np.cumsum(p / p.sum())
            lo = cdf[got - 1] if got else 0.0
            assert lo - NEAR[dtype] <= u <= cdf[got] + NEAR[dtype], (i, got, want, u, lo, cdf[got])


@pytest.mark.parametrize("temperature", [0.0, 0.9], ids=["greedy", "sampled"])
@pytest.mark.parametrize("batch", [1, 8, 64])
@pytest.mark.parametrize("dtype", DTYPES)
def test_decode_run_against_the_plain_implementation(tiny, dtype, batch, temperature):
    eng = Engine.from_folder(tiny.folder, dtype=dtype, max_tokens=64 * 4 * batch + 512,
                             max_slots=batch)
    sampler = DeviceSampler(eng.rt.device, eng.max_slots, eng.vocab_size)
    sampling = Sampling(temperature=temperature)
    prompts = prompts_of(tiny, batch)
    slots = [eng.open() for _ in prompts]
    for i, s in enumerate(slots):
        sampler.start(s, 100 + i)
    logits = eng.step([Entry(s, p) for s, p in zip(slots, prompts)])
    firsts = sampler.pick(logits, eng.last_slots, sampling).tolist()
    run = eng.decode_run(slots, firsts, [STEPS] * batch, sampler, sampling)
    with pytest.raises(InferError, match="decode run is open"):
        eng.step([Entry(slots[0], [1])])
    rows = []
    for i in range(STEPS):                       # two steps queued before the first is read
        run.launch()
        if i:
            rows.append(run.read())
    rows.append(run.read())
    with pytest.raises(InferError, match="opened for"):
        run.launch()
    run.finish()
    eng.rt.check()
    assert [eng.length(s) for s in slots] == [len(p) + STEPS for p in prompts]
    for b, p in enumerate(prompts):
        picks = [firsts[b]] + [r[b] for r in rows]
        check_picks(tiny, dtype, p, picks, temperature, 100 + b)
        assert eng.ids[slots[b]] == list(p) + picks[:-1]
    # the cache that the run left serves an ordinary step: the next logits are the plain ones
    b = batch // 2
    ids = list(prompts[b]) + [firsts[b]] + [r[b] for r in rows]
    if len(ids) <= tiny.config.max_position_embeddings:
        out = eng.step([Entry(slots[b], [ids[-1]])]).cpu().numpy()
        ok, err = close(out, tiny.reference(ids)[-1:], dtype)
        assert ok, err
    for s in slots:
        eng.close(s)
    assert all(eng.book.held_pages(g) == 0 for g in range(len(eng.plans)))


@pytest.mark.parametrize("dtype", DTYPES)
def test_decode_steps_equals_the_run_read_step_by_step(tiny_b_model, dtype):
    """``decode_steps`` (no pick is looked at in between; the picks come back as one device
    tensor) gives the picks of a run that is read after every step."""
    tiny = tiny_b_model
    eng = Engine.from_folder(tiny.folder, dtype=dtype, max_tokens=2048, max_slots=8)
    sampler = DeviceSampler(eng.rt.device, eng.max_slots, eng.vocab_size)
    sampling = Sampling(temperature=1.1)
    prompts = [tiny.tokens(n, seed=n) for n in (60, 3, 64, 31, 1)]
    got = []
    for mode in ("steps", "run"):
        slots = [eng.open() for _ in prompts]
        for i, s in enumerate(slots):
            sampler.start(s, 7 + i)
        logits = eng.step([Entry(s, p) for s, p in zip(slots, prompts)])
        firsts = sampler.pick(logits, eng.last_slots, sampling).tolist()
        if mode == "steps":
            got.append(eng.decode_steps(slots, firsts, 40, sampler, sampling).tolist())
            # picks that the host never read are unknown to prefix reuse
            assert eng.ids[slots[1]] == list(prompts[1]) + [firsts[1]] + [-1] * 39
        else:
            run = eng.decode_run(slots, firsts, [40] * len(slots), sampler, sampling)
            rows = []
            for _ in range(40):
                run.launch()
                rows.append(run.read())
            run.finish()
            got.append(rows)
        for s in slots:
            eng.close(s)
    assert got[0] == got[1]


def test_a_sequence_keeps_fewer_steps_than_were_launched(tiny_a_model):
    """What the host learns a step late: a sequence that ended is fed once more. Its length
    is committed without that step, and the sequence goes on from there as if the step had
    never run (the key it wrote lies beyond the length and is written over)."""
    tiny = tiny_a_model
    eng = Engine.from_folder(tiny.folder, dtype="float32", max_tokens=1024, max_slots=3)
    sampler = DeviceSampler(eng.rt.device, eng.max_slots, eng.vocab_size)
    greedy = Sampling()
    prompts = [tiny.tokens(n, seed=40 + n) for n in (62, 9, 30)]
    slots = [eng.open() for _ in prompts]
    logits = eng.step([Entry(s, p) for s, p in zip(slots, prompts)])
    firsts = sampler.pick(logits, eng.last_slots, greedy).tolist()
    run = eng.decode_run(slots, firsts, [10, 10, 10], sampler, greedy)
    rows = []
    for _ in range(6):
        run.launch()
        rows.append(run.read())
    with pytest.raises(InferError, match="finish"):
        run.finish([7, 6, 6])
    run.finish([6, 2, 0])                        # the second keeps two steps, the third none
    assert [eng.length(s) for s in slots] == [62 + 6, 9 + 2, 30]
    for b, keep in enumerate([6, 2, 0]):
        fed = [firsts[b]] + [r[b] for r in rows]
        ids = list(prompts[b]) + fed[:keep] + [5]
        out = eng.step([Entry(slots[b], [5])]).cpu().numpy()
        ok, err = close(out, tiny.reference(ids)[-1:], "float32")
        assert ok, (b, err)
    # a run reserves its pages when it is opened, all or nothing
    with pytest.raises(CacheError):
        eng.decode_run(slots, [1, 1, 1], [200, 200, 200], sampler, greedy)
    assert eng.run is None
    with pytest.raises(InferError, match="distinct slots"):
        eng.decode_run([slots[0], slots[0]], [1, 1], [2, 2], sampler, greedy)


@pytest.mark.parametrize("batch", [1, 2])
@pytest.mark.parametrize("name", ["C", "D"])
def test_a_long_sequence_is_dealt_out_over_more_ctas(name, batch, tmp_path_factory, monkeypatch):
    """One or two sequences that grow past the length from which the decode attention deals a
    sequence out over about one CTA per SM (through scratch memory and a second kernel, in the
    layer without a window): the run changes to the graph of its own in mid-run, and every
    pick stays the plain implementation's. The length is lowered to what a tiny model holds."""
    from mormot2_ai_b200 import kernels as K
    from mormot2_ai_b200.engine import batch as batch_module
    from tests.conftest import TinyModel
    tiny = TinyModel(name, str(tmp_path_factory.mktemp("long_" + name)))
    monkeypatch.setattr(batch_module, "LONG_CONTEXT", 150)
    calls = []
    plain_entry = K.attention_decode
    monkeypatch.setattr(K, "attention_decode",
                        lambda *a, **k: (calls.append(a[10]), plain_entry(*a, **k))[1])
    eng = Engine.from_folder(tiny.folder, dtype="bfloat16", max_tokens=1024, max_slots=2)
    sampler = DeviceSampler(eng.rt.device, eng.max_slots, eng.vocab_size)
    greedy = Sampling()
    prompts = [tiny.tokens(n, seed=70 + n) for n in (131, 90)[:batch]]
    slots = [eng.open() for _ in prompts]
    logits = eng.step([Entry(s, p) for s, p in zip(slots, prompts)])
    firsts = sampler.pick(logits, eng.last_slots, greedy).tolist()
    steps = 60
    run = eng.decode_run(slots, firsts, [steps] * batch, sampler, greedy)
    rows = []
    for _ in range(steps):
        run.launch()
        rows.append(run.read())
    run.finish()
    eng.rt.check()
    assert (batch, batch, False) in eng.graphs and (batch, batch, True) in eng.graphs
    assert calls and min(calls) > 8, calls          # more splits than a cluster holds
    for b, p in enumerate(prompts):
        check_picks(tiny, "bfloat16", p, [firsts[b]] + [r[b] for r in rows], 0.0, 0)
    # and an ordinary step of a long sequence: the logits are the plain ones
    ids = list(prompts[0]) + [firsts[0]] + [r[0] for r in rows]
    out = eng.step([Entry(slots[0], [ids[-1]])]).cpu().numpy()
    ok, err = close(out, tiny.reference(ids)[-1:], "bfloat16")
    assert ok, err


def test_batch_64_at_the_sizes_of_a_real_model():
    """Two layers with the sizes of a real model, 64 sequences of unequal lengths between 20
    and 700 tokens, decoded on the device: the decode products at 64 tokens, the cluster
    decode attention with sequences that end on different pages, the graph of 64 rows. The
    tensor-core path is fed the picks of the engine's own 32-bit path (so both see the same
    tokens) and its logits are compared with that path's at every step."""
    from mormot2_ai_b200 import DecoderModel, Qwen3Config, Runtime
    from mormot2_ai_b200.weights.random_init import random_tensors
    cfg = Qwen3Config.from_dict({
        "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "vocab_size": 151936,
        "hidden_size": 4096, "intermediate_size": 12288, "num_hidden_layers": 2,
        "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 128,
        "max_position_embeddings": 8192, "rms_norm_eps": 1e-6, "rope_theta": 1000000.0,
        "tie_word_embeddings": False, "hidden_act": "silu", "attention_bias": False})
    names = DecoderModel(cfg.to_model_spec()).tensors()
    weights = random_tensors(names, 6, 0.03, 0.1, torch.bfloat16, "cuda:0")
    kw = dict(max_tokens=64 * 768, max_context=768, max_slots=64, prefill_chunk=768,
              max_step_tokens=16384)
    fast = Engine(cfg, weights, Runtime(torch.bfloat16), **kw)
    slow = Engine(cfg, weights, Runtime(torch.float32), **kw)
    g = torch.Generator().manual_seed(4)
    lens = torch.randint(20, 700, (64,), generator=g).tolist()
    lens[3], lens[40] = 63, 64                      # the first decoded token opens a page
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in lens]
    sf, ss = [fast.open() for _ in prompts], [slow.open() for _ in prompts]
    for b0 in range(0, 64, 16):
        part = slice(b0, b0 + 16)
        a = fast.step([Entry(s, p) for s, p in zip(sf[part], prompts[part])])
        b = slow.step([Entry(s, p) for s, p in zip(ss[part], prompts[part])])
        ok, err = close(a.cpu().numpy(), b.cpu().numpy(), "bfloat16")
        assert ok, ("prompts", b0, err)
        tokens = b.argmax(dim=1).tolist() if b0 == 0 else tokens + b.argmax(dim=1).tolist()
    worst = 0.0
    for step in range(4):
        a = fast.step([Entry(s, [t]) for s, t in zip(sf, tokens)])
        b = slow.step([Entry(s, [t]) for s, t in zip(ss, tokens)])
        assert float(b.abs().max()) > 0.5
        for i in range(64):                    # every sequence's row in the common measure
            ok, err = close(a[i].cpu().numpy(), b[i].cpu().numpy(), "bfloat16")
            assert ok, (step, i, err)
            worst = max(worst, err)
        tokens = b.argmax(dim=1).tolist()
    # and on the device: the run's greedy picks are the 32-bit path's, or near ties of it
    sampler = DeviceSampler(fast.rt.device, 64, cfg.vocab_size)
    run = fast.decode_run(sf, tokens, [3] * 64, sampler, Sampling())
    for step in range(3):
        run.launch()
        picks = run.read()
        b = slow.step([Entry(s, [t]) for s, t in zip(ss, tokens)])
        top = b.topk(2, dim=1)
        for i, (p, ids, vals) in enumerate(zip(picks, top.indices.tolist(), top.values.tolist())):
            if p != ids[0]:
                assert float(b[i, ids[0]] - b[i, p]) < 6e-2 * float(b[i].std()), (step, i)
        tokens = picks
    run.finish()
    fast.rt.check()
    slow.rt.check()
