"""Generation through the entry points on a B200: greedy tokens equal to the plain
implementation's, seeded sampling that repeats, stop tokens, unequal prompts in batches that
follow one another, and the command line."""
import os
import subprocess
import sys

import numpy as np
import pytest

from mormot2_ai_b200 import LlmClient
from tests.conftest import ROOT

pytestmark = pytest.mark.gpu


def plain_greedy_with_margins(tiny, prompt, n):
    """Greedy tokens of the plain implementation and each step's top-1/top-2 margin."""
    ids, out, margins = list(prompt), [], []
    for _ in range(n):
        logits = tiny.reference(ids)[-1]
        order = np.argsort(-logits, kind="stable")
        out.append(int(order[0]))
        margins.append(float(logits[order[0]] - logits[order[1]]))
        ids.append(out[-1])
    return out, margins


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_through_the_entry_point(tiny, dtype):
    client = LlmClient(tiny.folder, dtype=dtype, max_batch=3, cache_tokens=1024)
    prompts = [tiny.tokens(n, seed=800 + n) for n in tiny.prompt_lens]
    got = client.generate(prompts, max_tokens=tiny.decode_steps, temperature=0.0, stop=[])
    for p, tokens in zip(prompts, got):
        want, margins = plain_greedy_with_margins(tiny, p, tiny.decode_steps)
        assert len(tokens) == tiny.decode_steps
        for i, (a, b) in enumerate(zip(tokens, want)):
            if a != b:
                # a different token is right only at a near tie of the plain logits
                assert dtype == "bfloat16" and margins[i] < 2e-2, (i, a, b, margins[i])
                break
    assert got[0] == client.greedy(prompts[0], tiny.decode_steps)
    assert all(client.engine.book.held_pages(g) == 0 for g in range(len(client.engine.plans)))


def test_stop_tokens_caps_and_batches(tiny_a_model):
    tiny = tiny_a_model
    client = LlmClient(tiny.folder, dtype="float32", max_batch=2, cache_tokens=512)
    prompts = [tiny.tokens(n, seed=900 + n) for n in (3, 9, 1, 20, 6)]
    free = client.generate(prompts, max_tokens=6, temperature=0.0, stop=[])
    assert [len(t) for t in free] == [6] * 5
    stop = free[1][2]
    outs = client.generate(prompts, max_tokens=6, temperature=0.0, stop=[stop], details=True)
    for o, f in zip(outs, free):
        if stop in f:
            assert o.tokens == f[:f.index(stop) + 1] and o.stopped     # the stop token is returned
        else:
            assert o.tokens == f and not o.stopped
    limit = tiny.config.max_position_embeddings
    long = client.generate([tiny.tokens(limit - 2, seed=1)], max_tokens=50, temperature=0.0, stop=[])
    assert len(long[0]) == 3                                            # limit - len + 1


def test_seeded_sampling_repeats_and_differs(tiny_b_model):
    tiny = tiny_b_model
    client = LlmClient(tiny.folder, dtype="float32", max_batch=4, cache_tokens=1024)
    prompts = [tiny.tokens(5, seed=s) for s in range(4)]
    kw = dict(max_tokens=12, temperature=1.5, stop=[])
    a = client.generate(prompts, seed=7, **kw)
    b = client.generate(prompts, seed=7, **kw)
    c = client.generate(prompts, seed=8, **kw)
    assert a == b and a != c
    d = client.generate(prompts, seed=7, top_k=4, top_p=0.9, **kw)
    assert d == client.generate(prompts, seed=7, top_k=4, top_p=0.9, **kw)
    # the same prompt in a batch and alone: sequence i draws from the stream of seed + i
    alone = client.generate([prompts[2]], seed=9, **kw)
    together = client.generate(prompts, seed=7, **kw)
    assert alone[0] == together[2]
    # the draws follow the plain sampler fed with the plain logits
    sampler = tiny.plain.PlainSampler(temperature=1.5, seed=9)
    ids, want = list(prompts[2]), []
    for _ in range(12):
        want.append(sampler.next(tiny.reference(ids)[-1]))
        ids.append(want[-1])
    assert alone[0] == want


def test_a_kernels_error_word_ends_generation_and_leaves_nothing_held(tiny_a_model):
    """A kernel whose bounded wait ran out writes a code into the runtime's error word. The
    failure is made on the host here (the code is written into the word, no kernel is made to
    wait): ``check`` and ``read_tokens`` raise and clear the word; in the generation loop the
    code arrives with a step's picks, the loop raises, and no slot, page or run stays open."""
    from mormot2_ai_b200 import KernelError
    from mormot2_ai_b200.engine.generate import EngineStepper, Request, generate
    from mormot2_ai_b200.sampling import Sampling
    tiny = tiny_a_model
    client = LlmClient(tiny.folder, dtype="bfloat16", max_batch=3, cache_tokens=1024)
    eng, rt = client.engine, client.engine.rt
    rt.error_word.fill_(2)
    with pytest.raises(KernelError, match="code 2"):
        rt.check()
    assert int(rt.error_word.item()) == 0
    rt.check()
    rt.error_word.fill_(9)
    with pytest.raises(KernelError, match="code 9"):
        rt.read_tokens(2)
    assert int(rt.error_word.item()) == 0
    prompts = [tiny.tokens(n, seed=950 + n) for n in (4, 70, 9)]
    good = client.generate(prompts, max_tokens=12, temperature=0.0, stop=[])

    class Faulty(EngineStepper):
        launches = 0

        def decode(self, members):
            run = super().decode(members)
            launch = run.launch

            def faulty_launch():
                launch()
                Faulty.launches += 1
                if Faulty.launches == 5:
                    rt.error_word.fill_(3)     # as a kernel of the fifth step would
            run.launch = faulty_launch
            return run

    with pytest.raises(KernelError, match="code 3"):
        generate(Faulty(eng, Sampling(), None, 3), [Request(p, 12) for p in prompts])
    assert eng.run is None and eng.book.slots.free == eng.max_slots
    assert all(eng.book.held_pages(g) == 0 for g in range(len(eng.plans)))
    assert int(rt.error_word.item()) == 0
    assert client.generate(prompts, max_tokens=12, temperature=0.0, stop=[]) == good


def test_command_line(tiny_a_model):
    tiny = tiny_a_model
    env = dict(os.environ)
    prompt = tiny.tokens(4, seed=1)
    p = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "llm-quickstart"), tiny.folder,
                        ",".join(map(str, prompt)), "f32", "--max-tokens", "5",
                        "--temperature", "0"], capture_output=True, text=True, timeout=600, env=env)
    assert p.returncode == 0, p.stderr[-2000:]
    got = [int(t) for t in p.stdout.strip().splitlines()[-1].split(",")]
    assert got == tiny.plain.greedy(tiny.plain_config, tiny.plain_weights, prompt, 5)
    p = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "llm-bench"), tiny.folder,
                        "20", "4", "bf16"], capture_output=True, text=True, timeout=600, env=env)
    assert p.returncode == 0, p.stderr[-2000:]
    assert "prefill: 20 tokens" in p.stdout and "decode: 3 tokens" in p.stdout
    assert "MiB, of which cache" in p.stdout and "kernel launches:" in p.stdout
    p = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "llm-bench"), tiny.folder,
                        "20", "4", "bf16", "--shares"], capture_output=True, text=True,
                       timeout=600, env=env)
    assert p.returncode == 0, p.stderr[-2000:]
    assert "products" in p.stdout and "attention" in p.stdout and "decode, mean of 4" in p.stdout
