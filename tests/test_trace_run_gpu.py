"""bin/trace_run as a user runs it: the same requests replayed whole, with the last 32 tokens
decoded one by one, and in batches of unequal lengths (with fewer pages than all requests need
together, so that slots and pages are used again), in float32 and in bfloat16, each compared
with the plain implementation."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest

from tests.conftest import ROOT, close

pytestmark = pytest.mark.gpu
TRACE_RUN = os.path.join(ROOT, "bin", "trace_run")


def replay(model, dtype, steps, out_dir, max_tokens, more=()):
    text = "".join(json.dumps(s) + "\n" for s in steps)
    p = subprocess.run([sys.executable, TRACE_RUN, "--model", model, "--dtype", dtype,
                        "--out", str(out_dir), "--max-tokens", str(max_tokens)] + list(more),
                       input=text, capture_output=True, text=True, timeout=900)
    assert p.returncode == 0, p.stderr[-3000:]
    done = [l for l in p.stdout.splitlines() if l.startswith("done ")]
    assert done == [f"done {s['step']}" for s in steps]
    return p


def logits_of(out_dir, step, vocab):
    path = os.path.join(str(out_dir), f"{step}.f32")
    return np.fromfile(path, dtype="<f4").reshape(-1, vocab)


def requests_of(tiny):
    limit = tiny.config.max_position_embeddings
    lens = [40, 33, limit, 70, 35, limit - 20]
    return {f"r{i}": tiny.tokens(n, seed=700 + i) for i, n in enumerate(lens)}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_whole_and_tail_by_one(tiny, dtype, tmp_path):
    reqs = requests_of(tiny)
    vocab = tiny.config.vocab_size
    steps, expect, n = [], {}, 0
    for rid, ids in reqs.items():                       # whole: every position wanted
        steps.append({"step": n, "entries": [{"id": rid, "tokens": ids,
                                              "want": list(range(len(ids)))}], "end": [rid]})
        expect[n] = [(rid, list(range(len(ids))))]
        n += 1
    for rid, ids in reqs.items():                       # the last 32 tokens one by one
        head = len(ids) - 32
        steps.append({"step": n, "entries": [{"id": rid + "t", "tokens": ids[:head],
                                              "want": [head - 1]}], "end": []})
        expect[n] = [(rid, [head - 1])]
        n += 1
        for t in range(head, len(ids)):
            steps.append({"step": n, "entries": [{"id": rid + "t", "tokens": [ids[t]],
                                                  "want": [0]}],
                          "end": [rid + "t"] if t == len(ids) - 1 else []})
            expect[n] = [(rid, [t])]
            n += 1
    limit = tiny.config.max_position_embeddings
    replay(tiny.folder, dtype, steps, tmp_path, max_tokens=limit)   # one request at a time
    refs = {rid: tiny.reference(ids) for rid, ids in reqs.items()}
    for step, wanted in expect.items():
        got = logits_of(tmp_path, step, vocab)
        want = np.concatenate([refs[rid][places] for rid, places in wanted])
        ok, err = close(got, want, dtype)
        assert ok, f"step {step} {wanted[0][0]}: relative error {err:.3g}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_unequal_batches(tiny, dtype, tmp_path):
    reqs = requests_of(tiny)
    vocab = tiny.config.vocab_size
    names = list(reqs)
    batches = [names[0:3], names[3:5], names[5:6]]
    decode = 9
    steps, expect, n = [], {}, 0
    for batch in batches:
        cut = {rid: len(reqs[rid]) - min(decode, 3 + 2 * names.index(rid)) for rid in batch}
        entries = [{"id": rid, "tokens": reqs[rid][:cut[rid]], "want": [0, cut[rid] - 1]}
                   for rid in batch]
        at = dict(cut)
        ended = [rid for rid in batch if at[rid] >= len(reqs[rid])]
        steps.append({"step": n, "entries": entries, "end": ended})
        expect[n] = [(rid, [0, cut[rid] - 1]) for rid in batch]
        n += 1
        live = [rid for rid in batch if rid not in ended]
        while live:
            entries = [{"id": rid, "tokens": [reqs[rid][at[rid]]], "want": [0]} for rid in live]
            expect[n] = [(rid, [at[rid]]) for rid in live]
            for rid in live:
                at[rid] += 1
            ended = [rid for rid in live if at[rid] >= len(reqs[rid])]
            steps.append({"step": n, "entries": entries, "end": ended})
            live = [rid for rid in live if rid not in ended]      # shorter requests end earlier
            n += 1
    most = max(sum(-(-len(reqs[rid]) // 64) * 64 for rid in batch) for batch in batches)
    replay(tiny.folder, dtype, steps, tmp_path, max_tokens=most)  # pages must be used again
    refs = {rid: tiny.reference(ids) for rid, ids in reqs.items()}
    for step, wanted in expect.items():
        got = logits_of(tmp_path, step, vocab)
        want = np.concatenate([refs[rid][places] for rid, places in wanted])
        ok, err = close(got, want, dtype)
        assert ok, f"step {step} {wanted}: relative error {err:.3g}"


def test_steps_without_wants_write_nothing(tiny_a_model, tmp_path):
    tiny = tiny_a_model
    ids = tiny.tokens(20, seed=9)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": ids[:10], "want": []}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": ids[10:], "want": [9]}], "end": ["a"]},
             {"step": 2, "entries": [], "end": []}]
    replay(tiny.folder, "float32", steps, tmp_path, max_tokens=64, more=["--manifest"])
    assert not os.path.exists(os.path.join(str(tmp_path), "0.f32"))
    got = logits_of(tmp_path, 1, tiny.config.vocab_size)
    ok, err = close(got, tiny.reference(ids)[-1:], "float32")
    assert ok, err
    # the same logits in the reference project's fixture format, read as its loader reads it
    import hashlib
    manifest = json.load(open(os.path.join(str(tmp_path), "manifest.json")))
    blob = open(os.path.join(str(tmp_path), manifest["blob"]["file"]), "rb").read()
    assert hashlib.sha256(blob).hexdigest() == manifest["blob"]["sha256"]
    assert len(blob) == manifest["blob"]["bytes"]
    (t,) = manifest["tensors"]
    assert t["name"] == "step1.logits" and t["dtype"] == "f32"
    assert t["shape"] == [1, tiny.config.vocab_size] and t["bytes"] == 4 * tiny.config.vocab_size
    part = blob[t["offset"]:t["offset"] + t["bytes"]]
    assert hashlib.sha256(part).hexdigest() == t["sha256"]
    assert np.array_equal(np.frombuffer(part, "<f4").reshape(t["shape"]), got)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_truncate_steps(tiny_b_model, dtype, tmp_path):
    """A request is cut back to a prefix and goes on with other tokens, beside a request that
    is left alone: the logits are those of the new sequence as a whole."""
    tiny = tiny_b_model
    a, b = tiny.tokens(80, seed=31), tiny.tokens(50, seed=32)
    other = tiny.tokens(12, seed=33)
    steps = [
        {"step": 0, "entries": [{"id": "a", "tokens": a, "want": [79]},
                                {"id": "b", "tokens": b, "want": [49]}], "end": []},
        {"step": 1, "truncate": [{"id": "a", "len": 17}],
         "entries": [{"id": "a", "tokens": other[:1], "want": [0]},
                     {"id": "b", "tokens": [9], "want": [0]}], "end": ["b"]},
        {"step": 2, "entries": [{"id": "a", "tokens": other[1:], "want": [0, 10]}], "end": ["a"]}]
    replay(tiny.folder, dtype, steps, tmp_path, max_tokens=256)
    vocab = tiny.config.vocab_size
    new = a[:17] + other
    ref_new, ref_b = tiny.reference(new), tiny.reference(b + [9])
    for step, want in ((1, np.stack([ref_new[17], ref_b[50]])), (2, ref_new[[18, 28]])):
        ok, err = close(logits_of(tmp_path, step, vocab), want, dtype)
        assert ok, f"step {step}: relative error {err:.3g}"
