"""The plain implementation itself (no GPU): its record against the reference project's
fixtures, properties of its parts, and its sampler."""
import json
import math
import os

import numpy as np
import pytest

from tests.plain import qwen3_plain as plain

HERE = os.path.dirname(os.path.abspath(__file__))
# the reference project's tests/data/infer-ref folder: named by MORMOT_REFERENCE_FIXTURES, else
# looked for in a checkout of the reference project beside this repository (../reference)
REFERENCE_FIXTURES = os.environ.get("MORMOT_REFERENCE_FIXTURES") or os.path.join(
    os.path.dirname(os.path.dirname(HERE)), "reference", "tests", "data", "infer-ref")


def test_golden_record_against_the_reference_fixtures():
    """tests/golden/reference_fixtures.json was written by
    tests/golden/check_reference_fixtures.py: the plain implementation on the reference's
    tiny Qwen3 models against the transformers float32 states stored with them."""
    rec = json.load(open(os.path.join(HERE, "golden", "reference_fixtures.json")))
    assert set(rec["sets"]) == {"tiny-qwen3", "tiny-qwen3/untied", "tiny-qwen3-sliding"}
    for name, entry in rec["sets"].items():
        for case, r in entry["cases"].items():
            assert r["argmax_equal"], (name, case)
            assert r.get("greedy_equal", True), (name, case)
            assert max(r["max_abs_diff"].values()) < 5e-6, (name, case, r["max_abs_diff"])


@pytest.mark.skipif(not os.path.isdir(REFERENCE_FIXTURES),
                    reason="no checkout of the reference project beside this repository; set "
                           "MORMOT_REFERENCE_FIXTURES to its tests/data/infer-ref")
def test_plain_matches_the_reference_fixtures_now():
    import hashlib
    for name in ("tiny-qwen3", "tiny-qwen3/untied", "tiny-qwen3-sliding"):
        folder = os.path.join(REFERENCE_FIXTURES, name)
        config, weights = plain.read_model_folder(folder)
        manifest = json.load(open(os.path.join(folder, "manifest.json")))
        blob = open(os.path.join(folder, "tensors.bin"), "rb").read()
        assert hashlib.sha256(blob).hexdigest() == manifest["blob"]["sha256"]
        t = {e["name"]: e for e in manifest["tensors"]}
        cases = sorted({k.split(".")[0] for k in t})
        assert cases
        for case in cases:
            e = t[case + ".ids"]
            ids = np.frombuffer(blob[e["offset"]:][:e["bytes"]], np.int32)
            e = t[case + ".logits"]
            want = np.frombuffer(blob[e["offset"]:][:e["bytes"]], np.float32).reshape(e["shape"])
            got = plain.forward(config, weights, ids.tolist())
            assert np.abs(got - want).max() < 5e-6, (name, case)


def test_inverse_frequencies_round_as_the_reference():
    inv = plain.inverse_frequencies(1e6, 32)
    assert inv.dtype == np.float32 and inv[0] == 1.0
    for i in (1, 7, 15):
        e = np.float32(2 * i / 32)
        assert inv[i] == np.float32(1.0 / float(np.float32(math.exp(math.log(1e6) * float(e)))))
    cos, sin = plain.rotary_tables(inv, [0, 4095])
    assert cos[0].tolist() == [1.0] * 16 and sin[0].tolist() == [0.0] * 16
    angle = np.float32(inv[1] * np.float32(4095))            # the angle itself in float32
    assert cos[1, 1] == np.float32(math.cos(float(angle)))


def test_attention_window_and_groups():
    rng = np.random.default_rng(0)
    n, nh, nkv, hd = 12, 4, 2, 8
    q = rng.standard_normal((n, nh * hd)).astype(np.float32)
    k = rng.standard_normal((n, nkv * hd)).astype(np.float32)
    v = rng.standard_normal((n, nkv * hd)).astype(np.float32)
    full = plain.causal_attention(q, k, v, nh, nkv, hd)
    assert np.array_equal(plain.causal_attention(q, k, v, nh, nkv, hd, window=n), full)
    w5 = plain.causal_attention(q, k, v, nh, nkv, hd, window=5)
    assert np.array_equal(w5[:5], full[:5]) and not np.allclose(w5[5:], full[5:])
    # row r with window w sees exactly the keys r-w+1..r
    cut = plain.causal_attention(q[3:8], k[3:8], v[3:8], nh, nkv, hd)
    assert np.allclose(w5[7], cut[4], atol=1e-6)
    # the first token attends to itself only: its output is its value (head h -> KV head h//2)
    for h in range(nh):
        assert np.allclose(full[0, h * hd:(h + 1) * hd], v[0, (h // 2) * hd:(h // 2 + 1) * hd])
    # heads of one group differ only through q
    q2 = q.copy()
    q2[:, hd:2 * hd] = q[:, :hd]
    same = plain.causal_attention(q2, k, v, nh, nkv, hd)
    assert np.array_equal(same[:, :hd], same[:, hd:2 * hd])


def test_norm_swiglu_rope():
    x = np.array([[3.0, 4.0]], dtype=np.float32)
    y = plain.rms_norm(x, np.array([1.0, 2.0], dtype=np.float32), 0.0)
    assert np.allclose(y, [[3 / math.sqrt(12.5), 8 / math.sqrt(12.5)]], rtol=1e-6)
    g = np.array([0.0, 1.0, -2.0], dtype=np.float32)
    assert np.allclose(plain.swiglu(g, np.ones(3, np.float32)),
                       [0.0, 1 / (1 + math.exp(-1)), -2 / (1 + math.exp(2))], rtol=1e-6)
    cos, sin = np.zeros((1, 2), np.float32), np.ones((1, 2), np.float32)   # a quarter turn
    r = plain.rope(np.array([[1.0, 2.0, 3.0, 4.0]], np.float32), 1, 4, cos, sin)
    assert r.tolist() == [[-3.0, -4.0, 1.0, 2.0]]


def test_argmax_ties_and_nan():
    nan, inf = float("nan"), float("inf")
    assert plain.arg_max(np.array([1.0, 3.0, 3.0, 2.0], np.float32)) == 1
    assert plain.arg_max(np.array([nan, -inf, nan], np.float32)) == 1
    assert plain.arg_max(np.array([nan, nan], np.float32)) == 0
    assert plain.arg_max(np.array([-0.0, 0.0], np.float32)) == 0
    assert plain.arg_max(np.array([-5.0, nan, -1.0], np.float32)) == 2


def test_splitmix64_stream():
    s = plain.PlainSampler(temperature=1.0, seed=0)
    # splitmix64 from state 0: first outputs e220a8397b1dcdaf, 6e789e6aa1b965f4 (Vigna)
    assert int(s.next_double() * 2 ** 53) == 0xE220A8397B1DCDAF >> 11
    assert int(s.next_double() * 2 ** 53) == 0x6E789E6AA1B965F4 >> 11


def test_sampler_filters():
    logits = np.log(np.array([0.5, 0.2, 0.2, 0.05, 0.05], dtype=np.float64)).astype(np.float32)
    def draws(**kw):
        s = plain.PlainSampler(seed=3, **kw)
        return [s.next(logits) for _ in range(400)]
    assert set(draws(temperature=0.0)) == {0}
    d = draws(temperature=1.0)
    assert set(d) == {0, 1, 2, 3, 4} and 150 < d.count(0) < 250
    assert set(draws(temperature=1.0, top_k=1)) == {0}
    assert set(draws(temperature=1.0, top_k=2)) == {0, 1, 2}       # the tie with the 2nd stays
    assert set(draws(temperature=1.0, top_p=0.6)) == {0, 1}        # 0.5 + 0.2 reaches 0.6
    assert set(draws(temperature=1.0, min_p=0.3)) == {0, 1, 2}     # at least 0.3 * 0.5
    assert set(draws(temperature=1.0, top_k=3, top_p=0.75)) == {0, 1}   # 0.7/0.9 >= 0.75
    a, b = plain.PlainSampler(temperature=0.8, seed=5), plain.PlainSampler(temperature=0.8, seed=5)
    assert [a.next(logits) for _ in range(50)] == [b.next(logits) for _ in range(50)]
    with pytest.raises(ValueError):
        plain.PlainSampler(top_p=0.0)
    bad = np.array([float("nan"), 1.0, float("-inf"), 1.5], np.float32)
    assert set(plain.PlainSampler(temperature=1.0, seed=1).next(bad) for _ in range(20)) <= {1, 3}
