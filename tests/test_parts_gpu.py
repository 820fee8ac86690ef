"""Each part alone against the plain implementation's function of the same name, and the
generality of putting parts together: a toy mixer with state of its own that is registered,
built and stepped without a change to the library's files; an order of layers that names a
layer twice; a layer that reads another layer's cache; a toy feed-forward with routing and a toy
position encoding, registered from here as well."""
import math

import numpy as np
import pytest
import torch

from mormot2_ai_b200 import (CacheError, ConfigError, DecoderModel, Engine, Entry, LayerSpec, ModelSpec,
                             PartSpec, Qwen3Config, Run, Runtime)
from mormot2_ai_b200.parts.block import settle
from mormot2_ai_b200.parts import (FEED_FORWARDS, MIXERS, NORMS, POSITIONS, Part, StateNeed,
                                   TensorNeed, register_mixer)
from mormot2_ai_b200.weights import random_tensors
from tests.conftest import close, tiny_b
from tests.gpu_helpers import DEV, make_line, make_step
from tests.plain import qwen3_plain as plain

pytestmark = pytest.mark.gpu
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def part_weights(part, dtype, seed=0):
    w = random_tensors(part.tensors(), seed, std=0.05, norm_std=0.1, dtype=torch.bfloat16)
    dev = {k: v.to(DT[dtype]).to(DEV) for k, v in w.items()}
    ref = {k: v.float().numpy() for k, v in w.items()}
    return dev, ref


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_norm_part(dtype):
    rt = Runtime(DT[dtype])
    part = NORMS.build(PartSpec("rmsnorm", {"name": "n.weight", "size": 200, "eps": 1e-5}), "p.")
    assert [t.name for t in part.tensors()] == ["p.n.weight"]
    dev, ref = part_weights(part, dtype)
    part.bind(dev, rt)
    x = torch.randn(6, 200, generator=torch.Generator().manual_seed(0))
    got = part.forward(x.to(DEV))
    ok, err = close(got.float().cpu(), plain.rms_norm(x.numpy(), ref["p.n.weight"], 1e-5), dtype)
    assert ok, err


def test_position_part():
    rt = Runtime(torch.float32)
    for theta, rot in ((1e4, 16), (1e6, 128), (5e5, 40)):
        part = POSITIONS.build(PartSpec("rope_half", {"theta": theta, "rot_dim": rot}))
        part.bind({}, rt)
        inv, rot_dim = part.frequencies()
        assert rot_dim == rot
        assert np.array_equal(inv.cpu().numpy(), plain.inverse_frequencies(theta, rot))
    assert POSITIONS.build(PartSpec("none")).frequencies() == (None, 0)
    with pytest.raises(ConfigError):
        POSITIONS.build(PartSpec("rope_half", {"theta": 1e4, "rot_dim": 7}))
    with pytest.raises(ConfigError, match="alibi"):
        POSITIONS.build(PartSpec("alibi"))


def attention_spec(hidden, nh, nkv, hd, window, head_norm=True):
    names = {"q": "q.weight", "k": "k.weight", "v": "v.weight", "o": "o.weight"}
    if head_norm:
        names.update({"q_norm": "qn.weight", "k_norm": "kn.weight"})
    return PartSpec("gqa_attention", {
        "hidden_size": hidden, "heads": nh, "kv_heads": nkv, "head_dim": hd,
        "head_norm_eps": 1e-6 if head_norm else None, "position": "rope", "window": window,
        "scale": 1 / math.sqrt(hd), "names": names})


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("hidden,nh,nkv,hd,window", [(96, 6, 2, 16, 0), (72, 3, 1, 48, 7),
                                                     (128, 4, 4, 64, 0)])
def test_attention_mixer_alone(dtype, hidden, nh, nkv, hd, window):
    """The mixer over two sequences (a prompt, then one more token each) equals the plain
    attention block without its norm and residual."""
    rt = Runtime(DT[dtype])
    rope = POSITIONS.build(PartSpec("rope_half", {"theta": 1e4, "rot_dim": hd}))
    rope.bind({}, rt)
    mixer = MIXERS.build(attention_spec(hidden, nh, nkv, hd, window), "l.", positions={"rope": rope})
    need = mixer.cache_need()
    assert (need.kv_heads, need.head_dim, need.window) == (nkv, hd, window)
    dev, ref = part_weights(mixer, dtype, seed=hd)
    mixer.bind(dev, rt)
    line = make_line(3, 128, nkv, hd, DT[dtype], window=window)
    g = torch.Generator().manual_seed(1)
    lens = [20, 9]
    hs = [(torch.randn(n + 1, hidden, generator=g)).to(DT[dtype]) for n in lens]
    cfg = {"num_attention_heads": nh, "num_key_value_heads": nkv, "head_dim": hd,
           "rms_norm_eps": 1e-6}

    def reference(h):
        n = h.shape[0]
        inv = plain.inverse_frequencies(1e4, hd)
        cos, sin = plain.rotary_tables(inv, range(n))
        x = h.float().numpy()
        q = plain.linear(x, ref["l.q.weight"])
        k = plain.linear(x, ref["l.k.weight"])
        v = plain.linear(x, ref["l.v.weight"])
        q = plain.rms_norm(q.reshape(n * nh, hd), ref["l.qn.weight"], 1e-6).reshape(n, nh * hd)
        k = plain.rms_norm(k.reshape(n * nkv, hd), ref["l.kn.weight"], 1e-6).reshape(n, nkv * hd)
        q, k = plain.rope(q, nh, hd, cos, sin), plain.rope(k, nkv, hd, cos, sin)
        a = plain.causal_attention(q, k, v, nh, nkv, hd, window)
        return plain.linear(a, ref["l.o.weight"])

    step = make_step([(2, 0, [0] * lens[0], []), (0, 0, [0] * lens[1], [])])
    h = torch.cat([hs[0][:lens[0]], hs[1][:lens[1]]]).to(DEV)
    x = torch.zeros(h.shape[0], hidden, device=DEV)
    pending = mixer.forward(h, x, step, line, None, True)
    if pending is not None:            # split sums that the next norm would add
        settle(x, pending)
    want = np.concatenate([reference(hs[0])[:lens[0]], reference(hs[1])[:lens[1]]])
    ok, err = close(x.cpu(), want, dtype)
    assert ok, err
    step = make_step([(2, lens[0], [0], []), (0, lens[1], [0], [])])
    h = torch.cat([hs[0][lens[0]:], hs[1][lens[1]:]]).to(DEV)
    x = torch.full((2, hidden), 1.5, device=DEV)            # added into the residual
    pending = mixer.forward(h, x, step, line, None, True)
    if pending is not None:
        settle(x, pending)
    want = np.stack([reference(hs[0])[-1], reference(hs[1])[-1]]) + 1.5
    ok, err = close(x.cpu(), want, dtype)
    assert ok, err


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("hidden,inter", [(96, 320), (64, 130), (200, 72)])
def test_feed_forward_part_alone(dtype, hidden, inter):
    rt = Runtime(DT[dtype])
    part = FEED_FORWARDS.build(PartSpec("swiglu", {
        "hidden_size": hidden, "intermediate_size": inter,
        "names": {"gate": "g.weight", "up": "u.weight", "down": "d.weight"}}), "m.")
    dev, ref = part_weights(part, dtype, seed=inter)
    part.bind(dev, rt)
    h = torch.randn(11, hidden, generator=torch.Generator().manual_seed(2)).to(DT[dtype])
    x = torch.full((11, hidden), -0.5, device=DEV)
    pending = part.forward(h.to(DEV), x, None)
    if pending is not None:
        settle(x, pending)
    hn = h.float().numpy()
    act = plain.swiglu(plain.linear(hn, ref["m.g.weight"]), plain.linear(hn, ref["m.u.weight"]))
    ok, err = close(x.cpu(), plain.linear(act, ref["m.d.weight"]) - 0.5, dtype)
    assert ok, err


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_block_alone(dtype, tiny_b_model):
    """One pre-norm residual block built from tiny B's layer 1 (the windowed one)."""
    tiny = tiny_b_model
    rt = Runtime(DT[dtype])
    model = DecoderModel(tiny.config.to_model_spec())
    layer = model.layers[1]
    weights = {k: torch.tensor(v).to(DT[dtype]).to(DEV) for k, v in tiny.plain_weights.items()}
    for p in list(model.positions.values()) + layer.parts():
        p.bind(weights, rt)
    n = 40
    x0 = torch.randn(n, tiny.config.hidden_size, generator=torch.Generator().manual_seed(3))
    x = x0.to(DEV)
    line = make_line(1, 64, 1, 32, DT[dtype], window=24)
    pending = layer.block.forward(x, make_step([(0, 0, [0] * n, [])]), line, None, True)
    if pending is not None:
        settle(x, pending)
    c = tiny.plain_config
    cos, sin = plain.rotary_tables(plain.inverse_frequencies(1e6, 32), range(n))
    want = plain.attention_block(x0.numpy(), tiny.plain_weights, "model.layers.1.", c, cos, sin, 24)
    want = plain.dense_block(want, tiny.plain_weights, "model.layers.1.", c)
    ok, err = close(x.cpu(), want, dtype)
    assert ok, err


# ------------------------------------------------------------------ generality
class RunningMeanMixer(Part):
    """A toy mixer with state of its own and no keys or values: it adds, to every token, the
    mean of all hidden rows of its sequence so far times a learned gain. The state per sequence
    is [hidden + 1]: the running sum and the count. Defined here, not in the library."""

    def __init__(self, spec, prefix="", positions=None):
        super().__init__(spec, prefix)
        self.hidden = spec.params["hidden_size"]
        self.name = prefix + "toy.gain"

    def tensors(self):
        return [TensorNeed(self.name, (self.hidden,), "vector")]

    def state_need(self):
        return StateNeed((self.hidden + 1,))

    def bind(self, weights, rt):
        self.gain = weights[self.name].float()

    def forward(self, h, x, step, line, state, writes_cache):
        starts = step.seq_start.tolist()
        for b, slot in enumerate(step.seq_slot.tolist()):       # a sequence's tokens in order
            rows = h[starts[b]:starts[b + 1]].float()
            sums = state[slot, :-1] + torch.cumsum(rows, 0)
            counts = state[slot, -1] + torch.arange(1, rows.shape[0] + 1, device=h.device)
            x[starts[b]:starts[b + 1]] += self.gain * sums / counts[:, None]
            state[slot, :-1] = sums[-1]
            state[slot, -1] = counts[-1]


def toy_spec(cfg, schedule, mixers):
    base = cfg.to_model_spec()
    layers = []
    for i, l in enumerate(base.layers):
        mixer = l.mixer
        if mixers[i] == "toy":
            mixer = PartSpec("running_mean", {"hidden_size": cfg.hidden_size})
        layers.append(LayerSpec(l.block, mixer, l.feed_forward, l.norms, l.prefix))
    return ModelSpec(base.architecture, base.vocab_size, base.hidden_size, base.max_positions,
                     base.embedding, base.positions, tuple(layers), tuple(schedule),
                     base.final_norm, base.head)


def build_engine(cfg, spec, dtype, seed=5):
    rt = Runtime(DT[dtype])
    model = DecoderModel(spec)
    weights = random_tensors(model.tensors(), seed, 0.05, 0.1, torch.bfloat16)
    ref = {k: v.float().numpy() for k, v in weights.items()}
    dev = {k: v.to(DT[dtype]).to(DEV) for k, v in weights.items()}
    return Engine(cfg, dev, rt, max_tokens=1024, model=model), ref


def plain_toy_forward(cfg, spec, w, ids):
    """The plain implementation, layer by layer in the spec's order, with the toy mixer and the
    shared cache restated for whole sequences."""
    c = cfg.to_dict()
    n = len(ids)
    cos, sin = plain.rotary_tables(plain.inverse_frequencies(cfg.rope_theta, cfg.head_dim), range(n))
    x = plain.embed(w["model.embed_tokens.weight"], ids)
    kv_of_line = {}
    for run in spec.schedule:
        l = spec.layers[run.layer]
        p = l.prefix
        if l.mixer.kind == "running_mean":
            h = plain.rms_norm(x, w[p + "input_layernorm.weight"], cfg.rms_norm_eps)
            mean = np.cumsum(h.astype(np.float64), 0) / np.arange(1, n + 1)[:, None]
            x = (x + (w[p + "toy.gain"] * mean).astype(np.float32)).astype(np.float32)
        else:
            st = {}
            if run.writes_cache:
                x_new = plain.attention_block(x, w, p, c, cos, sin, l.mixer.params["window"], st)
                kv_of_line[run.cache_line] = (st["k"], st["v"])
            else:                                   # q of this layer, k and v of another one
                k, v = kv_of_line[run.cache_line]
                h = plain.rms_norm(x, w[p + "input_layernorm.weight"], cfg.rms_norm_eps)
                nh, nkv, hd = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
                q = plain.linear(h, w[p + "self_attn.q_proj.weight"])
                q = plain.rms_norm(q.reshape(n * nh, hd), w[p + "self_attn.q_norm.weight"],
                                   cfg.rms_norm_eps).reshape(n, nh * hd)
                q = plain.rope(q, nh, hd, cos, sin)
                a = plain.causal_attention(q, k, v, nh, nkv, hd, l.mixer.params["window"])
                x_new = (x + plain.linear(a, w[p + "self_attn.o_proj.weight"])).astype(np.float32)
            x = x_new
        x = plain.dense_block(x, w, p, c)
    hN = plain.rms_norm(x, w["model.norm.weight"], cfg.rms_norm_eps)
    return plain.linear(hN, w["lm_head.weight"])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_mixer_with_state_is_registered_built_and_stepped(dtype):
    register_mixer("running_mean", RunningMeanMixer)
    cfg = tiny_b()
    schedule = [Run(0, 0), Run(1, 1), Run(2, 2)]
    spec = toy_spec(cfg, schedule, ["attn", "toy", "attn"])
    eng, ref = build_engine(cfg, spec, dtype)
    assert set(eng.model.state_needs) == {1} and set(eng.model.line_needs) == {0, 2}
    assert eng.cache.states[1].shape == (eng.max_slots, cfg.hidden_size + 1)
    rng = np.random.default_rng(0)
    a, b = rng.integers(0, cfg.vocab_size, 30).tolist(), rng.integers(0, cfg.vocab_size, 12).tolist()
    s0, s1 = eng.open(), eng.open()
    out = eng.step([Entry(s0, a[:20]), Entry(s1, b[:5])]).cpu().numpy()
    for row, ids in enumerate((a[:20], b[:5])):
        ok, err = close(out[row:row + 1], plain_toy_forward(cfg, spec, ref, ids)[-1:], dtype)
        assert ok, err
    for t in range(5):                                   # the state is carried token by token
        out = eng.step([Entry(s0, [a[20 + t]]), Entry(s1, [b[5 + t]])]).cpu().numpy()
        for row, ids in enumerate((a[:21 + t], b[:6 + t])):
            ok, err = close(out[row:row + 1], plain_toy_forward(cfg, spec, ref, ids)[-1:], dtype)
            assert ok, (t, err)
    eng.close(s0)
    s2 = eng.open()                                      # the slot again: its state starts at 0
    assert s2 == s0
    out = eng.step([Entry(s2, b)]).cpu().numpy()
    ok, err = close(out, plain_toy_forward(cfg, spec, ref, b)[-1:], dtype)
    assert ok, err


def test_a_failed_step_leaves_state_and_length_as_it_found_them():
    """A long prompt runs as several passes, each of which moves the toy mixer's state on. The
    third pass fails (made on the host: the mixer raises on a flagged call). The step then
    counts for nothing: length and state are those from before it, and the same step again
    gives the plain restatement's logits (the reference marks its state as not matching with
    ``fStateOk``, ``decoder.pas:436``, ``:3301``, ``:3348``)."""

    class Failing(RunningMeanMixer):
        fail_at = None
        calls = 0

        def forward(self, h, x, step, line, state, writes_cache):
            Failing.calls += 1
            if Failing.calls == Failing.fail_at:
                raise RuntimeError("made to fail")
            super().forward(h, x, step, line, state, writes_cache)

    register_mixer("running_mean", Failing)
    cfg = tiny_b()
    spec = toy_spec(cfg, [Run(0, 0), Run(1, 1), Run(2, 2)], ["attn", "toy", "attn"])
    rt = Runtime(DT["float32"])
    model = DecoderModel(spec)
    weights = random_tensors(model.tensors(), 5, 0.05, 0.1, torch.bfloat16)
    ref = {k: v.float().numpy() for k, v in weights.items()}
    dev = {k: v.float().to(DEV) for k, v in weights.items()}
    eng = Engine(cfg, dev, rt, max_tokens=1024, model=model, prefill_chunk=8, max_slots=2)
    rng = np.random.default_rng(3)
    ids = rng.integers(0, cfg.vocab_size, 50).tolist()
    other = rng.integers(0, cfg.vocab_size, 9).tolist()
    s0, s1 = eng.open(), eng.open()
    eng.step([Entry(s0, ids[:10]), Entry(s1, other[:4])])
    before = eng.cache.states[1].clone()
    Failing.calls, Failing.fail_at = 0, 3
    with pytest.raises(RuntimeError, match="made to fail"):
        eng.step([Entry(s0, ids[10:]), Entry(s1, other[4:])])     # 5 passes of 8 tokens
    Failing.fail_at = None
    assert eng.length(s0) == 10 and eng.length(s1) == 4
    assert torch.equal(eng.cache.states[1], before)
    out = eng.step([Entry(s0, ids[10:]), Entry(s1, other[4:])]).cpu().numpy()
    for row, seq in enumerate((ids, other)):
        ok, err = close(out[row:row + 1], plain_toy_forward(cfg, spec, ref, seq)[-1:], "float32")
        assert ok, (row, err)
    # state of fixed size cannot go back: only to nothing, or to where it is
    with pytest.raises(CacheError, match="cannot go back"):
        eng.truncate(s0, 20)
    eng.truncate(s0, 50)
    eng.truncate(s0, 0)
    assert float(eng.cache.states[1][s0].abs().max()) == 0.0
    out = eng.step([Entry(s0, other)]).cpu().numpy()
    ok, err = close(out, plain_toy_forward(cfg, spec, ref, other)[-1:], "float32")
    assert ok, err
    # a decode run that keeps fewer steps than it launched leaves state ahead of the length
    from mormot2_ai_b200 import Sampling
    from mormot2_ai_b200.sampling import DeviceSampler
    sampler = DeviceSampler(rt.device, eng.max_slots, eng.vocab_size)
    run = eng.decode_run([s0, s1], [1, 2], [4, 4], sampler, Sampling())
    run.launch(), run.launch()
    run.read(), run.read()
    run.finish([2, 1])
    assert eng.state_ok[s0] and not eng.state_ok[s1]
    with pytest.raises(CacheError, match="fixed-size state"):
        eng.step([Entry(s1, [3])])
    eng.step([Entry(s0, [3])])
    eng.truncate(s1, 0)
    eng.step([Entry(s1, [3])])
    register_mixer("running_mean", RunningMeanMixer)


def test_state_of_another_type_and_start_value():
    from mormot2_ai_b200.cache.storage import CacheStorage
    store = CacheStorage([], 4, torch.bfloat16, torch.device(DEV),
                         {3: StateNeed((2, 3), "int32", 7), 5: StateNeed((4,))})
    assert store.states[3].dtype == torch.int32 and store.states[5].dtype == torch.float32
    assert store.states[3].shape == (4, 2, 3) and int(store.states[3].min()) == 7
    store.states[3][1] += 5
    store.states[5][1] += 1.5
    idx = torch.tensor([1, 2], device=DEV)
    store.save_states(idx)
    store.states[3][1:3] = 0
    store.states[5][:] = 9.0
    store.restore_states(idx)
    assert store.states[3][1].tolist() == [[12] * 3] * 2 and store.states[3][2].tolist() == [[7] * 3] * 2
    assert store.states[5][1].tolist() == [1.5] * 4 and store.states[5][0].tolist() == [9.0] * 4
    store.reset_state(1)
    assert int(store.states[3][1].max()) == 7 and float(store.states[5][1].max()) == 0.0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_layer_twice_and_a_shared_cache(dtype):
    """The order of layers is data: layer 0 runs twice (each run with a cache line of its own)
    and the last run reads the keys and values that the run before it wrote."""
    cfg = Qwen3Config(vocab_size=300, hidden_size=64, num_hidden_layers=2, num_attention_heads=4,
                      num_key_value_heads=2, head_dim=16, intermediate_size=96,
                      max_position_embeddings=128, rms_norm_eps=1e-6, rope_theta=1e4,
                      tie_word_embeddings=False)
    schedule = [Run(0, 0), Run(1, 1), Run(0, 2), Run(1, 2, writes_cache=False)]
    spec = toy_spec(cfg, schedule, ["attn", "attn"])
    eng, ref = build_engine(cfg, spec, dtype)
    assert sorted(eng.model.line_needs) == [0, 1, 2]
    rng = np.random.default_rng(1)
    ids = rng.integers(0, 300, 40).tolist()
    want = plain_toy_forward(cfg, spec, ref, ids)
    s = eng.open()
    out = eng.step([Entry(s, ids[:33], [0, 32])]).cpu().numpy()
    ok, err = close(out, want[[0, 32]], dtype)
    assert ok, err
    for t in range(33, 40):
        ok, err = close(eng.step([Entry(s, [ids[t]])]).cpu().numpy(), want[t:t + 1], dtype)
        assert ok, (t, err)
    for bad in ([Run(0, 0), Run(1, 0)],                       # a line written twice
                [Run(1, 0, writes_cache=False), Run(0, 0)],   # read before it is written
                [Run(0, None)], [Run(5, 0)]):
        with pytest.raises(ConfigError):
            DecoderModel(toy_spec(cfg, bad, ["attn", "attn"]))


class TopOneExperts(Part):
    """A toy feed-forward with routing, defined here, not in the library: a router picks one
    of E small two-matrix experts per token (highest router logit, lowest index on a tie) and
    the expert's output, weighted by the softmax probability of its logit, is added to x."""

    def __init__(self, spec, prefix=""):
        super().__init__(spec, prefix)
        p = spec.params
        self.hidden, self.inter, self.experts = p["hidden_size"], p["inter"], p["experts"]
        self.base = prefix + "toy_moe."

    def tensors(self):
        e, h, i = self.experts, self.hidden, self.inter
        return [TensorNeed(self.base + "router", (e, h)), TensorNeed(self.base + "w1", (e * i, h)),
                TensorNeed(self.base + "w2", (e * h, i))]

    def bind(self, weights, rt):
        e, h, i = self.experts, self.hidden, self.inter
        self.router = weights[self.base + "router"].float()
        self.w1 = weights[self.base + "w1"].float().view(e, i, h)
        self.w2 = weights[self.base + "w2"].float().view(e, h, i)

    def forward(self, h, x, step):
        hf = h.float()
        logits = hf @ self.router.T                              # router logits in float32
        prob = torch.softmax(logits, dim=-1)
        pick = logits.argmax(dim=-1)
        for e in range(self.experts):
            rows = (pick == e).nonzero().flatten()
            if rows.numel():
                mid = torch.relu(hf[rows] @ self.w1[e].T)
                x[rows] += prob[rows, e, None] * (mid @ self.w2[e].T)
        return None


class SlowedRope(Part):
    """A toy position encoding, defined here: rotary over the first rot_dim values of a head
    only, with every position counted as position / factor (the frequencies divided by it)."""

    def __init__(self, spec, prefix=""):
        super().__init__(spec, prefix)
        self.theta, self.rot_dim = spec.params["theta"], spec.params["rot_dim"]
        self.factor = spec.params["factor"]

    def bind(self, weights, rt):
        inv = plain.inverse_frequencies(self.theta, self.rot_dim) / np.float32(self.factor)
        self.inv_freq = torch.from_numpy(inv.astype(np.float32)).to(rt.device)

    def frequencies(self):
        return self.inv_freq, self.rot_dim


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_routed_feed_forward_and_toy_position_encoding(dtype):
    """Two more kinds of parts from outside the library: layer 1's feed-forward routes each
    token to one of three experts, and every attention rotates with a position encoding that
    the library does not have (12 of 16 values of a head, positions slowed by 4)."""
    from mormot2_ai_b200.parts import register_feed_forward, register_position
    register_feed_forward("top_one_experts", TopOneExperts)
    register_position("slowed_rope", SlowedRope)
    cfg = Qwen3Config(vocab_size=300, hidden_size=64, num_hidden_layers=2, num_attention_heads=4,
                      num_key_value_heads=2, head_dim=16, intermediate_size=96,
                      max_position_embeddings=128, rms_norm_eps=1e-6, rope_theta=1e4,
                      tie_word_embeddings=False)
    base = cfg.to_model_spec()
    moe = PartSpec("top_one_experts", {"hidden_size": 64, "inter": 40, "experts": 3})
    layers = [base.layers[0],
              LayerSpec(base.layers[1].block, base.layers[1].mixer, moe, base.layers[1].norms,
                        base.layers[1].prefix)]
    name = next(iter(base.positions))
    positions = {name: PartSpec("slowed_rope", {"theta": 1e4, "rot_dim": 12, "factor": 4.0})}
    spec = ModelSpec(base.architecture, base.vocab_size, base.hidden_size, base.max_positions,
                     base.embedding, positions, tuple(layers), base.schedule, base.final_norm,
                     base.head)
    eng, w = build_engine(cfg, spec, dtype)

    def reference(ids):
        n, nh, nkv, hd, rot = len(ids), 4, 2, 16, 12
        inv = plain.inverse_frequencies(1e4, rot) / np.float32(4.0)
        cos, sin = plain.rotary_tables(inv.astype(np.float32), range(n))
        x = plain.embed(w["model.embed_tokens.weight"], ids)
        for li in range(2):
            p = f"model.layers.{li}."
            h = plain.rms_norm(x, w[p + "input_layernorm.weight"], 1e-6)
            q = plain.linear(h, w[p + "self_attn.q_proj.weight"])
            k = plain.linear(h, w[p + "self_attn.k_proj.weight"])
            v = plain.linear(h, w[p + "self_attn.v_proj.weight"])
            q = plain.rms_norm(q.reshape(n * nh, hd), w[p + "self_attn.q_norm.weight"], 1e-6)
            k = plain.rms_norm(k.reshape(n * nkv, hd), w[p + "self_attn.k_norm.weight"], 1e-6)
            q, k = q.reshape(n, nh, hd).copy(), k.reshape(n, nkv, hd).copy()
            q[:, :, :rot] = plain.rope(q[:, :, :rot].reshape(n, nh * rot), nh, rot, cos,
                                       sin).reshape(n, nh, rot)
            k[:, :, :rot] = plain.rope(k[:, :, :rot].reshape(n, nkv * rot), nkv, rot, cos,
                                       sin).reshape(n, nkv, rot)
            a = plain.causal_attention(q.reshape(n, nh * hd), k.reshape(n, nkv * hd), v, nh, nkv,
                                       hd, 0)
            x = (x + plain.linear(a, w[p + "self_attn.o_proj.weight"])).astype(np.float32)
            if li == 0:
                x = plain.dense_block(x, w, p, cfg.to_dict())
                continue
            h = plain.rms_norm(x, w[p + "post_attention_layernorm.weight"], 1e-6).astype(np.float64)
            logits = h @ w[p + "toy_moe.router"].astype(np.float64).T
            prob = np.exp(logits - logits.max(1, keepdims=True))
            prob /= prob.sum(1, keepdims=True)
            out = np.zeros_like(h)
            for t in range(n):
                e = int(logits[t].argmax())
                w1 = w[p + "toy_moe.w1"].reshape(3, 40, 64)[e].astype(np.float64)
                w2 = w[p + "toy_moe.w2"].reshape(3, 64, 40)[e].astype(np.float64)
                out[t] = prob[t, e] * (w2 @ np.maximum(w1 @ h[t], 0))
            x = (x + out).astype(np.float32)
        return plain.linear(plain.rms_norm(x, w["model.norm.weight"], 1e-6), w["lm_head.weight"])

    rng = np.random.default_rng(4)
    a, b = rng.integers(0, 300, 50).tolist(), rng.integers(0, 300, 23).tolist()
    ra, rb = reference(a), reference(b)
    s0, s1 = eng.open(), eng.open()
    out = eng.step([Entry(s0, a[:40], [0, 39]), Entry(s1, b[:9])]).cpu().numpy()
    ok, err = close(out, np.stack([ra[0], ra[39], rb[8]]), dtype)
    assert ok, err
    for t in range(10):
        out = eng.step([Entry(s0, [a[40 + t]]), Entry(s1, [b[9 + t]])]).cpu().numpy()
        ok, err = close(out, np.stack([ra[40 + t], rb[9 + t]]), dtype)
        assert ok, (t, err)
    eng.rt.check()
