"""The engine against the plain implementation on a B200, in float32 and in bfloat16, for both
tiny configurations: each request alone and whole; the last 32 tokens one by one; batches of
unequal lengths whose shorter requests end earlier, one batch after another so that slots and
pages are used again; long decoding; the first tokens of a sequence; prompts cut into passes
(which also turns the window's ring of pages on)."""
import numpy as np
import pytest
import torch

from mormot2_ai_b200 import CacheError, Engine, Entry, InferError
from tests.conftest import close

pytestmark = pytest.mark.gpu
DTYPES = ["float32", "bfloat16"]


def engine_of(tiny, dtype, **kw):
    kw.setdefault("max_tokens", 2048)
    return Engine.from_folder(tiny.folder, dtype=dtype, **kw)


def check(got, want, dtype, what):
    ok, err = close(got, want, dtype)
    assert ok, f"{what}: relative error {err:.3g} ({dtype})"


@pytest.mark.parametrize("dtype", DTYPES)
def test_each_request_alone_and_whole(tiny, dtype):
    eng = engine_of(tiny, dtype)
    limit = tiny.config.max_position_embeddings
    for n in tiny.prompt_lens + [limit]:
        ids = tiny.tokens(n, seed=n)
        slot = eng.open()
        out = eng.step([Entry(slot, ids, list(range(n)))])
        eng.close(slot)
        check(out.cpu().numpy(), tiny.reference(ids), dtype, f"whole prompt of {n}")
    eng.rt.check()


@pytest.mark.parametrize("dtype", DTYPES)
def test_last_32_tokens_one_by_one(tiny, dtype):
    eng = engine_of(tiny, dtype)
    for n in (40, tiny.config.max_position_embeddings - 3):
        ids = tiny.tokens(n, seed=100 + n)
        ref = tiny.reference(ids)
        slot = eng.open()
        head = n - 32
        out = eng.step([Entry(slot, ids[:head], [head - 1])])
        check(out.cpu().numpy(), ref[head - 1:head], dtype, f"prompt end at {head - 1}")
        for t in range(head, n):
            out = eng.step([Entry(slot, [ids[t]])])
            check(out.cpu().numpy(), ref[t:t + 1], dtype, f"decoded token at {t} of {n}")
        assert eng.length(slot) == n
        eng.close(slot)
    eng.rt.check()


@pytest.mark.parametrize("dtype", DTYPES)
def test_unequal_batches_with_slot_reuse(tiny, dtype):
    """Three slots and few pages for seven requests: batches of unequal lengths, the prompts in
    one step, then one token each; a request that ends leaves the batch and its slot and pages
    serve the next batch."""
    limit = tiny.config.max_position_embeddings
    lens = tiny.prompt_lens + [2, 65, 33, limit - tiny.decode_steps - 1]
    decode = [tiny.decode_steps, 3, 1, tiny.decode_steps, 5, 2, tiny.decode_steps][:len(lens)]
    lens = lens[:len(decode)]
    # just the pages that the fullest batch of three needs: later batches must reuse them
    pages = max(sum(-(-(n + d) // 64) for n, d in list(zip(lens, decode))[b0:b0 + 3])
                for b0 in range(0, len(lens), 3))
    eng = engine_of(tiny, dtype, max_tokens=64 * pages, max_slots=3)
    reqs = [tiny.tokens(n + d, seed=200 + i) for i, (n, d) in enumerate(zip(lens, decode))]
    refs = [tiny.reference(r) for r in reqs]
    used_slots = []
    for b0 in range(0, len(reqs), 3):
        idx = list(range(b0, min(b0 + 3, len(reqs))))
        slots = {i: eng.open() for i in idx}
        used_slots.append(sorted(slots.values()))
        out = eng.step([Entry(slots[i], reqs[i][:lens[i]]) for i in idx]).cpu().numpy()
        for row, i in enumerate(idx):
            check(out[row:row + 1], refs[i][lens[i] - 1:lens[i]], dtype, f"request {i} prompt")
        at = {i: lens[i] for i in idx}
        live = list(idx)
        while live:
            live = [i for i in live if at[i] < len(reqs[i])]
            for i in idx:
                if i not in live and i in slots:
                    eng.close(slots.pop(i))          # ended earlier: slot and pages go back
            if not live:
                break
            out = eng.step([Entry(slots[i], [reqs[i][at[i]]]) for i in live]).cpu().numpy()
            for row, i in enumerate(live):
                check(out[row:row + 1], refs[i][at[i]:at[i] + 1], dtype,
                      f"request {i} token {at[i]}")
                at[i] += 1
    assert used_slots[0] == used_slots[1] == [0, 1, 2]       # the same slots again
    assert all(eng.book.held_pages(g) == 0 for g in range(len(eng.plans)))
    assert eng.book.slots.free == 3
    eng.rt.check()


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding_to_the_context_limit(tiny, dtype):
    eng = engine_of(tiny, dtype)
    n = tiny.config.max_position_embeddings
    ids = tiny.tokens(n, seed=300)
    ref = tiny.reference(ids)
    slot = eng.open()
    out = eng.step([Entry(slot, ids[:3])])
    check(out.cpu().numpy(), ref[2:3], dtype, "prompt")
    worst = 0.0
    for t in range(3, n):
        out = eng.step([Entry(slot, [ids[t]])])
        ok, err = close(out.cpu().numpy(), ref[t:t + 1], dtype)
        assert ok, f"token {t}: relative error {err:.3g}"
        worst = max(worst, err)
    with pytest.raises(CacheError, match="exceed the context"):
        eng.step([Entry(slot, [1])])
    assert eng.length(slot) == n
    eng.close(slot)


@pytest.mark.parametrize("dtype", DTYPES)
def test_first_tokens_of_a_sequence(tiny, dtype):
    eng = engine_of(tiny, dtype)
    ids = tiny.tokens(6, seed=400)
    ref = tiny.reference(ids)
    slot = eng.open()
    for t in range(6):                      # from the very first token on, one by one
        out = eng.step([Entry(slot, [ids[t]])])
        check(out.cpu().numpy(), ref[t:t + 1], dtype, f"token {t}")
    eng.close(slot)
    slot = eng.open()                       # a prompt of one token, then two at once
    check(eng.step([Entry(slot, ids[:1])]).cpu().numpy(), ref[0:1], dtype, "first token")
    check(eng.step([Entry(slot, ids[1:3], [0, 1])]).cpu().numpy(), ref[1:3], dtype, "next two")
    eng.close(slot)


@pytest.mark.parametrize("dtype", DTYPES)
def test_prompts_cut_into_passes(tiny, dtype):
    """A small pass size cuts prompts into several passes of the model (and, for the windowed
    layer of tiny B, makes its cache a ring of pages smaller than the sequence): same logits."""
    eng = engine_of(tiny, dtype, prefill_chunk=16, max_step_tokens=40, max_slots=4)
    if any(p.window for p in eng.plans):
        assert any(p.ring_pages for p in eng.plans)
    limit = tiny.config.max_position_embeddings
    lens = [limit, limit - 60, 37, 16]
    reqs = [tiny.tokens(n, seed=500 + n) for n in lens]
    slots = [eng.open() for _ in reqs]
    wants = [[0, n // 2, n - 1] if n > 2 else [n - 1] for n in lens]
    before = eng.passes
    out = eng.step([Entry(s, r, w) for s, r, w in zip(slots, reqs, wants)]).cpu().numpy()
    assert eng.passes - before >= limit // 16
    row = 0
    for r, w in zip(reqs, wants):
        ref = tiny.reference(r)
        for place in w:
            check(out[row:row + 1], ref[place:place + 1], dtype, f"len {len(r)} place {place}")
            row += 1
    # decoding goes on from what the passes left (the longer one beyond the ring's first lap)
    ext = [r + tiny.tokens(4, seed=len(r)) for r in reqs[1:]]
    for t in range(4):
        out = eng.step([Entry(s, [e[len(r) + t]]) for s, e, r in
                        zip(slots[1:], ext, reqs[1:])]).cpu().numpy()
        for row, (e, r) in enumerate(zip(ext, reqs[1:])):
            ref = tiny.reference(e[:len(r) + t + 1])
            check(out[row:row + 1], ref[-1:], dtype, f"decode {t} after passes")
    eng.rt.check()


@pytest.mark.parametrize("dtype", DTYPES)
def test_truncate_and_go_on_equals_a_fresh_pass(tiny, dtype):
    """A sequence cut back to a prefix and fed other tokens gives the logits of a fresh pass
    over the new sequence (the reference's ``TinyPromptReuse``, ``test.infer.qwen3.pas:870-986``);
    whole pages beyond the cut come back to the pool."""
    eng = engine_of(tiny, dtype, max_tokens=1024, max_slots=2)
    first = tiny.tokens(120, seed=600)
    slot = eng.open()
    eng.step([Entry(slot, first)])
    held = [eng.book.held_pages(g) for g in range(len(eng.plans))]
    for cut, more in ((70, 9), (17, 50), (17, 3)):
        eng.truncate(slot, cut)
        assert eng.length(slot) == cut
        other = tiny.tokens(more, seed=601 + more)
        ids = first[:cut] + other
        out = eng.step([Entry(slot, other, list(range(more)))]).cpu().numpy()
        check(out, tiny.reference(ids)[cut:], dtype, f"after a cut to {cut}")
        first = ids
        out = eng.step([Entry(slot, [7])]).cpu().numpy()       # and a decode step after it
        first = first + [7]
        check(out, tiny.reference(first)[-1:], dtype, f"decoding after a cut to {cut}")
    assert [eng.book.held_pages(g) for g in range(len(eng.plans))] == [1] * len(eng.plans)
    assert held == [2] * len(eng.plans)
    with pytest.raises(CacheError, match="truncate"):
        eng.truncate(slot, eng.length(slot) + 1)
    # the same prefix again for another request: only what differs is fed
    request = first[:15] + tiny.tokens(6, seed=650)
    kept = eng.reuse(slot, request)
    assert kept == 15 == eng.length(slot) and eng.common(slot, request) == 15
    out = eng.step([Entry(slot, request[kept:])]).cpu().numpy()
    check(out, tiny.reference(request)[-1:], dtype, "after reuse")
    assert eng.reuse(slot, request) == len(request) - 1          # the last token is fed again
    out = eng.step([Entry(slot, request[-1:])]).cpu().numpy()
    check(out, tiny.reference(request)[-1:], dtype, "the same request again")
    eng.truncate(slot, 0)
    assert all(eng.book.held_pages(g) == 0 for g in range(len(eng.plans)))
    out = eng.step([Entry(slot, request[:3])]).cpu().numpy()
    check(out, tiny.reference(request[:3])[-1:], dtype, "after a cut to nothing")
    eng.rt.check()


@pytest.mark.parametrize("dtype", DTYPES)
def test_truncate_behind_a_windows_ring(tiny_b_model, dtype):
    """Tiny B's middle layer has a window of 24; with passes of 16 tokens its keys live in a
    ring of 2 pages. A cut whose next position would read keys that the ring has overwritten
    is refused and changes nothing; one that the ring still covers works."""
    tiny = tiny_b_model
    eng = engine_of(tiny, dtype, prefill_chunk=16, max_slots=2)
    ring = [g for g, p in enumerate(eng.plans) if p.ring_pages]
    assert ring and eng.plans[ring[0]].ring_pages == 2
    ids = tiny.tokens(200, seed=610)
    slot = eng.open()
    eng.step([Entry(slot, ids)])
    with pytest.raises(CacheError, match="no longer holds"):
        eng.truncate(slot, 100)                     # the ring holds keys from 128 on
    assert eng.length(slot) == 200
    out = eng.step([Entry(slot, [3])]).cpu().numpy()
    check(out, tiny.reference(ids + [3])[-1:], dtype, "after the refusal")
    eng.truncate(slot, 160)                         # reads keys from 137 on
    other = tiny.tokens(30, seed=611)
    out = eng.step([Entry(slot, other, [0, 13, 29])]).cpu().numpy()
    check(out, tiny.reference(ids[:160] + other)[[160, 173, 189]], dtype, "after the cut")
    assert eng.reuse(slot, ids[:90] + [1, 2]) == 0  # a prefix behind the ring: nothing is kept
    assert eng.length(slot) == 0
    eng.rt.check()


def test_refused_steps_change_nothing(tiny_a_model):
    tiny = tiny_a_model
    eng = engine_of(tiny, "float32", max_tokens=128, max_slots=2)
    s0, s1 = eng.open(), eng.open()
    ids = tiny.tokens(10)
    eng.step([Entry(s0, ids)])
    held = eng.book.held_pages(0)
    for bad, match in (([Entry(s0, [tiny.config.vocab_size])], "outside the vocabulary"),
                       ([Entry(s0, [-1])], "outside the vocabulary"),
                       ([Entry(s0, [])], "0 tokens"),
                       ([Entry(s0, [1]), Entry(s0, [2])], "twice"),
                       ([Entry(s0, [1], [1])], "wanted places"),
                       ([], "without entries")):
        with pytest.raises(InferError, match=match):
            eng.step(bad)
    with pytest.raises(CacheError, match="not open"):
        eng.step([Entry(7, [1])])
    with pytest.raises(CacheError):
        eng.step([Entry(s0, [1]), Entry(s1, tiny.tokens(128))])     # more pages than there are
    small = engine_of(tiny, "float32", max_tokens=128, max_slots=2, max_step_tokens=16)
    t0 = small.open()
    with pytest.raises(InferError, match="rows of logits"):          # wanted rows may repeat
        small.step([Entry(t0, ids, [0] * 17)])
    assert small.length(t0) == 0 and small.book.held_pages(0) == 0
    assert eng.length(s0) == 10 and eng.length(s1) == 0 and eng.book.held_pages(0) == held
    ref = tiny.reference(ids + [5])
    out = eng.step([Entry(s0, [5])]).cpu().numpy()
    check(out, ref[-1:], "float32", "the step after the refusals")
    with pytest.raises(CacheError):
        eng.open()                                                   # both slots are held


def test_padding_and_batch_mates_change_nothing(tiny_b_model):
    """The logits of a request do not depend on what else is in the batch."""
    tiny = tiny_b_model
    eng = engine_of(tiny, "float32")
    a, b, c = tiny.tokens(9, 1), tiny.tokens(50, 2), tiny.tokens(3, 3)
    s = eng.open()
    alone = eng.step([Entry(s, a, list(range(9)))]).cpu().numpy().copy()
    eng.close(s)
    slots = [eng.open() for _ in range(3)]
    out = eng.step([Entry(slots[0], b), Entry(slots[1], a, list(range(9))),
                    Entry(slots[2], c)]).cpu().numpy()
    assert np.abs(out[1:10] - alone).max() <= 2e-6


@pytest.mark.parametrize("lens", [(1100, 200), (4200,)], ids=["two_prompts", "long_prompt"])
def test_layers_of_full_size_bfloat16_against_float32(lens):
    """Two layers with the sizes of a real model (width 4096, 32 heads of 128 on 8, feed-forward
    12288, vocabulary 151936): the tensor-core path (products on CTA pairs for the prompts, the
    decode forms with split K, both tensor-core attention kernels) against the engine's own
    32-bit path on the same weights. The tiny configurations reach none of these kernel shapes."""
    from mormot2_ai_b200 import Qwen3Config
    cfg = Qwen3Config.from_dict({
        "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "vocab_size": 151936,
        "hidden_size": 4096, "intermediate_size": 12288, "num_hidden_layers": 2,
        "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 128,
        "max_position_embeddings": 8192, "rms_norm_eps": 1e-6, "rope_theta": 1000000.0,
        "tie_word_embeddings": False, "hidden_act": "silu", "attention_bias": False})
    from mormot2_ai_b200 import DecoderModel, Runtime
    from mormot2_ai_b200.weights.random_init import random_tensors
    names = DecoderModel(cfg.to_model_spec()).tensors()
    weights = random_tensors(names, 5, 0.03, 0.1, torch.bfloat16, "cuda:0")   # one set for both
    kw = dict(max_tokens=8192, max_context=4608, max_slots=4)
    fast = Engine(cfg, weights, Runtime(torch.bfloat16), **kw)
    slow = Engine(cfg, weights, Runtime(torch.float32), **kw)
    g = torch.Generator().manual_seed(3)
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in lens]

    def rel(a, b):
        """The bfloat16 path's logits against the 32-bit path's, in the measure and within the
        bound of every bfloat16 comparison of these tests."""
        ok, err = close(a.cpu().numpy(), b.cpu().numpy(), "bfloat16")
        return err if ok else float("inf")

    slots_f = [fast.open() for _ in prompts]
    slots_s = [slow.open() for _ in prompts]
    want = [[0, len(p) // 2, len(p) - 1] for p in prompts]
    a = fast.step([Entry(s, p, w) for s, p, w in zip(slots_f, prompts, want)])
    b = slow.step([Entry(s, p, w) for s, p, w in zip(slots_s, prompts, want)])
    assert float(b.abs().max()) > 0.5                      # logits of a size that means something
    assert rel(a, b) < float("inf")
    for step in range(3):                                   # decode: the token the 32-bit path picks
        last = [3 * i + 2 for i in range(len(prompts))]     # each prompt's last wanted row
        tokens = b[last].argmax(dim=1).tolist() if step == 0 else b.argmax(dim=1).tolist()
        a = fast.step([Entry(s, [t]) for s, t in zip(slots_f, tokens)])
        b = slow.step([Entry(s, [t]) for s, t in zip(slots_s, tokens)])
        assert rel(a, b) < float("inf"), step
    fast.rt.check()
    slow.rt.check()


ODD_CONFIGS = [
    # width, heads, kv heads, head size, feed-forward, vocabulary, layers, windows, tied
    (80, 5, 5, 48, 200, 1000, 3, (0, 40, 0), True),        # no grouping, heads of 48
    (72, 3, 1, 80, 104, 333, 2, (0, 0), True),             # heads of 80, an odd vocabulary
    (100, 5, 1, 112, 90, 127, 2, (65, 0), False),          # a width that is no multiple of 8
    (64, 2, 2, 256, 96, 260, 1, (0,), False),              # heads of 256
    (136, 7, 7, 96, 72, 515, 2, (0, 130), True),           # seven heads of 96
]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("sizes", ODD_CONFIGS, ids=[f"h{c[0]}_hd{c[3]}" for c in ODD_CONFIGS])
def test_other_sizes_whole_and_decoded(sizes, dtype, tmp_path):
    """Sizes that the four tiny configurations do not have (head sizes 48 to 256 in steps of 16,
    odd head counts, widths and vocabularies off every power of two): a batch of two unequal
    prompts, then tokens one by one, against the plain implementation."""
    from mormot2_ai_b200 import Qwen3Config, write_random_model
    from tests.plain import qwen3_plain as plain
    hidden, nh, nkv, hd, inter, vocab, layers, windows, tied = sizes
    cfg = Qwen3Config(vocab_size=vocab, hidden_size=hidden, num_hidden_layers=layers,
                      num_attention_heads=nh, num_key_value_heads=nkv, head_dim=hd,
                      intermediate_size=inter, max_position_embeddings=256, rms_norm_eps=1e-6,
                      rope_theta=1e5, tie_word_embeddings=tied, layer_windows=windows)
    folder = write_random_model(str(tmp_path / "m"), cfg, 11, std=0.05, norm_std=0.1)
    pc, pw = plain.read_model_folder(folder)
    eng = Engine.from_folder(folder, dtype=dtype, max_tokens=1024)
    rng = np.random.default_rng(hidden)
    seqs = [rng.integers(0, vocab, n).tolist() for n in (150, 67)]
    refs = [plain.forward(pc, pw, ids) for ids in seqs]
    heads = [130, 60]
    slots = [eng.open() for _ in seqs]
    out = eng.step([Entry(s, ids[:h], list(range(h))) for s, ids, h in zip(slots, seqs, heads)])
    check(out.cpu().numpy(), np.concatenate([r[:h] for r, h in zip(refs, heads)]), dtype,
          "prompts")
    for t in range(7):
        out = eng.step([Entry(s, [ids[h + t]]) for s, ids, h in zip(slots, seqs, heads)])
        check(out.cpu().numpy(), np.stack([r[h + t] for r, h in zip(refs, heads)]), dtype,
              f"decoded token {t}")
    eng.rt.check()


def test_kernel_classes_add_up_to_the_step(tiny_b_model):
    """``timed_step`` runs the kernels one by one and books each to its class: the classes
    add up to the step's time within a tenth, every class of the model is there, and the
    logits are those of an ordinary step."""
    tiny = tiny_b_model
    eng = engine_of(tiny, "bfloat16", max_slots=4)
    prompts = [tiny.tokens(n, seed=70 + n) for n in (200, 64, 9)]
    slots = [eng.open() for _ in prompts]
    eng.timed_step([Entry(s, p[:-2]) for s, p in zip(slots, prompts)])     # warms up
    # many rounds so that event overhead and launch gaps average out the same way in both sums
    inside = whole = 0.0
    for t in (-2, -1):
        logits, shares, total = eng.timed_step([Entry(s, [p[t]]) for s, p in zip(slots, prompts)])
        assert {"products", "attention", "norms", "rotary", "embedding"} <= set(shares)
        inside += sum(shares.values())
        whole += total
    want = np.stack([tiny.reference(p)[-1] for p in prompts])
    check(logits.cpu().numpy(), want, "bfloat16", "a timed step")
    for s in slots:
        eng.truncate(s, 0)
    logits, shares, total = eng.timed_step([Entry(s, p) for s, p in zip(slots, prompts)])
    check(logits.cpu().numpy(), want, "bfloat16", "a timed prefill")
    # the classes (the time between kernels is one of them) add up to the step within a tenth
    assert 0.9 * total <= sum(shares.values()) <= 1.001 * total, (shares, total)
    assert 0.9 * whole <= inside <= 1.001 * whole, (inside, whole)
    assert eng.use_graphs                                  # graphs are on again afterwards


@pytest.mark.parametrize("dtype", DTYPES)
def test_states_after_every_layer(tiny, dtype):
    """``Engine.on_state`` receives the residual after the embedding and after every entry of
    the layer order; the values are the plain implementation's, for a prompt and for a token
    decoded after it (the reference's ``CheckStates``, ``test.infer.qwen3.pas:385-436``)."""
    eng = engine_of(tiny, dtype)
    ids = tiny.tokens(70, seed=77)
    states = {}
    tiny.plain.forward(tiny.plain_config, tiny.plain_weights, ids, states)
    seen = {}
    eng.on_state = lambda name, x: seen.__setitem__(name, x.detach().float().cpu().numpy().copy())
    slot = eng.open()
    eng.step([Entry(slot, ids[:-1])])
    layers = tiny.config.num_hidden_layers
    assert list(seen) == ["embed"] + [f"run{i:02d}" for i in range(layers)]
    embed = tiny.plain.embed(tiny.plain_weights["model.embed_tokens.weight"], ids)
    assert np.array_equal(seen["embed"], embed[:-1])       # rows of the table, exactly
    for i in range(layers):
        check(seen[f"run{i:02d}"], states[f"layer{i:02d}"][:-1], dtype, f"prompt, layer {i}")
    seen.clear()
    eng.step([Entry(slot, ids[-1:])])                      # a decode step, run eagerly for this
    for i in range(layers):
        check(seen[f"run{i:02d}"], states[f"layer{i:02d}"][-1:], dtype, f"decode, layer {i}")
    eng.on_state = None
