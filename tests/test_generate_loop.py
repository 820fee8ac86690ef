"""The generation loop's decisions (no GPU), with a scripted stepper in place of the engine:
unequal prompts that start together, stop tokens, caps, sequences that end earlier and free
their slot at once, one batch after another, nothing held after an error."""
import pytest

from mormot2_ai_b200 import InferError, Sampling, sampling_from_config
from mormot2_ai_b200.engine.generate import Request, checked, generate, plan_batches


class ScriptedStepper:
    """Answers every sequence with the tokens of a script keyed by the prompt's first token."""

    def __init__(self, scripts, max_batch=4, pages=64, limit=128, fail_at=None):
        self.scripts, self._max_batch, self._pages, self._limit = scripts, max_batch, pages, limit
        self.free = list(range(max_batch))
        self.seq = {}           # slot -> [key, tokens fed so far, picks so far]
        self.calls = []         # per pick: [(slot, n tokens fed)]
        self.opened = self.closed = 0
        self.fail_at = fail_at

    def context_limit(self):
        return self._limit

    def max_batch(self):
        return self._max_batch

    def total_pages(self):
        return self._pages

    def open(self, seed):
        slot = self.free.pop(0)
        self.seq[slot] = [None, [], 0, seed]
        self.opened += 1
        return slot

    def close(self, slot):
        assert slot in self.seq, "closed twice"
        del self.seq[slot]
        self.free.append(slot)
        self.closed += 1

    def pick(self, entries):
        if self.fail_at is not None and len(self.calls) == self.fail_at:
            raise RuntimeError("device fault")
        self.calls.append([(slot, len(tokens)) for slot, tokens in entries])
        out = []
        for slot, tokens in entries:
            st = self.seq[slot]
            if st[0] is None:
                st[0] = tokens[0]
            st[1].extend(tokens)
            out.append(self.scripts[st[0]][st[2]])
            st[2] += 1
        return out


def test_unequal_batch_stops_and_caps():
    scripts = {1: [10, 11, 99, 12], 2: [20, 21, 22, 23, 24, 25], 3: [99]}
    st = ScriptedStepper(scripts)
    reqs = [Request([1, 5, 5], 10, {99}), Request([2], 4, {99}), Request([3] * 7, 10, {99})]
    out = generate(st, reqs)
    assert [o.tokens for o in out] == [[10, 11, 99], [20, 21, 22, 23], [99]]
    assert [o.stopped for o in out] == [True, False, True]
    # the prompts in one step with their unequal lengths, then one token each; a sequence that
    # ended is absent from the next step; the last token is never fed back
    assert st.calls[0] == [(0, 3), (1, 1), (2, 7)]
    assert st.calls[1] == [(0, 1), (1, 1)]
    assert st.calls[2] == [(0, 1), (1, 1)]
    assert st.calls[3] == [(1, 1)]
    assert len(st.calls) == 4 and st.opened == st.closed == 3 and len(st.free) == 4


def test_batches_one_after_another_reuse_slots():
    scripts = {k: [k * 10 + i for i in range(8)] for k in range(1, 8)}
    st = ScriptedStepper(scripts, max_batch=3)
    reqs = [Request([k] * k, 2 + k % 3) for k in range(1, 8)]
    out = generate(st, reqs)
    assert [o.tokens for o in out] == [scripts[k][:2 + k % 3] for k in range(1, 8)]
    assert [len(c) for c in st.calls if len(c) == 3][0] == 3
    firsts = [c for c in st.calls if any(n > 1 for _, n in c) or c == st.calls[0]]
    assert len(firsts) == 3                       # 7 requests on 3 slots: 3 batches
    assert st.opened == st.closed == 7
    assert {slot for c in st.calls for slot, _ in c} == {0, 1, 2}   # the same slots again


def test_caps_follow_the_context():
    reqs = checked([Request([1] * 120, 50), Request([1] * 128, 50), Request([1], 5)], 128)
    assert [r.max_new for r in reqs] == [9, 1, 5]      # limit - len(prompt) + 1
    with pytest.raises(InferError, match="empty prompt"):
        checked([Request([], 5)], 128)
    with pytest.raises(InferError, match="new tokens"):
        checked([Request([1], 0)], 128)
    with pytest.raises(InferError, match="exceeds the context"):
        checked([Request([1] * 129, 5)], 128)


def test_batches_respect_the_cache():
    reqs = [Request([1] * 100, 29), Request([1] * 60, 5), Request([1] * 10, 10),
            Request([1] * 200, 57)]
    assert plan_batches(reqs, 8, 4) == [[0, 1, 2], [3]]     # 2 + 1 + 1 pages, then 4
    assert plan_batches(reqs, 2, 64) == [[0, 1], [2, 3]]
    with pytest.raises(InferError, match="pages"):
        plan_batches(reqs, 8, 3)


def test_an_error_leaves_nothing_held():
    scripts = {1: [1, 2, 3, 4], 2: [5, 6, 7, 8]}
    st = ScriptedStepper(scripts, fail_at=1)
    with pytest.raises(RuntimeError):
        generate(st, [Request([1], 4), Request([2], 4)])
    assert st.opened == st.closed == 2 and not st.seq


def test_sampling_settings_and_defaults(tmp_path):
    assert Sampling().greedy and not Sampling().filtered
    assert Sampling(temperature=1e-31).greedy and not Sampling(temperature=0.5).greedy
    assert Sampling(temperature=1.0, top_k=5).filtered
    for bad in (dict(top_k=-1), dict(top_p=0.0), dict(top_p=1.5), dict(min_p=1.0),
                dict(min_p=-0.1), dict(temperature=float("nan")), dict(top_p=float("inf"))):
        with pytest.raises(InferError):
            Sampling(**bad)
    assert sampling_from_config(str(tmp_path)) == Sampling()          # no file: greedy
    p = tmp_path / "generation_config.json"
    p.write_text('{"do_sample": false, "temperature": 0.6, "top_k": 20}')
    assert sampling_from_config(str(tmp_path)) == Sampling()          # do_sample false: greedy
    p.write_text('{"do_sample": true}')
    assert sampling_from_config(str(p)) == Sampling(temperature=1.0, top_k=50)
    p.write_text('{"do_sample": true, "temperature": 0.6, "top_k": 20, "top_p": 0.95, "min_p": 0.05}')
    assert sampling_from_config(str(p)) == Sampling(0.6, 20, 0.95, 0.05)
    p.write_text('{"do_sample": true, "top_k": 2.5}')
    with pytest.raises(InferError, match="top_k"):
        sampling_from_config(str(p))
    p.write_text('{"do_sample": true, "temperature": true}')
    with pytest.raises(InferError, match="temperature"):
        sampling_from_config(str(p))
    p.write_text('[1]')
    with pytest.raises(InferError, match="JSON object"):
        sampling_from_config(str(p))
