"""The generation loop's decisions (no GPU), with a scripted stepper in place of the engine:
unequal prompts that start together, stop tokens, caps, sequences that end earlier and free
their slot at once, one batch after another, nothing held after an error."""
import pytest

from mormot2_ai_b200 import InferError, Sampling, sampling_from_config
from mormot2_ai_b200.engine.generate import (Request, checked, generate, pages_needed,
                                             plan_batches)


class ScriptedStepper:
    """Answers every sequence with the tokens of a script keyed by the prompt's first token.
    Its decode runs answer a launched step only when it is read, as a device would a step
    late; it records what was fed to whom."""

    def __init__(self, scripts, max_batch=4, pages=64, limit=128, fail_at=None, ring=0):
        self.scripts, self._max_batch, self._pages, self._limit = scripts, max_batch, pages, limit
        self._ring = ring
        self.free = list(range(max_batch))
        self.seq = {}           # slot -> [key, tokens fed so far, picks so far, seed]
        self.calls = []         # per step: [(slot, n tokens fed)]
        self.opened = self.closed = 0
        self.fail_at = fail_at
        self.open_runs = 0

    def context_limit(self):
        return self._limit

    def max_batch(self):
        return self._max_batch

    def pools(self):
        return [(self._pages, self._ring)]

    def open(self, seed):
        slot = self.free.pop(0)
        self.seq[slot] = [None, [], 0, seed]
        self.opened += 1
        return slot

    def close(self, slot):
        assert slot in self.seq, "closed twice"
        assert self.open_runs == 0, "closed while a run is open"
        del self.seq[slot]
        self.free.append(slot)
        self.closed += 1

    def _step(self, entries):
        if self.fail_at is not None and len(self.calls) == self.fail_at:
            raise RuntimeError("device fault")
        self.calls.append([(slot, len(tokens)) for slot, tokens in entries])
        out = []
        for slot, tokens in entries:
            st = self.seq[slot]
            if st[0] is None:
                st[0] = tokens[0]
            st[1].extend(tokens)
            script = self.scripts[st[0]]
            out.append(script[st[2]] if st[2] < len(script) else -7)   # beyond the script
            st[2] += 1
        return out

    def prefill(self, entries):
        return self._step(entries)

    def decode(self, members):
        self.open_runs += 1
        return ScriptedRun(self, members)


class ScriptedRun:
    def __init__(self, stepper, members):
        self.st, self.slots = stepper, [m[0] for m in members]
        self.last = [m[1] for m in members]
        self.max_steps = min(m[2] for m in members)
        self.queue = []
        self.launched = 0

    def launch(self):
        assert self.launched < self.max_steps, "launched beyond the first cap"
        # the device feeds every member its last pick, whatever the host knows by now
        picks = self.st._step([(s, [t]) for s, t in zip(self.slots, self.last)])
        self.last = picks
        self.queue.append(picks)
        self.launched += 1

    def read(self):
        return self.queue.pop(0)

    def finish(self, kept):
        assert not self.queue, "steps left unread"
        assert all(0 <= k <= self.launched for k in kept)
        self.kept = kept
        self.st.open_runs -= 1
        # what a member was fed beyond what it keeps does not count
        for slot, k in zip(self.slots, kept):
            st = self.st.seq[slot]
            extra = self.launched - k
            if extra:
                del st[1][-extra:]
                st[2] -= extra

    def abandon(self):
        self.st.open_runs -= 1


def test_unequal_batch_stops_and_caps():
    scripts = {1: [10, 11, 99, 12], 2: [20, 21, 22, 23, 24, 25], 3: [99]}
    st = ScriptedStepper(scripts)
    reqs = [Request([1, 5, 5], 10, {99}), Request([2], 4, {99}), Request([3] * 7, 10, {99})]
    out = generate(st, reqs)
    assert [o.tokens for o in out] == [[10, 11, 99], [20, 21, 22, 23], [99]]
    assert [o.stopped for o in out] == [True, False, True]
    # the prompts in one step with their unequal lengths, then one token each; a sequence
    # that ended at its prompt is absent from the first run
    assert st.calls[0] == [(0, 3), (1, 1), (2, 7)]
    assert st.calls[1] == [(0, 1), (1, 1)]
    assert st.calls[2] == [(0, 1), (1, 1)]
    # request 0 stops in the second decode step; request 1 reaches its cap of 4 picks in the
    # third, which is the run's last: no step is launched beyond a cap, and request 0's stop
    # token was fed in that third step only because the host read the second a step late
    assert len(st.calls) == 4 and st.calls[3] == [(0, 1), (1, 1)]
    assert st.opened == st.closed == 3 and len(st.free) == 4


def test_a_stop_read_a_step_late_costs_no_token():
    """A sequence stops while the others go on for long: the step that was queued before the
    host read the stop counts for the others, and the next run starts without the one that
    stopped."""
    scripts = {1: [10, 99, 11, 12, 13], 2: list(range(20, 40))}
    st = ScriptedStepper(scripts)
    out = generate(st, [Request([1], 10, {99}), Request([2, 2], 9, {99})])
    assert [o.tokens for o in out] == [[10, 99], list(range(20, 29))]
    two = [c for c in st.calls[1:] if len(c) == 2]
    one = [c for c in st.calls[1:] if len(c) == 1]
    # request 0: pick 10 at the prompt, 99 in decode step 1; step 2 was queued with both
    assert len(two) == 2 and len(one) == 9 - 1 - 2
    assert all(c == [(1, 1)] for c in one)


def test_batches_one_after_another_reuse_slots():
    scripts = {k: [k * 10 + i for i in range(8)] for k in range(1, 8)}
    st = ScriptedStepper(scripts, max_batch=3)
    reqs = [Request([k] * k, 2 + k % 3) for k in range(1, 8)]
    out = generate(st, reqs)
    assert [o.tokens for o in out] == [scripts[k][:2 + k % 3] for k in range(1, 8)]
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
    assert plan_batches(reqs, 8, [(4, 0)]) == [[0, 1, 2], [3]]     # 2 + 1 + 1 pages, then 4
    assert plan_batches(reqs, 2, [(64, 0)]) == [[0, 1], [2, 3]]
    with pytest.raises(InferError, match="pages"):
        plan_batches(reqs, 8, [(3, 0)])


def test_batches_count_pages_per_group():
    """A windowed group keeps a ring of pages per sequence however long it grows: its small
    pool must not refuse or split what fits (a full group of 512 pages beside a ring of 81)."""
    long = [Request([1] * 10000, 1) for _ in range(4)]
    assert pages_needed([(512, 0), (81, 81)], 10000) == [157, 81]
    assert plan_batches(long[:1], 1, [(512, 0), (81, 81)]) == [[0]]
    # four slots: the full pool holds three such requests (3 x 157 <= 512), the ring pool four
    assert plan_batches(long, 4, [(512, 0), (4 * 81, 81)]) == [[0, 1, 2], [3]]
    assert plan_batches(long, 4, [(1024, 0), (4 * 81, 81)]) == [[0, 1, 2, 3]]
    # and the ring pool limits when it is the scarce one
    assert plan_batches(long, 4, [(1024, 0), (2 * 81, 81)]) == [[0, 1], [2, 3]]
    with pytest.raises(InferError, match="needs 157 pages"):
        plan_batches(long[:1], 1, [(100, 0), (81, 81)])


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
