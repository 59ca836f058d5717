"""The generation loop's decisions, driven by a fake backend (CPU)."""
import pytest

from llmi_b200.engine.generate import Request, plan_batches, run_batches


class FakeBackend:
    """Chooses (sum of all tokens fed so far to the slot) % 50; records every step."""

    def __init__(self, n_slots):
        self.free_slots = list(range(n_slots))
        self.history = {}
        self.steps = []
        self.freed = []

    def alloc(self):
        s = self.free_slots.pop(0)
        self.history[s] = []
        return s

    def free(self, slot):
        assert slot in self.history, "freed twice"
        del self.history[slot]
        self.free_slots.append(slot)
        self.freed.append(slot)

    def step(self, entries):
        self.steps.append([(slot, r.index, list(toks)) for slot, r, toks in entries])
        out = []
        for slot, r, toks in entries:
            self.history[slot] += toks
            out.append(sum(self.history[slot]) % 50)
        return out


def expected_stream(prompt, n):
    hist, out = list(prompt), []
    for _ in range(n):
        out.append(sum(hist) % 50)
        hist.append(out[-1])
    return out


def test_prompts_run_together_then_one_token_each():
    reqs = [Request(0, [1, 2, 3], 4), Request(1, [7], 2), Request(2, [5, 5, 5, 5, 5], 4)]
    be = FakeBackend(3)
    steps = run_batches([reqs], be)
    assert steps == 4
    assert [len(t) for _, _, t in be.steps[0]] == [3, 1, 5]                    # whole prompts, one step
    assert all(len(t) == 1 for st in be.steps[1:] for _, _, t in st)           # then one token each
    assert [len(st) for st in be.steps] == [3, 3, 2, 2]                        # request 1 left after two tokens
    for r in reqs:
        assert r.output == expected_stream(r.prompt, r.max_new) and r.finish == "length"
    assert len(be.steps[-1]) == 2 and sorted(be.freed) == [0, 1, 2] and not be.history
    # the last chosen token is never fed forward
    fed = [t for st in be.steps for _, i, t in st if i == 0]
    assert fed == [[1, 2, 3]] + [[t] for t in reqs[0].output[:-1]]


def test_stop_token_is_kept_and_ends_the_sequence_at_once():
    free = expected_stream([4, 9], 6)
    stop = free[2]
    reqs = [Request(0, [4, 9], 6), Request(1, [30], 6)]
    be = FakeBackend(2)
    run_batches([reqs], be, stop_ids=[stop])
    first_stop = free.index(stop)
    assert reqs[0].output == free[:first_stop + 1] and reqs[0].finish == "stop"
    other = expected_stream([30], 6)
    cut = next((i + 1 for i, t in enumerate(other) if t == stop), 6)
    assert reqs[1].output == other[:cut]
    assert be.freed[0] == 0 or reqs[1].finish == "stop"


def test_batches_run_one_after_another_and_reuse_slots():
    reqs = [Request(i, [i + 1] * (i + 1), 3) for i in range(5)]
    batches = plan_batches(reqs, max_batch=2, max_tokens=64 * 2)
    assert [[r.index for r in b] for b in batches] == [[0, 1], [2, 3], [4]]
    be = FakeBackend(2)                       # only two slots exist: later batches must reuse them
    run_batches(batches, be)
    for r in reqs:
        assert r.output == expected_stream(r.prompt, 3)
    assert len(be.freed) == 5 and set(be.freed) == {0, 1}
    # nothing joins a running batch: every step's requests belong to one batch
    for st in be.steps:
        ids = {i for _, i, _ in st}
        assert any(ids <= {r.index for r in b} for b in batches)


def test_plan_respects_cache_tokens_and_order():
    reqs = [Request(0, [1] * 60, 5), Request(1, [1] * 10, 200), Request(2, [1] * 64, 1), Request(3, [1], 1)]
    # needs in cache tokens: 64, 256 (10 + 199 -> 4 pages), 64, 64
    b = plan_batches(reqs, max_batch=8, max_tokens=320)
    assert [[r.index for r in x] for x in b] == [[0, 1], [2, 3]]
    with pytest.raises(ValueError, match="needs 256 cache tokens"):
        plan_batches(reqs, max_batch=8, max_tokens=128)


def test_zero_new_tokens_runs_nothing():
    reqs = [Request(0, [1, 2], 0), Request(1, [3], 1)]
    be = FakeBackend(1)
    assert run_batches([reqs], be) == 1
    assert reqs[0].output == [] and reqs[0].finish == "length" and reqs[1].output == expected_stream([3], 1)
