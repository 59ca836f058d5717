"""The index block of a step, checked on the CPU: what plan_step writes, and that the patched block of a
continued decode step (continue_decode_step) is the block that planning anew would give."""
import numpy as np
import pytest
import torch

from llmi_b200.cache.pages import CacheError
from llmi_b200.cache.storage import KVRequest, SequenceCache
from llmi_b200.engine.batch import SequenceStep, StepError, continue_decode_step, plan_step


class HostBuffers:
    """Stands in for StepBuffers without a GPU: two alternating host blocks and a 'device' block."""

    def __init__(self, n=8192):
        self.hosts = [torch.zeros(n, dtype=torch.int32), torch.zeros(n, dtype=torch.int32)]
        self.dev = torch.zeros(n, dtype=torch.int32)
        self.turn = 0
        self.serial = 0

    def stage(self, n):
        self.turn ^= 1
        self.serial += 1
        self.hosts[self.turn].fill_(-99)            # whatever a block held before must not matter
        return self.hosts[self.turn], self.dev

    def upload(self, n):
        self.dev[:n] = self.hosts[self.turn][:n]


def make_cache(window=0, n_slots=6, max_tokens=64 * 24):
    reqs = [(KVRequest(2, 16, 0), 2)]
    if window:
        reqs.append((KVRequest(1, 16, window), 1))
    return SequenceCache(reqs, [], max_tokens=max_tokens, max_positions=1000, dtype=torch.float32, device="meta",
                         page_size=64, n_slots=n_slots)


def test_block_of_a_prompt_step():
    cache = make_cache()
    a, b = cache.alloc_slot(), cache.alloc_slot()
    buf = HostBuffers()
    ctx = plan_step(cache, [SequenceStep(a, [5, 6, 7], [0, 2]), SequenceStep(b, [9, 8], [1])], 50, buf)
    assert ctx.token_ids.tolist() == [5, 6, 7, 9, 8]
    assert ctx.tok_seq.tolist() == [0, 0, 0, 1, 1]
    assert ctx.tok_pos.tolist() == [0, 1, 2, 0, 1]
    assert ctx.want_rows.tolist() == [0, 2, 4]
    assert ctx.seq_q_start.tolist() == [0, 3, 5]
    assert ctx.seq_kv_len.tolist() == [3, 2]
    assert ctx.seq_slot.tolist() == [a, b]
    assert not ctx.decode and ctx.max_kv_len == 3
    pages = ctx.pages_of(cache.kv_groups[0])
    assert pages.shape == (2, 1) and pages[0, 0] != pages[1, 0]


def test_block_of_a_step_that_continues_by_several_tokens():
    """Sequences already hold tokens; one goes on by three, one by one, one starts: positions go on from each
    sequence's length, lengths are length + new tokens, and the page tables cover the earlier positions too."""
    cache = make_cache()
    a, b, c = cache.alloc_slot(), cache.alloc_slot(), cache.alloc_slot()
    buf = HostBuffers()
    plan_step(cache, [SequenceStep(a, [1] * 62, []), SequenceStep(b, [2] * 10, [])], 50, buf)
    ctx = plan_step(cache, [SequenceStep(a, [5, 6, 7], [2]), SequenceStep(b, [9], [0]), SequenceStep(c, [1, 2], [0, 1])], 50, buf)
    assert not ctx.decode
    assert ctx.tok_pos.tolist() == [62, 63, 64, 10, 0, 1]
    assert ctx.tok_seq.tolist() == [0, 0, 0, 1, 2, 2]
    assert ctx.seq_kv_len.tolist() == [65, 11, 2]
    assert ctx.seq_q_start.tolist() == [0, 3, 4, 6]
    assert ctx.want_rows.tolist() == [2, 3, 4, 5]
    assert ctx.host_q_lens == [3, 1, 2] and ctx.host_kv_lens == [65, 11, 2]
    pages = ctx.pages_of(cache.kv_groups[0])
    assert pages.shape == (3, 2) and pages[0, 1] >= 0 and pages[1, 1] == -1
    assert cache.length(a) == 65 and cache.length(b) == 11 and cache.length(c) == 2


def test_block_of_a_prompt_step_padded_to_a_shape():
    """A prompt step padded for replay: token rows of no sequence (-1) up to the asked number, padding sequences
    without tokens, wanted rows that point nowhere, page tables of the asked width — and the real entries, the
    cache's lengths and the last entry of the sequence starts as in the step without padding."""
    cache = make_cache()
    a, b, c = cache.alloc_slot(), cache.alloc_slot(), cache.alloc_slot()
    buf = HostBuffers()
    plan_step(cache, [SequenceStep(a, [1] * 70, [])], 50, buf)
    ctx = plan_step(cache, [SequenceStep(a, [5, 6, 7], [0, 2]), SequenceStep(b, [9, 8], [1]), SequenceStep(c, [4], [])], 50, buf,
                    pad_seqs_to=4, pad_pages_to=4, pad_tokens_to=64, pad_want_to=4)
    assert not ctx.decode and ctx.n_tokens == 64 and ctx.n_seqs == 4 and ctx.n_want == 4 and ctx.n_want_real == 3
    assert ctx.token_ids.tolist() == [5, 6, 7, 9, 8, 4] + [-1] * 58
    assert ctx.tok_seq.tolist() == [0, 0, 0, 1, 1, 2] + [-1] * 58
    assert ctx.tok_pos.tolist() == [70, 71, 72, 0, 1, 0] + [0] * 58
    assert ctx.want_rows.tolist() == [0, 2, 4, -1]
    assert ctx.seq_q_start.tolist() == [0, 3, 5, 6, 6]
    assert ctx.seq_kv_len.tolist() == [73, 2, 1, 0]
    assert ctx.seq_slot.tolist() == [a, b, c, -1]
    assert ctx.host_q_lens is None and ctx.n_q_blocks == 64 // 128 + 4
    pages = ctx.pages_of(cache.kv_groups[0])
    assert pages.shape == (4, 4) and (pages[3] == -1).all() and pages[0, 1] >= 0 and pages[0, 2] == -1
    assert cache.length(a) == 73 and cache.length(b) == 2 and cache.length(c) == 1
    cache.check()


@pytest.mark.parametrize("window", [0, 100])
def test_continued_decode_step_equals_planning_anew(window):
    """Two caches in lockstep: one is stepped by plan_step every time, the other by continue_decode_step.
    Lengths start near a page's end so that pages are taken (and, with a window, given back) on the way."""
    caches = [make_cache(window), make_cache(window)]
    bufs = [HostBuffers(), HostBuffers()]
    starts = [60, 127, 3, 190]
    slots = []
    for c in caches:
        ss = [c.alloc_slot() for _ in starts]
        for s, n in zip(ss, starts):
            c.extend(s, n)
        slots.append(ss)
    assert slots[0] == slots[1]
    rng = np.random.default_rng(0)
    prev = None
    for step in range(140):
        toks = rng.integers(0, 50, len(starts)).tolist()
        seqs = [SequenceStep(s, [t], [0]) for s, t in zip(slots[0], toks)]
        ref = plan_step(caches[0], seqs, 50, bufs[0], pad_seqs_to=4, pad_pages_to=8)
        n = ref.layout.n_int32
        if prev is None:
            prev = plan_step(caches[1], seqs, 50, bufs[1], pad_seqs_to=4, pad_pages_to=8)
        else:
            continue_decode_step(caches[1], prev, toks, 50, bufs[1])
        assert prev.layout.n_int32 == n
        assert torch.equal(bufs[0].dev[:n], bufs[1].dev[:n]), f"step {step}"
        assert prev.max_kv_len == ref.max_kv_len
        for c in caches:
            c.check()
    for g0, g1 in zip(caches[0].kv_groups, caches[1].kv_groups):
        assert g0.pool.n_free == g1.pool.n_free
        for s in slots[0]:
            assert g0.pool.table(s) == g1.pool.table(s) and g0.pool.length(s) == g1.pool.length(s)


def test_continued_decode_step_refusals_change_nothing():
    cache = make_cache(max_tokens=64 * 2, n_slots=2)
    a, b = cache.alloc_slot(), cache.alloc_slot()
    cache.extend(a, 63)
    cache.extend(b, 64)                  # both pages are taken now; b's next token needs a third
    buf = HostBuffers()
    with pytest.raises(CacheError, match="cache is full"):
        plan_step(cache, [SequenceStep(a, [1], [0]), SequenceStep(b, [1], [0])], 50, buf, pad_seqs_to=2, pad_pages_to=2)
    cache.free_slot(b)
    b = cache.alloc_slot()
    cache.extend(b, 5)
    ctx = plan_step(cache, [SequenceStep(a, [1], [0]), SequenceStep(b, [1], [0])], 50, buf, pad_seqs_to=2, pad_pages_to=2)
    assert (cache.length(a), cache.length(b)) == (64, 6)
    with pytest.raises(StepError, match="out of range"):
        continue_decode_step(cache, ctx, [1, 50], 50, buf)
    with pytest.raises(CacheError, match="cache is full"):      # a's next token needs a page, none is free
        continue_decode_step(cache, ctx, [1, 2], 50, buf)
    assert (cache.length(a), cache.length(b)) == (64, 6)
    for g in cache.kv_groups:
        assert g.pool.length(a) == 64 and g.pool.length(b) == 6
    cache.check()
    cache.free_slot(b)
    with pytest.raises(CacheError, match="not live"):
        continue_decode_step(cache, ctx, [1, 2], 50, buf)


def test_a_step_that_does_not_fit_a_windowed_group_reserves_nothing():
    """A global group with room and a windowed group without: the step is refused before anything is reserved, in
    every group and for every slot, for a prompt step and for a continued decode step."""
    reqs = [(KVRequest(2, 16, 0), 1), (KVRequest(1, 16, 64), 1)]
    cache = SequenceCache(reqs, [], max_tokens=64 * 4, max_positions=1000, dtype=torch.float32, device="meta",
                          page_size=64, n_slots=4)
    glob, win = cache.kv_groups[0].pool, cache.kv_groups[1].pool
    a, b = cache.alloc_slot(), cache.alloc_slot()
    buf = HostBuffers()
    plan_step(cache, [SequenceStep(a, [1] * 64, []), SequenceStep(b, [1] * 64, [])], 50, buf)     # 2 of 4 pages each group
    c = cache.alloc_slot()
    before = (glob.n_free, win.n_free, cache.length(a), cache.length(b), cache.length(c))
    with pytest.raises(CacheError, match="full"):        # a and b take one page each, c would need two more
        plan_step(cache, [SequenceStep(a, [1], []), SequenceStep(b, [1], []), SequenceStep(c, [1] * 65, [])], 50, buf)
    assert (glob.n_free, win.n_free, cache.length(a), cache.length(b), cache.length(c)) == before
    assert glob.length(a) == 64 and win.length(a) == 64
    cache.check()
    # the windowed group alone is out of pages: fill it with a third sequence whose window holds two pages
    plan_step(cache, [SequenceStep(c, [1] * 128, [])], 50, buf)
    assert win.n_free == 0 and glob.n_free == 0
    ctx = None
    with pytest.raises(CacheError, match="full"):
        plan_step(cache, [SequenceStep(a, [1], [])], 50, buf)
    assert cache.length(a) == 64 and glob.length(a) == 64 and win.length(a) == 64
    cache.check()


def test_a_window_gives_back_a_long_prompts_dead_pages_at_the_next_step():
    """After a prompt of five pages a window of 64 positions needs two of them: the first decode step gives back
    the other three at once, not one at every later page end, and both ways of growing agree."""
    for grow in ("plan", "continue"):
        reqs = [(KVRequest(1, 16, 64), 1)]
        cache = SequenceCache(reqs, [], max_tokens=64 * 6, max_positions=1000, dtype=torch.float32, device="meta",
                              page_size=64, n_slots=2)
        pool = cache.kv_groups[0].pool
        a = cache.alloc_slot()
        buf = HostBuffers()
        plan_step(cache, [SequenceStep(a, [1] * 300, [])], 50, buf)
        assert pool.n_free == 1
        ctx = plan_step(cache, [SequenceStep(a, [2], [0])], 50, buf, pad_seqs_to=1, pad_pages_to=8)
        # position 300 sees 237..300: pages 0, 1, 2 are dead (page 3 starts at 192)
        assert pool.n_free == 4 and pool.table(a)[:3] == [-1, -1, -1] and pool.table(a)[3] >= 0
        if grow == "continue":
            continue_decode_step(cache, ctx, [3], 50, buf)
        else:
            plan_step(cache, [SequenceStep(a, [3], [0])], 50, buf)
        assert pool.n_free == 4 and cache.length(a) == 302
        cache.check()


def snapshot(cache):
    g = cache.kv_groups[0].pool
    return (sorted(g._free), {s: list(t) for s, t in g._pages.items()}, dict(g._length), dict(cache._length),
            g.matrix.copy().tolist())


def test_a_step_laid_out_ahead_equals_planning_anew_and_can_be_taken_back():
    """prepare_continue / finish_continue (the next decode step's block made while the device still runs this one)
    against plan_step, over page ends; a reservation that is not used leaves no trace, whatever happens meanwhile."""
    from llmi_b200.engine.batch import finish_continue, prepare_continue
    rng = np.random.default_rng(1)
    starts = [60, 127, 3, 190]
    caches, bufs, slots = [make_cache(), make_cache()], [HostBuffers(), HostBuffers()], []
    for c, b in zip(caches, bufs):
        ss = [c.alloc_slot() for _ in starts]
        plan_step(c, [SequenceStep(s, [1] * n, []) for s, n in zip(ss, starts)], 50, b)
        slots.append(ss)
    prev = None
    for step in range(140):
        toks = rng.integers(0, 50, len(starts)).tolist()
        ref = plan_step(caches[0], [SequenceStep(s, [t], [0]) for s, t in zip(slots[0], toks)], 50, bufs[0], pad_seqs_to=4, pad_pages_to=8)
        if prev is None:
            prev = plan_step(caches[1], [SequenceStep(s, [t], [0]) for s, t in zip(slots[1], toks)], 50, bufs[1], pad_seqs_to=4, pad_pages_to=8)
        else:
            before = snapshot(caches[1])
            lens = [caches[1].length(s) for s in slots[1]]
            pending = prepare_continue(caches[1], prev, bufs[1])
            assert [caches[1].length(s) for s in slots[1]] == lens        # a reservation does not count as length
            if step % 7 == 3:                          # now and then something else comes first: the reservation goes back
                caches[1].settle()                     # and the step is planned the ordinary way
                assert snapshot(caches[1]) == before
                prev = plan_step(caches[1], [SequenceStep(s, [t], [0]) for s, t in zip(slots[1], toks)], 50, bufs[1],
                                 pad_seqs_to=4, pad_pages_to=8)
            else:
                finish_continue(caches[1], prev, pending, toks, 50, bufs[1])
            assert [caches[1].length(s) for s in slots[1]] == [n + 1 for n in lens]
        n = ref.layout.n_int32
        assert bufs[0].dev[:n].tolist() == bufs[1].dev[:n].tolist(), step
        assert prev.max_kv_len == ref.max_kv_len
        caches[1].check()


def test_reservations_ahead_and_everything_else_that_touches_the_cache():
    from llmi_b200.engine.batch import finish_continue, prepare_continue
    cache = make_cache(max_tokens=64 * 4, n_slots=4)
    a, b = cache.alloc_slot(), cache.alloc_slot()
    buf = HostBuffers()
    plan_step(cache, [SequenceStep(a, [1] * 63, []), SequenceStep(b, [1] * 64, [])], 50, buf)
    ctx = plan_step(cache, [SequenceStep(a, [1], [0]), SequenceStep(b, [1], [0])], 50, buf, pad_seqs_to=2, pad_pages_to=4)
    pool = cache.kv_groups[0].pool
    assert pool.n_free == 1                               # a: 1 page (64 positions), b: 2 pages
    # the next step ahead: a opens its second page
    before = snapshot(cache)
    prepare_continue(cache, ctx, buf)
    assert pool.n_free == 0 and cache.length(a) == 64 and cache.length(b) == 65
    # a sequence ends instead: its slot is freed with the reservation; the other's reservation goes back on the next touch
    cache.free_slot(a)
    assert cache.length(b) == 65
    c = cache.alloc_slot()                                # settles
    assert pool.n_free == 2 and pool.length(b) == 65 and cache.length(b) == 65
    cache.check()
    # a prompt in between (plan_step) takes the reservation back before it reserves its own room
    ctx = plan_step(cache, [SequenceStep(b, [1], [0])], 50, buf, pad_seqs_to=1, pad_pages_to=4)
    prepare_continue(cache, ctx, buf)
    plan_step(cache, [SequenceStep(c, [1] * 128, [])], 50, buf)       # would not fit if b's reservation... it does fit: 2 pages free
    assert cache.length(b) == 66 and cache.length(c) == 128 and pool.n_free == 0
    # no room for a reservation: refused, nothing changes; a bad token takes the reservation back
    ctx = plan_step(cache, [SequenceStep(b, [1], [0])], 50, buf, pad_seqs_to=1, pad_pages_to=4)
    for _ in range(60):
        pending = prepare_continue(cache, ctx, buf)
        finish_continue(cache, ctx, pending, [1], 50, buf)
    assert cache.length(b) == 127
    pending = prepare_continue(cache, ctx, buf)
    with pytest.raises(StepError, match="out of range"):
        finish_continue(cache, ctx, pending, [50], 50, buf)
    assert cache.length(b) == 127 and pool.length(b) == 127
    pending = prepare_continue(cache, ctx, buf)
    finish_continue(cache, ctx, pending, [2], 50, buf)
    before = snapshot(cache)
    with pytest.raises(CacheError, match="full"):          # position 128 needs a page and none is free
        prepare_continue(cache, ctx, buf)
    assert snapshot(cache) == before
    cache.check()
    # a windowed group cannot reserve ahead
    w = make_cache(window=100)
    s = w.alloc_slot()
    ctx = plan_step(w, [SequenceStep(s, [1], [0])], 50, buf, pad_seqs_to=1, pad_pages_to=4)
    assert not w.can_speculate()
    with pytest.raises(CacheError, match="windowed"):
        prepare_continue(w, ctx, buf)


def test_shapes_that_prompt_steps_are_padded_to():
    """Token rows go up to 16, 32, a multiple of 64 (of 128 from 512 tokens on); longer prompts are not padded."""
    from llmi_b200.engine.graphs import bucket, prompt_bucket
    assert [prompt_bucket(n) for n in (1, 16, 17, 32, 33, 64, 65, 500, 512, 513, 640, 641, 1024)] == \
        [16, 16, 32, 32, 64, 64, 128, 512, 512, 640, 640, 768, 1024]
    assert prompt_bucket(1025) == 0 and prompt_bucket(4096) == 0
    for n in range(1, 1025):
        assert prompt_bucket(n) >= n and prompt_bucket(n) - n < 128
    assert [bucket(n) for n in (1, 2, 3, 5, 8, 9, 64, 65)] == [1, 2, 4, 8, 8, 16, 64, 128]
