"""The scheduler's decisions, on the host with a stand-in for the model: admission order, the
token budget, portions, decode rows, preemption when pages run out, finishing and freeing."""
import pytest

from llm_steadyinfer_b200.cache import CacheLayout, CacheManager
from llm_steadyinfer_b200.engine.scheduler import RequestRejected, Scheduler, SeqState
from llm_steadyinfer_b200.parts.base import CacheNeed, StateNeed
from llm_steadyinfer_b200.sampling import SamplingParams


def make(num_pages=64, page_size=4, max_seqs=4, budget=16, max_len=256, max_gen=8, prefix=False, eos=(), layout=None):
    layout = layout or CacheLayout([CacheNeed(1, 8, None)], [None])
    cache = CacheManager(layout, page_size, num_pages, max_seqs, prefix)
    return Scheduler(cache, max_seqs, max_len, max_gen, token_budget=budget, eos_token_ids=eos), cache


def run_step(s, cache, next_token=lambda seq: 100 + len(seq.outputs)):
    """What the engine does around the model: commit the lengths, hand back one token per wanted row."""
    items = s.schedule()
    for it in items:
        assert cache.length(it.seq.id) == it.start, "a portion starts where the cache ends"
        assert cache.blocks_for(it.start + it.count) <= len(cache.table(0, it.seq.id)), "pages are there"
        cache.commit(it.seq.id, it.start + it.count)
    sampled = {it.seq.id: next_token(it.seq) for it in items if it.want_logits}
    s.update(items, sampled)
    cache.check_invariant()
    return items


def test_portions_under_the_budget_and_decode_rows_first():
    s, cache = make(budget=16)
    a = s.add_request(list(range(40)))
    b = s.add_request(list(range(5)))
    it = run_step(s, cache)
    assert [(i.seq.id, i.start, i.count, i.want_logits) for i in it] == [(a, 0, 16, False)]
    it = run_step(s, cache)
    assert [(i.seq.id, i.start, i.count) for i in it] == [(a, 16, 16)]
    it = run_step(s, cache)                                   # a's last 8, then 5 of b fill the budget
    assert [(i.seq.id, i.start, i.count, i.want_logits) for i in it] == [(a, 32, 8, True), (b, 0, 5, True)]
    it = run_step(s, cache)                                   # both decode now
    assert [(i.seq.id, i.start, i.count, i.want_logits) for i in it] == [(a, 40, 1, True), (b, 5, 1, True)]
    c = s.add_request(list(range(30)))
    it = run_step(s, cache)                                   # decode rows first, then the new prompt
    assert [(i.seq.id, i.count) for i in it] == [(a, 1), (b, 1), (c, 16)]


def test_finishing_frees_and_reasons():
    s, cache = make(max_gen=3, eos=[7])
    a = s.add_request([1, 2, 3])
    b = s.add_request([4, 5], SamplingParams(max_tokens=10))
    c = s.add_request([6], SamplingParams(max_tokens=10, ignore_eos=True, stop_token_ids=(9,)))
    toks = {a: [11, 12, 13, 14], b: [21, 7, 22], c: [7, 8, 9, 10]}
    while s.has_unfinished():
        run_step(s, cache, lambda seq: toks[seq.id][len(seq.outputs)])
    fin = {q.id: q for q in s.finished}
    assert fin[a].outputs == [11, 12, 13] and fin[a].finish_reason == "length"
    assert fin[b].outputs == [21, 7] and fin[b].finish_reason == "eos"
    assert fin[c].outputs == [7, 8, 9] and fin[c].finish_reason == "eos"
    assert cache.free_pages() == 64 and not cache.requests


def test_rejections_and_max_gen_clamp():
    s, cache = make(max_len=16, num_pages=3, max_gen=100)
    with pytest.raises(RequestRejected):
        s.add_request([])
    with pytest.raises(RequestRejected):
        s.add_request(list(range(16)))                        # no room to generate
    with pytest.raises(RequestRejected):
        s.add_request(list(range(12)))                        # 13 tokens do not fit 3 pages of 4
    s.add_request(list(range(10)))
    assert s.waiting[0].max_gen == 6                          # clamped to max_len - prompt


def test_admission_is_fcfs_and_waits_for_pages_and_slots():
    s, cache = make(num_pages=10, max_seqs=2, budget=64, max_gen=2)
    a = s.add_request(list(range(20)))                        # 5 pages
    b = s.add_request(list(range(24)))                        # 6 pages: does not fit beside a
    c = s.add_request(list(range(4)))                         # would fit, but b is first in line
    it = run_step(s, cache)
    assert [i.seq.id for i in it] == [a] and [q.id for q in s.waiting] == [b, c]
    while any(q.id == a for q in s.running):
        run_step(s, cache)
    it = run_step(s, cache)
    assert {i.seq.id for i in it} == {b, c}
    d = s.add_request([1])
    run_step(s, cache)
    assert [q.id for q in s.waiting] == [d], "two are running: the third waits for a slot"


def test_decode_growth_preempts_the_newest_and_it_recomputes():
    s, cache = make(num_pages=6, page_size=4, max_seqs=3, budget=64, max_gen=12)
    a = s.add_request(list(range(7)))                         # 2 pages
    b = s.add_request(list(range(6)))                         # 2 pages
    c = s.add_request(list(range(5)))                         # 2 pages: the pool is full
    run_step(s, cache)                                        # prompts, first tokens: 8, 7, 6 tokens known
    assert cache.free_pages() == 0
    it = run_step(s, cache)                                   # a writes position 7: still page 2
    assert [i.seq.id for i in it] == [a, b, c]
    it = run_step(s, cache)                                   # a needs a third page: c, the newest, gives one
    seqs = {q.id: q for q in list(s.running) + list(s.waiting)}
    assert seqs[c].state is SeqState.PREEMPTED and s.waiting[0].id == c
    assert [i.seq.id for i in it] == [a, b]
    assert seqs[c].num_computed == 4 and cache.length(c) == 4 and len(cache.table(0, c)) == 1
    assert seqs[c].outputs == [100, 101], "generated tokens are kept"
    n_before = s.num_preemptions
    while s.has_unfinished():
        run_step(s, cache)
    fin = {q.id: q for q in s.finished}
    assert all(fin[r].finish_reason == "length" and len(fin[r].outputs) == 12 for r in (a, b, c))
    assert fin[c].num_preemptions >= 1 and s.num_preemptions >= n_before
    assert cache.free_pages() == 6


def test_recompute_after_preemption_runs_known_tokens_as_a_portion():
    s, cache = make(num_pages=4, page_size=4, max_seqs=2, budget=64, max_gen=6)
    a = s.add_request(list(range(6)))
    b = s.add_request(list(range(6)))
    for _ in range(3):
        run_step(s, cache)                                    # both hold 2 pages, 8 tokens known each
    it = run_step(s, cache)                                   # a needs page 3 -> b preempted (keeps 1 page)
    assert [i.seq.id for i in it] == [a]
    bq = s.waiting[0]
    assert bq.id == b and bq.num_computed == 4
    while any(q.id == a for q in s.running):
        run_step(s, cache)
    it = run_step(s, cache)                                   # b comes back: recomputes 4..end in one portion
    assert [(i.seq.id, i.start, i.want_logits) for i in it] == [(b, 4, True)]
    assert it[0].count == len(bq.prompt) + len(bq.outputs) - 1 - 4, "all known tokens but the newest were stored before"
    while s.has_unfinished():
        run_step(s, cache)
    assert cache.free_pages() == 4


def test_alone_and_too_large_is_aborted_not_hung():
    s, cache = make(num_pages=2, page_size=4, max_seqs=2, budget=64, max_gen=50)
    a = s.add_request(list(range(5)))
    steps = 0
    while s.has_unfinished():
        run_step(s, cache)
        steps += 1
        assert steps < 20
    assert s.finished[0].finish_reason == "aborted" and len(s.finished[0].outputs) == 4   # 5 + 4 = 9 > 8 slots
    assert cache.free_pages() == 2


def test_newest_waits_for_older_ones_instead_of_cutting_them():
    s, cache = make(num_pages=5, page_size=4, max_seqs=2, budget=64, max_gen=6)
    a = s.add_request(list(range(11)))                        # 3 pages, room for 12 tokens
    b = s.add_request(list(range(6)))                         # 2 pages, room for 8
    run_step(s, cache); run_step(s, cache)                    # a: 13 known? no: a has 12 known -> needs page at 13
    while s.has_unfinished():
        run_step(s, cache)
    fin = {q.id: q for q in s.finished}
    assert len(fin[a].outputs) == 6 and len(fin[b].outputs) == 6
    assert fin[a].num_preemptions == 0, "the older request is never cut for the newer one"


def test_adaptive_budget_moves_one_doubling_per_step():
    s, cache = make(num_pages=4096, page_size=16, max_seqs=8, budget="adaptive", max_len=20000, max_gen=4)
    assert s.token_budget == 1024
    s.add_request(list(range(9000)))
    counts = []
    for _ in range(4):
        counts.append(run_step(s, cache)[0].count)
    assert counts == [2048, 4096, 2856][:len(counts)] or counts[:2] == [2048, 4096]
    for i in range(6):
        s.add_request(list(range(3)))
    s.add_request(list(range(9000)))
    for _ in range(3):
        run_step(s, cache)
    assert s.token_budget <= 2048, "decode pressure above a half shrinks the budget"


def test_prefix_hits_skip_computed_pages():
    s, cache = make(num_pages=32, page_size=4, max_seqs=1, budget=64, max_gen=2, prefix=True)
    shared = list(range(50, 62))
    a = s.add_request(shared + [1, 2, 3])
    while s.has_unfinished():
        run_step(s, cache)
    b = s.add_request(shared + [9])
    it = run_step(s, cache)
    assert [(i.start, i.count, i.want_logits) for i in it] == [(12, 1, True)]
    assert it[0].seq.prefix_hit_tokens == 12
    while s.has_unfinished():
        run_step(s, cache)
    cache.check_invariant()


def test_decode_step_decided_ahead_of_its_tokens():
    """``schedule_ahead``: the step after a step in flight, decided before that step's tokens are known. It
    holds the same requests one position further (their tokens fed on the device), leaves out a request that
    ends by length with the unread token, admits a waiting request with its prompt beside them, and declines
    (None) when a page is missing."""
    s, cache = make(num_pages=8, page_size=4, max_seqs=3, budget=64, max_gen=6)
    a = s.add_request([1, 2, 3], SamplingParams(max_tokens=6))
    b = s.add_request([4, 5, 6, 7, 8], SamplingParams(max_tokens=2))
    run_step(s, cache)                                  # prompts, first tokens
    items = s.schedule()                                # a decode step, "launched": lengths committed, not read
    assert [(it.seq.id, it.start, it.count) for it in items] == [(a, 3, 1), (b, 5, 1)]
    for it in items:
        cache.commit(it.seq.id, it.start + 1)
    ahead = s.schedule_ahead(items)
    # b has one output and may have two: the unread token ends it, so only a goes on
    assert [(it.seq.id, it.start, it.count, it.want_logits) for it in ahead] == [(a, 4, 1, True)]
    assert cache.blocks_for(6) <= len(cache.table(0, a))
    s.update(items, {a: 50, b: 51})
    for it in ahead:
        cache.commit(it.seq.id, it.start + 1)
    s.update(ahead, {a: 52})
    seq_a = next(q for q in s.running if q.id == a)
    assert seq_a.outputs[-2:] == [50, 52] and seq_a.num_computed == 5
    assert [q.id for q in s.finished] == [b]
    cache.check_invariant()
    assert all(it.fed for it in ahead)
    # a waiting request is admitted blind as well: its prompt runs beside the row that is fed
    items = s.schedule()
    for it in items:
        cache.commit(it.seq.id, it.start + 1)
    c = s.add_request([9] * 3)
    ahead = s.schedule_ahead(items)
    assert [(it.seq.id, it.start, it.count, it.want_logits, it.fed) for it in ahead] == \
        [(a, 6, 1, True, True), (c, 0, 3, True, False)]
    s.update(items, {a: 53})
    for it in ahead:
        cache.commit(it.seq.id, it.start + it.count)
    s.update(ahead, {a: 54, c: 60})
    assert seq_a.outputs[-2:] == [53, 54] and next(q for q in s.running if q.id == c).outputs == [60]
    cache.check_invariant()


def test_prompt_portions_go_on_in_the_step_ahead():
    """A prompt cut by the budget: the step ahead takes its next portion from where the step in flight leaves
    it, and the portion that reaches the prompt's end asks for logits; the step after that feeds its token."""
    s, cache = make(num_pages=16, page_size=4, max_seqs=2, budget=4, max_gen=4)
    a = s.add_request(list(range(1, 11)), SamplingParams(max_tokens=4))
    items = s.schedule()
    assert [(it.start, it.count, it.want_logits) for it in items] == [(0, 4, False)]
    cache.commit(a, 4)
    ahead = s.schedule_ahead(items)
    assert [(it.start, it.count, it.want_logits, it.fed) for it in ahead] == [(4, 4, False, False)]
    s.update(items, {})
    cache.commit(a, 8)
    third = s.schedule_ahead(ahead)
    assert [(it.start, it.count, it.want_logits, it.fed) for it in third] == [(8, 2, True, False)]
    s.update(ahead, {})
    cache.commit(a, 10)
    fourth = s.schedule_ahead(third)
    assert [(it.start, it.count, it.want_logits, it.fed) for it in fourth] == [(10, 1, True, True)]
    s.update(third, {a: 77})
    cache.commit(a, 11)
    s.update(fourth, {a: 78})
    assert s.running[0].outputs == [77, 78] and s.running[0].num_computed == 11
    cache.check_invariant()


def test_no_step_ahead_without_a_page():
    s, cache = make(num_pages=2, page_size=4, max_seqs=2, budget=64, max_gen=8)
    a = s.add_request([1, 2, 3, 4, 5, 6], SamplingParams(max_tokens=8))
    run_step(s, cache)                                  # 6 tokens: both pages taken
    items = s.schedule()                                # position 6 fits the second page
    cache.commit(a, 7)
    ahead = s.schedule_ahead(items)                     # position 7 still fits
    assert ahead is not None and ahead[0].start == 7
    s.update(items, {a: 70})
    cache.commit(a, 8)
    assert s.schedule_ahead(ahead) is None              # position 8 needs a third page: left to schedule()
    s.update(ahead, {a: 71})


def test_step_ahead_counts_pages_row_by_row():
    """Two requests that each need a new page for the step ahead and one free page: the step ahead is
    declined (the page that the first took stays with it), nothing is raised."""
    s, cache = make(num_pages=5, page_size=4, max_seqs=2, budget=64, max_gen=8)
    a = s.add_request([1, 2, 3], SamplingParams(max_tokens=8))
    b = s.add_request([4, 5, 6], SamplingParams(max_tokens=8))
    run_step(s, cache)                                  # prompts: one page each, lengths 3
    items = s.schedule()                                # position 3 of both: still the first page
    for it in items:
        cache.commit(it.seq.id, 4)
    assert cache.free_pages(0) == 3
    taken = cache.groups[0].pool.allocate(2)              # someone else takes two pages: one is left
    assert s.schedule_ahead(items) is None              # position 4 needs a second page for both
    s.update(items, {a: 7, b: 8})
    assert cache.free_pages(0) == 0
    cache.groups[0].pool.release(taken[0]); cache.groups[0].pool.release(taken[1])
    cache.check_invariant()


@pytest.mark.parametrize("reserve", ["prompt", "portion"])
@pytest.mark.parametrize("windowed", [False, True], ids=["one_group", "window_and_state"])
@pytest.mark.parametrize("seed", range(12))
def test_random_serving_with_and_without_steps_ahead(seed, windowed, reserve):
    """A stand-in model (the token of request r at output index i is a fixed function of both) under random
    arrivals, small pools, stop tokens and shared prefixes: with steps decided ahead where the scheduler allows
    it and without, every request ends with the same tokens and reason, and the cache keeps its books."""
    import random

    def token(seq, index):
        return (hash((seq.id, index)) % 97) + 3

    def serve(ahead):
        rng = random.Random(seed)
        # windowed: a layer with all keys, a layer with a window of 6 (its pages come back while requests
        # run, and nothing of a preempted request can be kept) and a layer with state of fixed size
        layout = CacheLayout([CacheNeed(1, 8, None), CacheNeed(1, 8, 6), None],
                             [None, None, StateNeed((3,))]) if windowed else None
        s, cache = make(num_pages=rng.choice([12, 20, 40]), page_size=4, max_seqs=4, budget=rng.choice([8, 32]),
                        max_len=64, max_gen=12, prefix=True, eos=(5, 6, 7), layout=layout)
        s.reserve = reserve
        shared = [11, 12, 13, 14, 15, 16, 17, 18]
        todo = []
        for i in range(16):
            prompt = [20 + rng.randrange(50) for _ in range(rng.choice([1, 3, 6, 10, 17]))]
            if rng.random() < 0.3:
                prompt = shared + prompt
            todo.append((rng.randrange(0, 30), prompt, SamplingParams(max_tokens=rng.choice([1, 2, 5, 12])), i))
        inflight, step, aheads = None, 0, 0
        while todo or s.has_unfinished() or inflight:
            for t in [t for t in todo if t[0] <= step]:
                todo.remove(t)
                s.add_request(t[1], t[2], req_id=f"r{t[3]}")
            step += 1
            items = inflight if inflight is not None else s.schedule()
            if inflight is None:
                for it in items:
                    cache.commit(it.seq.id, it.start + it.count)
            inflight = None
            if ahead and items:
                nxt = s.schedule_ahead(items)
                if nxt is not None:
                    for it in nxt:
                        cache.commit(it.seq.id, it.start + it.count)
                    inflight = nxt
                    aheads += 1
            # the index of the token a row draws: outputs so far, plus one when the row was decided ahead
            sampled = {it.seq.id: token(it.seq, it.start + it.count - len(it.seq.prompt)) for it in items if it.want_logits}
            s.update(items, sampled)
            cache.check_invariant()
            assert step < 5000
        assert not cache.requests
        return {q.id: (q.outputs, q.finish_reason) for q in s.finished}, aheads

    plain, _ = serve(False)
    piped, aheads = serve(True)
    assert plain == piped
    assert aheads > 0
    for outs, reason in plain.values():
        assert reason in ("eos", "length") and len(outs) >= 1, (outs, reason)


def test_an_id_cannot_be_live_twice():
    s, cache = make()
    s.add_request([1, 2, 3], req_id="a")
    with pytest.raises(RequestRejected):
        s.add_request([4, 5], req_id="a")
    run_step(s, cache)
    with pytest.raises(RequestRejected):
        s.add_request([4, 5], req_id="a")                # running now
    while s.has_unfinished():
        run_step(s, cache)
    s.add_request([4, 5], req_id="a")                    # ended: the id is free again
    assert s.add_request([6], req_id=None) != "a"


def test_default_seed_is_the_same_in_every_process():
    """A request that names no seed gets one from a digest of its id, not from Python's salted hash."""
    import subprocess
    import sys
    from llm_steadyinfer_b200.engine.scheduler import default_seed
    s, _ = make()
    s.add_request([1, 2, 3], SamplingParams(temperature=0.8), req_id="chat-17")
    s.add_request([1, 2, 3], SamplingParams(temperature=0.8, seed=5), req_id="chat-18")
    seeds = {q.id: q.seed for q in s.waiting}
    assert seeds == {"chat-17": default_seed("chat-17"), "chat-18": 5}
    assert default_seed("chat-17") != default_seed("chat-18") and 0 <= default_seed(("a", 1)) < 2 ** 31
    code = "from llm_steadyinfer_b200.engine.scheduler import default_seed; print(default_seed('chat-17'))"
    for salt in ("1", "2"):
        out = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, check=True,
                             env={**__import__("os").environ, "PYTHONHASHSEED": salt,
                                  "PYTHONPATH": __import__("os").path.dirname(__import__("os").path.dirname(__file__))})
        assert int(out.stdout) == default_seed("chat-17")


def test_a_waiting_prompt_is_hashed_once():
    """While a request waits at the head of the queue for pages, every step asks the prefix index about it;
    the chained hashes of its prompt are made at the first asking and kept."""
    s, cache = make(num_pages=6, page_size=4, max_seqs=4, budget=64, max_gen=3, prefix=True)
    calls = []
    real = cache.chain_hashes
    cache.chain_hashes = lambda tokens: calls.append(len(tokens)) or real(tokens)
    s.add_request(list(range(20)))               # 5 pages + growth: fills the pool
    run_step(s, cache)
    s.add_request(list(range(100, 112)))         # 3 pages: waits until the first one ends
    n = 0
    while s.has_unfinished():
        run_step(s, cache)
        n += 1
    assert n >= 3 and calls.count(12) == 1 and calls.count(20) == 1
    cache.check_invariant()


def test_admission_on_the_first_portion_preempts_for_later_portions():
    """``reserve="portion"``: requests are admitted when their first portion's pages are free, so more run than
    the pool holds prompts of; an older request's later portion has the newest ones preempted, they wait, come
    back and recompute, and every request finishes."""
    s, cache = make(num_pages=14, page_size=4, max_seqs=4, budget=8, max_gen=3)
    s.reserve = "portion"
    ids = [s.add_request(list(range(100 * i, 100 * i + 24))) for i in range(4)]     # 6 pages each, 24 in all: 14 there
    first = run_step(s, cache)
    assert len(s.running) == 4, "all four were admitted on two pages each"
    assert [(it.seq.id, it.start, it.count) for it in first] == [(ids[0], 0, 8)]
    n = 0
    while s.has_unfinished():
        items = run_step(s, cache)
        assert all(it.seq.state is SeqState.RUNNING or it.seq.state is SeqState.FINISHED for it in items)
        n += 1
        assert n < 400, "the schedule must end"
    assert s.num_preemptions >= 1 and s.num_recomputed_tokens >= 0
    assert sorted(q.id for q in s.finished) == sorted(ids)
    assert all(q.finish_reason == "length" and len(q.outputs) == 3 for q in s.finished)
    assert cache.free_pages(0) == 14
    cache.check_invariant()


def test_portion_admission_aborts_what_can_never_fit():
    s, cache = make(num_pages=4, page_size=4, max_seqs=2, budget=8, max_gen=2)
    s.reserve = "portion"
    a = s.add_request(list(range(15)))            # 15 + 1 tokens fit 4 pages: accepted; its portions fill the pool
    while s.has_unfinished():
        run_step(s, cache)
    assert s.finished[0].id == a and s.finished[0].finish_reason in ("length", "aborted")
    cache.check_invariant()
    assert cache.free_pages(0) == 4


def test_newer_requests_with_one_page_each_give_it_up_for_an_older_portion():
    """``reserve="portion"`` with a portion of one page: every request is admitted on one page and the pool is
    full of one-page holders. The oldest request's next portion then needs a page that only a newer request's
    last page can give: that request gives it, waits and starts again, and every request finishes. (Victims that
    always kept their first page left the older request waiting for ever.)"""
    s, cache = make(num_pages=5, page_size=4, max_seqs=5, budget=4, max_gen=2)
    s.reserve = "portion"
    ids = [s.add_request(list(range(50 * i, 50 * i + 10))) for i in range(5)]       # 3 pages each, 5 in the pool
    n = 0
    while s.has_unfinished():
        items = run_step(s, cache)
        n += 1
        assert items or n < 3, "a step with nothing to run while requests wait: the schedule has stalled"
        assert n < 400, "the schedule must end"
    assert s.num_preemptions >= 1
    assert sorted(q.id for q in s.finished) == sorted(ids)
    assert all(q.finish_reason == "length" and len(q.outputs) == 2 for q in s.finished)
    assert cache.free_pages(0) == 5
    cache.check_invariant()
