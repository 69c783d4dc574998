"""Cache manager and scheduler decisions (no GPU)."""
import random

import pytest

from llmario_b200.cache import (CacheError, CacheFull, CacheManager, FixedState, PagedKV,
                                PagePool)
from llmario_b200.engine.scheduler import FINISHED, RUNNING, WAITING, Request, Scheduler
from llmario_b200.sampling import SamplingParams


def manager(n_pages=16, page=4, max_requests=4, ctx=64, window=None, layers=2, state=False):
    needs = [PagedKV(2, 8, None)] * layers + ([PagedKV(2, 8, window)] if window else [])
    if state:
        needs.append(FixedState((3,)))
    return CacheManager(needs, [None] * len(needs), page, n_pages, max_requests, ctx)


# ------------------------------------------------------------------------------ pool
def test_pool_all_or_nothing_and_double_free():
    p = PagePool(4)
    assert p.alloc(5) is None and p.free == 4
    a = p.alloc(3)
    assert p.free == 1 and len(set(a)) == 3
    p.release(a[:1])
    with pytest.raises(CacheError):
        p.release(a[:1])         # freed twice
    with pytest.raises(CacheError):
        p.release([99])
    assert p.held() == 2


def test_freed_pages_are_used_again_oldest_first():
    p = PagePool(3)
    a = p.alloc(3)
    p.release([a[1]])
    p.release([a[0]])
    assert p.alloc(2) == [a[1], a[0]]


# ------------------------------------------------------------------------------ manager
def test_grouping_by_need():
    m = manager(window=6, layers=3)
    assert len(m.groups) == 2
    assert m.groups[0].entries == [0, 1, 2] and m.groups[1].entries == [3]
    m2 = CacheManager([PagedKV(2, 8), PagedKV(2, 8), None], [None, None, 0], 4, 8, 2, 32)
    assert m2._where[2] == m2._where[0]          # reads the first entry's cache
    with pytest.raises(CacheError):
        CacheManager([None, PagedKV(2, 8)], [None, 0], 4, 8, 2, 32)


def test_reserve_refuses_and_changes_nothing():
    m = manager(n_pages=5)
    m.open("a"), m.open("b")
    m.reserve([("a", 9)])
    m.advance("a", 9)
    m.take_table_updates()
    before = (m.free_pages(), m.pages_of("a"), m.pages_of("b"))
    with pytest.raises(CacheFull) as e:
        m.reserve([("a", 4), ("b", 8)])      # a needs 1 more, b needs 2, 2 free
    assert (e.value.needed, e.value.free) == (3, 2)
    assert (m.free_pages(), m.pages_of("a"), m.pages_of("b")) == before
    assert all(len(u) == 0 for u in m.take_table_updates())
    m.reserve([("a", 3), ("b", 8)])          # a fits its pages, b takes the last two
    assert m.free_pages() == [0]
    m.check_invariants()


def test_step_contract_errors():
    m = manager(ctx=16)
    m.open("a")
    with pytest.raises(CacheError, match="twice"):
        m.reserve([("a", 1), ("a", 1)])
    with pytest.raises(CacheError, match="exceed the context"):
        m.reserve([("a", 17)])
    with pytest.raises(CacheError, match="unknown request"):
        m.reserve([("zz", 1)])
    with pytest.raises(CacheError, match="already open"):
        m.open("a")
    for r in "bcd":
        m.open(r)
    with pytest.raises(CacheError, match="no free request slot"):
        m.open("e")


def test_window_pages_go_back_when_passed():
    m = manager(n_pages=8, page=4, window=6, layers=1, ctx=64)
    full, win = 0, 1
    m.open("a")
    at = 0
    for n in (5, 4, 1, 1, 1, 9, 2):
        m.reserve([("a", n)])
        m.advance("a", n)
        at += n
        pages = m.pages_of("a", win)
        # a later query at position >= at reaches back to at - 6 + 1
        first_needed = max(0, at - 6 + 1) // 4
        assert all(p == -1 for p in pages[:first_needed])
        assert all(p >= 0 for p in pages[first_needed:])
        assert all(p >= 0 for p in m.pages_of("a", full))
        m.check_invariants()
    assert m.counters["window_releases"] == first_needed
    assert m.free_pages()[win] > m.free_pages()[full]
    m.close("a")
    assert m.free_pages() == [8, 8]
    m.check_invariants()


def test_truncate_and_state_rules():
    m = manager(n_pages=8)
    m.open("a")
    m.reserve([("a", 14)])
    m.advance("a", 14)
    m.truncate("a", 5)
    assert m.length("a") == 5 and len(m.pages_of("a")) == 2 and m.free_pages() == [6]
    with pytest.raises(CacheError):
        m.truncate("a", 9)
    s = manager(state=True)
    s.open("a")
    s.reserve([("a", 3)])
    s.advance("a", 3)
    with pytest.raises(CacheError, match="cannot be rewound"):
        s.truncate("a", 1)
    w = manager(window=6, layers=1)
    w.open("a")
    w.reserve([("a", 20)])
    w.advance("a", 20)
    with pytest.raises(CacheError, match="already given back"):
        w.truncate("a", 6)


def test_table_updates_one_per_cell():
    m = manager(n_pages=4, max_requests=1)
    m.open("a")
    m.reserve([("a", 8)])
    m.advance("a", 8)
    first = m.pages_of("a")
    m.close("a")
    m.open("b")                       # same slot, pages handed out again
    m.reserve([("b", 4)])
    (u,) = m.take_table_updates()
    cells = {(int(s), int(j)): int(p) for s, j, p in u}
    assert len(cells) == len(u)       # no cell twice: any order of application is right
    assert cells[(0, 0)] == m.pages_of("b")[0] and cells[(0, 1)] == -1


@pytest.mark.parametrize("seed", range(5))
def test_random_orders_lose_nothing(seed):
    rng = random.Random(seed)
    m = manager(n_pages=24, page=4, max_requests=5, ctx=40, window=7, layers=2, state=True)
    live = {}
    n = 0
    for _ in range(600):
        op = rng.random()
        if op < 0.25 and m.free_slots():
            n += 1
            m.open(n)
            live[n] = 0
        elif op < 0.8 and live:
            chosen = rng.sample(sorted(live), rng.randint(1, len(live)))
            growth = [(r, rng.randint(1, 9)) for r in chosen if live[r] < 30]
            if growth:
                try:
                    m.reserve(growth)
                    for r, k in growth:
                        m.advance(r, k)
                        live[r] += k
                except CacheFull:
                    pass
        elif live:
            r = rng.choice(sorted(live))
            m.close(r)
            del live[r]
        m.check_invariants()
        for r, length in live.items():
            assert m.length(r) == length
    for r in list(live):
        m.close(r)
    m.check_invariants()
    assert m.free_pages() == [24, 24] and m.free_slots() == 5


# ------------------------------------------------------------------------------ scheduler
def req(rid, n_prompt, max_tokens=4):
    return Request(rid, list(range(1, n_prompt + 1)), SamplingParams(temperature=0, max_tokens=max_tokens))


def run_plan(s, plan, token=7):
    """Pretend the step ran: grow the cache as the step function would, then complete."""
    for e in plan.entries:
        if not s.cache.has(e.request.id):
            s.cache.open(e.request.id)
    s.cache.reserve([(e.request.id, e.count) for e in plan.entries])
    for e in plan.entries:
        s.cache.advance(e.request.id, e.count)
    return s.complete(plan, {e.request.id: token for e in plan.entries if e.samples})


def test_portions_under_the_budget_then_decodes_first():
    """The reference's rule (sched/src/lib.rs:318-326): (a,0,8), then (a,8,10) + (b,0,3)."""
    s = Scheduler(manager(n_pages=64, ctx=64), token_budget=8)
    a, b = req("a", 10), req("b", 3)
    s.add(a), s.add(b)
    p1 = s.plan()
    assert [(e.request.id, e.start, e.count, e.samples) for e in p1.entries] == [("a", 0, 8, False)]
    run_plan(s, p1)
    p2 = s.plan()
    assert [(e.request.id, e.start, e.count, e.samples) for e in p2.entries] == \
        [("a", 8, 2, True), ("b", 0, 3, True)]
    run_plan(s, p2)
    c = req("c", 20)
    s.add(c)
    p3 = s.plan()        # decodes first, one token each, then c's first portion in what is left
    assert [(e.request.id, e.start, e.count) for e in p3.entries] == \
        [("a", 10, 1), ("b", 3, 1), ("c", 0, 6)]
    assert p3.tokens == 8


def test_finish_reasons_and_pages_come_back():
    m = manager(n_pages=16, ctx=12)
    s = Scheduler(m, token_budget=32, eos_token_ids=[99])
    a, b, c = req("a", 3, max_tokens=2), req("b", 3, max_tokens=50), req("c", 9, max_tokens=50)
    for r in (a, b, c):
        s.add(r)
    done = run_plan(s, s.plan())
    assert not done
    done = run_plan(s, s.plan())
    assert done == [a] and a.finish_reason == "length" and a.output == [7, 7]
    done = run_plan(s, s.plan(), token=99)     # end of sequence
    assert {r.id for r in done} == {"b", "c"} and b.finish_reason == "stop"
    assert m.free_pages() == [16] and not s.has_work()
    d = req("d", 9, max_tokens=50)             # runs into the context of 12
    s.add(d)
    while s.has_work():
        run_plan(s, s.plan())
    assert d.finish_reason == "length" and d.sequence_len == 12
    e = req("e", 3, max_tokens=3)
    e.params.ignore_eos = True
    s.add(e)
    while s.has_work():
        run_plan(s, s.plan(), token=99)
    assert e.finish_reason == "length" and e.output == [99, 99, 99]


def test_refuses_bad_prompts():
    s = Scheduler(manager(ctx=16))
    with pytest.raises(ValueError, match="empty"):
        s.add(req("a", 0))
    with pytest.raises(ValueError, match="does not fit the context"):
        s.add(req("a", 16))


def test_pages_run_out_newest_is_preempted_and_recomputed():
    m = manager(n_pages=6, page=4, ctx=64, max_requests=4)
    s = Scheduler(m, token_budget=64)
    a, b = req("a", 11, max_tokens=6), req("b", 11, max_tokens=6)
    s.add(a), s.add(b)
    run_plan(s, s.plan())           # both prompts: 3 pages each, pool full, 12 tokens each
    assert m.free_pages() == [0]
    p = s.plan()                    # both decode at position 11: fits the held pages
    assert not p.preempted and len(p.entries) == 2
    run_plan(s, p)
    p = s.plan()                    # position 12 needs a fourth page each: none free
    assert p.preempted == [b] and b.state == WAITING and b.computed == 0 and b.preemptions == 1
    assert [(e.request.id, e.count) for e in p.entries] == [("a", 1)]   # b waits: no room
    assert s.waiting[0] is b
    run_plan(s, p)
    while a.state != FINISHED:
        run_plan(s, s.plan())
    # b comes back and recomputes prompt + what it had generated, in one portion
    p = s.plan()
    assert [(e.request.id, e.start, e.count, e.samples) for e in p.entries] == \
        [("b", 0, 11 + len(b.output), True)]
    while s.has_work():
        run_plan(s, s.plan())
    assert len(b.output) == 6 and m.free_pages() == [6]
    assert s.counters["preemptions"] == 1
    m.check_invariants()


def test_a_request_too_large_for_the_cache_fails_alone():
    m = manager(n_pages=3, page=4, ctx=64)
    s = Scheduler(m, token_budget=64)
    a = req("a", 10, max_tokens=30)
    s.add(a)
    run_plan(s, s.plan())
    while s.has_work():
        p = s.plan()
        if p.failed:
            break
        run_plan(s, p)
    assert a.state == FINISHED and a.finish_reason == "error" and "KV cache full" in a.error
    assert m.free_pages() == [3]
    big = req("big", 40)
    s.add(big)
    p = s.plan()        # the prompt is cut to what fits, then sticks: fails alone
    while s.has_work() and not p.failed:
        run_plan(s, p)
        p = s.plan()
    assert big.finish_reason == "error" and m.free_pages() == [3]


def test_prompt_portion_shrinks_to_free_pages():
    m = manager(n_pages=5, page=4, ctx=64)
    s = Scheduler(m, token_budget=64)
    a, b = req("a", 10, max_tokens=8), req("b", 30, max_tokens=2)
    s.add(a), s.add(b)
    p = s.plan()
    # a takes 3 pages; b gets what is left: 2 pages = 8 tokens of its prompt
    assert [(e.request.id, e.count) for e in p.entries] == [("a", 10), ("b", 8)]


@pytest.mark.parametrize("seed", range(3))
def test_random_load_finishes_everything(seed):
    rng = random.Random(seed)
    m = manager(n_pages=12, page=4, ctx=48, max_requests=3, window=9, layers=1)
    s = Scheduler(m, token_budget=16)
    reqs = [req(i, rng.randint(1, 20), max_tokens=rng.randint(1, 12)) for i in range(12)]
    pending = list(reqs)
    steps = 0
    while pending or s.has_work():
        if pending and rng.random() < 0.4:
            s.add(pending.pop(0))
        if s.has_work():
            p = s.plan()
            assert p.tokens <= 16
            assert len({e.request.id for e in p.entries}) == len(p.entries)
            run_plan(s, p, token=rng.randint(0, 5))
            m.check_invariants()
        steps += 1
        assert steps < 5000
    assert all(r.state == FINISHED and r.finish_reason in ("length", "stop") for r in reqs)
    assert all(len(r.output) == r.params.max_tokens or r.sequence_len == 48 for r in reqs)
    assert m.free_pages() == [12, 12]


# ------------------------------------------------------------------------------ the step ahead
def launch(s, plan):
    """What the step function does to the cache when a plan is queued."""
    for e in plan.entries:
        if not s.cache.has(e.request.id):
            s.cache.open(e.request.id)
    s.cache.reserve([(e.request.id, e.count) for e in plan.entries])
    for e in plan.entries:
        s.cache.advance(e.request.id, e.count)


def finish(s, plan, token=7):
    return s.complete(plan, {e.request.id: token for e in plan.entries if e.samples})


def test_a_step_is_planned_ahead_on_what_is_certain():
    """While a step runs, the step after it is planned on the requests as they will stand when it
    ends without an end-of-sequence token: the rest of a prompt, the admission of a request that
    waits, one more token for every request that decodes (its input is the token in flight)."""
    s = Scheduler(manager(n_pages=64, ctx=64), token_budget=8, eos_token_ids=[99])
    a, b = req("a", 10, max_tokens=3), req("b", 3, max_tokens=50)
    s.add(a), s.add(b)
    p1 = s.plan()                       # a's first portion fills the budget: b still waits
    assert [(e.request.id, e.start, e.count, e.samples) for e in p1.entries] == [("a", 0, 8, False)]
    launch(s, p1)
    p2 = s.plan_ahead(p1)               # the rest of a, and b is admitted: both draw a token
    assert [(e.request.id, e.start, e.count, e.samples) for e in p2.entries] == \
        [("a", 8, 2, True), ("b", 0, 3, True)]
    assert b.state == "running" and not s.waiting
    launch(s, p2)
    assert finish(s, p1) == []
    p3 = s.plan_ahead(p2)               # the tokens p2 draws are the inputs of p3
    assert [(e.request.id, e.start, e.count, e.samples) for e in p3.entries] == \
        [("a", 10, 1, True), ("b", 3, 1, True)]
    launch(s, p3)
    finish(s, p2)
    p4 = s.plan_ahead(p3)               # a's third and last token will be the one p4 draws
    assert [e.request.id for e in p4.entries] == ["a", "b"]
    launch(s, p4)
    finish(s, p3)
    p5 = s.plan_ahead(p4)               # a ends for certain with p4: only b goes on
    assert [(e.request.id, e.start) for e in p5.entries] == [("b", 5)]
    launch(s, p5)
    assert finish(s, p4) == [a] and a.output == [7, 7, 7] and a.finish_reason == "length"
    # b draws an end-of-sequence token in p5 while p6 is already queued for it
    p6 = s.plan_ahead(p5)
    launch(s, p6)
    assert finish(s, p5, token=99) == [b] and b.finish_reason == "stop"
    assert finish(s, p6) == [] and b.output == [7, 7, 7, 99]     # the row too many is passed over
    assert s.plan_ahead(p6) is None and not s.has_work()
    assert s.cache.free_pages() == [64]
    s.cache.check_invariants()
    assert s.counters["steps_planned_ahead"] == 5 and s.counters["steps_planned"] == 6


def test_what_a_step_planned_ahead_leaves_to_the_next_plan():
    m = manager(n_pages=4, page=4, max_requests=2, ctx=64)
    s = Scheduler(m, token_budget=64)
    a, b, c = req("a", 7, 50), req("b", 7, 50), req("c", 3, 50)
    s.add(a), s.add(b), s.add(c)        # two request slots: c waits
    p = s.plan()
    launch(s, p)
    assert [e.request.id for e in p.entries] == ["a", "b"]
    # c cannot be admitted while a and b hold both slots: the next step is a and b alone
    ahead = s.plan_ahead(p)
    assert [(e.request.id, e.start, e.count) for e in ahead.entries] == [("a", 7, 1), ("b", 7, 1)]
    assert [r.id for r in s.waiting] == ["c"]
    finish(s, p)
    s.abort(c)
    launch(s, ahead)                    # a and b at 8 tokens each: all four pages are full
    assert s.plan_ahead(ahead) is None  # the next token of each needs a page that is not there:
    finish(s, ahead)                    # who gives way is decided with all facts known
    p = s.plan()
    assert [r.id for r in p.preempted] == ["b"] and [e.request.id for e in p.entries] == ["a"]
    # a request that arrives while a step runs is admitted into the step planned ahead
    s3 = Scheduler(manager(n_pages=64, max_requests=3, ctx=64), token_budget=64)
    d, e = req("d", 5, 50), req("e", 5, 50)
    s3.add(d), s3.add(e)
    p = s3.plan()
    launch(s3, p)
    f = req("f", 4, 50)
    s3.add(f)
    ahead = s3.plan_ahead(p)
    assert [(x.request.id, x.start, x.count) for x in ahead.entries] == \
        [("d", 5, 1), ("e", 5, 1), ("f", 0, 4)]
    assert f.state == "running"
    # all slots taken and one request ends for certain with the token in flight: it is left out
    # of the step ahead but keeps its slot until the flying step is reported, so the request
    # that waits comes in with the plan after that
    s4 = Scheduler(manager(n_pages=64, max_requests=2, ctx=64), token_budget=64)
    g, h, i = req("g", 5, 2), req("h", 5, 50), req("i", 4, 50)
    s4.add(g), s4.add(h), s4.add(i)
    p = s4.plan()
    launch(s4, p)
    p2 = s4.plan_ahead(p)               # g's first token is in flight: it has one more to draw
    assert [x.request.id for x in p2.entries] == ["g", "h"]
    launch(s4, p2)
    finish(s4, p)
    p3 = s4.plan_ahead(p2)              # g's last token is in flight
    assert [x.request.id for x in p3.entries] == ["h"] and [r.id for r in s4.waiting] == ["i"]
    launch(s4, p3)
    assert [r.id for r in finish(s4, p2)] == ["g"]
    p4 = s4.plan_ahead(p3)
    assert [(x.request.id, x.start, x.count) for x in p4.entries] == [("h", 7, 1), ("i", 0, 4)]
    # penalties do not stand in the way: the sampler counts the token in flight on the device
    pen = req("p", 3, 50)
    pen.params.repeat_penalty = 1.3
    s2 = Scheduler(manager(n_pages=64, ctx=64), token_budget=8)
    s2.add(pen)
    p = s2.plan()
    launch(s2, p)
    ahead = s2.plan_ahead(p)
    assert pen.params.penalties_active and [(x.request.id, x.start) for x in ahead.entries] == [("p", 3)]


# ------------------------------------------------------------------------------ native core vs plain model
@pytest.mark.parametrize("seed", range(6))
def test_native_bookkeeping_agrees_with_the_plain_model(seed):
    """The C++ core and the plain Python model under ``tests/plain`` are driven with the same
    random operations (open, grow in mixed steps, truncate, close, misuse) and must give the
    same answers at every turn: slots, page ids in order, free pages, refusals with their
    numbers, table changes, slots to be zeroed."""
    import random

    from llmario_b200.cache import CacheError, CacheFull
    from plain.cache_plain import PlainCache, PlainError, PlainFull

    rng = random.Random(seed)
    page = rng.choice([1, 4, 8])
    windows = [None, rng.choice([5, 9, 17])] if seed % 2 else [None]
    n_pages = rng.choice([6, 14, 30])
    ctx = rng.choice([24, 50])
    max_req = rng.choice([2, 4])
    needs = [PagedKV(2, 16, w) for w in windows]
    native = CacheManager(needs, [None] * len(needs), page, n_pages, max_req, ctx)
    plain = PlainCache([n_pages] * len(windows), windows, page, max_req, ctx)
    live = []
    names = iter(range(10 ** 6))

    def both(op_native, op_plain):
        """Run an operation on both; they succeed together or fail together."""
        try:
            a, ea = op_native(), None
        except (CacheError, CacheFull) as e:
            a, ea = None, e
        try:
            b, eb = op_plain(), None
        except (PlainError, PlainFull) as e:
            b, eb = None, e
        assert (ea is None) == (eb is None), (ea, eb)
        if isinstance(ea, CacheFull) or isinstance(eb, PlainFull):
            assert isinstance(ea, CacheFull) and isinstance(eb, PlainFull)
            assert (ea.group, ea.needed, ea.free) == (eb.group, eb.needed, eb.free)
        return a, b, ea is None

    for step in range(400):
        op = rng.random()
        if op < 0.2:
            rid = f"r{next(names)}"
            a, b, ok = both(lambda: native.open(rid), lambda: plain.open(rid))
            if ok:
                assert a == b
                live.append(rid)
        elif op < 0.7 and live:
            k = rng.randint(1, min(3, len(live)))
            chosen = rng.sample(live, k)
            if rng.random() < 0.05:
                chosen.append(chosen[0])                     # misuse: twice in one step
            growth = [(r, rng.choice([0, 1, 1, 2, 5, 11]) if rng.random() < 0.9 else 40)
                      for r in chosen]
            _, _, ok = both(lambda: native.reserve(growth), lambda: plain.reserve(growth))
            if ok:
                for r, n in growth:
                    both(lambda: native.advance(r, n), lambda: plain.advance(r, n))
        elif op < 0.8 and live:
            r = rng.choice(live)
            to = rng.randint(0, plain.requests[r]["length"] + 1)
            both(lambda: native.truncate(r, to), lambda: plain.truncate(r, to))
        elif op < 0.95 and live:
            r = live.pop(rng.randrange(len(live)))
            both(lambda: native.close(r), lambda: plain.close(r))
        else:
            both(lambda: native.advance("nobody", 1), lambda: plain.advance("nobody", 1))
        # the same state after every operation
        assert native.free_pages() == [len(f) for f in plain.free]
        assert native.free_slots() == len(plain.free_slots)
        for r in live:
            assert native.info(r) == (plain.requests[r]["slot"], plain.requests[r]["length"])
            for g in range(len(windows)):
                assert native.pages_of(r, g) == plain.requests[r]["pages"][g]
                assert native.pages_needed(r, 3) == plain.pages_needed(r, 3)
        if step % 7 == 0:
            got = [sorted(map(tuple, u.tolist())) for u in native.take_table_updates()]
            assert got == plain.take_updates()
            assert native.take_fresh_slots() == plain.take_fresh()
        native.check_invariants()
    for r in live:
        native.close(r), plain.close(r)
    assert native.free_pages() == [n_pages] * len(windows)


@pytest.mark.parametrize("seed", range(8))
def test_native_scheduler_agrees_with_the_plain_model(seed):
    """The scheduler decides in native code; a plain Python model of the same rules lives under
    tests/plain.  Both get the same random load (arrivals, lengths, limits, end-of-sequence
    tokens, aborts, steps planned ahead, so few pages that requests are preempted and one is
    too large for the cache) and must make the same plans, step by step."""
    from plain.scheduler_plain import PlainScheduler, Request as PlainRequest

    rng = random.Random(100 + seed)
    window = rng.choice([None, 9])
    budget = rng.choice([5, 16, 64])
    pages = rng.choice([8, 12, 40])

    def make():
        return manager(n_pages=pages, page=4, ctx=48, max_requests=3, window=window, layers=1)

    native = Scheduler(make(), token_budget=budget, eos_token_ids=[3])
    plain = PlainScheduler(make(), token_budget=budget, eos_token_ids=[3])
    specs = [(i, rng.randint(1, 40), rng.randint(1, 12), rng.random() < 0.3) for i in range(14)]
    pending = list(specs)
    both = {}

    def same_plan(a, b):
        assert [(e.request.id, e.start, e.count, e.samples) for e in a.entries] == \
               [(e.request.id, e.start, e.count, e.samples) for e in b.entries]
        assert [r.id for r in a.preempted] == [r.id for r in b.preempted]
        assert [r.id for r in a.failed] == [r.id for r in b.failed]

    def same_state():
        assert [r.id for r in native.waiting] == [r.id for r in plain.waiting]
        assert [r.id for r in native.running] == [r.id for r in plain.running]
        for rid, (a, b) in both.items():
            assert (a.state, a.computed, a.output, a.finish_reason, a.preemptions) == \
                   (b.state, b.computed, b.output, b.finish_reason, b.preemptions), rid
        assert native.cache.free_pages() == plain.cache.free_pages()
        na, pl = native.counters, plain.counters
        assert all(na[k] == pl.get(k, 0) for k in na), (na, pl)

    steps = 0
    while pending or native.has_work():
        assert native.has_work() == plain.has_work()
        if pending and rng.random() < 0.4:
            i, n, mt, ig = pending.pop(0)
            params = SamplingParams(temperature=0, max_tokens=mt, ignore_eos=ig)
            a = Request(i, list(range(1, n + 1)), params)
            b = PlainRequest(i, list(range(1, n + 1)), params)
            both[i] = (a, b)
            native.add(a), plain.add(b)
        if native.running and rng.random() < 0.05:
            victim = rng.choice(native.running).id
            native.abort(both[victim][0]), plain.abort(both[victim][1])
            same_state()
        if native.has_work():
            pa, pb = native.plan(), plain.plan()
            same_plan(pa, pb)
            launch(native, pa), launch(plain, pb)
            tokens = {e.request.id: rng.randint(0, 5) for e in pa.entries if e.samples}
            # the step after, decided before this one's tokens are known
            aa, ab = native.plan_ahead(pa), plain.plan_ahead(pb)
            assert (aa is None) == (ab is None)
            native.complete(pa, tokens), plain.complete(pb, tokens)
            same_state()
            if aa is not None:
                same_plan(aa, ab)
                live_a = [e for e in aa.entries if e.request.state == RUNNING]
                live_b = [e for e in ab.entries if e.request.state == RUNNING]
                for s, live in ((native, live_a), (plain, live_b)):
                    for e in live:                  # (a step planned ahead may admit a request)
                        if not s.cache.has(e.request.id):
                            s.cache.open(e.request.id)
                    s.cache.reserve([(e.request.id, e.count) for e in live])
                    for e in live:
                        s.cache.advance(e.request.id, e.count)
                tokens = {e.request.id: rng.randint(0, 5) for e in aa.entries}
                native.complete(aa, tokens), plain.complete(ab, tokens)
                same_state()
            native.cache.check_invariants()
        steps += 1
        assert steps < 5000
    assert all(a.state == FINISHED for a, _ in both.values())
    assert native.cache.free_pages() == [pages] * len(native.cache.groups)


def test_abort_and_names_used_again():
    """A waiting request can be dropped before it ever ran; a request id can be used again once
    its request is over (finished, failed or aborted); the cache manager forgets the key it had
    promised."""
    m = manager(n_pages=16, page=4, ctx=32, max_requests=2)
    s = Scheduler(m, token_budget=8)
    a, b = req("a", 6, max_tokens=2), req("b", 5, max_tokens=2)
    s.add(a), s.add(b)
    s.abort(b)                                   # never admitted
    assert b.state == FINISHED and b.finish_reason == "aborted" and list(s.waiting) == [a]
    while s.has_work():
        run_plan(s, s.plan())
    assert a.finish_reason == "length" and len(a.output) == 2
    a2 = req("a", 3, max_tokens=1)               # the same id again
    s.add(a2)
    p = s.plan()
    assert [(e.request is a2, e.start, e.count, e.samples) for e in p.entries] == [(True, 0, 3, True)]
    s.abort(a2)                                  # while it is running and holds pages
    assert a2.finish_reason == "aborted" and not s.has_work()
    assert m.free_pages() == [16] * len(m.groups) and m.free_slots() == 2
    m.check_invariants()
    assert not m.live_requests()
    with pytest.raises(ValueError):
        s.add(req("c", 0))
    big = req("big", 31, max_tokens=4)           # fits the context, not the 16 pages of 4
    m2 = manager(n_pages=4, page=4, ctx=64, max_requests=2)
    s2 = Scheduler(m2, token_budget=64)
    s2.add(big)
    p = s2.plan()
    if p.entries:                                # the prompt is fed in portions until pages run out
        while s2.has_work() and not p.failed:
            run_plan(s2, p)
            p = s2.plan()
    assert big in p.failed and big.finish_reason == "error" and "KV cache full" in big.error
    s2.add(req("big", 3, max_tokens=1))          # its id is free again, and so are its pages
    run_plan(s2, s2.plan())
    assert not s2.has_work() and m2.free_pages() == [4] * len(m2.groups)
