"""The scheduler's decisions: admission, portions under the token budget,
decoding, finishing, and what happens when pages run out."""
import numpy as np
import pytest

from crane_b200.cache import GroupSpec, PageTable
from crane_b200.engine.scheduler import Scheduler


def make(pages=16, page_size=16, max_running=4, budget=64, chunk=32, max_seq_len=256):
    t = PageTable([GroupSpec(pages, page_size)], max_requests=max_running)
    return t, Scheduler(t, max_running, budget, chunk, max_seq_len)


def feed(s, plan, token=5):
    """Answers every entry that asked for a token."""
    out = {}
    for e in plan:
        if e.sample:
            out[e.request_id] = s.on_token(e.request_id, token)
    return out


def test_prompt_is_cut_into_portions_under_the_budget():
    t, s = make(budget=48, chunk=32)
    s.add(1, list(range(100)), 4, [])
    seen = []
    for _ in range(4):
        plan = s.schedule()
        assert len(plan) == 1 and sum(len(e.tokens) for e in plan) <= 48
        seen.append((plan[0].start, len(plan[0].tokens), plan[0].sample))
        feed(s, plan)
    assert seen == [(0, 32, False), (32, 32, False), (64, 32, False), (96, 4, True)]
    assert list(s.schedule()[0].tokens) == [5]                   # now it decodes


def test_decoding_requests_come_first_and_portions_fill_the_rest():
    t, s = make(budget=40, chunk=32)
    s.add(1, [1, 2, 3], 10, [])
    feed(s, s.schedule())                                          # request 1 now decodes
    s.add(2, list(range(90)), 10, [])
    plan = s.schedule()
    assert [(e.request_id, len(e.tokens)) for e in plan] == [(1, 1), (2, 32)]
    feed(s, plan)
    plan = s.schedule()
    assert [(e.request_id, e.start, len(e.tokens)) for e in plan] == [(1, 4, 1), (2, 32, 32)]
    assert sum(len(e.tokens) for e in plan) <= 40


def test_fifo_admission_up_to_max_running():
    t, s = make(max_running=2, budget=64, chunk=8)
    for rid in (1, 2, 3):
        s.add(rid, [1] * 8, 2, [])
    plan = s.schedule()
    assert [e.request_id for e in plan] == [1, 2] and s.num_waiting == 1
    feed(s, plan)
    plan = s.schedule()
    assert [e.request_id for e in plan] == [1, 2]
    done = feed(s, plan)
    assert done == {1: "length", 2: "length"}
    assert [e.request_id for e in s.schedule()] == [3]             # admitted once a slot is free
    assert t.live() == 1


def test_finish_reasons_and_pages_come_back():
    t, s = make()
    s.add(1, [1, 2, 3], 5, [9])
    feed(s, s.schedule(), token=4)
    assert s.on_token(1, 4) is None or True
    plan = s.schedule()
    assert s.on_token(1, 9) == "stop"                              # an EOS token stops it ...
    st = s.state(1)
    assert st.finish_reason == "stop" and s.tokens(1)[-1] == 9     # ... and stays in the tokens
    assert t.free_pages() == 16 and t.live() == 0
    s.drop(1)
    with pytest.raises(KeyError):
        s.state(1)


def test_prompt_limits():
    t, s = make(max_seq_len=20)
    with pytest.raises(ValueError, match="refused"):
        s.add(1, [1] * 21, 5, [])
    with pytest.raises(ValueError, match="refused"):
        s.add(1, [], 5, [])
    assert s.add(2, [1] * 20, 5, []) == "finished"                 # no room to generate
    assert s.state(2).finish_reason == "length"
    s.add(3, [1] * 18, 50, [])                                     # max_new_tokens is clamped to 2
    feed(s, s.schedule())
    assert feed(s, s.schedule()) == {3: "length"}
    assert s.stats()["rejected"] == 2


def test_preemption_when_pages_run_out():
    # 6 pages of 4 tokens; two requests of 8 prompt tokens decode until the pool is full
    t, s = make(pages=6, page_size=4, max_running=2, budget=32, chunk=16, max_seq_len=64)
    s.add(1, [1] * 8, 10, [])
    s.add(2, [2] * 8, 10, [])
    preempted_at = None
    for step in range(40):
        plan = s.schedule()
        if s.last_preempted():
            preempted_at = step
            assert s.last_preempted() == [2]                       # the most recently admitted
            assert [e.request_id for e in plan] == [1]             # and its entry is gone
            feed(s, plan, token=3)
            break
        feed(s, plan, token=3)
    assert preempted_at is not None
    st = s.state(2)
    assert not st.running and st.computed == 0 and st.preemptions == 1
    assert st.num_tokens > 8                                       # it keeps what it generated
    t.check()
    # request 1 runs on; when it ends, request 2 is recomputed from all its tokens and goes on
    before = s.tokens(2)
    guard = 0
    while s.state(1).finish_reason is None:
        feed(s, s.schedule(), token=3)
        guard += 1
        assert guard < 100
    plan = s.schedule()
    e = [e for e in plan if e.request_id == 2][0]
    assert e.start == 0 and list(e.tokens) == before[:len(e.tokens)]
    feed(s, plan, token=3)
    guard = 0
    while s.has_work():
        feed(s, s.schedule(), token=3)
        guard += 1
        assert guard < 200
    assert s.state(2).finish_reason == "length" and len(s.tokens(2)) == 18
    assert t.free_pages() == 6
    t.check()


def test_a_request_that_cannot_fit_is_ended_not_hung():
    t, s = make(pages=2, page_size=4, max_running=2, budget=32, chunk=16, max_seq_len=64)
    s.add(1, [1] * 6, 30, [])
    reasons = []
    for _ in range(10):
        plan = s.schedule()
        if s.last_failed():
            reasons = s.last_failed()
            break
        feed(s, plan, token=3)
    assert reasons == [1] and s.state(1).finish_reason == "cache_too_small"
    assert len(s.tokens(1)) == 9                                   # 8 cached tokens + the one it could not place
    assert t.free_pages() == 2 and not s.has_work()


def test_first_portion_shrinks_to_the_pool_when_alone():
    t, s = make(pages=2, page_size=4, max_running=2, budget=32, chunk=16, max_seq_len=64)
    s.add(1, [1] * 12, 3, [])
    plan = s.schedule()
    assert len(plan[0].tokens) == 8                                # what two pages hold


def test_cancel():
    t, s = make()
    s.add(1, [1] * 40, 5, [])
    s.schedule()
    s.cancel(1)
    assert s.state(1).finish_reason == "cancelled" and t.free_pages() == 16 and not s.has_work()


@pytest.mark.parametrize("seed", range(4))
def test_random_load_never_breaks_budget_or_books(seed):
    rng = np.random.default_rng(seed)
    t, s = make(pages=24, page_size=8, max_running=4, budget=48, chunk=24, max_seq_len=120)
    lens, next_id, finished = {}, 1, {}
    for step in range(500):
        if rng.random() < 0.15 and next_id < 40:
            n = int(rng.integers(1, 90))
            s.add(next_id, rng.integers(0, 100, n).tolist(), int(rng.integers(1, 30)), [7])
            lens[next_id] = n
            next_id += 1
        plan = s.schedule()
        assert sum(len(e.tokens) for e in plan) <= 48
        assert len({e.request_id for e in plan}) == len(plan) <= 4
        for e in plan:
            assert t.length(e.request_id) == e.start + len(e.tokens)
            assert e.sample == (e.start + len(e.tokens) == s.state(e.request_id).num_tokens)
        for e in plan:
            if e.sample:
                r = s.on_token(e.request_id, int(rng.integers(0, 12)))
                if r:
                    finished[e.request_id] = r
        for rid in s.last_failed():
            finished[rid] = "cache_too_small"
        t.check()
    while s.has_work():
        for e in s.schedule():
            if e.sample:
                r = s.on_token(e.request_id, 7)
                if r:
                    finished[e.request_id] = r
    assert set(finished) == set(lens)
    assert t.free_pages() == 24 and t.live() == 0
    st = s.stats()
    assert st["finished"] == len(lens) and st["requests"] == len(lens)


# ---- tokens that are planned before they are known --------------------------
def test_placeholder_lets_the_next_step_be_planned():
    t, s = make()
    s.add(1, [1, 2, 3], 4, [9])
    plan = s.schedule()
    assert plan[0].sample
    s.expect_tokens([1])
    nxt = s.schedule()                                             # planned with the token unknown
    assert [(e.start, list(e.tokens), e.sample) for e in nxt] == [(3, [-1], True)]
    assert s.resolve_tokens([1], [7]) == [None]
    assert s.tokens(1) == [1, 2, 3, 7]
    s.expect_tokens([1])
    assert s.tokens(1) == [1, 2, 3, 7, -1]
    assert s.resolve_tokens([1], [8]) == [None]
    assert s.tokens(1) == [1, 2, 3, 7, 8]


def test_stop_token_voids_what_was_planned_beyond_it():
    t, s = make()
    s.add(1, [1, 2, 3], 10, [9])
    s.schedule()
    s.expect_tokens([1])
    s.schedule()                                                   # one step too far
    s.expect_tokens([1])
    assert s.resolve_tokens([1], [9]) == ["stop"]
    assert s.tokens(1) == [1, 2, 3, 9]
    assert t.free_pages() == 16 and t.live() == 0                  # pages are back
    assert s.resolve_tokens([1], [4]) == ["stop"]                  # the late token changes nothing
    assert s.tokens(1) == [1, 2, 3, 9]
    assert not s.has_work()


def test_last_token_by_count_is_not_planned_past():
    t, s = make()
    s.add(1, [1, 2, 3], 2, [])
    s.schedule()
    s.expect_tokens([1])
    assert len(s.schedule()) == 1
    s.expect_tokens([1])                                           # the second of two tokens
    assert s.schedule() == [] and s.has_work()                     # nothing more, but not done
    assert s.resolve_tokens([1], [5]) == [None]
    assert s.schedule() == []
    assert s.resolve_tokens([1], [6]) == ["length"]
    assert s.tokens(1) == [1, 2, 3, 5, 6]
    assert not s.has_work() and t.live() == 0


def test_cancel_drops_placeholders():
    t, s = make()
    s.add(1, [1, 2, 3], 8, [])
    s.schedule()
    s.expect_tokens([1])
    s.cancel(1)
    assert s.tokens(1) == [1, 2, 3] and s.state(1).finish_reason == "cancelled"
    assert s.resolve_tokens([1], [5]) == ["cancelled"]
    assert s.tokens(1) == [1, 2, 3]


def test_placeholders_and_preemption_give_the_same_tokens_as_plain_decoding():
    """The same requests, once answered at once and once a step late, under a
    pool so small that requests are preempted: same tokens for every request."""
    def run(late):
        t, s = make(pages=6, page_size=4, max_running=3, budget=16, chunk=8, max_seq_len=64)
        for rid, n in ((1, 5), (2, 7), (3, 3)):
            s.add(rid, list(range(1, n + 1)), 9, [])
        pending, steps = None, 0
        def answer(ids):
            toks = [(rid * 31 + len(s.tokens(rid)) * 7) % 50 for rid in ids]
            if late:
                # the oldest placeholder sits one before the end if a newer one follows
                toks = [(rid * 31 + (len(s.tokens(rid)) - s.tokens(rid).count(-1)) * 7) % 50
                        for rid in ids]
                return s.resolve_tokens(ids, toks)
            return s.on_tokens(ids, toks)
        while s.has_work() and steps < 400:
            steps += 1
            plan = s.schedule()
            ids = [e.request_id for e in plan if e.sample]
            for e in plan:
                assert (np.asarray(e.tokens[:-1]) >= 0).all()     # only a last token may be unknown
            if late:
                s.expect_tokens(ids)
                if pending:
                    answer(pending)
                pending = ids
            elif ids:
                answer(ids)
            t.check()
        if late and pending:
            answer(pending)
        assert steps < 400
        return {rid: s.tokens(rid) for rid in (1, 2, 3)}, s.stats()["preemptions"]
    plain, p0 = run(False)
    late, p1 = run(True)
    assert plain == late
    assert p0 > 0 and p1 > 0
    assert all(len(v) - n == 9 for v, n in zip(plain.values(), (5, 7, 3)))
