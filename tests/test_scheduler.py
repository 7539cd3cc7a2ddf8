"""The scheduler's decisions, on the host, with the cache manager's bookkeeping only."""
import pytest

from tinyinfer_b200.cache import CacheManager
from tinyinfer_b200.engine import Request, Scheduler
from tinyinfer_b200.parts import PagedKVSpec
from tinyinfer_b200.sampling import SamplingParams


def _setup(num_pages=64, max_num_seqs=4, budget=32, chunk=None, max_position=1024, eos=()):
    cache = CacheManager([PagedKVSpec(2, 16, None)], page_size=16, num_pages=num_pages,
                         max_requests=max_num_seqs)
    return cache, Scheduler(cache, max_num_seqs=max_num_seqs, max_batched_tokens=budget,
                            chunk=chunk, max_position=max_position, eos_token_ids=eos)


def _run_step(cache, sched, token=5):
    """What the generation loop does with a plan, without a model: every sampling entry gets ``token``."""
    plan = sched.schedule()
    cache.reserve_step([(s.request.req_id, s.count) for s in plan])
    for s in plan:
        assert s.start == cache.length(s.request.req_id) - s.count == s.request.computed
    finished = sched.step_done(plan, [token] * sum(s.samples for s in plan))
    cache.check()
    return plan, finished


def _req(i, n, max_tokens=4):
    return Request(req_id=i, prompt=list(range(1, n + 1)), params=SamplingParams(max_tokens=max_tokens))


def test_budget_and_portions():
    cache, sched = _setup(budget=32, chunk=None)
    sched.add(_req("a", 50))
    sched.add(_req("b", 10))
    plan, _ = _run_step(cache, sched)
    assert [(s.request.req_id, s.start, s.count, s.samples) for s in plan] == [("a", 0, 32, False)]
    plan, _ = _run_step(cache, sched)          # a's rest, then b with what the budget leaves
    assert [(s.request.req_id, s.start, s.count, s.samples) for s in plan] == \
        [("a", 32, 18, True), ("b", 0, 10, True)]
    plan, _ = _run_step(cache, sched)          # both decode
    assert [(s.request.req_id, s.count, s.samples) for s in plan] == [("a", 1, True), ("b", 1, True)]


def test_chunk_caps_a_portion_and_decodes_come_first():
    cache, sched = _setup(budget=20, chunk=16)
    sched.add(_req("a", 3, max_tokens=10))
    _run_step(cache, sched)
    sched.add(_req("b", 40))
    plan, _ = _run_step(cache, sched)
    assert [(s.request.req_id, s.count) for s in plan] == [("a", 1), ("b", 16)]
    plan, _ = _run_step(cache, sched)
    assert [(s.request.req_id, s.start, s.count) for s in plan] == [("a", 4, 1), ("b", 16, 16)]
    plan, _ = _run_step(cache, sched)
    assert [(s.request.req_id, s.start, s.count, s.samples) for s in plan] == \
        [("a", 5, 1, True), ("b", 32, 8, True)]


def test_admission_is_bounded_by_request_slots():
    cache, sched = _setup(max_num_seqs=2, budget=64)
    for i in range(3):
        sched.add(_req(i, 4, max_tokens=2))
    plan, _ = _run_step(cache, sched)
    assert [s.request.req_id for s in plan] == [0, 1]
    plan, finished = _run_step(cache, sched)                    # second token: both finish
    assert [r.req_id for r in finished] == [0, 1] and all(r.finish_reason == "length" for r in finished)
    plan, _ = _run_step(cache, sched)
    assert [s.request.req_id for s in plan] == [2]
    assert cache.live_requests() == [2]


def test_finishing_rules():
    cache, sched = _setup(eos=(9,), max_position=8)
    sched.add(_req("eos", 3, max_tokens=50))
    _, fin = _run_step(cache, sched, token=9)
    assert fin[0].finish_reason == "stop" and fin[0].output == [9] and cache.live_requests() == []
    sched.add(Request("stop", [1, 2], SamplingParams(max_tokens=50, stop_token_ids=(7,))))
    _, fin = _run_step(cache, sched, token=7)
    assert fin[0].finish_reason == "stop"
    sched.add(_req("ctx", 6, max_tokens=50))
    _run_step(cache, sched)                                      # 7 tokens known
    _, fin = _run_step(cache, sched)                             # 8 = max_position: stop
    assert fin[0].finish_reason == "context" and len(fin[0].tokens) == 8
    sched.add(_req("long", 9))                                   # prompt beyond the context
    assert not sched.has_work()


def test_requests_that_can_never_fit_finish_at_once():
    cache, sched = _setup(num_pages=4)
    r = _req("big", 60, max_tokens=10)                           # 70 tokens need 5 pages
    sched.add(r)
    assert r.finish_reason == "too_long" and not sched.has_work()
    with pytest.raises(ValueError, match="empty prompt"):
        sched.add(Request("e", []))
    # a group with a window needs the window only, but that much it does need
    for pages, fits in ((4, True), (3, False)):
        cache = CacheManager([PagedKVSpec(2, 16, 40)], page_size=16, num_pages=pages, max_requests=2)
        sched = Scheduler(cache, max_num_seqs=2, max_batched_tokens=16, max_position=1024)
        r = _req("w", 200, max_tokens=100)                       # 41 keys: 3 pages and one at the edge
        sched.add(r)
        assert (r.finish_reason is None) == fits
        while fits and sched.has_work():
            plan, _ = _run_step(cache, sched)
            for s in plan:
                if cache.has_request(s.request.req_id):
                    cache.release_passed(s.request.req_id)
        assert not fits or (r.finish_reason == "length" and len(r.output) == 100)


def test_pages_run_out_newest_is_preempted_and_recomputed():
    cache, sched = _setup(num_pages=4, max_num_seqs=3, budget=64)
    sched.add(_req("old", 30, max_tokens=30))                    # 2 pages, grows into a 3rd and 4th
    sched.add(_req("new", 30, max_tokens=30))                    # 2 pages
    _run_step(cache, sched)
    assert cache.free_pages() == [0]
    _run_step(cache, sched)                                      # 31 tokens in the cache
    _run_step(cache, sched)                                      # 32: both requests' pages are full
    plan, _ = _run_step(cache, sched)                            # both need a page: none is free
    assert [s.request.req_id for s in plan] == ["old"]
    new = sched.waiting[0]
    assert new.req_id == "new" and new.preemptions == 1 and new.computed == 0 and len(new.output) == 3
    assert sched.num_preemptions == 1 and cache.live_requests() == ["old"]
    # the old one runs on; when it finishes, the preempted one is recomputed from its 33 tokens
    seen_recompute = False
    for _ in range(80):
        if not sched.has_work():
            break
        plan, _ = _run_step(cache, sched)
        for s in plan:
            if s.request.req_id == "new" and s.count > 1:
                assert s.start == 0 and s.count == 33 and s.samples    # prompt 30 + 3 generated
                seen_recompute = True
    assert seen_recompute and not sched.has_work()
    assert len(new.output) == 30 and cache.free_pages() == [4]


def test_a_lone_request_preempts_itself_rather_than_deadlock():
    cache, sched = _setup(num_pages=2, max_num_seqs=2, budget=64, max_position=64)
    a = _req("a", 16, max_tokens=10)
    b = _req("b", 16, max_tokens=10)
    sched.add(a)
    sched.add(b)
    for _ in range(100):
        if not sched.has_work():
            break
        _run_step(cache, sched)
    assert a.finish_reason == b.finish_reason == "length" and len(a.output) == len(b.output) == 10
    assert sched.num_preemptions >= 1 and cache.free_pages() == [2]


def test_portion_is_shortened_to_the_pages_there_are():
    cache, sched = _setup(num_pages=3, max_num_seqs=2, budget=64)
    sched.add(_req("a", 20, max_tokens=2))                       # 2 pages
    _run_step(cache, sched)
    sched.add(_req("b", 10, max_tokens=2))                       # 1 page: fits
    plan, _ = _run_step(cache, sched)
    assert [(s.request.req_id, s.count) for s in plan] == [("a", 1), ("b", 10)]


def test_lookahead_tells_the_next_step_only_when_it_is_certain():
    """The step after a running one can be told ahead when all its requests choose a token now,
    none ends by its length, nothing waits and the pages are there."""
    cache, sched = _setup(num_pages=5, max_num_seqs=2, budget=64, eos=(9,))
    sched.add(_req("a", 20, max_tokens=3))
    sched.add(_req("b", 31, max_tokens=5))
    sched.add(_req("c", 4))                                     # waits for a request slot
    plan = sched.schedule()
    cache.reserve_step([(s.request.req_id, s.count) for s in plan])
    assert sched.lookahead(plan) is None                        # c waits for admission
    sched.waiting.clear()
    told = sched.lookahead(plan)
    assert [(s.request.req_id, s.start, s.count, s.samples) for s in told] == \
        [("a", 20, 1, True), ("b", 31, 1, True)]
    # the step told ahead is put on the device; only then are the first step's tokens known
    cache.reserve_step([(s.request.req_id, s.count) for s in told])
    sched.step_done(plan, [5, 5])
    third = sched.lookahead(told)
    assert [(s.request.req_id, s.start) for s in third] == [("a", 21), ("b", 32)]
    cache.reserve_step([(s.request.req_id, s.count) for s in third])
    sched.step_done(told, [5, 5])
    assert sched.lookahead(third) is None                       # a's third token is its last
    fin = sched.step_done(third, [5, 5])
    assert [r.req_id for r in fin] == ["a"] and fin[0].output == [5, 5, 5]
    plan = sched.schedule()
    assert [(s.request.req_id, s.start) for s in plan] == [("b", 33)]
    cache.check()


def test_lookahead_needs_the_pages_and_no_unfinished_prompt():
    cache, sched = _setup(num_pages=4, max_num_seqs=2, budget=40, chunk=None)
    sched.add(_req("a", 32, max_tokens=9))                      # two full pages: its next token needs a third
    sched.add(_req("b", 16, max_tokens=9))                      # cut: 8 tokens fit the budget
    plan = sched.schedule()
    assert [(s.request.req_id, s.count, s.samples) for s in plan] == [("a", 32, True), ("b", 8, False)]
    cache.reserve_step([(s.request.req_id, s.count) for s in plan])
    assert sched.lookahead(plan) is None                        # b is still inside its prompt
    sched.step_done(plan, [5])
    plan = sched.schedule()
    cache.reserve_step([(s.request.req_id, s.count) for s in plan])
    assert [(s.request.req_id, s.count) for s in plan] == [("a", 1), ("b", 8)]
    assert sched.lookahead(plan) is None                        # all four pages are taken: b's 17th token has none
    cache.check()


def test_a_request_that_stops_drops_the_token_of_the_step_told_ahead():
    cache, sched = _setup(eos=(9,))
    sched.add(_req("a", 3, max_tokens=50))
    sched.add(_req("b", 5, max_tokens=50))
    plan = sched.schedule()
    cache.reserve_step([(s.request.req_id, s.count) for s in plan])
    told = sched.lookahead(plan)
    cache.reserve_step([(s.request.req_id, s.count) for s in told])
    fin = sched.step_done(plan, [9, 4])                         # a stops on the token nobody knew
    assert [r.req_id for r in fin] == ["a"] and cache.live_requests() == ["b"]
    assert sched.lookahead(told) is None                        # the batch has changed
    assert sched.step_done(told, [7, 8]) == []
    a, b = plan[0].request, plan[1].request
    assert a.output == [9] and a.finish_reason == "stop"
    assert b.output == [4, 8] and b.computed == 6
    plan = sched.schedule()
    assert [(s.request.req_id, s.start, s.count) for s in plan] == [("b", 6, 1)]
    cache.check()
