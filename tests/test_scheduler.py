"""The scheduler's decisions (no GPU): admission, portions under a token budget, decoding,
finishing and freeing, and what happens when pages run out.  The model is a stub that
returns a fixed function of the tokens run so far."""
import torch

from lgml_b200.cache import CacheManager, PagedKV
from lgml_b200.engine.scheduler import GenRequest, Scheduler
from lgml_b200.sampling import SamplingParams


def make(n_pages=8, slots=4, ubatch=512, budget=2048, max_position=4096, repeat_stop=0):
    cm = CacheManager({0: PagedKV(1, 8)}, n_pages=n_pages, max_slots=slots, dtype=torch.float32, device="cpu")
    return Scheduler(cm, max_position=max_position, ubatch=ubatch, max_batch_tokens=budget, repeat_stop_tokens=repeat_stop), cm


def req(rid, n_prompt, max_new, stop=()):
    return GenRequest(id=rid, prompt=list(range(1, n_prompt + 1)), max_new_tokens=max_new, params=SamplingParams.neutral(0.0), stop_ids=stop)


def stub_token(r):
    """What the stub model 'samples': a function of the tokens the request holds."""
    return (sum(r.tokens) * 31 + len(r.tokens)) % 1000 + 1000


def drive(s, cm, log=None, limit=10000):
    for _ in range(limit):
        if s.idle:
            return
        plan = s.plan()
        if log is not None:
            log.append([(e.request.id, len(e.tokens), e.sample) for e in plan])
        for e in plan:                          # the runner would commit the cached tokens
            cm.commit(e.request.cache_req, len(e.tokens))
        cm.check()
        s.complete(plan, {e.request.id: stub_token(e.request) for e in plan if e.sample})
    raise AssertionError("the scheduler did not finish")


def solo(n_prompt, max_new, **kw):
    s, cm = make(**kw)
    r = req("solo", n_prompt, max_new)
    s.add(r)
    drive(s, cm)
    return r.generated


def test_prompt_is_cut_into_portions_then_decoded():
    s, cm = make(ubatch=100, n_pages=8)
    r = req("a", 250, 3)
    s.add(r)
    log = []
    drive(s, cm, log)
    assert log[:3] == [[("a", 100, False)], [("a", 100, False)], [("a", 50, True)]]
    assert log[3:] == [[("a", 1, True)], [("a", 1, True)]]
    assert r.finish_reason == "length" and len(r.generated) == 3
    assert cm.n_free_pages == 8 and not cm.live


def test_token_budget_bounds_a_step_and_decodes_go_first():
    s, cm = make(ubatch=64, budget=100, n_pages=16)
    a, b = req("a", 10, 50), req("b", 300, 2)
    s.add(a)
    s.add(b)
    log = []
    drive(s, cm, log)
    assert all(sum(n for _, n, _ in step) <= 100 for step in log)
    assert log[0] == [("a", 10, True), ("b", 64, False)]
    assert log[1][0] == ("a", 1, True) and log[1][1] == ("b", 64, False)     # a decoded token beside a prompt portion
    assert len(a.generated) == 50 and len(b.generated) == 2


def test_fifo_admission_and_slot_limit():
    s, cm = make(slots=2, n_pages=16)
    rs = [req(i, 20, 4) for i in range(5)]
    for r in rs:
        s.add(r)
    log = []
    drive(s, cm, log)
    assert all(len(step) <= 2 for step in log)
    first_seen = [next(i for i, step in enumerate(log) if any(e[0] == r.id for e in step)) for r in rs]
    assert first_seen == sorted(first_seen)
    assert all(len(r.generated) == 4 for r in rs)
    assert cm.n_free_pages == 16


def test_admission_waits_for_room_for_prompt_plus_one():
    s, cm = make(n_pages=3, slots=4)
    a, b = req("a", 100, 10), req("b", 128, 5)          # b needs 3 pages for 129 tokens; a holds 2
    s.add(a)
    s.add(b)
    log = []
    drive(s, cm, log)
    b_first = next(i for i, step in enumerate(log) if any(e[0] == "b" for e in step))
    a_last = max(i for i, step in enumerate(log) if any(e[0] == "a" for e in step))
    assert b_first > a_last
    assert len(b.generated) == 5 and s.stats["preemptions"] == 0


def test_stop_token_and_position_limit():
    s, cm = make(max_position=40)
    r = req("a", 30, 100)
    s.add(r)
    drive(s, cm)
    assert r.finish_reason == "length" and len(r.prompt) + len(r.generated) == 40
    s, cm = make()
    r = req("a", 5, 100)
    expect_first = stub_token(r)
    r.stop_ids = (expect_first,)
    s.add(r)
    drive(s, cm)
    assert r.finish_reason == "stop" and r.generated == [expect_first]


def test_repeat_guard():
    s, cm = make(repeat_stop=4)
    r = req("a", 5, 100)
    s.add(r)
    for _ in range(100):
        if s.idle:
            break
        plan = s.plan()
        for e in plan:
            cm.commit(e.request.cache_req, len(e.tokens))
        s.complete(plan, {e.request.id: 7 for e in plan if e.sample})
    assert r.finish_reason == "length" and r.generated == [7, 7, 7, 7]


def test_out_of_pages_preempts_the_latest_and_the_reply_is_whole():
    """Two requests outgrow a pool that held both prompts: the later one is preempted, gives
    its pages back, is prefilled again from prompt + generated, and ends with the same
    reply as alone."""
    want_a, want_b = solo(60, 80, n_pages=8), solo(50, 90, n_pages=8)
    s, cm = make(n_pages=3, slots=4)
    a, b = req("a", 60, 80), req("b", 50, 90)
    s.add(a)
    s.add(b)
    log = []
    drive(s, cm, log)
    assert s.stats["preemptions"] >= 1 and b.preemptions >= 1 and a.preemptions == 0
    assert a.generated == want_a and b.generated == want_b
    assert a.finish_reason == "length" and b.finish_reason == "length"
    # after the preemption b came back as one long prompt
    refill = [n for step in log for rid, n, _ in step if rid == "b" and n > 1]
    assert len(refill) >= 2 and refill[-1] > 50
    assert cm.n_free_pages == 3 and not cm.live
    cm.check()


def test_alone_and_out_of_pages_ends_with_length():
    s, cm = make(n_pages=2)
    r = req("a", 100, 500)
    s.add(r)
    drive(s, cm)
    assert r.finish_reason == "length"
    assert len(r.prompt) + len(r.generated) == 128 + 1         # the last sampled token has no cell and needs none
    assert cm.n_free_pages == 2


def test_prompts_that_can_never_fit_are_refused():
    import pytest

    s, cm = make(n_pages=2, max_position=1000)
    with pytest.raises(ValueError, match="cache pool"):
        s.add(req("big", 128, 1))
    with pytest.raises(ValueError, match="context"):
        s.add(req("long", 1000, 1))
    with pytest.raises(ValueError, match="empty"):
        s.add(GenRequest(id="e", prompt=[], max_new_tokens=1))


def drive_ahead(s, cm, log=None, limit=10000):
    """As an engine that launches a decode step before it has seen the ids of the step before:
    the step after ``inflight`` is planned (and 'launched': committed) first, then ``inflight``
    is completed."""
    inflight = None
    for _ in range(limit):
        if inflight is None:
            if s.idle:
                return
            inflight = s.plan()
            for e in inflight:
                cm.commit(e.request.cache_req, len(e.tokens))
            if log is not None:
                log.append(("plan", [(e.request.id, len(e.tokens)) for e in inflight]))
            continue
        nxt = s.plan_ahead(inflight)
        if nxt is not None:
            for e in nxt:
                cm.commit(e.request.cache_req, 1)
            if log is not None:
                log.append(("ahead", [(e.request.id, len(e.tokens)) for e in nxt]))
        cm.check()
        s.complete(inflight, {e.request.id: stub_token(e.request) for e in inflight if e.sample and e.request.finish_reason is None})
        cm.check()
        inflight = nxt
    raise AssertionError("the scheduler did not finish")


def test_planning_ahead_gives_the_same_replies():
    outs = []
    for ahead in (False, True):
        s, cm = make(ubatch=64, budget=128, n_pages=12, slots=3)
        rs = [req("a", 70, 40), req("b", 130, 25), req("c", 5, 60), req("d", 64, 64)]
        for r in rs:
            s.add(r)
        (drive_ahead if ahead else drive)(s, cm)
        assert cm.n_free_pages == 12 and not cm.live
        outs.append([(r.generated, r.finish_reason) for r in rs])
    assert outs[0] == outs[1]


def test_planning_ahead_only_when_nothing_but_an_end_token_can_change_the_plan():
    s, cm = make(ubatch=64, n_pages=8, slots=2)
    a = req("a", 10, 5)
    s.add(a)
    p0 = s.plan()
    cm.commit(a.cache_req, 10)
    # one request, decoding, tokens left: the next step can be planned before the id is known
    p1 = s.plan_ahead(p0)
    assert p1 is not None and [(e.request.id, len(e.tokens), e.sample) for e in p1] == [("a", 1, True)]
    cm.commit(a.cache_req, 1)
    s.complete(p0, {"a": 7})
    # a request waits: admission comes first
    s.add(req("b", 10, 5))
    assert s.plan_ahead(p1) is None
    s.complete(p1, {"a": 8})
    p2 = s.plan()                       # a decodes, b's prompt is admitted
    assert sorted((e.request.id, len(e.tokens)) for e in p2) == [("a", 1), ("b", 10)]
    for e in p2:
        cm.commit(e.request.cache_req, len(e.tokens))
    p3 = s.plan_ahead(p2)               # both sample in p2: both can go on
    assert p3 is not None and len(p3) == 2
    for e in p3:
        cm.commit(e.request.cache_req, 1)
    s.complete(p2, {"a": 9, "b": 9})
    # a has 3 of 5; after p3 it has 4, after the next 5: that step can still be planned ahead,
    # the one after it cannot (the limit ends a there)
    p4 = s.plan_ahead(p3)
    assert p4 is not None
    for e in p4:
        cm.commit(e.request.cache_req, 1)
    s.complete(p3, {"a": 9, "b": 9})
    assert s.plan_ahead(p4) is None
    s.complete(p4, {"a": 9, "b": 9})
    assert a.finish_reason == "length" and len(a.generated) == 5
    cm.check()


def test_an_end_token_drops_the_step_planned_ahead():
    s, cm = make(n_pages=8, slots=2)
    a, b = req("a", 10, 50, stop=(77,)), req("b", 20, 50)
    s.add(a)
    s.add(b)
    p0 = s.plan()
    for e in p0:
        cm.commit(e.request.cache_req, len(e.tokens))
    p1 = s.plan_ahead(p0)
    for e in p1:
        cm.commit(e.request.cache_req, 1)
    done = s.complete(p0, {"a": 77, "b": 5})          # a ends while its next token is under way
    assert done == [a] and a.finish_reason == "stop" and a.generated == [77]
    cm.check()
    assert s.plan_ahead(p1) is None                   # the batch changed
    s.complete(p1, {"a": 123, "b": 6})                # a's extra token is dropped
    assert a.generated == [77] and b.generated == [5, 6] and b.n_cached == 21
    cm.check()
    assert len(cm.live) == 1


def test_planning_ahead_stops_when_a_page_is_missing():
    s, cm = make(n_pages=2, slots=1)
    a = req("a", 120, 50)
    s.add(a)
    inflight = s.plan()
    cm.commit(a.cache_req, 120)
    n = 0
    while True:
        nxt = s.plan_ahead(inflight)
        if nxt is None:
            break
        cm.commit(a.cache_req, 1)
        s.complete(inflight, {"a": 3})
        inflight = nxt
        n += 1
    assert a.cache_req.n_tokens == 128 and n == 8    # both pages full: the next token needs a third
    s.complete(inflight, {"a": 3})
    assert s.plan() == [] and a.finish_reason == "length"   # alone and out of pages
    cm.check()


# ---------------------------------------------------------------------------------------------
# prefix cache
# ---------------------------------------------------------------------------------------------

def make_prefix(n_pages=8, slots=4, **kw):
    cm = CacheManager({0: PagedKV(1, 8)}, n_pages=n_pages, max_slots=slots, dtype=torch.float32, device="cpu", prefix_cache=True)
    return Scheduler(cm, max_position=4096, ubatch=kw.get("ubatch", 512), max_batch_tokens=kw.get("budget", 2048), repeat_stop_tokens=0), cm


def test_a_prompt_that_begins_like_an_earlier_one_runs_only_the_rest():
    s, cm = make_prefix()
    a = req("a", 200, 2)
    s.add(a)
    drive(s, cm)
    assert s.stats["prefix_tokens"] == 0 and cm.groups[0].pool.n_cached == 3      # 200 + 2 tokens: three full pages stay findable
    b = req("b", 200, 2)                                                          # the same prompt
    s.add(b)
    log = []
    drive(s, cm, log)
    assert log[0] == [("b", 200 - 192, True)] and s.stats["prefix_tokens"] == 192
    assert b.generated == a.generated                                             # the stub's tokens depend on the tokens alone
    c = GenRequest(id="c", prompt=list(range(1, 101)) + [7] * 100, max_new_tokens=1, params=SamplingParams.neutral(0.0))
    s.add(c)                                                                      # 100 tokens in common: one full page
    log = []
    drive(s, cm, log)
    assert log[0] == [("c", 200 - 64, True)]
    cm.check()
    assert not cm.live and cm.groups[0].pool.n_held == 0


def test_admission_counts_cached_pages_once():
    """A pool of 4 pages whose 3 cached pages are the new prompt's prefix: the prompt needs 4 pages,
    3 of them are the cached ones, and that fits; another prompt of the same length does not."""
    s, cm = make_prefix(n_pages=4, slots=2)
    a = req("a", 193, 1)
    s.add(a)
    drive(s, cm)
    assert cm.groups[0].pool.n_cached == 3 and cm.n_free_pages == 4
    b = req("b", 250, 2)                      # begins like a (192 tokens in common), needs 4 pages in all
    s.add(b)
    drive(s, cm)
    assert b.finish_reason == "length" and len(b.generated) == 2 and s.stats["prefix_tokens"] == 192
    assert cm.groups[0].pool.evicted_total == 0


def test_a_preempted_request_takes_up_its_own_pages_again():
    s, cm = make_prefix(n_pages=6, slots=2, ubatch=64)
    a, b = req("a", 130, 70), GenRequest(id="b", prompt=list(range(500, 630)), max_new_tokens=70, params=SamplingParams.neutral(0.0))
    s.add(a)
    s.add(b)
    drive(s, cm)
    assert s.stats["preemptions"] >= 1 and s.stats["prefix_tokens"] >= 128       # the victim found its first pages again
    assert a.generated == solo_prefix(130, 70, a.prompt) and b.generated == solo_prefix(130, 70, b.prompt)
    assert not cm.live and cm.groups[0].pool.n_held == 0


def solo_prefix(n_prompt, max_new, prompt):
    s, cm = make_prefix(n_pages=16)
    r = GenRequest(id="solo", prompt=list(prompt), max_new_tokens=max_new, params=SamplingParams.neutral(0.0))
    s.add(r)
    drive(s, cm)
    return r.generated


def test_a_preempted_request_that_was_already_planned_gives_its_tokens_back():
    """The latest request is decoding and is planned first; an older one, still reading its prompt
    in portions, then finds no page and preempts it.  The victim's token leaves the plan and returns
    to the step's budget (the portion planned after it is a token longer for it), and the victim
    is not let in again in the same call."""
    s, cm = make(n_pages=5, slots=4, ubatch=32, budget=2048)
    a, c, b = req("a", 150, 4), req("c", 150, 4), req("b", 3, 200)
    for r in (a, c, b):
        s.add(r)
    seen = False
    for _ in range(400):
        if s.idle:
            break
        before = s.stats["preemptions"]
        was_running = [r.id for r in s.running]
        plan = s.plan()
        s.max_batch_tokens = 40              # all three are let in by the first call; from then on the budget binds
        if s.stats["preemptions"] > before and "b" in was_running and not seen:
            seen = True
            ids = [e.request.id for e in plan]
            assert "b" not in ids and b in s.waiting and b.cache_req is None      # out of the plan, not back in at once
            assert sum(len(e.tokens) for e in plan) == 40                         # its token went to the next portion
            assert [(e.request.id, len(e.tokens)) for e in plan] == [("a", 22), ("c", 18)]
        for e in plan:
            cm.commit(e.request.cache_req, len(e.tokens))
        cm.check()
        s.complete(plan, {e.request.id: stub_token(e.request) for e in plan if e.sample})
    assert seen and s.idle
    assert b.preemptions >= 1 and len(b.generated) == 200 and b.generated == solo_of(3, 200)
    assert cm.n_free_pages == 5 and not cm.live


def solo_of(n_prompt, max_new):
    s, cm = make(n_pages=8)
    r = req("b", n_prompt, max_new)
    s.add(r)
    drive(s, cm)
    return r.generated
