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
