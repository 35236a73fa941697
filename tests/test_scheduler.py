"""The scheduler's decisions, on scripted traces with no model: tokens are
'sampled' by appending to `token_ids` by hand.  The scenarios restate Azimml/shrike's
tests/test_block_manager.py:60-99, tests/test_scheduler.py:21-66 and
tests/test_review_regressions.py:17-78."""

from shrike_b200.cache import CacheManager, KVGroupSpec
from shrike_b200.engine.request import Request, SamplingParams, Status
from shrike_b200.engine.scheduler import Scheduler

GROUP = KVGroupSpec((0,), 2, 16, None)


def make(num_pages, page_size=4, budget=8, max_running=8):
    manager = CacheManager([GROUP], page_size, num_pages, max_running)
    return manager, Scheduler(manager, max_tokens_per_step=budget, max_running=max_running)


def request(n, **kw):
    return Request(token_ids=list(range(n)), sampling=SamplingParams(**kw))


def run_step(scheduler, sample=True):
    batch = scheduler.schedule()
    scheduler.postprocess(batch)
    if sample:
        for req, _ in batch:
            if req.num_computed_tokens >= req.num_tokens:
                req.token_ids.append(0)
    return [(req.req_id, n) for req, n in batch]


def test_long_prompt_is_cut_under_the_budget_and_leftover_admits_the_next():
    manager, scheduler = make(64, budget=8)
    long, short = request(20), request(3)
    scheduler.add(long)
    scheduler.add(short)
    assert run_step(scheduler) == [(long.req_id, 8)]
    assert run_step(scheduler) == [(long.req_id, 8)]
    # 4 tokens finish the long prompt; the leftover budget of 4 admits the short one
    assert run_step(scheduler) == [(long.req_id, 4), (short.req_id, 3)]
    # both decode now: single tokens, in admission order
    assert run_step(scheduler) == [(long.req_id, 1), (short.req_id, 1)]


def test_singles_come_before_portions():
    manager, scheduler = make(64, budget=16)
    first = request(2)
    scheduler.add(first)
    run_step(scheduler)
    second = request(9)
    scheduler.add(second)
    batch = scheduler.schedule()
    assert [(r.req_id, n) for r, n in batch] == [(first.req_id, 1), (second.req_id, 9)]


def test_one_token_prompt_is_a_single():
    manager, scheduler = make(8)
    only = request(1)
    scheduler.add(only)
    assert run_step(scheduler) == [(only.req_id, 1)]
    assert only.num_tokens == 2 and only.status is Status.RUNNING


def test_pool_exhaustion_preempts_the_newest_and_recomputes_it():
    manager, scheduler = make(4, page_size=4, budget=32)
    old, new = request(7), request(7)
    scheduler.add(old)
    scheduler.add(new)
    assert run_step(scheduler) == [(old.req_id, 7), (new.req_id, 7)]   # 2 + 2 pages: pool full
    assert run_step(scheduler) == [(old.req_id, 1), (new.req_id, 1)]   # token 8 fits the held pages
    # token 9 of `old` needs a third page: the newest (`new`) is preempted and, sitting
    # at the head of the queue, is retried in the same step: 9 tokens need 3 pages, only
    # 1 is free, so it waits.
    batch = run_step(scheduler)
    assert batch == [(old.req_id, 1)]
    assert scheduler.num_preemptions == 1
    assert new.status is Status.WAITING and new.num_computed_tokens == 0 and new.cache is None
    assert scheduler.waiting[0] is new and new.num_tokens == 9       # keeps what it generated
    scheduler.finish(old, "length")
    assert manager.whole()
    # re-admitted whole: only the prompt is prefilled as a portion, history is replayed token by token
    assert run_step(scheduler, sample=False) == [(new.req_id, 7)]
    assert run_step(scheduler, sample=False) == [(new.req_id, 1)]
    assert new.num_computed_tokens == 8 and new.num_tokens == 9


def test_a_request_that_is_itself_the_newest_sits_the_step_out():
    manager, scheduler = make(2, page_size=4, budget=32)
    only = request(8)
    scheduler.add(only)
    assert run_step(scheduler) == [(only.req_id, 8)]
    # the 9th token needs a page and none is free: it preempts itself, is skipped in the
    # running pass, and (now at the head of the queue, pool empty) is admitted again in
    # the same step with its prompt only.  The engine refuses such a request at
    # add_request, because it could never finish.
    assert run_step(scheduler, sample=False) == [(only.req_id, 8)]
    assert scheduler.num_preemptions == 1 and only.status is Status.RUNNING
    assert only.num_computed_tokens == 8 and only.num_tokens == 9


def test_max_running_caps_admission():
    manager, scheduler = make(64, budget=64, max_running=2)
    reqs = [request(3) for _ in range(4)]
    for r in reqs:
        scheduler.add(r)
    assert [rid for rid, _ in run_step(scheduler)] == [reqs[0].req_id, reqs[1].req_id]
    assert len(scheduler.running) == 2 and len(scheduler.waiting) == 2
    scheduler.finish(reqs[0], "length")
    assert reqs[2].req_id in [rid for rid, _ in run_step(scheduler)]


def test_head_of_line_blocking_is_fcfs():
    manager, scheduler = make(4, page_size=4, budget=64)
    holder, big, small = request(8), request(12), request(2)
    scheduler.add(holder)
    run_step(scheduler)            # holds 2 of 4 pages
    scheduler.add(big)             # needs 3 pages: does not fit
    scheduler.add(small)           # would fit, but may not overtake
    batch = run_step(scheduler)
    assert [rid for rid, _ in batch] == [holder.req_id]
    assert list(scheduler.waiting) == [big, small]
    scheduler.finish(holder, "length")
    assert [rid for rid, _ in run_step(scheduler)] == [big.req_id, small.req_id]


def test_budget_zero_leaves_later_running_requests_out():
    manager, scheduler = make(64, budget=2)
    reqs = [request(1) for _ in range(3)]
    for r in reqs:
        scheduler.add(r)
    assert len(run_step(scheduler)) == 2
    assert len(run_step(scheduler)) == 2   # two running decode; the third is still waiting
    assert len(scheduler.waiting) == 1


def test_finish_and_abort_give_everything_back():
    manager, scheduler = make(16, budget=64)
    a, b, c = request(5), request(9), request(3)
    for r in (a, b):
        scheduler.add(r)
    run_step(scheduler)
    scheduler.add(c)
    scheduler.finish(a, "stop")
    assert a.status is Status.FINISHED and a.finish_reason == "stop" and a.cache is None
    scheduler.abort(b)     # running
    scheduler.abort(c)     # still waiting
    assert not scheduler.has_work and manager.whole()
    assert b.finish_reason == "aborted" and c.finish_reason == "aborted"


def test_empty_schedule_when_nothing_fits():
    manager, scheduler = make(1, page_size=4, budget=64)
    scheduler.add(request(9))
    assert scheduler.schedule() == []
    assert scheduler.has_work


def test_preempt_newest_is_an_operators_lever_and_a_preempted_request_may_still_finish():
    manager, scheduler = make(num_pages=16)
    a, b = request(6, max_new_tokens=4), request(5, max_new_tokens=4)
    scheduler.add(a)
    scheduler.add(b)
    run_step(scheduler)
    assert scheduler.running == [a, b]
    assert scheduler.preempt_newest() is b and scheduler.num_preemptions == 1
    assert b.status is Status.WAITING and b.num_computed_tokens == 0 and b.cache is None and scheduler.waiting[0] is b
    scheduler.finish(b, "length")          # the step in flight when it was preempted produced its last token
    assert b.status is Status.FINISHED and not scheduler.waiting
    scheduler.finish(a, "stop")
    assert manager.whole() and scheduler.preempt_newest() is None


def test_a_portion_never_outgrows_a_windowed_groups_pool():
    """A group with a window has a small pool of its own.  The scheduler cuts a prompt so that
    the window and the portion fit in it, however large the token budget is."""
    full, window = KVGroupSpec((0,), 2, 16, None), KVGroupSpec((1,), 2, 16, 6)
    manager = CacheManager([full, window], 4, [64, 6], 4)      # the windowed pool: 6 pages of 4
    scheduler = Scheduler(manager, max_tokens_per_step=64, max_running=4)
    assert manager.portion_limit() == (6 - 2) * 4 - 6 + 2 == 12
    long_prompt = request(50, max_new_tokens=2)
    scheduler.add(long_prompt)
    fed = []
    while not long_prompt.prefill_done:
        batch = scheduler.schedule()
        assert batch, "the prompt can never be scheduled"
        fed.append(batch[0][1])
        scheduler.postprocess(batch)
    assert max(fed) == 12 and sum(fed) == 50 and scheduler.num_preemptions == 0
    scheduler.finish(long_prompt, "length")
    assert manager.whole()
