"""The scheduler's decisions, with a stub in place of the step function."""

import random

import pytest

from kairyu_b200.cache import CacheLayout, CacheManager
from kairyu_b200.engine.scheduler import EngineRequest, Scheduler, Status
from kairyu_b200.parts.base import PagedKVSpec


def make(num_pages=17, page_size=4, **kwargs):
    layout = CacheLayout.from_slot_specs({0: (PagedKVSpec(1, 16),)})
    cache = CacheManager(layout, num_pages=num_pages, page_size=page_size, max_requests=kwargs.get("max_num_seqs", 8))
    return Scheduler(cache, **kwargs), cache


def request(name, prompt_len, max_new=4, **kwargs):
    return EngineRequest(name, tuple(range(1, prompt_len + 1)), max_new_tokens=max_new, **kwargs)


def run_step(scheduler, cache, token=7):
    """What the engine does around one plan, with a constant sampled token."""
    plan = scheduler.schedule()
    sampled = {}
    for chunk in plan.scheduled:
        assert cache.get(chunk.request_id).num_tokens == chunk.start
        cache.advance(chunk.request_id, chunk.start + chunk.num_tokens)
        if chunk.samples:
            sampled[chunk.request_id] = token
    finished = scheduler.update(sampled)
    cache.check()
    return plan, finished


def test_prompt_is_cut_under_the_token_budget_and_decodes_come_first():
    scheduler, cache = make(max_num_batched_tokens=8)
    scheduler.add_request(request("a", 19))
    sizes = []
    for _ in range(3):
        plan, _ = run_step(scheduler, cache)
        assert len(plan.scheduled) == 1 and plan.scheduled[0].is_prefill
        sizes.append(plan.scheduled[0].num_tokens)
    assert sizes == [8, 8, 3] and plan.scheduled[0].samples
    scheduler.add_request(request("b", 20))
    plan, _ = run_step(scheduler, cache)
    assert [(c.request_id, c.num_tokens, c.is_prefill) for c in plan.scheduled] == [("a", 1, False), ("b", 7, True)]
    assert sum(c.num_tokens for c in plan.scheduled) <= 8


def test_prefill_chunk_size_caps_a_portion():
    scheduler, cache = make(max_num_batched_tokens=100, prefill_chunk_size=6, num_pages=40)
    scheduler.add_request(request("a", 15))
    sizes = [run_step(scheduler, cache)[0].scheduled[0].num_tokens for _ in range(3)]
    assert sizes == [6, 6, 3]


def test_partial_prefills_are_limited_and_share_the_budget():
    scheduler, cache = make(max_num_batched_tokens=10, max_num_partial_prefills=2, num_pages=60)
    for name in "abc":
        scheduler.add_request(request(name, 30))
    plan, _ = run_step(scheduler, cache)
    # the first admission takes the whole budget; nobody else fits this step
    assert [(c.request_id, c.num_tokens) for c in plan.scheduled] == [("a", 10)]
    plan, _ = run_step(scheduler, cache)
    assert [(c.request_id, c.num_tokens) for c in plan.scheduled] == [("a", 10)]
    # c is never admitted while a and b are both mid-prompt
    seen = set()
    for _ in range(4):
        plan, _ = run_step(scheduler, cache)
        seen |= {c.request_id for c in plan.scheduled if c.is_prefill and not c.samples}
        assert len([c for c in plan.scheduled if c.is_prefill and not c.samples]) <= 2


def test_finish_reasons():
    scheduler, cache = make()
    scheduler.add_request(request("len", 3, max_new=2))
    scheduler.add_request(request("eos", 3, max_new=9, eos_token_ids=(7,)))
    scheduler.add_request(request("ign", 3, max_new=3, eos_token_ids=(7,), ignore_eos=True))
    scheduler.add_request(request("min", 3, max_new=9, stop_token_ids=(7,), min_tokens=3))
    done = {}
    for _ in range(6):
        _, finished = run_step(scheduler, cache)
        for name in finished:
            done[name] = (scheduler.finish_reason(name), len(scheduler.output_tokens(name)))
    assert done == {"len": ("length", 2), "eos": ("stop", 1), "ign": ("length", 3), "min": ("stop", 3)}
    assert cache.live_requests == 0 and not scheduler.has_unfinished()


def test_bad_requests_are_refused_at_the_door():
    scheduler, _ = make(max_model_len=20)
    with pytest.raises(ValueError, match="at least one prompt token"):
        scheduler.add_request(request("a", 0))
    with pytest.raises(ValueError, match="max_model_len"):
        scheduler.add_request(request("a", 18, max_new=3))
    scheduler.add_request(request("a", 5))
    with pytest.raises(ValueError, match="already known"):
        scheduler.add_request(request("a", 5))
    with pytest.raises(ValueError, match="not awaiting"):
        scheduler.update({"a": 1})
    with pytest.raises(TypeError):
        scheduler.update({"a": "1"})


def test_head_of_queue_waits_for_pages_and_a_hopeless_prompt_is_rejected():
    scheduler, cache = make(num_pages=9, page_size=4)  # 8 usable pages = 32 tokens
    scheduler.add_request(request("a", 20, max_new=3))
    scheduler.add_request(request("b", 16, max_new=2))
    scheduler.add_request(request("huge", 40, max_new=2))
    plan, _ = run_step(scheduler, cache)
    assert [c.request_id for c in plan.scheduled] == ["a"]  # b needs 4 pages, 3 are free: it waits
    assert scheduler.state("b").status is Status.WAITING
    finished_at = {}
    for step in range(12):
        plan, finished = run_step(scheduler, cache)
        for name in finished + plan.rejected:
            finished_at[name] = step
    assert scheduler.finish_reason("huge") == "length" and scheduler.output_tokens("huge") == ()
    assert scheduler.finish_reason("a") == "length" and len(scheduler.output_tokens("a")) == 3
    assert len(scheduler.output_tokens("b")) == 2 and finished_at["b"] > finished_at["a"]
    assert scheduler.counters["rejections"] == 1


def test_decode_out_of_pages_preempts_the_youngest_request_without_outputs():
    scheduler, cache = make(num_pages=7, page_size=4, max_num_batched_tokens=6)  # 6 usable pages
    scheduler.add_request(request("old", 7, max_new=8))  # grows to 14 cached tokens: 4 pages in the end
    run_step(scheduler, cache)  # 6 tokens
    run_step(scheduler, cache)  # 1 token, samples
    # young is admitted while 4 pages are free, takes them portion by portion, and gets stuck
    # one page short once old has grown; old's next page then has to come from young
    scheduler.add_request(request("young", 16, max_new=2))
    events = []
    for _ in range(30):
        if not scheduler.has_unfinished():
            break
        plan, finished = run_step(scheduler, cache)
        events.append((tuple(c.request_id for c in plan.scheduled), plan.preempted))
    assert scheduler.counters["preemptions"] >= 1
    assert any("young" in preempted for _, preempted in events) or scheduler.state("young").preemptions >= 1
    assert scheduler.state("old").preemptions == 0
    assert len(scheduler.output_tokens("old")) == 8 and len(scheduler.output_tokens("young")) == 2
    assert cache.live_requests == 0


def test_preempted_request_with_outputs_recomputes_them():
    scheduler, cache = make(num_pages=5, page_size=4, max_num_batched_tokens=50)  # 4 usable pages
    scheduler.add_request(request("a", 4, max_new=12))
    scheduler.add_request(request("b", 4, max_new=12))
    steps = 0
    while scheduler.has_unfinished() and steps < 200:
        plan, _ = run_step(scheduler, cache)
        for chunk in plan.scheduled:
            state = scheduler.state(chunk.request_id) if chunk.request_id in scheduler._states else None
        steps += 1
    # 2 x 15 tokens do not fit 16 slots at once: one was preempted with outputs and fed them again
    assert scheduler.counters["preemptions"] >= 1
    assert len(scheduler.output_tokens("a")) == 12 and len(scheduler.output_tokens("b")) == 12


def test_lone_request_that_outgrows_the_cache_ends_with_length():
    scheduler, cache = make(num_pages=3, page_size=4)  # 8 token slots
    scheduler.add_request(request("a", 6, max_new=10))
    for _ in range(12):
        if not scheduler.has_unfinished():
            break
        run_step(scheduler, cache)
    assert scheduler.finish_reason("a") == "length"
    assert 1 <= len(scheduler.output_tokens("a")) < 10
    assert cache.live_requests == 0


def test_abort_frees_pages():
    scheduler, cache = make()
    scheduler.add_request(request("a", 10))
    scheduler.add_request(request("b", 10))
    run_step(scheduler, cache)
    scheduler.abort("a")
    assert scheduler.finish_reason("a") == "abort" and "a" not in cache
    scheduler.abort("b")
    scheduler.abort("nobody")
    assert cache.live_requests == 0 and not scheduler.has_unfinished()


@pytest.mark.parametrize("seed", range(6))
def test_random_workloads_finish_and_leave_the_cache_empty(seed):
    rng = random.Random(seed)
    scheduler, cache = make(
        num_pages=rng.choice([9, 14, 30]), page_size=rng.choice([2, 4, 8]), max_num_batched_tokens=rng.choice([5, 16, 64]),
        max_num_seqs=4, max_num_partial_prefills=rng.choice([1, 2]),
    )
    wanted = {}
    for index in range(12):
        prompt, new = rng.randint(1, 24), rng.randint(1, 12)
        scheduler.add_request(request(f"r{index}", prompt, max_new=new))
        wanted[f"r{index}"] = new
    steps = 0
    while scheduler.has_unfinished():
        plan, _ = run_step(scheduler, cache)
        assert sum(c.num_tokens for c in plan.scheduled) <= scheduler.budget
        assert len({c.request_id for c in plan.scheduled}) == len(plan.scheduled)
        steps += 1
        assert steps < 2000, "the scheduler stopped making progress"
    assert cache.live_requests == 0
    for name, new in wanted.items():
        reason = scheduler.finish_reason(name)
        assert reason == "length"
        outputs = len(scheduler.output_tokens(name))
        assert outputs == new or (outputs < new and not cache.can_hold(len(scheduler.state(name).request.prompt_token_ids) + new - 1))


# ------------------------------------------------------------------ schedule-ahead


def test_a_sampled_token_in_flight_can_be_fed_before_it_is_known():
    scheduler, cache = make(num_pages=16, page_size=4)
    scheduler.add_request(EngineRequest("a", tuple(range(1, 6)), max_new_tokens=3))
    first = scheduler.schedule().scheduled
    assert [(c.start, c.num_tokens, c.samples) for c in first] == [(0, 5, True)]
    assert scheduler.state("a").in_flight == 1
    ahead = scheduler.schedule().scheduled  # planned before update(): feeds the token in flight
    assert [(c.start, c.num_tokens, c.samples) for c in ahead] == [(5, 1, True)]
    assert ahead[0].start >= scheduler.state("a").total_tokens  # its value is not known to the host
    assert scheduler.state("a").in_flight == 2
    assert scheduler.schedule().scheduled[0].start == 6          # a third: max_new_tokens = 3 allows it
    assert scheduler.schedule().scheduled == ()                  # but no fourth
    assert scheduler.update({"a": 11}) == () and scheduler.state("a").in_flight == 2
    assert scheduler.update({"a": 12}) == ()
    assert scheduler.update({"a": 13}) == ("a",)
    assert scheduler.output_tokens("a") == (11, 12, 13) and scheduler.finish_reason("a") == "length"
    cache.check()


def test_tokens_that_arrive_after_a_stop_are_dropped_and_in_flight_requests_are_not_victims():
    scheduler, cache = make(num_pages=16, page_size=4)
    scheduler.add_request(EngineRequest("a", (1, 2, 3), max_new_tokens=8, stop_token_ids=(42,)))
    scheduler.schedule()
    scheduler.schedule()  # ahead
    assert scheduler.update({"a": 42}) == ("a",)      # the stop: finished with one token still in flight
    assert scheduler.update({"a": 7}) == ()           # the late token is dropped
    assert scheduler.output_tokens("a") == (42,)
    assert "a" not in cache
    # a request with a token in flight is never chosen as a victim
    scheduler.add_request(EngineRequest("b", (1, 2, 3, 4), max_new_tokens=4))
    scheduler.add_request(EngineRequest("c", (5, 6, 7, 8), max_new_tokens=4))
    scheduler.schedule()
    assert scheduler._pick_victim("b", set()) is None and scheduler.state("c").in_flight == 1
    scheduler.update({"b": 1, "c": 2})
    assert scheduler._pick_victim("b", set()) == "c"


def test_the_request_behind_a_blocked_head_goes_first_once():
    """kairyu/engine/core/scheduler.py:28, 1543-1577: while the head waits for pages and something
    runs, its direct successor may be admitted, once; a second successor waits behind the head."""
    scheduler, cache = make(num_pages=9, page_size=4, max_num_batched_tokens=64)  # 8 pages
    scheduler.add_request(request("running", 10, max_new=8))   # 5 pages by its end
    run_step(scheduler, cache)
    scheduler.add_request(request("big", 24, max_new=2))       # 7 pages: must wait for "running"
    scheduler.add_request(request("small", 5, max_new=2))      # 2 pages: fits beside "running"
    scheduler.add_request(request("small2", 5, max_new=2))
    plan, _ = run_step(scheduler, cache)
    assert [c.request_id for c in plan.scheduled] == ["running", "small"]
    assert scheduler.state("big").bypasses == 1 and scheduler.state("big").status is Status.WAITING
    plan, _ = run_step(scheduler, cache)
    # the head has been passed once: small2 stays behind it although it would fit
    assert sorted(c.request_id for c in plan.scheduled) == ["running", "small"]
    assert scheduler.num_waiting == 2
    for _ in range(40):
        if not scheduler.has_unfinished():
            break
        run_step(scheduler, cache)
    assert not scheduler.has_unfinished()
    for name, count in (("running", 8), ("big", 2), ("small", 2), ("small2", 2)):
        assert len(scheduler.output_tokens(name)) == count


def test_nothing_passes_a_blocked_head_when_nothing_runs():
    scheduler, cache = make(num_pages=5, page_size=4, max_num_batched_tokens=64)  # 4 pages
    scheduler.add_request(request("too-big", 30))   # 8 pages: can never fit
    scheduler.add_request(request("fits", 6, max_new=2))
    plan, _ = run_step(scheduler, cache)
    assert plan.rejected == ("too-big",) and [c.request_id for c in plan.scheduled] == ["fits"]


def test_priority_scheduling_orders_the_waiting_queue():
    """Lower priority values are admitted first, first come first served among equals; a preempted
    request goes back to its place by its arrival (kairyu/engine/core/scheduler.py:191-199)."""
    scheduler, cache = make(num_pages=40, max_num_batched_tokens=6, max_num_partial_prefills=1, priority_scheduling=True)
    for name, priority in (("late-low", 5), ("first", 0), ("urgent", -1), ("second", 0)):
        scheduler.add_request(EngineRequest(name, tuple(range(1, 7)), max_new_tokens=1, priority=priority))
    order = []
    for _ in range(8):
        plan, _ = run_step(scheduler, cache)
        order.extend(c.request_id for c in plan.scheduled if c.start == 0)
    assert order == ["urgent", "first", "second", "late-low"]
    # without the option the queue is first come, first served
    scheduler, cache = make(num_pages=40, max_num_batched_tokens=6, max_num_partial_prefills=1)
    for name, priority in (("a", 5), ("b", 0)):
        scheduler.add_request(EngineRequest(name, tuple(range(1, 7)), max_new_tokens=1, priority=priority))
    plan, _ = run_step(scheduler, cache)
    assert plan.scheduled[0].request_id == "a"


def test_preempted_request_keeps_its_place_under_priority_scheduling():
    scheduler, cache = make(num_pages=6, page_size=4, max_num_batched_tokens=64, priority_scheduling=True)  # 5 pages
    scheduler.add_request(EngineRequest("old", tuple(range(1, 8)), max_new_tokens=8, priority=1))
    scheduler.add_request(EngineRequest("young", tuple(range(51, 60)), max_new_tokens=8, priority=1))
    scheduler.add_request(EngineRequest("later-but-urgent", tuple(range(1, 4)), max_new_tokens=1, priority=0))
    preempted = []
    for _ in range(60):
        if not scheduler.has_unfinished():
            break
        plan, _ = run_step(scheduler, cache)
        preempted.extend(plan.preempted)
    assert not scheduler.has_unfinished() and preempted
    assert [len(scheduler.output_tokens(name)) for name in ("old", "young", "later-but-urgent")] == [8, 8, 1]


def test_a_prompt_stays_one_token_short_while_finishing_it_could_strand_running_decodes():
    """kairyu/engine/core/scheduler.py:636-677.  Two requests decode and will need 4 pages each in
    the end; 9 pages exist.  A third prompt fits beside them now, but as a decoding request it
    could not be pushed out cheaply when they grow: it is fed up to its last token and waits
    there, is the one to be preempted when a decode needs its page, and finishes its prompt once
    a decoding request has ended."""
    scheduler, cache = make(num_pages=10, page_size=4, max_num_batched_tokens=64)  # 9 usable pages
    scheduler.add_request(request("a", 6, max_new=10))  # 16 tokens in the end: 4 pages
    scheduler.add_request(request("b", 6, max_new=10))
    plan, _ = run_step(scheduler, cache)
    assert [(c.request_id, c.num_tokens, c.samples) for c in plan.scheduled] == [("a", 6, True), ("b", 6, True)]
    scheduler.add_request(request("c", 7, max_new=6))  # 13 tokens in the end: 4 pages; 9 - 8 leave 1
    plan, _ = run_step(scheduler, cache)
    by_id = {c.request_id: c for c in plan.scheduled}
    assert (by_id["c"].num_tokens, by_id["c"].samples, by_id["c"].is_prefill) == (6, False, True)
    assert scheduler.state("c").remaining == 1 and not scheduler.state("c").decoding
    waited = 0
    preempted = []
    finished_at = {}
    for step in range(60):
        if not scheduler.has_unfinished():
            break
        plan, finished = run_step(scheduler, cache)
        preempted.extend(plan.preempted)
        for name in finished:
            finished_at[name] = step
        if "c" in scheduler.running_ids() and not scheduler.state("c").decoding and not any(c.request_id == "c" for c in plan.scheduled):
            waited += 1
    assert waited > 0
    assert set(preempted) <= {"c"}  # a and b never lose their outputs
    assert scheduler.state("a").preemptions == 0 and scheduler.state("b").preemptions == 0
    assert [len(scheduler.output_tokens(name)) for name in "abc"] == [10, 10, 6]
    assert finished_at["c"] > min(finished_at["a"], finished_at["b"])
    assert cache.live_requests == 0


def test_a_prompt_may_finish_when_nothing_decodes_or_it_wants_one_token():
    scheduler, cache = make(num_pages=5, page_size=4, max_num_batched_tokens=64)  # 4 usable pages
    scheduler.add_request(request("a", 6, max_new=30))  # could never reach its limit; the first to decode goes on anyway
    plan, _ = run_step(scheduler, cache)
    assert plan.scheduled[0].samples
    scheduler.add_request(request("one", 5, max_new=1))  # produces a single token: nothing to protect it from
    plan, _ = run_step(scheduler, cache)
    assert {c.request_id: c.samples for c in plan.scheduled} == {"a": True, "one": True}


def test_a_windowed_group_admits_a_prompt_longer_than_its_pool():
    """A group that keeps a window of keys needs the window and one portion, not the whole prompt:
    a prompt of more tokens than the pool has room for is admitted and runs through."""
    layout = CacheLayout.from_slot_specs({0: (PagedKVSpec(1, 16, 8),)})  # window of 8 tokens
    cache = CacheManager(layout, num_pages=9, page_size=4, max_requests=4)  # 8 usable pages: 32 tokens
    scheduler = Scheduler(cache, max_num_batched_tokens=8)
    scheduler.add_request(request("long", 70, max_new=5))
    steps = 0
    while scheduler.has_unfinished() and steps < 100:
        plan, _ = run_step(scheduler, cache)
        assert plan.scheduled and not plan.rejected
        steps += 1
    assert scheduler.finish_reason("long") == "length" and len(scheduler.output_tokens("long")) == 5
    # with portions larger than the pool can hold beside the window, the prompt is refused at the door
    scheduler = Scheduler(cache, max_num_batched_tokens=64)
    scheduler.add_request(request("hopeless", 70, max_new=5))
    plan, _ = run_step(scheduler, cache)
    assert plan.rejected == ("hopeless",)
