"""Prefix sharing: the tree of whole pages, the cache manager with it on, the
scheduler's admissions over it, and the engine's outputs with and without it."""

import random

import pytest

import torch_kernels
from test_engine_gpu import engine_weights, plain_generate, prompts_of
from tiny_configs import TINY

from kairyu_b200 import LLM, SamplingParams, TokensPrompt
from kairyu_b200.cache import CacheLayout, CacheManager
from kairyu_b200.cache.prefix import PrefixIndex
from kairyu_b200.engine.scheduler import EngineRequest, Scheduler
from kairyu_b200.parts.base import PagedKVSpec, StateSpec


# ---------------------------------------------------------------------- the tree
def test_tree_matches_whole_pages_and_takes_back_oldest_unread_leaf_first():
    tree = PrefixIndex(page_size=2)
    a = tree.insert(None, (1, 2), (10,), readers=0)
    b = tree.insert(a, (3, 4), (11,), readers=0)
    c = tree.insert(a, (5, 6), (12,), readers=0)
    assert [n.pages for n in tree.match([1, 2, 3, 4, 9])] == [(10,), (11,)]
    assert [n.pages for n in tree.match([1, 2, 3, 4, 9], max_pages=1)] == [(10,)]
    assert tree.match([1, 3, 3, 4]) == [] and tree.match([1]) == []
    assert tree.num_unread == 3
    tree.check()
    # a reader protects its whole path; the other leaf goes first, then nothing more
    path = tree.match([1, 2, 3, 4])
    tree.acquire(path)
    assert tree.num_unread == 1
    assert tree.evict(5) == [(12,)] and not c.alive
    tree.check()
    tree.drop(path)
    assert tree.num_unread == 2
    # the leaf before the page it hangs from
    assert tree.evict(1) == [(11,)] and tree.evict(1) == [(10,)] and tree.evict(1) == []
    assert tree.num_nodes == 0 and not a.alive and not b.alive
    tree.check()


def test_tree_evicts_by_last_use_and_refuses_wrong_calls():
    tree = PrefixIndex(page_size=1)
    old = tree.insert(None, (1,), (5,), readers=0)
    new = tree.insert(None, (2,), (6,), readers=0)
    tree.acquire([old])
    tree.drop([old])  # read after `new` was inserted: now the younger of the two
    assert tree.evict(1) == [(6,)]
    with pytest.raises(ValueError, match="already in the tree"):
        tree.insert(None, (1,), (7,), readers=0)
    with pytest.raises(ValueError, match="holds 1 tokens"):
        tree.insert(None, (1, 2), (7,), readers=0)
    with pytest.raises(ValueError, match="more readers"):
        tree.insert(old, (3,), (7,), readers=1)
    with pytest.raises(ValueError, match="more often"):
        tree.drop([old])
    assert new.alive is False


def test_tree_heap_stays_small_under_many_reads():
    tree = PrefixIndex(page_size=1)
    node = tree.insert(None, (1,), (5,), readers=0)
    for _ in range(2000):
        tree.acquire([node])
        tree.drop([node])
    assert len(tree._heap) < 200
    tree.check()
    assert tree.evict(1) == [(5,)]


# ---------------------------------------------------------------------- the cache manager
def layout(groups=1):
    return CacheLayout.from_slot_specs({index: (PagedKVSpec(2, 16 * (index + 1)),) for index in range(groups)})


def fill(cache, name, tokens):
    """Admit, compute every token, as a request that runs to its end does."""
    record = cache.admit(name, tokens)
    assert cache.ensure_capacity(name, len(tokens))
    cache.advance(name, len(tokens))
    return record


def test_manager_shares_published_pages_and_leaves_the_last_token():
    cache = CacheManager(layout(2), num_pages=12, page_size=4, max_requests=4, prefix_sharing=True)
    tokens = list(range(100, 110))  # 2 whole pages and 2 tokens
    first = fill(cache, "a", tokens)
    assert first.num_cached_tokens == 0
    assert cache.publish("a", tokens) == 2 and cache.publish("a", tokens) == 0
    cache.check()
    shared = [cache.block_table("a", group)[:2] for group in range(2)]
    # same tokens: both whole pages; the tables start with the very same pages in every group
    second = cache.admit("b", tokens)
    assert second.num_tokens == second.num_cached_tokens == 8
    assert [cache.block_table("b", group) for group in range(2)] == shared
    # a prompt that ends on the page edge leaves its last page to compute
    third = cache.admit("c", tokens[:8])
    assert third.num_cached_tokens == 4
    # diverging in the second page
    fourth = cache.admit("d", tokens[:5] + [7, 7, 7, 7])
    assert fourth.num_cached_tokens == 4
    cache.check()
    assert cache.ensure_capacity("b", 10) and cache.block_table("b", 0)[2] not in cache.block_table("a", 0)
    free_before = cache.free_pages()
    for name in "abcd":
        cache.release(name)
    cache.check()
    # a's tail page and b's own page went back; the two published pages stay, unread
    assert cache.free_pages() == free_before + 2 and cache.prefix.num_unread == 2
    assert cache.available_pages() == cache.free_pages() + 2 == 11


def test_manager_takes_unread_pages_back_when_a_pool_is_short():
    cache = CacheManager(layout(), num_pages=7, page_size=2, max_requests=4, prefix_sharing=True)
    old, new = [1, 2, 3, 4, 5], [9, 8, 7, 6, 5]
    for name, tokens in (("old", old), ("new", new)):
        fill(cache, name, tokens)
        cache.publish(name, tokens)
        cache.release(name)
    assert cache.free_pages() == 2 and cache.prefix.num_unread == 4
    reader = cache.admit("reader", new)  # holds new's two pages
    assert reader.num_cached_tokens == 4
    cache.admit("big")
    assert cache.ensure_capacity("big", 8)  # 4 pages: the 2 free ones and old's 2
    cache.check()
    assert cache.prefix.num_nodes == 2 and cache.admit("again", old).num_cached_tokens == 0
    assert not cache.ensure_capacity("again", 2)  # nothing free, nothing unread
    cache.release("big")
    assert cache.ensure_capacity("again", 2)
    cache.check()


def test_manager_keeps_its_own_copy_where_the_tree_has_the_page_already():
    cache = CacheManager(layout(), num_pages=12, page_size=2, max_requests=4, prefix_sharing=True)
    tokens = [4, 5, 6, 7, 8]
    fill(cache, "a", tokens)
    fill(cache, "b", tokens)  # admitted before a published: computes its own pages
    assert cache.publish("a", tokens) == 2 and cache.publish("b", tokens) == 0
    cache.check()
    held = cache.pools[0].num_held
    cache.release("b")
    assert cache.pools[0].num_held == held - 3  # all of b's pages were its own
    cache.release("a")
    cache.check()
    assert cache.pools[0].num_held == 2


def test_manager_refuses_prefix_sharing_for_windows_and_state():
    windowed = CacheLayout.from_slot_specs({0: (PagedKVSpec(2, 16, window=8),)})
    with pytest.raises(ValueError, match="prefix sharing needs"):
        CacheManager(windowed, num_pages=8, page_size=4, max_requests=2, prefix_sharing=True)
    stateful = CacheLayout.from_slot_specs({0: (PagedKVSpec(2, 16), StateSpec((3,)))})
    with pytest.raises(ValueError, match="prefix sharing needs"):
        CacheManager(stateful, num_pages=8, page_size=4, max_requests=2, prefix_sharing=True)


@pytest.mark.parametrize("seed", range(8))
def test_manager_random_orders_with_sharing(seed):
    rng = random.Random(seed)
    page_size = rng.choice([1, 2, 4])
    cache = CacheManager(layout(rng.choice([1, 2])), num_pages=24, page_size=page_size, max_requests=5, prefix_sharing=True)
    live: dict[str, tuple[list[int], int]] = {}
    counter = 0
    for _ in range(800):
        action = rng.random()
        if action < 0.25 and len(live) < 5:
            name = f"r{counter}"
            counter += 1
            tokens = [rng.randrange(2) for _ in range(rng.randrange(1, 30))]  # two token values: prefixes collide
            record = cache.admit(name, tokens)
            assert record.num_tokens % page_size == 0 and record.num_tokens < len(tokens)
            live[name] = (tokens, record.num_tokens)
        elif action < 0.7 and live:
            name = rng.choice(sorted(live))
            tokens, done = live[name]
            grow = min(rng.choice([1, 1, 2, 5, 17]), len(tokens) - done)
            if grow and cache.ensure_capacity(name, done + grow, query_start=done):
                cache.advance(name, done + grow)
                live[name] = (tokens, done + grow)
        elif action < 0.85 and live:
            name = rng.choice(sorted(live))
            cache.publish(name, live[name][0])
        elif live:
            name = rng.choice(sorted(live))
            cache.release(name)
            del live[name]
        cache.check()
        # what the tree holds for a live request is what that request's tokens say
        for name, (tokens, done) in live.items():
            record = cache.get(name)
            node_keys = [key for node in record.shared for key in node.key]
            assert node_keys == tokens[: len(node_keys)] and len(node_keys) <= max(done, record.num_cached_tokens)
    for name in list(live):
        cache.release(name)
    cache.check()
    assert all(pool.num_held == cache.prefix.num_nodes == cache.prefix.num_unread for pool in cache.pools)


# ---------------------------------------------------------------------- the scheduler
def make_scheduler(num_pages=17, page_size=4, **kwargs):
    cache = CacheManager(layout(), num_pages=num_pages, page_size=page_size, max_requests=8, prefix_sharing=True)
    return Scheduler(cache, **kwargs), cache


def run_step(scheduler, cache, token=7):
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


def test_scheduler_publishes_after_the_first_token_and_later_requests_start_behind():
    scheduler, cache = make_scheduler(max_num_batched_tokens=64)
    prompt = tuple(range(1, 12))  # 11 tokens: 2 whole pages
    scheduler.add_request(EngineRequest("a", prompt, max_new_tokens=6))
    scheduler.add_request(EngineRequest("same-step", prompt, max_new_tokens=2))
    plan, _ = run_step(scheduler, cache)
    # admitted in one step: nothing was published yet, both compute everything
    assert [(c.request_id, c.start, c.num_tokens) for c in plan.scheduled] == [("a", 0, 11), ("same-step", 0, 11)]
    assert cache.prefix.num_nodes == 2  # a's prompt pages, published when its first token came
    scheduler.add_request(EngineRequest("b", prompt + (50, 51), max_new_tokens=2))
    plan, _ = run_step(scheduler, cache)
    chunk = [c for c in plan.scheduled if c.request_id == "b"][0]
    assert (chunk.start, chunk.num_tokens, chunk.samples) == (8, 5, True)
    assert scheduler.state("b").num_cached_tokens == 8 and scheduler.state("a").num_cached_tokens == 0
    assert cache.block_table("b", 0)[:2] == cache.block_table("a", 0)[:2]
    while scheduler.has_unfinished():
        run_step(scheduler, cache)
    assert cache.live_requests == 0
    # a's finish published its generated page too: prompt(11) + 5 fed outputs = 16 tokens = 4 pages
    again = prompt + (7, 7, 7, 7, 7, 7)
    scheduler.add_request(EngineRequest("c", again, max_new_tokens=1))
    plan, _ = run_step(scheduler, cache)
    assert (plan.scheduled[0].start, plan.scheduled[0].num_tokens) == (16, 1)
    assert scheduler.prefix_hit_rate == pytest.approx((8 + 16) / (11 + 11 + 13 + 17))


def test_scheduler_counts_unread_pages_as_room_and_preemption_publishes_nothing():
    scheduler, cache = make_scheduler(num_pages=7, page_size=4, max_num_batched_tokens=64)  # 6 pages
    scheduler.add_request(EngineRequest("a", tuple(range(1, 18)), max_new_tokens=1))  # 17 tokens: 5 pages
    run_step(scheduler, cache)
    assert cache.free_pages() == 2 and cache.prefix.num_unread == 4
    # 5 pages are needed, 2 are free: the four unread ones make room
    scheduler.add_request(EngineRequest("b", tuple(range(101, 118)), max_new_tokens=3))
    plan, _ = run_step(scheduler, cache)
    assert plan.scheduled and plan.scheduled[0].num_tokens == 17 and cache.prefix.counters["evicted_pages"] == 3
    # b has published its 4 prompt pages and holds them; c cannot be admitted beside it and waits
    scheduler.add_request(EngineRequest("c", tuple(range(201, 214)), max_new_tokens=1))
    plan, _ = run_step(scheduler, cache)
    assert [c.request_id for c in plan.scheduled] == ["b"] and scheduler.num_waiting == 1
    while scheduler.has_unfinished():
        run_step(scheduler, cache)
    assert scheduler.finish_reason("c") == "length" and len(scheduler.output_tokens("c")) == 1


def test_scheduler_preempted_request_finds_its_published_prompt_again():
    scheduler, cache = make_scheduler(num_pages=6, page_size=4, max_num_batched_tokens=64)  # 5 pages
    scheduler.add_request(EngineRequest("old", tuple(range(1, 8)), max_new_tokens=8))   # 7 tokens
    scheduler.add_request(EngineRequest("young", tuple(range(51, 60)), max_new_tokens=8))  # 9 tokens
    preempted = []
    for _ in range(40):
        if not scheduler.has_unfinished():
            break
        plan, _ = run_step(scheduler, cache)
        preempted.extend(plan.preempted)
    assert not scheduler.has_unfinished() and preempted
    assert len(scheduler.output_tokens("old")) == 8 and len(scheduler.output_tokens("young")) == 8
    cache.check()
    assert cache.live_requests == 0


@pytest.mark.parametrize("seed", range(6))
def test_scheduler_random_workloads_with_sharing_finish_and_keep_the_invariants(seed):
    rng = random.Random(seed)
    scheduler, cache = make_scheduler(
        num_pages=rng.choice([10, 16, 40]), page_size=rng.choice([2, 4]), max_num_batched_tokens=rng.choice([5, 16, 64])
    )
    stems = [tuple(rng.randrange(3) for _ in range(rng.randrange(4, 14))) for _ in range(3)]
    for index in range(14):
        prompt = rng.choice(stems) + tuple(rng.randrange(3) for _ in range(rng.randrange(0, 6)))
        scheduler.add_request(EngineRequest(f"r{index}", prompt, max_new_tokens=rng.randrange(1, 7)))
    for _ in range(600):
        if not scheduler.has_unfinished():
            break
        run_step(scheduler, cache, token=rng.randrange(3))
    assert not scheduler.has_unfinished() and cache.live_requests == 0
    for index in range(14):
        state = scheduler.state(f"r{index}")
        assert state.finish_reason == "length"
        if cache.can_hold(len(state.request.prompt_token_ids) + state.request.max_new_tokens):
            assert len(state.outputs) == state.request.max_new_tokens  # else it ended when the cache was full
    assert scheduler.counters["cached_prompt_tokens"] > 0


# ---------------------------------------------------------------------- the engine
@pytest.fixture
def cpu_kernels(monkeypatch):
    torch_kernels.install(monkeypatch)


def test_engine_outputs_do_not_change_with_prefix_caching(cpu_kernels):
    config, seed, page_size = TINY["llama"]
    llm = LLM.from_random(
        config, seed=seed, dtype="float32", device="cpu", page_size=page_size, num_pages=40,
        enable_prefix_caching=True, max_num_batched_tokens=48,
    )
    weights = engine_weights(llm)
    stem = prompts_of(config, [37], seed=300)[0]
    tails = prompts_of(config, [1, 9, 20], seed=301)
    prompts = [stem + tail for tail in tails]
    params = SamplingParams(temperature=0.0, max_tokens=10)
    first = llm.generate(TokensPrompt(tuple(prompts[0])), params)[0]
    assert first.metrics["num_cached_tokens"] == 0
    outputs = llm.generate([TokensPrompt(tuple(p)) for p in prompts], params)
    whole_pages = len(stem) // page_size * page_size
    assert outputs[0].metrics["num_cached_tokens"] == (len(prompts[0]) + 9) // page_size * page_size
    assert [o.metrics["num_cached_tokens"] for o in outputs[1:]] == [whole_pages, whole_pages]
    for prompt, output in zip(prompts, outputs):
        assert list(output.outputs[0].token_ids) == plain_generate(config, weights, prompt, 10)
    assert list(first.outputs[0].token_ids) == list(outputs[0].outputs[0].token_ids)
    llm.engine.cache.check()
    assert llm.engine.cache.live_requests == 0 and llm.engine.scheduler.prefix_hit_rate > 0.4


def test_engine_with_prefix_caching_few_pages_and_depth_two(cpu_kernels):
    config, seed, page_size = TINY["odd"]
    llm = LLM.from_random(
        config, seed=seed, dtype="float32", device="cpu", page_size=page_size, num_pages=12,
        enable_prefix_caching=True, max_num_batched_tokens=9, max_num_seqs=3, pipeline_depth=2,
    )
    weights = engine_weights(llm)
    stem = prompts_of(config, [19], seed=310)[0]
    prompts = [stem + tail for tail in prompts_of(config, [2, 11, 5, 8, 3, 14], seed=311)]
    params = SamplingParams(temperature=0.0, max_tokens=12)
    for round_ in range(2):
        outputs = llm.generate([TokensPrompt(tuple(p)) for p in prompts], params)
        for prompt, output in zip(prompts, outputs):
            assert list(output.outputs[0].token_ids) == plain_generate(config, weights, prompt, 12)
        llm.engine.cache.check()
        assert llm.engine.cache.live_requests == 0
    assert llm.engine.cache.prefix.counters["evicted_pages"] > 0
    assert llm.engine.scheduler.counters["cached_prompt_tokens"] > 0


@pytest.mark.parametrize("seed", [3, 11, 29, 57])
def test_everything_on_equals_everything_off_on_random_workloads(cpu_kernels, seed):
    """Schedule-ahead, prefix caching and log-probability reports together, on prompts that share
    stems, over pools so small that requests wait, are preempted and unread pages are taken back:
    tokens, finish reasons and stop reasons are those of the plain configuration, twice in a row."""
    rng = random.Random(seed)
    name = rng.choice(["llama", "qwen3", "odd"])
    config, model_seed, page_size = TINY[name]
    count = rng.randint(3, 8)
    stems = [prompts_of(config, [rng.randint(1, 40)], seed=1000 + seed * 7 + i)[0] for i in range(2)]
    prompts = [rng.choice(stems) + prompts_of(config, [rng.randint(0, 25)], seed=2000 + seed * 11 + i)[0] for i in range(count)]
    limits = [rng.randint(1, 14) for _ in range(count)]
    options = dict(
        num_pages=rng.randint(10, 20), max_num_batched_tokens=rng.choice([5, 16, 64]), max_num_seqs=rng.choice([2, 4, 8]), page_size=page_size
    )
    results = {}
    stops = None
    for variant in ("off", "on"):
        extra = dict(pipeline_depth=1) if variant == "off" else dict(pipeline_depth=2, enable_prefix_caching=True)
        llm = LLM.from_random(config, seed=model_seed, dtype="float32", device="cpu", **options, **extra)
        if stops is None:  # tokens the free run produces, so that some requests stop early
            free = llm.generate([TokensPrompt(tuple(p)) for p in prompts], [SamplingParams(temperature=0.0, max_tokens=m) for m in limits])
            stops = [o.outputs[0].token_ids[len(o.outputs[0].token_ids) // 2] if i % 2 == 0 else None for i, o in enumerate(free)]
        params = [
            SamplingParams(
                temperature=0.0 if i % 3 else 0.7, seed=5 + i, max_tokens=limits[i], stop_token_ids=[stops[i]] if stops[i] is not None else [],
                logprobs=(i % 4 if variant == "on" and i % 2 else None),
            )
            for i in range(count)
        ]
        for round_ in range(2):  # the second round finds its prompts in the prefix tree
            outputs = llm.generate([TokensPrompt(tuple(p)) for p in prompts], params)
            results[(variant, round_)] = [(o.outputs[0].token_ids, o.outputs[0].finish_reason, o.outputs[0].stop_reason) for o in outputs]
            for output, asked in zip(outputs, params):
                completion = output.outputs[0]
                if asked.logprobs is None:
                    assert completion.logprobs is None
                else:
                    assert len(completion.logprobs) == len(completion.token_ids)
                    assert all(list(entry)[0] == token for entry, token in zip(completion.logprobs, completion.token_ids))
            llm.engine.cache.check()
            assert llm.engine.cache.live_requests == 0 and not llm.engine._pending and not llm.engine._logprobs
    assert all(value == results[("off", 0)] for value in results.values())
