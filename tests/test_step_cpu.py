"""The step function, cache and replay cuts on the CPU, with the kernels replaced
by their plain torch statements (tests/torch_kernels.py).  This checks the host
side: metadata packing, block tables, page reuse, wanted rows.  The kernels
themselves are checked on the GPU."""

import numpy as np
import pytest

import plain_model
import torch_kernels
import traces
from golden_inputs import golden_weights
from tiny_configs import TINY

from kairyu_b200.cache import CacheLayout, CacheManager, CacheStorage
from kairyu_b200.engine.engine import build_model
from kairyu_b200.engine.runner import ModelRunner, StepEntry, StepError


def make_runner(name, *, num_pages, page_size=None, dtype="float32", max_requests=8):
    config, seed, default_page = TINY[name]
    page_size = page_size or default_page
    model, _ = build_model(config, dtype=dtype, device="cpu")
    weights = golden_weights(config, seed)
    tensors = {spec.name: weights[spec.alias_of or spec.name if spec.name not in weights else spec.name] for spec in model.tensor_specs()}
    model.load({k: v.to(model.dtype) for k, v in tensors.items()})
    layout = CacheLayout.from_slot_specs(model.cache_slot_specs())
    cache = CacheManager(layout, num_pages=num_pages, page_size=page_size, max_requests=max_requests)
    storage = CacheStorage(layout, num_pages=num_pages, page_size=page_size, max_requests=max_requests, dtype=model.dtype, device="cpu")
    runner = ModelRunner(model, cache, storage, max_model_len=config["max_position_embeddings"], decode_mode="eager", check_tables=True, debug_poison=True)
    return runner, config, weights


def plain_logits(config, weights, requests):
    return {name: plain_model.forward_logits(config, weights, tokens).numpy() for name, tokens in requests.items()}


def assert_matches(result, expected, tolerance):
    worst = 0.0
    for (name, position), row in result.items():
        worst = max(worst, float(np.abs(row - expected[name][position]).max()))
    assert worst < tolerance, f"max abs difference {worst}"
    return worst


@pytest.fixture(autouse=True)
def cpu_kernels(monkeypatch):
    torch_kernels.install(monkeypatch)


@pytest.mark.parametrize("name", ["llama", "qwen3", "odd", "wide", "yarn"])
def test_whole_prompts_match_plain(name):
    runner, config, weights = make_runner(name, num_pages=40)
    requests = traces.make_requests(config["vocab_size"], [1, 7, 33, 50], seed=11)
    result = traces.run_in_process(runner, traces.trace_whole(requests))
    assert len(result) == sum(len(t) for t in requests.values())
    assert_matches(result, plain_logits(config, weights, requests), 2e-5)
    assert runner.cache.live_requests == 0


@pytest.mark.parametrize("name", ["llama", "qwen3"])
def test_every_cut_gives_the_same_logits(name):
    runner, config, weights = make_runner(name, num_pages=40)
    requests = traces.make_requests(config["vocab_size"], [70, 45, 101, 38, 64, 83], seed=5)
    expected = plain_logits(config, weights, requests)
    for steps in (traces.trace_decode_tail(requests), traces.trace_chunks(requests)):
        assert_matches(traces.run_in_process(runner, steps), expected, 2e-5)
    mixed = traces.trace_mixed(requests, seed=3)
    assert max(len(step["entries"]) for step in mixed) > 1
    assert_matches(traces.run_in_process(runner, mixed), expected, 2e-5)


def test_mixed_trace_reuses_pages_of_a_small_pool():
    config, _, page_size = TINY["qwen3"]
    requests = traces.make_requests(config["vocab_size"], [70, 45, 101, 38, 64, 83, 90, 55], seed=9)
    steps = traces.trace_mixed(requests, seed=1)
    pool_tokens = traces.peak_tokens(steps)
    total = sum(len(t) for t in requests.values())
    assert pool_tokens < total  # pages have to be used again
    runner, config, weights = make_runner("qwen3", num_pages=pool_tokens // page_size + 1)
    result = traces.run_in_process(runner, steps)
    assert_matches(result, plain_logits(config, weights, requests), 2e-5)


def test_stale_pages_do_not_leak_into_a_new_request():
    """Poison every page that is given back: a step that read stale keys would return NaN."""
    runner, config, weights = make_runner("llama", num_pages=12)
    requests = traces.make_requests(config["vocab_size"], [60, 50, 70, 40], seed=2)
    expected = plain_logits(config, weights, requests)
    for name, tokens in requests.items():
        logits = runner.step([StepEntry(name, tokens, tuple(range(len(tokens))))])
        assert np.abs(logits.numpy() - expected[name]).max() < 2e-5
        pages = [p for p in runner.cache.block_table(name, 0) if p >= 0]
        runner.cache.release(name)
        runner.storage.poison_pages(0, pages)


def test_wanted_rows_only():
    runner, config, weights = make_runner("llama", num_pages=20)
    tokens = traces.make_requests(config["vocab_size"], [30], seed=4)["r0"]
    expected = plain_model.forward_logits(config, weights, tokens).numpy()
    assert runner.step([StepEntry("a", tokens[:10], ())]) is None
    logits = runner.step([StepEntry("a", tokens[10:30], (0, 19, 7))])
    assert logits.shape == (3, config["vocab_size"])
    for row, position in enumerate((10, 29, 17)):
        assert np.abs(logits[row].numpy() - expected[position]).max() < 2e-5


def test_step_rejects_bad_entries():
    runner, config, _ = make_runner("llama", num_pages=20)
    with pytest.raises(StepError):
        runner.step([])
    with pytest.raises(StepError):
        runner.step([StepEntry("a", [], ())])
    with pytest.raises(StepError):
        runner.step([StepEntry("a", [config["vocab_size"]], ())])
    with pytest.raises(StepError):
        runner.step([StepEntry("a", [1, 2], (2,))])
    with pytest.raises(StepError):
        runner.step([StepEntry("a", [1], ()), StepEntry("a", [2], ())])
    with pytest.raises(StepError):
        runner.step([StepEntry("a", [1] * (config["max_position_embeddings"] + 1), ())])


def test_step_runs_out_of_pages_loudly():
    from kairyu_b200.cache import OutOfPages

    runner, config, _ = make_runner("llama", num_pages=3)  # two usable pages of 16
    runner.step([StepEntry("a", [1] * 32, ())])
    with pytest.raises(OutOfPages):
        runner.step([StepEntry("a", [1], ())])


def test_table_check_catches_a_page_named_twice(monkeypatch):
    """With check_tables the step function refuses a step whose block tables share a page (the cache
    manager never makes one; the check is the host-side guard the reference has, prefill.py:105-178)."""
    torch_kernels.install(monkeypatch)
    runner, _, _ = make_runner("llama", num_pages=12, page_size=8)
    runner.step([StepEntry("a", list(range(10)), ()), StepEntry("b", list(range(5)), ())])
    runner.cache.get("b").tables[0][0] = runner.cache.get("a").tables[0][1]  # corrupt: b now names a page of a
    with pytest.raises(StepError, match="is named by"):
        runner.step([StepEntry("a", [1], (0,)), StepEntry("b", [2], (0,))])


def test_descriptor_table_never_frees_what_a_call_may_still_point_at(monkeypatch):
    """A kernel call takes the host addresses of up to three encoded descriptors before it launches.
    When the table of descriptors is full it is set aside, not cleared: the last `limit` descriptors
    handed out stay referenced, whatever the order of insertions and repeated uses."""
    import ctypes
    import random
    import weakref

    import kairyu_b200.kernels as kernels

    class Buffer:  # stands for a ctypes buffer; weakly referencable
        pass

    monkeypatch.setattr(kernels, "_TENSOR_MAP_LIMIT", 4)
    monkeypatch.setattr(kernels, "_tensor_maps", {})
    monkeypatch.setattr(kernels, "_tensor_maps_before", {})
    rng = random.Random(0)
    recent: list = []  # weak references to the last three descriptors handed out
    for step in range(500):
        key = ("k", rng.randrange(12))
        held = kernels._held_map(key)
        if held is None:
            held = Buffer()
            kernels._keep_map(key, held)
        recent.append(weakref.ref(held))
        del held
        recent = recent[-3:]
        assert all(ref() is not None for ref in recent), step
    assert len(kernels._tensor_maps) <= 4 and len(kernels._tensor_maps_before) <= 4
    del ctypes


def _padding_graph(runner, bucket):
    """The host side of a captured decode graph (mirror, layout, row state) without a device."""
    from kairyu_b200.engine.runner import _Graph

    host, layout, _ = runner._pack((), pad_rows=bucket, max_pages=runner.max_pages_per_request, include_want=False)
    held = _Graph(None, None, None, 0, layout)
    held.mirror = host.numpy().copy()
    held.row_state = [None] * bucket
    return held


def _mirror_table(runner, held, bucket, row, group=0):
    width = runner.max_pages_per_request
    base = held.layout["tables"][0] + (group * bucket + row) * width
    return list(held.mirror[base : base + width])


def _decode_rows(runner, names):
    rows = []
    for name in names:
        start = runner.cache.get(name).num_tokens
        assert runner.cache.ensure_capacity(name, start + 1, query_start=start)
        rows.append((StepEntry(name, [1], (0,)), start, start + 1))
    return rows


def test_graph_mirror_follows_a_request_that_was_released_and_admitted_again():
    """A request that comes back under the same id (after a preemption, or an id used again) holds
    other pages; the row of the graph's metadata it lands on must show the new table, not the old
    pages topped up."""
    runner, _, _ = make_runner("llama", num_pages=12, page_size=4)
    cache = runner.cache
    bucket = 2
    held = _padding_graph(runner, bucket)
    assert _mirror_table(runner, held, bucket, 0) == [0] * runner.max_pages_per_request

    def fill(name, tokens):
        cache.admit(name)
        assert cache.ensure_capacity(name, tokens, query_start=0)
        cache.advance(name, tokens)

    fill("a", 9)
    fill("b", 5)
    rows = _decode_rows(runner, ["a", "b"])
    runner._update_mirror(held, rows, bucket)
    for row, name in enumerate(["a", "b"]):
        table = cache.block_table(name, 0)
        assert _mirror_table(runner, held, bucket, row)[: len(table)] == table
    first_pages = list(cache.block_table("a", 0))
    cache.release("a")
    fill("c", 7)  # takes some of a's pages
    fill("a", 10)  # same id, other pages, same number of them
    assert cache.block_table("a", 0) != first_pages
    rows = _decode_rows(runner, ["a", "b"])
    runner._update_mirror(held, rows, bucket)
    table = cache.block_table("a", 0)
    mirrored = _mirror_table(runner, held, bucket, 0)
    assert mirrored[: len(table)] == table and set(mirrored[len(table) :]) == {-1}
    # the same admission growing by a page is topped up in place
    cache.advance("a", 12)
    rows = _decode_rows(runner, ["a", "b"])
    runner._update_mirror(held, rows, bucket)
    table = cache.block_table("a", 0)
    assert len(table) == 4 and _mirror_table(runner, held, bucket, 0)[:4] == table
    # a row that empties becomes padding again: the reserved page and the scratch state slot
    runner._update_mirror(held, _decode_rows(runner, ["b"]), bucket)
    assert _mirror_table(runner, held, bucket, 1) == [0] * runner.max_pages_per_request
    assert held.mirror[held.layout["state_slots"][0] + 1] == cache.scratch_state_slot
