"""Long prompts cut at random, in bfloat16, on a small model whose attention has the head size
(128) and head count (16 query heads on 4 KV heads) that send its prompt portions through every
way the tcgen05 prefill attention spreads its query tiles: one tile a block, a long and a short
tile a block, two tiles side by side over 128-key tiles, and a tile's keys shared among blocks.

Each seed draws a few requests of up to 6,000 tokens and cuts them into portions drawn from
sizes between 2 tokens and the whole prompt, with decoded tokens of other requests beside them
and a pool so small that pages are used again.  Logits at chosen positions are compared with the
plain model (kairyu tests/unit/test_model_parity.py:78-114 compares whole against chunked the
same way); the bound is what rounding every operation to bfloat16 costs the plain model itself.
"""

import random

import pytest
import torch

import parity
import traces

pytestmark = pytest.mark.gpu

PAGE = 16
CONFIG = {
    "architectures": ["Qwen3ForCausalLM"], "hidden_size": 256, "num_hidden_layers": 2, "num_attention_heads": 16,
    "num_key_value_heads": 4, "head_dim": 128, "intermediate_size": 384, "vocab_size": 512, "rope_theta": 1000000.0,
    "max_position_embeddings": 8192, "rms_norm_eps": 1e-6, "tie_word_embeddings": False, "hidden_act": "silu",
}
SEED = 9
SIZES = (2, 17, 64, 128, 129, 300, 512, 1024, 2048, 10_000)
BF16_FACTOR = 1.25


def random_cut(requests, rng):
    """Steps in which one request brings a portion of random size while up to three others, whose
    prompts are done but for their last eight tokens, bring one token each."""
    steps = []
    decoding: dict[str, int] = {}
    for name, tokens in requests.items():
        head = len(tokens) - 8
        start = 0
        while start < head:
            size = min(rng.choice(SIZES), head - start)
            entries = [{"id": name, "tokens": tokens[start : start + size], "want": list(range(size))}]
            ended = []
            for other in list(decoding):
                if rng.random() < 0.6:
                    place = decoding[other]
                    entries.append({"id": other, "tokens": [requests[other][place]], "want": [0]})
                    decoding[other] = place + 1
                    if place + 1 == len(requests[other]):
                        ended.append(other)
                        del decoding[other]
            steps.append({"step": len(steps), "entries": entries, "end": ended})
            start += size
        decoding[name] = head
        if len(decoding) > 3:  # finish the oldest before the next prompt starts
            oldest = next(iter(decoding))
            while oldest in decoding:
                place = decoding[oldest]
                last = place + 1 == len(requests[oldest])
                steps.append({"step": len(steps), "entries": [{"id": oldest, "tokens": [requests[oldest][place]], "want": [0]}], "end": [oldest] if last else []})
                decoding[oldest] = place + 1
                if last:
                    del decoding[oldest]
    while decoding:
        entries, ended = [], []
        for other in list(decoding):
            place = decoding[other]
            entries.append({"id": other, "tokens": [requests[other][place]], "want": [0]})
            decoding[other] = place + 1
            if place + 1 == len(requests[other]):
                ended.append(other)
                del decoding[other]
        steps.append({"step": len(steps), "entries": entries, "end": ended})
    return steps


@pytest.fixture(scope="module")
def model():
    from golden_inputs import golden_weights_on
    from kairyu_b200.engine.engine import random_model

    torch.backends.cuda.matmul.allow_tf32 = False
    torch.set_float32_matmul_precision("highest")
    weights = golden_weights_on(CONFIG, SEED, "cuda")
    held = {k: v.float() for k, v in parity.in_bf16(weights, False).items()}
    built, _ = random_model(CONFIG, SEED, dtype="bfloat16", device="cuda")
    return {"weights": weights, "held": held, "model": built}


def make_runner(built, num_pages):
    from kairyu_b200.cache import CacheLayout, CacheManager, CacheStorage
    from kairyu_b200.engine.runner import ModelRunner

    layout = CacheLayout.from_slot_specs(built.cache_slot_specs())
    cache = CacheManager(layout, num_pages=num_pages, page_size=PAGE, max_requests=8)
    storage = CacheStorage(layout, num_pages=num_pages, page_size=PAGE, max_requests=8, dtype=built.dtype, device="cuda")
    return ModelRunner(built, cache, storage, max_model_len=8192, decode_mode="cuda_graph", max_graph_batch=8, check_tables=True, debug_poison=True)


@pytest.mark.parametrize("seed", range(5))
def test_long_prompts_cut_at_random(model, seed):
    rng = random.Random(seed)
    lengths = [rng.choice((rng.randint(2000, 6000), rng.randint(300, 1500), rng.randint(20, 200))) for _ in range(rng.randint(3, 5))]
    lengths[0] = rng.randint(4200, 6000)  # one that is long enough for every kernel
    requests = traces.make_requests(CONFIG["vocab_size"], lengths, seed=500 + seed)
    keep = {name: parity.keep_positions(len(tokens), spread=12, tail=10) for name, tokens in requests.items()}
    truth = parity.plain_rows(CONFIG, model["held"], requests, keep)
    rounded = parity.plain_rows(CONFIG, parity.in_bf16(model["weights"], False), requests, keep)
    bound = BF16_FACTOR * parity.worst_error(rounded, truth)
    steps = random_cut(requests, rng)
    pool = traces.peak_tokens(steps) // PAGE + 2
    runner = make_runner(model["model"], pool)
    result = traces.run_in_process(runner, parity.thin_wants(steps, keep))
    runner.check_errors()
    assert result.keys() == truth.keys()
    error = parity.worst_error(result, truth)
    print(f"[parity] long prompts, seed {seed}, lengths {lengths}, {len(steps)} steps: worst error {error:.3e}, bound {bound:.3e}")
    assert error < bound, (error, bound, parity.rows_beyond(result, truth, bound))
    whole = traces.run_in_process(make_runner(model["model"], sum(lengths) // PAGE + 8), parity.thin_wants(traces.trace_whole(requests), keep))
    assert parity.worst_error(whole, truth) < bound


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_steps_of_portions_are_captured_and_replayed(dtype):
    """The same shapes of step come again and again (portions of 48 and 100 tokens, with and without
    decoded tokens beside them): the third time a shape comes it is captured, from then on replayed.  Every
    logits row equals, bit for bit, what a runner that launches every step kernel by kernel gives
    in 32-bit (the kernels are the same, and a captured step's filler row touches no request), and
    stays within the bfloat16 bound of the plain model."""
    from golden_inputs import golden_weights_on
    from kairyu_b200.cache import CacheLayout, CacheManager, CacheStorage
    from kairyu_b200.engine.engine import random_model
    from kairyu_b200.engine.runner import ModelRunner

    built, _ = random_model(CONFIG, SEED, dtype=dtype, device="cuda")
    weights = golden_weights_on(CONFIG, SEED, "cuda")
    requests = traces.make_requests(CONFIG["vocab_size"], [400, 333, 290, 410, 377, 305], seed=900)
    steps = []
    names = list(requests)
    live: dict[str, int] = {}
    for index, name in enumerate(names):
        tokens = requests[name]
        start = 0
        while start < len(tokens) - 4:
            size = min(48 if (start // 48) % 2 == 0 else 100, len(tokens) - 4 - start)
            entries = [{"id": name, "tokens": tokens[start : start + size], "want": [size - 1]}]
            ended = []
            for other, place in list(live.items()):
                entries.append({"id": other, "tokens": [requests[other][place]], "want": [0]})
                live[other] = place + 1
                if place + 1 == len(requests[other]):
                    ended.append(other)
                    del live[other]
            steps.append({"step": len(steps), "entries": entries, "end": ended})
            start += size
        live[name] = len(tokens) - 4
    while live:
        entries, ended = [], []
        for other, place in list(live.items()):
            entries.append({"id": other, "tokens": [requests[other][place]], "want": [0]})
            live[other] = place + 1
            if place + 1 == len(requests[other]):
                ended.append(other)
                del live[other]
        steps.append({"step": len(steps), "entries": entries, "end": ended})

    def runner_with(portion_graphs):
        layout = CacheLayout.from_slot_specs(built.cache_slot_specs())
        cache = CacheManager(layout, num_pages=160, page_size=PAGE, max_requests=8)
        storage = CacheStorage(layout, num_pages=160, page_size=PAGE, max_requests=8, dtype=built.dtype, device="cuda")
        return ModelRunner(built, cache, storage, max_model_len=1024, decode_mode="cuda_graph", max_graph_batch=8,
                           check_tables=True, debug_poison=True, portion_graphs=portion_graphs)

    captured = runner_with(True)
    assert captured.portion_graphs
    result = traces.run_in_process(captured, steps)
    captured.check_errors()
    assert captured.counters["portion_graph_captures"] >= 2 and captured.counters["portion_graph_replays"] >= 4
    plain_runner = runner_with(False)
    assert not plain_runner.portion_graphs
    launched = traces.run_in_process(plain_runner, steps)
    assert plain_runner.counters["portion_graph_captures"] == 0
    if dtype == "float32":
        parity.assert_same_bits(result, launched, "captured against launched")
    held = {k: v.float() for k, v in parity.in_bf16(weights, False).items()} if dtype == "bfloat16" else weights
    truth = parity.plain_rows(CONFIG, held, requests)
    truth = {key: row for key, row in truth.items() if key in result}
    bound = 2e-5 if dtype == "float32" else BF16_FACTOR * parity.worst_error(
        {k: v for k, v in parity.plain_rows(CONFIG, parity.in_bf16(weights, False), requests).items() if k in result}, truth)
    for rows in (result, launched):
        assert rows.keys() == truth.keys()
        assert parity.worst_error(rows, truth) < bound, (parity.worst_error(rows, truth), bound)
    # the same steps again on the runner that has its graphs: the same bits
    parity.assert_same_bits(result, traces.run_in_process(captured, steps), "a second pass over the captured steps")


def test_captured_shapes_are_bounded(monkeypatch):
    """More shapes of step than the runner keeps graphs for, taking turns: the first three stay (a kept
    shape gives way only after it has not come for a while, or shapes that take turns would evict one
    another for ever), the others are launched kernel by kernel; once the kept ones have gone unused for
    long enough, new shapes take their places.  Every step gives the bits of a runner that launches
    kernel by kernel (32-bit)."""
    import kairyu_b200.engine.runner as runner_module
    from kairyu_b200.cache import CacheLayout, CacheManager, CacheStorage
    from kairyu_b200.engine.engine import random_model
    from kairyu_b200.engine.runner import ModelRunner, StepEntry

    monkeypatch.setattr(runner_module, "MAX_PORTION_GRAPHS", 3)
    monkeypatch.setattr(runner_module, "PORTION_EVICT_AFTER", 12)
    built, _ = random_model(CONFIG, SEED, dtype="float32", device="cuda")

    def runner_with(portion_graphs):
        layout = CacheLayout.from_slot_specs(built.cache_slot_specs())
        cache = CacheManager(layout, num_pages=64, page_size=PAGE, max_requests=4)
        storage = CacheStorage(layout, num_pages=64, page_size=PAGE, max_requests=4, dtype=built.dtype, device="cuda")
        return ModelRunner(built, cache, storage, max_model_len=512, decode_mode="cuda_graph", max_graph_batch=4, portion_graphs=portion_graphs)

    captured, launched = runner_with(True), runner_with(False)
    generator = torch.Generator().manual_seed(4)

    def run(sizes, turns):
        for turn in range(turns):
            for size in sizes:
                tokens = torch.randint(0, CONFIG["vocab_size"], (size,), generator=generator).tolist()
                rows = []
                for runner in (captured, launched):
                    logits = runner.step([StepEntry("p", tokens, (size - 1,))])
                    rows.append(logits.clone())
                    runner.cache.release("p")
                assert torch.equal(rows[0], rows[1]), (turn, size)
                assert len(captured._portion_graphs) <= 3

    run([16, 32, 48, 64, 80], 5)  # five shapes take turns: three are kept
    assert captured.counters["portion_graph_captures"] == 3
    replays = captured.counters["portion_graph_replays"]
    assert replays >= 6
    run([96, 112], 12)  # the kept ones go unused: the new shapes take their places
    assert captured.counters["portion_graph_captures"] == 5
    assert captured.counters["portion_graph_replays"] > replays
    captured.check_errors()
