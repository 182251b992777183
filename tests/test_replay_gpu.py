"""Replay on the GPU: the same requests whole, with the last 32 tokens decoded
one by one, in portions of changing size, and mixed with other requests over a
pool so small that pages are used again; in 32-bit and in bfloat16; in process
and through ``bin/trace_run``; all compared with the plain implementation."""

import numpy as np
import pytest
import torch

import plain_model
import traces
from golden_inputs import as_held_in_bf16, golden_weights
from tiny_configs import TINY

pytestmark = pytest.mark.gpu

FP32_TOL = 2e-5
BF16_TOL = 2e-2  # absolute, on logits of magnitude ~1 (the reference's own bf16 bound, tests/gpu/test_tensor_decode_gpu.py:62-87)

LENGTHS = [70, 45, 101, 38, 64, 83, 90, 55]


def write_model(tmp_path_factory, name, dtype):
    from kairyu_b200.weights import write_random_model

    config, seed, _ = TINY[name]
    folder = tmp_path_factory.mktemp(f"{name}-{dtype}")
    write_random_model(config, folder, seed=seed, dtype=dtype)
    return folder


@pytest.fixture(scope="module", params=["llama", "qwen3", "odd", "wide", "yarn"])
def case(request, tmp_path_factory):
    name = request.param
    config, seed, page_size = TINY[name]
    folder = write_model(tmp_path_factory, name, "float32")
    weights = golden_weights(config, seed)
    requests = traces.make_requests(config["vocab_size"], LENGTHS, seed=21)
    expected32 = {n: plain_model.forward_logits(config, weights, t).numpy() for n, t in requests.items()}
    rounded = as_held_in_bf16(weights)
    expected16 = {n: plain_model.forward_logits(config, rounded, t).numpy() for n, t in requests.items()}
    return dict(name=name, config=config, folder=folder, page_size=page_size, requests=requests, expected={"float32": expected32, "bfloat16": expected16})


def make_runner(case, dtype, *, num_pages, decode_mode="eager"):
    from kairyu_b200.cache import CacheLayout, CacheManager, CacheStorage
    from kairyu_b200.engine.engine import load_model
    from kairyu_b200.engine.runner import ModelRunner

    model, _ = load_model(case["folder"], dtype=dtype, device="cuda")
    layout = CacheLayout.from_slot_specs(model.cache_slot_specs())
    cache = CacheManager(layout, num_pages=num_pages, page_size=case["page_size"], max_requests=8)
    storage = CacheStorage(layout, num_pages=num_pages, page_size=case["page_size"], max_requests=8, dtype=model.dtype, device="cuda")
    return ModelRunner(model, cache, storage, max_model_len=case["config"]["max_position_embeddings"], decode_mode=decode_mode, max_graph_batch=8, check_tables=True, debug_poison=True)


def worst(result, expected):
    return max(float(np.abs(row - expected[name][position]).max()) for (name, position), row in result.items())


def off_rows(result, expected, tolerance):
    """For a failure's message: the rows beyond the tolerance, as (request, position, error)."""
    errors = [(name, position, float(np.abs(row - expected[name][position]).max())) for (name, position), row in result.items()]
    return [entry for entry in errors if not entry[2] < tolerance][:12]


def cuts(case):
    requests = case["requests"]
    return {
        "whole": traces.trace_whole(requests),
        "tail": traces.trace_decode_tail(requests, 32),
        "chunks": traces.trace_chunks(requests),
        "mixed": traces.trace_mixed(requests, seed=3),
    }


@pytest.mark.parametrize("dtype,tolerance", [("float32", FP32_TOL), ("bfloat16", BF16_TOL)])
@pytest.mark.parametrize("decode_mode", ["eager", "cuda_graph"])
def test_every_cut_matches_plain(case, dtype, tolerance, decode_mode):
    all_cuts = cuts(case)
    small_pool = traces.peak_tokens(all_cuts["mixed"]) // case["page_size"] + 1
    total = sum(len(t) for t in case["requests"].values())
    assert small_pool * case["page_size"] < total + case["page_size"]
    runner = make_runner(case, dtype, num_pages=max(small_pool, 8), decode_mode=decode_mode)
    results = {}
    for cut, steps in all_cuts.items():
        results[cut] = traces.run_in_process(runner, steps)
        assert len(results[cut]) == total
        assert worst(results[cut], case["expected"][dtype]) < tolerance, (cut, off_rows(results[cut], case["expected"][dtype], tolerance))
    if decode_mode == "cuda_graph":
        assert runner.counters["graph_replays"] > 0
    if dtype == "float32":
        # the 32-bit kernels sum in an order that depends on the position only:
        # every cut gives the same bits
        for cut in ("tail", "chunks", "mixed"):
            for key, row in results["whole"].items():
                assert np.array_equal(row, results[cut][key]), (cut, key)


@pytest.mark.parametrize("dtype,tolerance", [("float32", FP32_TOL), ("bfloat16", BF16_TOL)])
def test_trace_run_program(case, dtype, tolerance, tmp_path):
    steps = traces.trace_mixed(case["requests"], seed=8)
    result = traces.run_program(
        case["folder"], tmp_path, steps, dtype=dtype, max_tokens=traces.peak_tokens(steps), vocab=case["config"]["vocab_size"],
        extra=["--page-size", str(case["page_size"])],
    )
    assert worst(result, case["expected"][dtype]) < tolerance
    tail = traces.trace_decode_tail(dict(list(case["requests"].items())[:2]), 32)
    out = tmp_path / "tail"
    result = traces.run_program(
        case["folder"], out, tail, dtype=dtype, max_tokens=traces.peak_tokens(tail), vocab=case["config"]["vocab_size"],
    )
    assert worst(result, case["expected"][dtype]) < tolerance


def test_trace_run_steps_without_wants_write_no_file(case, tmp_path):
    tokens = case["requests"]["r0"]
    steps = [
        {"step": 0, "entries": [{"id": "a", "tokens": tokens[:20], "want": []}], "end": []},
        {"step": 1, "entries": [{"id": "a", "tokens": tokens[20:22], "want": [1]}], "end": ["a"]},
    ]
    result = traces.run_program(case["folder"], tmp_path, steps, dtype="float32", max_tokens=64, vocab=case["config"]["vocab_size"])
    assert not (tmp_path / "0.f32").exists()
    assert list(result) == [("a", 21)]
    assert float(np.abs(result[("a", 21)] - case["expected"]["float32"]["r0"][21]).max()) < FP32_TOL


def test_first_tokens_of_a_sequence(case):
    """Position 0 alone, then positions 0..2: the shortest contexts."""
    runner = make_runner(case, "float32", num_pages=8)
    from kairyu_b200.engine.runner import StepEntry

    tokens = case["requests"]["r1"]
    expected = case["expected"]["float32"]["r1"]
    one = runner.step([StepEntry("a", tokens[:1], (0,))]).cpu().numpy()
    assert np.abs(one[0] - expected[0]).max() < FP32_TOL
    two = runner.step([StepEntry("a", tokens[1:3], (0, 1))]).cpu().numpy()
    assert np.abs(two - expected[1:3]).max() < FP32_TOL


@pytest.mark.parametrize("dtype,tolerance", [("float32", FP32_TOL), ("bfloat16", BF16_TOL)])
def test_long_decoding(case, dtype, tolerance):
    """One request decoded token by token over many pages (and, for bf16, past a split of the decode kernel)."""
    config = case["config"]
    length = min(config["max_position_embeddings"], 300)
    tokens = traces.make_requests(config["vocab_size"], [length], seed=77)["r0"]
    weights = golden_weights(config, TINY[case["name"]][1])
    if dtype == "bfloat16":
        weights = as_held_in_bf16(weights)
    expected = plain_model.forward_logits(config, weights, tokens).numpy()
    runner = make_runner(case, dtype, num_pages=length // case["page_size"] + 3, decode_mode="cuda_graph")
    steps = traces.trace_decode_tail({"r0": tokens}, tail=length - 3)
    result = traces.run_in_process(runner, steps)
    assert worst(result, {"r0": expected}) < tolerance


def test_graph_replays_of_several_rows_survive_other_work_between_steps(case):
    """Replays read index tensors made at capture time; allocations and kernels
    between steps (a sampler, say) must not land on them."""
    from kairyu_b200.engine.runner import StepEntry
    import kairyu_b200.kernels as kernels

    requests = dict(list(case["requests"].items())[:4])
    expected = case["expected"]["float32"]
    runner = make_runner(case, "float32", num_pages=40, decode_mode="cuda_graph")
    head = 20
    runner.step([StepEntry(name, tokens[:head], ()) for name, tokens in requests.items()])
    for index in range(head, head + 12):
        logits = runner.step([StepEntry(name, [tokens[index]], (0,)) for name, tokens in requests.items()])
        scratch = [torch.empty(4, dtype=torch.int32, device="cuda") for _ in range(8)]
        for tensor in scratch:
            kernels.argmax(logits, tensor)
        for row, name in enumerate(requests):
            assert np.abs(logits[row].cpu().numpy() - expected[name][index]).max() < FP32_TOL
    assert runner.counters["graph_replays"] >= 12
