"""The step function at the layer sizes of the models the benchmark runs: the
Llama-3.1-8B and Qwen3-8B shapes with two layers (every other size real: width 4096,
32 query and 8 KV heads of 128, feed-forward 14336 or 12288, vocabulary 128256 or
151936, llama3 position scaling over 8192 or per-head q/k norms), random weights.

Compared with the plain implementation (run on the GPU in fp32 with no reduced-precision
matrix mode: the CPU is too slow at these sizes; the code is the same file), in 32-bit and in
bfloat16: the four cuts of a set of requests (whole, tail decoded, portions, mixed over a
small pool), and decode steps of 12 to 64 live rows through graphs of every batch bucket.
Logits are asked for at chosen positions only (a row is half a megabyte).

Follows kairyu tests/unit/test_model_parity.py:78-114 (whole, then chunked through one pool)
and tests/unit/test_batched_decode.py:40,92 (several rows decoded together).
"""

import pytest
import torch

import parity
import traces

pytestmark = pytest.mark.gpu

PAGE = 16
LENGTHS = [300, 45, 531, 150, 64, 283, 190, 97]

LLAMA31_8B = {
    "architectures": ["LlamaForCausalLM"], "hidden_size": 4096, "num_hidden_layers": 2, "num_attention_heads": 32,
    "num_key_value_heads": 8, "head_dim": 128, "intermediate_size": 14336, "vocab_size": 128256, "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0, "original_max_position_embeddings": 8192},
    "max_position_embeddings": 8192, "rms_norm_eps": 1e-5, "tie_word_embeddings": False, "hidden_act": "silu",
}
QWEN3_8B = {
    "architectures": ["Qwen3ForCausalLM"], "hidden_size": 4096, "num_hidden_layers": 2, "num_attention_heads": 32,
    "num_key_value_heads": 8, "head_dim": 128, "intermediate_size": 12288, "vocab_size": 151936, "rope_theta": 1000000.0,
    "max_position_embeddings": 40960, "rms_norm_eps": 1e-6, "tie_word_embeddings": False, "hidden_act": "silu",
}
# The width and head count of Llama-3.1-70B (8192, 64 query heads on 8 KV heads) with a narrower
# feed-forward and vocabulary: products that write the residual are launched with more blocks than
# a scaling epilogue adds up, so these steps take the norm kernels at every row count.
WIDE_70B = {
    "architectures": ["LlamaForCausalLM"], "hidden_size": 8192, "num_hidden_layers": 2, "num_attention_heads": 64,
    "num_key_value_heads": 8, "head_dim": 128, "intermediate_size": 7168, "vocab_size": 32000, "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0, "original_max_position_embeddings": 8192},
    "max_position_embeddings": 8192, "rms_norm_eps": 1e-5, "tie_word_embeddings": False, "hidden_act": "silu",
}
SHAPES = {"llama31_8b": (LLAMA31_8B, 2), "qwen3_8b": (QWEN3_8B, 3), "width_8192": (WIDE_70B, 4)}

# Every bound is what the same arithmetic costs the plain model itself.
# 32-bit: the truth is the plain model in 64-bit; the plain model in 32-bit is a few 1e-5 from it on
# these logits (size up to 7, sums over 14336 terms); the engine, whose products add each output's
# terms in order (256 at a time, then the blocks' sums), stays within half of that (measured: 0.19 to
# 0.32 times; with one accumulator over all of k it was 1.0 to 1.5 times).
# bfloat16: the truth is the plain model in 32-bit on the weights rounded to bfloat16; the engine,
# which keeps the residual and all statistics in 32-bit, may not be further from it than the plain
# model is when it rounds every operation's result to bfloat16, with a quarter more for library
# products that may choose other algorithms on another day (measured: 0.7 to 0.8 times).
FP32_FACTOR = 0.5
BF16_FACTOR = 1.25


def no_reduced_precision():
    torch.backends.cuda.matmul.allow_tf32 = False
    torch.backends.cudnn.allow_tf32 = False
    torch.set_float32_matmul_precision("highest")


@pytest.fixture(scope="module", params=sorted(SHAPES))
def shape(request):
    from golden_inputs import golden_weights_on

    no_reduced_precision()
    config, seed = SHAPES[request.param]
    weights = golden_weights_on(config, seed, "cuda")  # fp32, by checkpoint name; what init_random draws
    requests = traces.make_requests(config["vocab_size"], LENGTHS, seed=31)
    keep = {name: parity.keep_positions(len(tokens)) for name, tokens in requests.items()}
    held = {"float32": weights, "bfloat16": {k: v.float() for k, v in parity.in_bf16(weights, False).items()}}
    case = dict(name=request.param, config=config, seed=seed, requests=requests, keep=keep, held=held, expected={}, bound={})
    yield case
    case.clear()
    torch.cuda.empty_cache()


def truth_and_bound(case, dtype, requests=None, keep=None):
    """(the logits to compare with, how far from them the engine may be)."""
    cached = requests is None
    if cached and dtype in case["expected"]:
        return case["expected"][dtype], case["bound"][dtype]
    requests = case["requests"] if requests is None else requests
    keep = case["keep"] if keep is None else keep
    config = case["config"]
    if dtype == "float32":
        truth = parity.plain_rows(config, {k: v.double() for k, v in case["held"]["float32"].items()}, requests, keep)
        bound = FP32_FACTOR * parity.worst_error(parity.plain_rows(config, case["held"]["float32"], requests, keep), truth)
    else:
        truth = parity.plain_rows(config, case["held"]["bfloat16"], requests, keep)
        bound = BF16_FACTOR * parity.worst_error(parity.plain_rows(config, parity.in_bf16(case["held"]["float32"], False), requests, keep), truth)
    if cached:
        case["expected"][dtype], case["bound"][dtype] = truth, bound
    return truth, bound


def make_runner(case, dtype, *, num_pages, max_graph_batch=8, decode_mode="cuda_graph", max_model_len=2048):
    from kairyu_b200.cache import CacheLayout, CacheManager, CacheStorage
    from kairyu_b200.engine.engine import random_model
    from kairyu_b200.engine.runner import ModelRunner

    model, _ = random_model(case["config"], case["seed"], dtype=dtype, device="cuda")
    layout = CacheLayout.from_slot_specs(model.cache_slot_specs())
    requests_at_once = max(max_graph_batch, 8)
    cache = CacheManager(layout, num_pages=num_pages, page_size=PAGE, max_requests=requests_at_once)
    storage = CacheStorage(layout, num_pages=num_pages, page_size=PAGE, max_requests=requests_at_once, dtype=model.dtype, device="cuda")
    return ModelRunner(
        model, cache, storage, max_model_len=max_model_len, decode_mode=decode_mode, max_graph_batch=max_graph_batch,
        check_tables=True, debug_poison=True,
    )


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_every_cut_at_real_layer_sizes(shape, dtype):
    expected, bound = truth_and_bound(shape, dtype)
    requests, keep = shape["requests"], shape["keep"]
    cuts = {
        "whole": traces.trace_whole(requests),
        "tail": traces.trace_decode_tail(requests, 32),
        "chunks": traces.trace_chunks(requests, sizes=(24, 7, 2, 130, 3, 64, 2, 257)),
        "mixed": traces.trace_mixed(requests, seed=3),
    }
    small_pool = traces.peak_tokens(cuts["mixed"]) // PAGE + 1
    assert small_pool * PAGE < sum(LENGTHS) + PAGE  # pages are used again
    runner = make_runner(shape, dtype, num_pages=small_pool)
    results = {}
    for cut, steps in cuts.items():
        results[cut] = traces.run_in_process(runner, parity.thin_wants(steps, keep))
        assert results[cut].keys() == expected.keys()
        error = parity.worst_error(results[cut], expected)
        print(f"[parity] {shape['name']} {dtype} {cut}: worst error {error:.3e}, bound {bound:.3e}")
        assert error < bound, (cut, error, bound, parity.rows_beyond(results[cut], expected, bound))
    assert runner.counters["graph_replays"] > 0
    if dtype == "float32":
        for cut in ("tail", "chunks", "mixed"):  # position-only summation orders: every cut gives the same bits
            parity.assert_same_bits(results["whole"], results[cut], cut)
    else:
        del runner
        again = make_runner(shape, dtype, num_pages=small_pool)  # a second engine: what is not a race gives the same bits
        for cut in ("tail", "mixed"):
            parity.assert_same_bits(results[cut], traces.run_in_process(again, parity.thin_wants(cuts[cut], keep)), cut)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_decode_steps_of_many_rows_at_real_layer_sizes(shape, dtype):
    """12, 16, 24, 40 and 64 live requests decoded together: graphs of the batch buckets beyond 8, where
    the products, the norms and the position encoding go through other kernels than up to 8 rows."""
    config = shape["config"]
    tail = 5
    runner = make_runner(shape, dtype, num_pages=64 * 6 + 1, max_graph_batch=64)
    for rows in (12, 16, 24, 40, 64):
        generator = torch.Generator().manual_seed(rows)
        lengths = torch.randint(tail + 1, 80, (rows,), generator=generator).tolist()
        requests = {f"m{rows}-{i}": t for i, t in enumerate(traces.make_requests(config["vocab_size"], lengths, seed=40 + rows).values())}
        keep = {name: list(range(len(tokens) - tail - 1, len(tokens))) for name, tokens in requests.items()}
        expected, bound = truth_and_bound(shape, dtype, requests, keep)
        before = runner.counters["graph_replays"]
        result = traces.run_in_process(runner, parity.trace_many_rows(requests, tail))
        assert runner.counters["graph_replays"] - before == tail
        assert result.keys() == expected.keys()
        error = parity.worst_error(result, expected)
        print(f"[parity] {shape['name']} {dtype} {rows} rows: worst error {error:.3e}, bound {bound:.3e}")
        assert error < bound, (rows, error, bound, parity.rows_beyond(result, expected, bound))


def test_a_long_prompt_at_real_layer_sizes(shape):
    """One prompt of 4,300 tokens in bfloat16, whole (its attention goes to the kernel that takes two
    query tiles a block), in portions of 1,024 (one tile a block) and of 512 and less (the later
    portions' keys are shared among blocks), with the last tokens decoded: every cut within the bound."""
    from ctypes import c_int

    import kairyu_b200.kernels as kernels

    config = shape["config"]
    if config["hidden_size"] != 4096:
        pytest.skip("one width is enough here")
    length = 4300
    heads = config["num_attention_heads"]
    assert kernels._fn("attention_prefill_tc5", "kb_attention_prefill_tc5_two_tiles", [c_int] * 5)(128, heads, -(-length // 256), PAGE, length) == 1
    assert kernels._fn("attention_prefill_tc5", "kb_attention_prefill_tc5_splits", [c_int] * 4)(128, heads, 4, 4000) > 1
    requests = traces.make_requests(config["vocab_size"], [length], seed=77)
    keep = {name: sorted(set(range(0, length, 389)) | set(range(length - 6, length))) for name in requests}
    expected, bound = truth_and_bound(shape, "bfloat16", requests, keep)
    cuts = {
        "whole": traces.trace_whole(requests),
        "portions of 1024": traces.trace_chunks(requests, sizes=(1024,)),
        "portions of 512 and less": traces.trace_chunks(requests, sizes=(512, 300, 512, 128, 512, 2, 512)),
        "tail decoded": traces.trace_decode_tail(requests, 5),
    }
    runner = make_runner(shape, "bfloat16", num_pages=length // PAGE + 3, max_model_len=4608)
    for cut, steps in cuts.items():
        result = traces.run_in_process(runner, parity.thin_wants(steps, keep))
        assert result.keys() == expected.keys()
        error = parity.worst_error(result, expected)
        print(f"[parity] {shape['name']} long prompt, {cut}: worst error {error:.3e}, bound {bound:.3e}")
        assert error < bound, (cut, error, bound, parity.rows_beyond(result, expected, bound))
    runner.check_errors()
