"""Every attention kernel inside the engine: single-layer models whose head size and page size pick, between
them, the tcgen05 prefill kernel, the TMA-fed decode kernel, the mma.sync pair and the fp32-arithmetic
kernel; replayed whole, with a decoded tail (CUDA graphs) and in portions, against the plain implementation."""

import numpy as np
import pytest

import plain_model
import traces
from golden_inputs import as_held_in_bf16, golden_weights

pytestmark = pytest.mark.gpu

# (architecture, heads, kv heads, head size, page size): which bf16 attention kernels they reach
SHAPES = {
    "tc5+tma d128 p16": ("LlamaForCausalLM", 4, 2, 128, 16),
    "tc5+tma d64 p64": ("Qwen3ForCausalLM", 6, 1, 64, 64),
    "tc5+tma d128 p128": ("LlamaForCausalLM", 2, 2, 128, 128),
    "mma prefill, tma decode d256 p8": ("LlamaForCausalLM", 2, 1, 256, 8),
    "mma prefill, tma decode d192 p32": ("Qwen3ForCausalLM", 3, 3, 192, 32),
    "mma pair d64 p4": ("LlamaForCausalLM", 4, 2, 64, 4),
    "mma pair d80 p16": ("Qwen3ForCausalLM", 4, 1, 80, 16),
    "group of 16": ("LlamaForCausalLM", 16, 1, 64, 16),
}


def config_of(shape):
    architecture, heads, kv_heads, head_dim, _ = shape
    return {
        "architectures": [architecture], "hidden_size": 96, "num_hidden_layers": 1, "num_attention_heads": heads,
        "num_key_value_heads": kv_heads, "head_dim": head_dim, "intermediate_size": 112, "vocab_size": 211,
        "rope_theta": 30000.0, "max_position_embeddings": 400, "rms_norm_eps": 1e-5, "tie_word_embeddings": True,
        "hidden_act": "silu",
    }


@pytest.mark.parametrize("dtype,tolerance", [("bfloat16", 2e-2), ("float32", 2e-5)])
@pytest.mark.parametrize("name", sorted(SHAPES))
def test_cuts_match_plain(name, dtype, tolerance, tmp_path):
    from kairyu_b200.cache import CacheLayout, CacheManager, CacheStorage
    from kairyu_b200.engine.engine import load_model
    from kairyu_b200.engine.runner import ModelRunner
    from kairyu_b200.weights import write_random_model

    shape = SHAPES[name]
    config, page_size, seed = config_of(shape), shape[4], 9
    folder = write_random_model(config, tmp_path / "model", seed=seed, dtype="float32")
    weights = golden_weights(config, seed)
    if dtype == "bfloat16":
        weights = as_held_in_bf16(weights)
    requests = traces.make_requests(config["vocab_size"], [150, 45, 270], seed=23)
    expected = {n: plain_model.forward_logits(config, weights, t).numpy() for n, t in requests.items()}
    model, _ = load_model(folder, dtype=dtype, device="cuda")
    layout = CacheLayout.from_slot_specs(model.cache_slot_specs())
    num_pages = sum(-(-len(t) // page_size) for t in requests.values()) + 4
    cache = CacheManager(layout, num_pages=num_pages, page_size=page_size, max_requests=4)
    storage = CacheStorage(layout, num_pages=num_pages, page_size=page_size, max_requests=4, dtype=model.dtype, device="cuda")
    runner = ModelRunner(model, cache, storage, max_model_len=400, decode_mode="cuda_graph", max_graph_batch=4)
    for steps in (traces.trace_whole(requests), traces.trace_decode_tail(requests, 32), traces.trace_chunks(requests)):
        result = traces.run_in_process(runner, steps)
        worst = max(float(np.abs(row - expected[n][p]).max()) for (n, p), row in result.items())
        assert worst < tolerance, worst
    runner.check_errors()
    assert runner.counters["graph_replays"] > 0
