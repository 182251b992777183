#!/usr/bin/env python3
"""Measures decoding and prefill of the Llama-3.1-8B shape (random bf16 weights)
on one B200 and prints one JSON line.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

A "step" is one decode step of the whole batch.  ``value`` is decoded tokens a
second of the step function plus token selection, timed on the device with CUDA
events; ``e2e`` is the same through ``LLM.generate`` (host token ids in, host
token ids out).  The line also carries the prefill of a 2,048-token prompt, the
roofline fraction of the decode step, decoding at batch 1 and 64, the clocks
seen during the timed region, and how many of this package's kernels ran in it.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

# The headline configuration: the Llama-3.1-8B shape
MODEL = {
    "architectures": ["LlamaForCausalLM"],
    "hidden_size": 4096,
    "num_hidden_layers": 32,
    "num_attention_heads": 32,
    "num_key_value_heads": 8,
    "head_dim": 128,
    "intermediate_size": 14336,
    "vocab_size": 128256,
    "rope_theta": 500000.0,
    "rope_scaling": {
        "rope_type": "llama3",
        "factor": 8.0,
        "low_freq_factor": 1.0,
        "high_freq_factor": 4.0,
        "original_max_position_embeddings": 8192,
    },
    "max_position_embeddings": 8192,
    "rms_norm_eps": 1e-5,
    "tie_word_embeddings": False,
    "hidden_act": "silu",
}
FULL_LAYERS = 32
SEED = 2
CONTEXT_LEN = 8192
PROMPT_LEN = 2048
GEN_LEN = 256
PAGE_SIZE = 16
PREFILL_TOKENS = 2048

# Further shapes (Qwen3-8B and Qwen3-32B) for --shape; the default run and its JSON
# contract are those of the headline configuration above.
SHAPES = {
    "llama31-8b": None,
    "qwen3-8b": dict(
        model={
            "architectures": ["Qwen3ForCausalLM"], "hidden_size": 4096, "num_hidden_layers": 36, "num_attention_heads": 32,
            "num_key_value_heads": 8, "head_dim": 128, "intermediate_size": 12288, "vocab_size": 151936, "rope_theta": 1000000.0,
            "max_position_embeddings": 40960, "rms_norm_eps": 1e-6, "tie_word_embeddings": False, "hidden_act": "silu",
        },
        name="Qwen3-8B shape", seed=3, prompt_len=2048, gen_len=256, context_len=8192,
    ),
    "qwen3-32b": dict(
        model={
            "architectures": ["Qwen3ForCausalLM"], "hidden_size": 5120, "num_hidden_layers": 64, "num_attention_heads": 64,
            "num_key_value_heads": 8, "head_dim": 128, "intermediate_size": 25600, "vocab_size": 151936, "rope_theta": 1000000.0,
            "max_position_embeddings": 40960, "rms_norm_eps": 1e-6, "tie_word_embeddings": False, "hidden_act": "silu",
        },
        name="Qwen3-32B shape", seed=4, prompt_len=1024, gen_len=128, context_len=8192,
    ),
    # Further sizes of the two families: a head size of 64 with tied embeddings, small widths where
    # launches weigh more, and 70B-sized layers (fewer of them than the model has, named in config).
    "llama32-1b": dict(
        model={
            "architectures": ["LlamaForCausalLM"], "hidden_size": 2048, "num_hidden_layers": 16, "num_attention_heads": 32,
            "num_key_value_heads": 8, "head_dim": 64, "intermediate_size": 8192, "vocab_size": 128256, "rope_theta": 500000.0,
            "rope_scaling": dict(MODEL["rope_scaling"], factor=32.0), "max_position_embeddings": 131072, "rms_norm_eps": 1e-5,
            "tie_word_embeddings": True, "hidden_act": "silu",
        },
        name="Llama-3.2-1B shape", seed=5, prompt_len=2048, gen_len=256, context_len=8192,
    ),
    "qwen3-1.7b": dict(
        model={
            "architectures": ["Qwen3ForCausalLM"], "hidden_size": 2048, "num_hidden_layers": 28, "num_attention_heads": 16,
            "num_key_value_heads": 8, "head_dim": 128, "intermediate_size": 6144, "vocab_size": 151936, "rope_theta": 1000000.0,
            "max_position_embeddings": 40960, "rms_norm_eps": 1e-6, "tie_word_embeddings": True, "hidden_act": "silu",
        },
        name="Qwen3-1.7B shape", seed=6, prompt_len=2048, gen_len=256, context_len=8192,
    ),
    "qwen3-14b": dict(
        model={
            "architectures": ["Qwen3ForCausalLM"], "hidden_size": 5120, "num_hidden_layers": 40, "num_attention_heads": 40,
            "num_key_value_heads": 8, "head_dim": 128, "intermediate_size": 17408, "vocab_size": 151936, "rope_theta": 1000000.0,
            "max_position_embeddings": 40960, "rms_norm_eps": 1e-6, "tie_word_embeddings": False, "hidden_act": "silu",
        },
        name="Qwen3-14B shape", seed=7, prompt_len=2048, gen_len=256, context_len=8192,
    ),
    "llama31-70b": dict(
        model={
            "architectures": ["LlamaForCausalLM"], "hidden_size": 8192, "num_hidden_layers": 80, "num_attention_heads": 64,
            "num_key_value_heads": 8, "head_dim": 128, "intermediate_size": 28672, "vocab_size": 128256, "rope_theta": 500000.0,
            "rope_scaling": dict(MODEL["rope_scaling"]), "max_position_embeddings": 131072, "rms_norm_eps": 1e-5,
            "tie_word_embeddings": False, "hidden_act": "silu",
        },
        name="Llama-3.1-70B shape", seed=8, prompt_len=1024, gen_len=128, context_len=8192,
    ),
}
MODEL_NAME = "Llama-3.1-8B shape"

FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def load_peaks() -> tuple[dict, str]:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        try:
            with open(path) as handle:
                data = json.load(handle)
            peaks = dict(FALLBACK_PEAKS)
            for key in peaks:
                if isinstance(data.get(key), (int, float)):
                    peaks[key] = float(data[key])
            return peaks, "measured"
        except (OSError, ValueError):
            pass
    return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region runs."""

    QUERY = (
        "clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
        "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"
    )

    def __init__(self, device_index: int = 0) -> None:
        self.process = None
        self.device_index = device_index

    def start(self) -> None:
        try:
            self.process = subprocess.Popen(
                ["nvidia-smi", f"--id={self.device_index}", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE,
                stderr=subprocess.DEVNULL,
                text=True,
            )
        except OSError:
            self.process = None

    def stop(self) -> dict:
        if self.process is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.process.terminate()
        try:
            output, _ = self.process.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.process.kill()
            output, _ = self.process.communicate()
        clocks, maxima, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in output.splitlines():
            fields = [field.strip() for field in line.split(",")]
            if len(fields) < 8:
                continue
            try:
                clocks.append(float(fields[0]))
                maxima.append(float(fields[1]))
            except ValueError:
                continue
            for name, value in zip(names, fields[4:8]):
                if value.lower() == "active":
                    reasons.add(name)
        return {
            "sm_mhz": statistics.median(clocks) if clocks else None,
            "sm_max_mhz": max(maxima) if maxima else None,
            "reasons": sorted(reasons),
            "samples": len(clocks),
        }


def layers_that_fit(layers: int, max_batch: int) -> int:
    """The most layers, up to ``layers``, whose bf16 weights (held twice while random weights are drawn and
    packed) and whose cache for ``max_batch`` requests fit in nine tenths of the device's free memory."""
    import torch

    hidden, inter = MODEL["hidden_size"], MODEL["intermediate_size"]
    head_dim = MODEL.get("head_dim") or hidden // MODEL["num_attention_heads"]
    q, kv = MODEL["num_attention_heads"] * head_dim, MODEL["num_key_value_heads"] * head_dim
    layer_weights = 2 * (hidden * (q + 2 * kv) + q * hidden + 3 * hidden * inter)
    tables = 2 * MODEL["vocab_size"] * hidden * (1 if MODEL.get("tie_word_embeddings") else 2)
    tokens = max_batch * (-(-(PROMPT_LEN + GEN_LEN + 64) // PAGE_SIZE)) * PAGE_SIZE
    layer_cache = 2 * 2 * kv * tokens
    free, _ = torch.cuda.mem_get_info()
    room = 0.9 * free - 2 * tables - (4 << 30)  # workspace, logits, graphs
    return max(0, min(layers, int(room // (2 * layer_weights + layer_cache))))


def build_engine(layers: int, max_batch: int):
    import torch

    from kairyu_b200.config.engine_config import EngineConfig
    from kairyu_b200.engine.engine import Engine

    config = dict(MODEL)
    config["num_hidden_layers"] = layers
    per_request = -(-(PROMPT_LEN + GEN_LEN + 64) // PAGE_SIZE)
    engine_config = EngineConfig(
        dtype="bfloat16",
        page_size=PAGE_SIZE,
        num_pages=max_batch * per_request + 1,
        # room to prefill the whole default batch in one step, so that the end-to-end run's
        # decode steps are pure decode steps (prompt portions would otherwise ride along)
        max_num_batched_tokens=max(PREFILL_TOKENS, 8 * PROMPT_LEN),
        max_num_seqs=max(max_batch, 1),
        max_model_len=CONTEXT_LEN,
        max_num_partial_prefills=1,
        pipeline_depth=2,  # schedule-ahead: step N+1 is launched while step N runs (end-to-end run)
        seed=SEED,
    )
    engine = Engine.from_random(config, SEED, engine_config)
    torch.cuda.synchronize()
    return engine, config


def random_tokens(count: int, vocab: int, seed: int) -> list[int]:
    import torch

    generator = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (count,), generator=generator).tolist()


def time_decode(engine, batch: int, steps: int, warmup: int, sample_clocks: bool):
    """Device time of ``steps`` decode steps of ``batch`` requests that each hold a
    PROMPT_LEN-token prompt: step function + greedy token selection."""
    import torch

    from kairyu_b200.engine.runner import StepEntry
    from kairyu_b200.sampling.params import SamplingParams
    from kairyu_b200.sampling.sampler import SamplingRow

    runner, cache = engine.runner, engine.cache
    vocab = MODEL["vocab_size"]
    names = [f"bench{index}" for index in range(batch)]
    for index, name in enumerate(names):
        runner.step([StepEntry(name, random_tokens(PROMPT_LEN, vocab, 100 + index), ())])
    feed = [random_tokens(batch, vocab, 1000 + step) for step in range(warmup + steps)]
    rows = [SamplingRow(name, SamplingParams(temperature=0.0), 0) for name in names]

    def one(step: int):
        logits = runner.step([StepEntry(name, [feed[step][index]], (0,)) for index, name in enumerate(names)])
        return engine.sampler.sample(logits, rows)

    for step in range(warmup):
        one(step)
    torch.cuda.synchronize()
    sampler = ClockSampler()
    if sample_clocks:
        sampler.start()
        time.sleep(0.3)
    launches_before = runner.counters["kernel_launches"]
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    start.record()
    for step in range(warmup, warmup + steps):
        one(step)
    stop.record()
    torch.cuda.synchronize()
    milliseconds = start.elapsed_time(stop)
    clocks = sampler.stop() if sample_clocks else None
    launches = runner.counters["kernel_launches"] - launches_before + steps  # + one argmax per step
    runner.check_errors()
    context = PROMPT_LEN + warmup + steps / 2.0  # mean tokens a request holds during the timed steps
    for name in names:
        cache.release(name)
    return milliseconds, launches, clocks, context


def time_prefill(engine, iterations: int = 5, warmup: int = 3):
    import torch

    from kairyu_b200.engine.runner import StepEntry

    runner, cache = engine.runner, engine.cache
    tokens = random_tokens(PREFILL_TOKENS, MODEL["vocab_size"], 7)
    times = []
    for index in range(warmup + iterations):
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        start.record()
        runner.step([StepEntry("prefill", tokens, (PREFILL_TOKENS - 1,))])
        stop.record()
        torch.cuda.synchronize()
        cache.release("prefill")
        if index >= warmup:
            times.append(start.elapsed_time(stop))
    return statistics.median(times)


def time_short_prefill(engine, tokens: int = 128, iterations: int = 5, warmup: int = 4) -> float:
    """Wall-clock milliseconds from a short prompt's step call to its logits on the device (what a first
    token waits for): below a few hundred tokens the step is a replayed graph once its shape has come
    three times, which the warm-up steps see to."""
    import torch

    from kairyu_b200.engine.runner import StepEntry

    runner, cache = engine.runner, engine.cache
    prompt = random_tokens(tokens, MODEL["vocab_size"], 11)
    times = []
    for index in range(warmup + iterations):
        torch.cuda.synchronize()
        begin = time.perf_counter()
        runner.step([StepEntry("short", prompt, (tokens - 1,))])
        torch.cuda.synchronize()
        if index >= warmup:
            times.append((time.perf_counter() - begin) * 1e3)
        cache.release("short")
    return statistics.median(times)


def prefill_flops(config: dict, tokens: int) -> float:
    hidden, inter = config["hidden_size"], config["intermediate_size"]
    heads, kv_heads, dim = config["num_attention_heads"], config["num_key_value_heads"], config["head_dim"]
    per_token = 2 * hidden * (heads + 2 * kv_heads) * dim + 2 * heads * dim * hidden + 2 * hidden * 2 * inter + 2 * inter * hidden
    linear = per_token * tokens * config["num_hidden_layers"]
    attention = 4 * heads * dim * (tokens * (tokens + 1) / 2) * config["num_hidden_layers"]  # causal half of QK^T and PV
    head = 2 * hidden * config["vocab_size"]  # one row of logits
    return float(linear + attention + head)


def time_e2e(engine, batch: int, steps: int):
    """Decode tokens/s through ``LLM.generate``: (time of 1+steps tokens) - (time of 1 token)."""
    import torch

    from kairyu_b200 import SamplingParams, TokensPrompt
    from kairyu_b200.entrypoints.llm import LLM

    llm = LLM.from_engine(engine)
    prompts = [TokensPrompt(tuple(random_tokens(PROMPT_LEN, MODEL["vocab_size"], 200 + index))) for index in range(batch)]

    def run(max_tokens: int) -> float:
        torch.cuda.synchronize()
        begin = time.perf_counter()
        outputs = llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=max_tokens, ignore_eos=True))
        torch.cuda.synchronize()
        elapsed = time.perf_counter() - begin
        assert all(len(output.outputs[0].token_ids) == max_tokens for output in outputs)
        return elapsed

    run(2)  # warm: graphs for this batch size
    short = min(run(1) for _ in range(2))
    long = min(run(1 + steps) for _ in range(2))
    seconds = max(long - short, 1e-9)
    meta_ints = batch * 10 + 2 + batch * (CONTEXT_LEN // PAGE_SIZE)  # the packed int32 step description
    return batch * steps / seconds, meta_ints * 4, batch * 4 + 4


def time_mixed(layers: int) -> dict:
    """The mixed workload through ``LLM.generate``: 32 requests with prompt lengths
    uniform in [128, 4096], prompts cut into portions of 512 tokens beside the decodes of the others,
    128 generated tokens each.  Returns prompt+generated tokens a second and generated tokens a second."""
    import torch

    from kairyu_b200 import SamplingParams, TokensPrompt
    from kairyu_b200.config.engine_config import EngineConfig
    from kairyu_b200.engine.engine import Engine
    from kairyu_b200.entrypoints.llm import LLM

    config = dict(MODEL)
    config["num_hidden_layers"] = layers
    generator = torch.Generator().manual_seed(SEED)
    lengths = torch.randint(128, 4097, (32,), generator=generator).tolist()
    engine_config = EngineConfig(
        dtype="bfloat16", page_size=PAGE_SIZE, num_pages=sum(-(-(n + 128 + 16) // PAGE_SIZE) for n in lengths) + 1,
        max_num_batched_tokens=512 + 32, prefill_chunk_size=512, max_num_seqs=32, max_model_len=CONTEXT_LEN,
        max_num_partial_prefills=1, pipeline_depth=2, seed=SEED,
    )
    engine = Engine.from_random(config, SEED, engine_config)
    llm = LLM.from_engine(engine)
    prompts = [TokensPrompt(tuple(random_tokens(n, MODEL["vocab_size"], 300 + i))) for i, n in enumerate(lengths)]
    params = SamplingParams(temperature=0.0, max_tokens=128, ignore_eos=True)
    llm.generate(prompts[:4], SamplingParams(temperature=0.0, max_tokens=4, ignore_eos=True))  # warm
    engine.warm_up(32, max(lengths) + 128)  # a serving engine's decode graphs exist before its first request
    torch.cuda.synchronize()
    begin = time.perf_counter()
    outputs = llm.generate(prompts, params)
    torch.cuda.synchronize()
    seconds = time.perf_counter() - begin
    generated = sum(len(output.outputs[0].token_ids) for output in outputs)
    engine.runner.check_errors()
    return {
        "mixed_b32_total_tok_s": (sum(lengths) + generated) / seconds,
        "mixed_b32_generated_tok_s": generated / seconds,
        "mixed_b32_seconds": seconds,
    }


def time_shared_prefix(layers: int) -> dict:
    """16 requests that share a 2,048-token stem (a system prompt) and differ in a 128-token tail,
    64 generated tokens each, through ``LLM.generate`` with prefix caching off and on.  Prompts are
    prefilled one at a time in portions of 512 tokens, so every request after the first is admitted
    when the stem's pages have been published."""
    import torch

    from kairyu_b200 import SamplingParams, TokensPrompt
    from kairyu_b200.config.engine_config import EngineConfig
    from kairyu_b200.engine.engine import Engine
    from kairyu_b200.entrypoints.llm import LLM

    config = dict(MODEL)
    config["num_hidden_layers"] = layers
    stem = random_tokens(2048, MODEL["vocab_size"], 400)
    prompts = [TokensPrompt(tuple(stem + random_tokens(128, MODEL["vocab_size"], 401 + i))) for i in range(16)]
    warm = [TokensPrompt(tuple(random_tokens(600, MODEL["vocab_size"], 450 + i))) for i in range(4)]
    params = SamplingParams(temperature=0.0, max_tokens=64, ignore_eos=True)
    result: dict = {}
    for caching in (False, True):
        engine_config = EngineConfig(
            dtype="bfloat16", page_size=PAGE_SIZE, num_pages=20 * (-(-(2048 + 128 + 64 + 16) // PAGE_SIZE)) + 1,
            max_num_batched_tokens=512 + 16, prefill_chunk_size=512, max_num_seqs=16, max_model_len=CONTEXT_LEN,
            max_num_partial_prefills=1, pipeline_depth=2, enable_prefix_caching=caching, seed=SEED,
        )
        engine = Engine.from_random(config, SEED, engine_config)
        llm = LLM.from_engine(engine)
        llm.generate(warm, SamplingParams(temperature=0.0, max_tokens=4, ignore_eos=True))
        engine.warm_up(16, 2048 + 128 + 64)
        torch.cuda.synchronize()
        begin = time.perf_counter()
        outputs = llm.generate(prompts, params)
        torch.cuda.synchronize()
        seconds = time.perf_counter() - begin
        engine.runner.check_errors()
        generated = sum(len(output.outputs[0].token_ids) for output in outputs)
        key = "shared_prefix_cached" if caching else "shared_prefix_plain"
        result[key + "_seconds"] = seconds
        result[key + "_generated_tok_s"] = generated / seconds
        if caching:
            result["shared_prefix_cached_tokens"] = sum(output.metrics["num_cached_tokens"] for output in outputs)
            result["shared_prefix_prompt_tokens"] = sum(len(prompt.prompt_token_ids) for prompt in prompts)
        del llm, engine
        torch.cuda.empty_cache()
    return result


def time_kernels(engine, config: dict, batch: int, peaks: dict) -> dict:
    """The step's dominant kernels, each timed alone: one launch per layer of the model (every layer
    has weights and cache pages of its own, 0.4 GB a layer, so no launch finds its operands in the
    126 MB L2), the launches of one kernel captured in a CUDA graph and timed with CUDA events.
    Decode products and decode attention are judged by the bytes they have to read over the measured
    copy bandwidth, prefill attention and the prefill products by their FLOPs over the measured
    library product peak."""
    import torch

    import kairyu_b200.kernels as kernels
    from kairyu_b200.engine.workspace import Workspace

    device = engine.device
    blocks = engine.model.blocks
    hidden, inter = config["hidden_size"], config["intermediate_size"]
    heads, kv_heads, dim = config["num_attention_heads"], config["num_key_value_heads"], config["head_dim"]
    page = engine.page_size
    workspace = Workspace(device)
    bf16 = torch.bfloat16

    def rand(*shape):
        return (torch.randn(*shape, device=device, dtype=torch.float32) * 0.5).to(bf16)

    def timed(launch, repeats: int = 3) -> float:
        """Median microseconds of one launch: ``launch(layer)`` for every layer, in a graph."""
        for layer in range(min(2, len(blocks))):
            launch(layer)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side), torch.cuda.graph(graph):
            for layer in range(len(blocks)):
                launch(layer)
        torch.cuda.current_stream().wait_stream(side)
        graph.replay()
        torch.cuda.synchronize()
        times = []
        for _ in range(repeats):
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            graph.replay()
            stop.record()
            torch.cuda.synchronize()
            times.append(start.elapsed_time(stop) * 1e3 / len(blocks))
        return statistics.median(times)

    def by_bytes(us: float, count: float) -> dict:
        achieved = count / (us * 1e-6) / 1e9
        return {"us": us, "achieved": achieved, "unit": "GB/s", "frac": achieved / peaks["hbm_gbs"]}

    def by_flops(us: float, count: float, library: bool = False) -> dict:
        achieved = count / (us * 1e-6) / 1e12
        entry = {"us": us, "achieved": achieved, "unit": "TFLOP/s", "frac": achieved / peaks["bf16_tflops"]}
        if library:
            entry["library"] = True  # the product is the library's (cuBLAS through torch), as the reference's is
        return entry

    result = {}
    q_size, kv_size = heads * dim, kv_heads * dim
    qkv_width = q_size + 2 * kv_size
    # ---- decode products at the headline batch (weights streamed once)
    x_h, x_q, x_i = rand(batch, hidden), rand(batch, q_size), rand(batch, inter)
    out_qkv = torch.empty(batch, qkv_width, device=device, dtype=bf16)
    out_h = torch.empty(batch, hidden, device=device, dtype=bf16)
    out_i = torch.empty(batch, inter, device=device, dtype=bf16)
    result["qkv_product_decode"] = by_bytes(timed(lambda l: kernels.linear(x_h, blocks[l].mixer.w_qkv, None, out_qkv)), qkv_width * hidden * 2)
    result["o_product_decode"] = by_bytes(timed(lambda l: kernels.linear(x_q, blocks[l].mixer.w_o, None, out_h)), hidden * q_size * 2)
    result["gate_up_product_decode"] = by_bytes(
        timed(lambda l: kernels.linear_swiglu(x_h, blocks[l].ffn.w_gate_up, out_i, workspace)), 2 * inter * hidden * 2)
    result["down_product_decode"] = by_bytes(timed(lambda l: kernels.linear(x_i, blocks[l].ffn.w_down, None, out_h)), hidden * inter * 2)
    head_weight = engine.model.head.weight
    logits = torch.empty(batch, head_weight.shape[0], device=device, dtype=torch.float32)
    head_us = timed(lambda l: kernels.linear(x_h, head_weight, None, logits)) if head_weight.numel() * 2 > 200e6 else None
    if head_us is not None:  # one weight, but eight times the L2: every launch streams it whole
        result["lm_head_decode"] = by_bytes(head_us, head_weight.numel() * 2)
    # ---- decode attention: ``batch`` rows of PROMPT_LEN + 15 keys each over this layer's pages
    context = PROMPT_LEN + 15
    pages_per_row = -(-context // page)
    usable = engine.num_pages - 1
    if batch * pages_per_row <= usable:
        table = (torch.arange(batch * pages_per_row, device=device, dtype=torch.int32) + 1).view(batch, pages_per_row).contiguous()
        seq_lens = torch.full((batch,), context, device=device, dtype=torch.int32)
        rows = torch.arange(batch, device=device, dtype=torch.int32)
        q = rand(batch, qkv_width)
        mixed = torch.empty(batch, q_size, device=device, dtype=bf16)
        k_all, v_all = engine.storage.k[0], engine.storage.v[0]
        scale = dim ** -0.5

        def decode_attention(l):
            kernels.attention_decode_mma(
                q, mixed, k_all[l], v_all[l], seq_lens=seq_lens, block_table=table, decode_rows=rows, decode_tokens=rows,
                num_rows=batch, max_seq_len=context, num_q_heads=heads, scale=scale, workspace=workspace,
            )

        result["attention_decode"] = by_bytes(timed(decode_attention), batch * context * kv_size * 2 * 2)
        # ---- prefill attention: one row of PREFILL_TOKENS tokens
        tokens = PREFILL_TOKENS
        if -(-tokens // page) <= usable:
            tile = kernels.attention_prefill_tile_rows(dim)
            tiles = -(-tokens // tile)
            table1 = (torch.arange(-(-tokens // page), device=device, dtype=torch.int32) + 1).view(1, -1).contiguous()
            qo = torch.tensor([0, tokens], device=device, dtype=torch.int32)
            lens1 = torch.tensor([tokens], device=device, dtype=torch.int32)
            tile_rows = torch.zeros(tiles, device=device, dtype=torch.int32)
            tile_starts = torch.arange(tiles, device=device, dtype=torch.int32) * tile
            q_many = rand(tokens, qkv_width)
            mixed_many = torch.empty(tokens, q_size, device=device, dtype=bf16)

            def prefill_attention(l):
                kernels.attention_prefill_mma(
                    q_many, mixed_many, k_all[l], v_all[l], qo_indptr=qo, seq_lens=lens1, block_table=table1, tile_rows=tile_rows,
                    tile_starts=tile_starts, num_tiles=tiles, num_q_heads=heads, scale=scale,
                )

            result["attention_prefill"] = by_flops(timed(prefill_attention), 4.0 * heads * dim * tokens * (tokens + 1) / 2)
            # ---- prefill products (the library's)
            xm_h, xm_q, xm_i = rand(tokens, hidden), rand(tokens, q_size), rand(tokens, inter)
            om_qkv = torch.empty(tokens, qkv_width, device=device, dtype=bf16)
            om_h = torch.empty(tokens, hidden, device=device, dtype=bf16)
            om_gu = torch.empty(tokens, 2 * inter, device=device, dtype=bf16)
            result["qkv_product_prefill"] = by_flops(timed(lambda l: kernels.linear(xm_h, blocks[l].mixer.w_qkv, None, om_qkv)), 2.0 * tokens * hidden * qkv_width, True)
            result["o_product_prefill"] = by_flops(timed(lambda l: kernels.linear(xm_q, blocks[l].mixer.w_o, None, om_h)), 2.0 * tokens * hidden * q_size, True)
            result["gate_up_product_prefill"] = by_flops(timed(lambda l: kernels.linear(xm_h, blocks[l].ffn.w_gate_up, None, om_gu)), 2.0 * tokens * hidden * 2 * inter, True)
            result["down_product_prefill"] = by_flops(timed(lambda l: kernels.linear(xm_i, blocks[l].ffn.w_down, None, om_h)), 2.0 * tokens * hidden * inter, True)
    torch.cuda.synchronize()
    return result


def reference_arm(args) -> int:
    """The unmodified reference through its own public API, from the copy of its package under
    baseline/_ref (``baseline/reference_bench.py`` drives it; nothing of this package is imported
    on that path)."""
    ref_root = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref_root, "kairyu")):
        print(json.dumps({
            "impl": "reference",
            "unavailable": "no copy of ytworks/kairyu under baseline/_ref (pip cannot build it offline: its build backend, "
            "hatchling, is not in the wheelhouse; the package is pure Python, so copying its kairyu/ folder there installs it)",
        }))
        return 0
    try:
        from baseline.reference_bench import run_reference

        workload = dict(
            name=MODEL_NAME, prompt_len=PROMPT_LEN, gen_len=GEN_LEN, page_size=PAGE_SIZE, context_len=CONTEXT_LEN, seed=SEED,
            ref_root=ref_root, layers=args.layers, layers_full=FULL_LAYERS, clock_sampler=ClockSampler,
        )
        line = run_reference(args, MODEL, workload)
    except Exception as error:  # the reference arm must never take the driver down
        line = {"impl": "reference", "unavailable": f"{type(error).__name__}: {str(error)[:300]}"}
    print(json.dumps(line))
    return 0


def main() -> int:
    global MODEL, MODEL_NAME, FULL_LAYERS, SEED, PROMPT_LEN, GEN_LEN, CONTEXT_LEN
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=128)
    parser.add_argument("--warmup", type=int, default=8)
    parser.add_argument("--impl", choices=["ours", "reference"], default="ours")
    parser.add_argument("--batch", type=int, default=8)
    parser.add_argument("--layers", type=int, default=FULL_LAYERS, help="fewer layers only where memory or time needs it")
    parser.add_argument("--no-points", action="store_true", help="skip the batch 1 / 64 points and the end-to-end run")
    parser.add_argument("--shape", choices=sorted(SHAPES), default="llama31-8b", help="another shape than the default (its own lengths)")
    parser.add_argument("--mixed", action="store_true", help="add the mixed workload of 32 requests (chunked prefill beside decode)")
    parser.add_argument("--shared-prefix", action="store_true", help="add the shared-stem workload of 16 requests, prefix caching off and on")
    parser.add_argument("--prompt-len", type=int, default=None, help="another prompt length than the shape's (with --gen-len, within the context length)")
    parser.add_argument("--gen-len", type=int, default=None)
    parser.add_argument("--context-len", type=int, default=None, help="another context length than the shape's (longer prompts)")
    args = parser.parse_args()
    if SHAPES[args.shape] is not None:
        shape = SHAPES[args.shape]
        MODEL, MODEL_NAME, SEED = shape["model"], shape["name"], shape["seed"]
        PROMPT_LEN, GEN_LEN, CONTEXT_LEN = shape["prompt_len"], shape["gen_len"], shape["context_len"]
        if args.layers == FULL_LAYERS:
            args.layers = MODEL["num_hidden_layers"]
        FULL_LAYERS = MODEL["num_hidden_layers"]
    if args.context_len is not None:
        CONTEXT_LEN = args.context_len
        MODEL = dict(MODEL, max_position_embeddings=max(MODEL["max_position_embeddings"], CONTEXT_LEN))
    if args.prompt_len is not None:
        PROMPT_LEN = args.prompt_len
    if args.gen_len is not None:
        GEN_LEN = args.gen_len
    if PROMPT_LEN + GEN_LEN > CONTEXT_LEN:
        print(f"bench.py: prompt {PROMPT_LEN} + generation {GEN_LEN} exceeds the context length {CONTEXT_LEN}", file=sys.stderr)
        return 1
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    if args.impl == "reference":
        return reference_arm(args)
    if args.warmup < 3:
        args.warmup = 3

    import torch

    if not torch.cuda.is_available():
        print("bench.py: no CUDA device; kairyu_b200 has no CPU path", file=sys.stderr)
        return 1
    torch.cuda.set_device(0)
    peaks, peak_source = load_peaks()
    max_batch = max(args.batch, 1 if args.no_points else 64)
    fitting = layers_that_fit(args.layers, max_batch)
    if fitting < 1:
        print("bench.py: not even one layer of this shape and its cache fit the device's free memory", file=sys.stderr)
        return 1
    if fitting < args.layers:
        print(f"bench.py: {args.layers} layers of this shape do not fit the device beside their cache; running {fitting} "
              "(the line's config names both numbers)", file=sys.stderr)
        args.layers = fitting
    engine, config = build_engine(args.layers, max_batch)
    model = engine.model
    weight_bytes = model.bytes_streamed_per_step()
    kv_bytes_per_token = 2 * config["num_hidden_layers"] * config["num_key_value_heads"] * config["head_dim"] * 2

    milliseconds, launches, clocks, context = time_decode(engine, args.batch, args.steps, args.warmup, True)
    ms_per_step = milliseconds / args.steps
    value = args.batch * args.steps / (milliseconds / 1e3)
    step_bytes = weight_bytes + args.batch * context * kv_bytes_per_token
    achieved = step_bytes / (ms_per_step / 1e3) / 1e9

    prefill_ms = time_prefill(engine)
    flops = prefill_flops(config, PREFILL_TOKENS)
    prefill = {
        "value": PREFILL_TOKENS / (prefill_ms / 1e3),
        "tokens": PREFILL_TOKENS,
        "ms": prefill_ms,
        "frac": flops / (prefill_ms / 1e3) / (peaks["bf16_tflops"] * 1e12),  # of the burst cuBLAS peak
        "frac_of_sustained": flops / (prefill_ms / 1e3) / (peaks["bf16_tflops_sustained"] * 1e12),
    }

    points = {}
    e2e = None
    kernel_block = None

    def roofline_point(batch: int, step_ms: float, tokens_held: float) -> dict:
        moved = weight_bytes + batch * tokens_held * kv_bytes_per_token
        rate = moved / (step_ms / 1e3) / 1e9
        return {"batch": batch, "ms_per_step": step_ms, "gbytes": moved / 1e9, "achieved": rate, "frac": rate / peaks["hbm_gbs"]}

    roofline_points = {f"decode_b{args.batch}": roofline_point(args.batch, ms_per_step, context)}
    if not args.no_points:
        for batch in (1, 16, 32, 64):
            if batch == args.batch:
                continue
            steps = max(16, min(args.steps, 64))
            ms, _, _, held = time_decode(engine, batch, steps, args.warmup, False)
            key = f"decode_b{batch}"
            if batch in (1, 64):
                points[key] = batch * steps / (ms / 1e3)
            roofline_points[key] = roofline_point(batch, ms / steps, held)
        points["prefill_128_tokens_ms"] = time_short_prefill(engine)
        kernel_block = time_kernels(engine, config, args.batch, peaks)
        rate, h2d, d2h = time_e2e(engine, args.batch, min(args.steps, 64))
        e2e = {"value": rate, "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h}
    if args.mixed:
        del engine
        torch.cuda.empty_cache()
        points.update(time_mixed(args.layers))
        engine = None
    if args.shared_prefix:
        del engine
        torch.cuda.empty_cache()
        points.update(time_shared_prefix(args.layers))

    line = {
        "metric": f"decode tok/s @bs{args.batch} ({MODEL_NAME}, {PROMPT_LEN}-token prompts)",
        "value": value,
        "unit": "tokens/s",
        "n_gpus": 1,
        "steps": args.steps,
        "warmup": args.warmup,
        "ms_per_step": ms_per_step,
        "higher_is_better": True,
        "scaling": "weak",
        "vs_baseline": None,
        "dtype": "bf16",
        "data": "synthetic: seeded random token ids, seeded random weights (no checkpoint, no dataset)",
        "impl": "ours",
        "config": {
            "model": MODEL_NAME,
            "layers": config["num_hidden_layers"],
            "layers_full": FULL_LAYERS,
            "hidden": config["hidden_size"],
            "heads": config["num_attention_heads"],
            "kv_heads": config["num_key_value_heads"],
            "head_dim": config["head_dim"],
            "intermediate": config["intermediate_size"],
            "vocab": config["vocab_size"],
            "global_batch": args.batch,
            "seq_len": PROMPT_LEN,
            "gen_len": GEN_LEN,
            "context_len": CONTEXT_LEN,
            "page_size": PAGE_SIZE,
            "parallelism": "single_gpu",
            "pipeline_depth": 2,
            "l2": "inputs>L2 (weights and cache exceed the 126 MB L2)",
            "peaks": peak_source,
        },
        "prefill": prefill,
        "roofline": {
            "bound": "hbm",
            "achieved": achieved,
            "peak": peaks["hbm_gbs"],
            "unit": "GB/s",
            "frac": achieved / peaks["hbm_gbs"],
        },
        "roofline_points": roofline_points,
        "points": points,
        "clocks": clocks,
        "gpu_launches": launches,
    }
    if e2e is not None:
        line["e2e"] = e2e
    if kernel_block is not None:
        line["kernels"] = kernel_block
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
