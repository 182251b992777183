"""Generation through the Python entry point on the GPU, compared with the
plain implementation: the two tiny workloads (greedy; temperature + top-p with
seeds), portions under a token budget, preemption when pages run out."""

import pytest
import torch

import plain_model
from tiny_configs import TINY

pytestmark = pytest.mark.gpu


def plain_generate(config, weights, prompt, steps, params=None, request_seed=0):
    tokens = list(prompt)
    for position in range(steps):
        logits = plain_model.forward_logits(config, weights, tokens)[-1]
        if params is None:
            token = int(logits.argmax())
        else:
            token = plain_model.sample_token(logits, base_seed=request_seed, position=position, **params)
        tokens.append(token)
    return tokens[len(prompt):]


def prompts_of(config, lengths, seed):
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, config["vocab_size"], (n,), generator=g).tolist() for n in lengths]


def test_greedy_workload_tiny_llama():
    """4 prompts of 1, 7, 33 and 50 tokens, 16 greedy tokens each, page size 16, fp32."""
    from kairyu_b200 import LLM, SamplingParams, TokensPrompt

    config, seed, page_size = TINY["llama"]
    llm = LLM.from_random(config, seed=seed, dtype="float32", page_size=page_size, num_pages=32)
    weights = {spec.name: None for spec in llm.engine.model.tensor_specs()}
    weights = engine_weights(llm)
    prompts = prompts_of(config, [1, 7, 33, 50], seed=100)
    outputs = llm.generate([TokensPrompt(tuple(p)) for p in prompts], SamplingParams(temperature=0.0, max_tokens=16))
    for prompt, output in zip(prompts, outputs):
        assert output.prompt_token_ids == tuple(prompt)
        assert list(output.outputs[0].token_ids) == plain_generate(config, weights, prompt, 16)
        assert output.outputs[0].finish_reason == "length"


def engine_weights(llm):
    """The engine's own (random, device-generated) weights by HF tensor name, as fp32 CPU tensors."""
    model = llm.engine.model
    out = {}
    for index, block in enumerate(model.blocks):
        p = f"model.layers.{index}"
        mixer, ffn = block.mixer, block.ffn
        q, kv = mixer.q_size, mixer.kv_size
        out[f"{p}.self_attn.q_proj.weight"] = mixer.w_qkv[:q]
        out[f"{p}.self_attn.k_proj.weight"] = mixer.w_qkv[q : q + kv]
        out[f"{p}.self_attn.v_proj.weight"] = mixer.w_qkv[q + kv :]
        out[f"{p}.self_attn.o_proj.weight"] = mixer.w_o
        if mixer.b_qkv is not None:
            out[f"{p}.self_attn.q_proj.bias"] = mixer.b_qkv[:q]
            out[f"{p}.self_attn.k_proj.bias"] = mixer.b_qkv[q : q + kv]
            out[f"{p}.self_attn.v_proj.bias"] = mixer.b_qkv[q + kv :]
        if mixer.b_o is not None:
            out[f"{p}.self_attn.o_proj.bias"] = mixer.b_o
        if mixer.q_norm_weight is not None:
            out[f"{p}.self_attn.q_norm.weight"] = mixer.q_norm_weight
            out[f"{p}.self_attn.k_norm.weight"] = mixer.k_norm_weight
        inter = ffn.intermediate_size
        out[f"{p}.mlp.gate_proj.weight"] = ffn.w_gate_up[:inter]
        out[f"{p}.mlp.up_proj.weight"] = ffn.w_gate_up[inter:]
        out[f"{p}.mlp.down_proj.weight"] = ffn.w_down
        out[f"{p}.input_layernorm.weight"] = block.mixer_norm.weight
        out[f"{p}.post_attention_layernorm.weight"] = block.ffn_norm.weight
    out["model.embed_tokens.weight"] = model.embedding.weight
    out["model.norm.weight"] = model.final_norm.weight
    out["lm_head.weight"] = model.head.weight
    return {k: v.detach().float().cpu() for k, v in out.items()}


def test_sampled_workload_tiny_qwen3():
    """6 prompts of 1..120 tokens, portions of 24, temperature 0.8 / top-p 0.9 with seeds, 24 tokens, page size 8, fp32."""
    from kairyu_b200 import LLM, SamplingParams, TokensPrompt

    config, seed, page_size = TINY["qwen3"]
    llm = LLM.from_random(config, seed=seed, dtype="float32", page_size=page_size, num_pages=128, prefill_chunk_size=24)
    weights = engine_weights(llm)
    g = torch.Generator().manual_seed(7)
    lengths = torch.randint(1, 121, (6,), generator=g).tolist()
    prompts = prompts_of(config, lengths, seed=101)
    params = [SamplingParams(temperature=0.8, top_p=0.9, seed=1000 + i, max_tokens=24) for i in range(6)]
    outputs = llm.generate([TokensPrompt(tuple(p)) for p in prompts], params)
    for index, (prompt, output) in enumerate(zip(prompts, outputs)):
        expected = plain_generate(config, weights, prompt, 24, dict(temperature=0.8, top_p=0.9), request_seed=1000 + index)
        assert list(output.outputs[0].token_ids) == expected
    again = llm.generate([TokensPrompt(tuple(p)) for p in prompts], params)
    assert [o.outputs[0].token_ids for o in again] == [o.outputs[0].token_ids for o in outputs]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_generation_under_a_small_budget_and_few_pages(dtype):
    """A token budget of 7 cuts prompts into many portions beside decodes; so few
    pages that requests wait and are preempted; the greedy tokens stay those of
    the plain implementation (fp32) or agree with it almost everywhere (bf16)."""
    from kairyu_b200 import LLM, SamplingParams, TokensPrompt

    config, seed, page_size = TINY["odd"]
    llm = LLM.from_random(config, seed=seed, dtype=dtype, page_size=page_size, num_pages=9, max_num_batched_tokens=7, max_num_seqs=4)
    weights = engine_weights(llm)
    prompts = prompts_of(config, [30, 14, 46, 31, 15, 47], seed=102)
    outputs = llm.generate([TokensPrompt(tuple(p)) for p in prompts], SamplingParams(temperature=0.0, max_tokens=20))
    assert llm.engine.scheduler.counters["preemptions"] > 0
    llm.engine.cache.check()
    assert llm.engine.cache.live_requests == 0
    agree = total = 0
    for prompt, output in zip(prompts, outputs):
        expected = plain_generate(config, weights, prompt, 20)
        got = list(output.outputs[0].token_ids)
        assert len(got) == 20
        if dtype == "float32":
            assert got == expected
        # count agreement up to the first divergence (after it the contexts differ)
        for a, b in zip(got, expected):
            total += 1
            if a != b:
                break
            agree += 1
    if dtype == "bfloat16":
        assert agree / total > 0.9


@pytest.mark.parametrize("name,dtype", [("llama", "float32"), ("wide", "bfloat16"), ("qwen3", "bfloat16")])
def test_schedule_ahead_gives_the_same_tokens(name, dtype):
    """pipeline_depth=2 launches step N+1 before step N's tokens reach the host (its rows read
    them from the device); the tokens, stops included, are those of pipeline_depth=1."""
    from kairyu_b200 import LLM, SamplingParams, TokensPrompt

    config, seed, page_size = TINY[name]
    prompts = prompts_of(config, [5, 21, 40, 9, 64], seed=120)
    results = {}
    stop = None
    for depth in (1, 2):
        llm = LLM.from_random(config, seed=seed, dtype=dtype, page_size=page_size, num_pages=64, pipeline_depth=depth)
        if stop is None:  # a token request 0 produces on its own: make it a stop token for it
            free = llm.generate(TokensPrompt(tuple(prompts[0])), SamplingParams(temperature=0.0, max_tokens=12))[0]
            stop = free.outputs[0].token_ids[5]
        params = [SamplingParams(temperature=0.0, max_tokens=24, stop_token_ids=[stop])] + [
            SamplingParams(temperature=0.0, max_tokens=m) for m in (3, 1, 30, 17)
        ]
        outputs = llm.generate([TokensPrompt(tuple(p)) for p in prompts], params)
        results[depth] = [(o.outputs[0].token_ids, o.outputs[0].finish_reason) for o in outputs]
        llm.engine.cache.check()
        assert llm.engine.cache.live_requests == 0
        assert (llm.engine.runner.counters["future_tokens"] > 0) == (depth == 2)
        if depth == 2:
            assert llm.engine.runner.counters["graph_replays"] > 0
    assert results[1] == results[2]
    assert results[2][0][1] == "stop" and results[2][0][0][-1] == stop and len(results[2][0][0]) <= 6
    if dtype == "float32":
        weights = engine_weights(LLM.from_random(config, seed=seed, dtype=dtype, page_size=page_size, num_pages=64))
        assert list(results[2][3][0]) == plain_generate(config, weights, prompts[3], 30)


@pytest.mark.parametrize("seed", [0, 5])
def test_schedule_ahead_on_random_workloads_under_page_pressure(seed):
    """bf16, CUDA graphs, a pool so small that requests wait and are preempted, random limits and stops:
    pipeline_depth=2 gives the tokens and finish reasons of pipeline_depth=1."""
    import random

    from kairyu_b200 import LLM, SamplingParams, TokensPrompt

    rng = random.Random(seed)
    config, model_seed, page_size = TINY["wide"]
    count = rng.randint(4, 8)
    lengths = [rng.randint(1, 90) for _ in range(count)]
    limits = [rng.randint(1, 20) for _ in range(count)]
    options = dict(num_pages=rng.randint(24, 40), max_num_batched_tokens=rng.choice([9, 32, 128]), max_num_seqs=rng.choice([3, 8]))
    prompts = prompts_of(config, lengths, seed=300 + seed)
    results, stops = {}, None
    for depth in (1, 2):
        llm = LLM.from_random(config, seed=model_seed, dtype="bfloat16", page_size=page_size, pipeline_depth=depth, **options)
        if stops is None:
            free = llm.generate([TokensPrompt(tuple(p)) for p in prompts], [SamplingParams(temperature=0.0, max_tokens=m) for m in limits])
            stops = [o.outputs[0].token_ids[len(o.outputs[0].token_ids) // 2] if i % 2 == 0 else None for i, o in enumerate(free)]
        params = [
            SamplingParams(temperature=0.0 if i % 3 else 0.7, seed=5 + i, max_tokens=limits[i], stop_token_ids=[stops[i]] if stops[i] is not None else [])
            for i in range(count)
        ]
        outputs = llm.generate([TokensPrompt(tuple(p)) for p in prompts], params)
        results[depth] = [(o.outputs[0].token_ids, o.outputs[0].finish_reason, o.outputs[0].stop_reason) for o in outputs]
        llm.engine.cache.check()
        assert llm.engine.cache.live_requests == 0 and not llm.engine.has_unfinished()
        llm.engine.runner.check_errors()
    assert results[1] == results[2]


def test_stop_token_and_eos():
    from kairyu_b200 import LLM, SamplingParams, TokensPrompt

    config, seed, page_size = TINY["llama"]
    llm = LLM.from_random(config, seed=seed, dtype="float32", page_size=page_size, num_pages=32)
    prompt = prompts_of(config, [9], seed=103)[0]
    free = llm.generate(TokensPrompt(tuple(prompt)), SamplingParams(temperature=0.0, max_tokens=12))[0].outputs[0].token_ids
    stop_at = free[4]
    first = free.index(stop_at)
    out = llm.generate(TokensPrompt(tuple(prompt)), SamplingParams(temperature=0.0, max_tokens=12, stop_token_ids=[stop_at]))[0].outputs[0]
    assert out.token_ids == free[: first + 1]
    assert out.finish_reason == "stop" and out.stop_reason == stop_at
    # min_tokens masks the stop token until enough tokens exist
    out = llm.generate(
        TokensPrompt(tuple(prompt)), SamplingParams(temperature=0.0, max_tokens=12, stop_token_ids=[stop_at], min_tokens=first + 2)
    )[0].outputs[0]
    assert len(out.token_ids) >= first + 2
    assert stop_at not in out.token_ids[: first + 2]
    # EOS from the model config ends a request unless ignore_eos
    llm.eos_token_ids = (stop_at,)
    out = llm.generate(TokensPrompt(tuple(prompt)), SamplingParams(temperature=0.0, max_tokens=12))[0].outputs[0]
    assert out.token_ids == free[: first + 1] and out.finish_reason == "stop"
    out = llm.generate(TokensPrompt(tuple(prompt)), SamplingParams(temperature=0.0, max_tokens=12, ignore_eos=True))[0].outputs[0]
    assert out.token_ids == free


def test_penalties_change_greedy_tokens_as_the_plain_rule_says():
    from kairyu_b200 import LLM, SamplingParams, TokensPrompt

    config, seed, page_size = TINY["llama"]
    llm = LLM.from_random(config, seed=seed, dtype="float32", page_size=page_size, num_pages=32)
    weights = engine_weights(llm)
    prompt = prompts_of(config, [15], seed=104)[0]
    params = SamplingParams(temperature=0.0, max_tokens=10, repetition_penalty=1.6, frequency_penalty=0.4, presence_penalty=0.3)
    got = list(llm.generate(TokensPrompt(tuple(prompt)), params)[0].outputs[0].token_ids)
    tokens = list(prompt)
    outputs = []
    for _ in range(10):
        logits = plain_model.forward_logits(config, weights, tokens)[-1]
        logits = plain_model.apply_penalties(logits, prompt, outputs, repetition=1.6, frequency=0.4, presence=0.3)
        token = int(logits.argmax())
        outputs.append(token)
        tokens.append(token)
    assert got == outputs


def test_kernels_refuse_cpu_tensors():
    import kairyu_b200.kernels as kernels

    with pytest.raises(kernels.KernelError):
        kernels.rmsnorm(torch.zeros(2, 8), torch.ones(8), 1e-5, torch.zeros(2, 8))


@pytest.mark.parametrize("name,dtype,depth", [("llama", "float32", 1), ("odd", "float32", 2), ("wide", "bfloat16", 2), ("qwen3", "bfloat16", 1)])
def test_prefix_caching_gives_the_same_tokens(name, dtype, depth):
    """Requests that start with the same tokens read the pages an earlier request computed
    (kairyu tests/unit/test_engine_hf_parity.py:115-133): the tokens are those of the plain
    implementation (fp32), or agree with it as far as generation without sharing does (bf16);
    with so few pages that unread shared pages are taken back and the stem is computed again."""
    from kairyu_b200 import LLM, SamplingParams, TokensPrompt

    config, seed, page_size = TINY[name]
    stem = prompts_of(config, [5 * page_size + 3], seed=130)[0]
    prompts = [stem + tail for tail in prompts_of(config, [1, 12, 2 * page_size, 7, 30, 3], seed=131)]
    other = prompts_of(config, [9 * page_size], seed=132)  # pushes the stem's pages out in between
    params = SamplingParams(temperature=0.0, max_tokens=16)
    llm = LLM.from_random(
        config, seed=seed, dtype=dtype, page_size=page_size, num_pages=22, max_num_seqs=3,
        max_num_batched_tokens=40, enable_prefix_caching=True, pipeline_depth=depth,
    )
    llm.engine.runner.check_tables = True
    weights = engine_weights(llm)
    rounds = []
    for workload in (prompts, other, prompts[::-1]):
        outputs = llm.generate([TokensPrompt(tuple(p)) for p in workload], params)
        rounds.append(outputs)
        llm.engine.cache.check()
        assert llm.engine.cache.live_requests == 0
    assert llm.engine.scheduler.counters["cached_prompt_tokens"] >= 5 * page_size * 4
    assert llm.engine.cache.prefix.counters["evicted_pages"] > 0
    assert max(o.metrics["num_cached_tokens"] for o in rounds[0]) >= 5 * page_size
    agree = total = 0
    for workload, outputs in zip((prompts, other, prompts[::-1]), rounds):
        for prompt, output in zip(workload, outputs):
            expected = plain_generate(config, weights, prompt, 16)
            got = list(output.outputs[0].token_ids)
            assert len(got) == 16
            if dtype == "float32":
                assert got == expected
            for a, b in zip(got, expected):
                total += 1
                if a != b:
                    break
                agree += 1
    if dtype == "bfloat16":
        assert agree / total > 0.9


@pytest.mark.parametrize("dtype,depth", [("float32", 1), ("float32", 2), ("bfloat16", 2)])
def test_logprobs_of_generated_tokens(dtype, depth):
    """``logprobs=k``: per generated token the chosen token's log-probability and the k largest, from
    the raw logits (kairyu/engine/core/sampler.py:1423-1437); compared with the plain model's
    log-softmax (fp32), or with its bf16 bound on logits (bf16), for greedy, sampled and penalised rows."""
    from kairyu_b200 import LLM, SamplingParams, TokensPrompt

    config, seed, page_size = TINY["wide"]
    llm = LLM.from_random(config, seed=seed, dtype=dtype, page_size=page_size, num_pages=64, max_num_batched_tokens=24, pipeline_depth=depth)
    weights = engine_weights(llm)
    prompts = prompts_of(config, [9, 30, 4, 17], seed=140)
    params = [
        SamplingParams(temperature=0.0, max_tokens=6, logprobs=3),
        SamplingParams(temperature=0.9, top_k=12, seed=5, max_tokens=5, logprobs=0),
        SamplingParams(temperature=0.0, max_tokens=4),
        SamplingParams(temperature=0.0, max_tokens=7, logprobs=5, repetition_penalty=1.4, presence_penalty=0.3),
    ]
    outputs = llm.generate([TokensPrompt(tuple(p)) for p in prompts], params)
    assert outputs[2].outputs[0].logprobs is None and outputs[2].outputs[0].cumulative_logprob is None
    tolerance = 2e-4 if dtype == "float32" else 5e-2
    for index in (0, 1, 3):
        completion, k = outputs[index].outputs[0], params[index].logprobs
        tokens = list(prompts[index])
        total = 0.0
        assert len(completion.logprobs) == len(completion.token_ids)
        for token, entry in zip(completion.token_ids, completion.logprobs):
            logits = plain_model.forward_logits(config, weights, tokens)[-1]
            expected, chosen = plain_model.logprob_entry(logits, token, k)
            assert list(entry)[0] == token and len(entry) in (max(k, 1), k + 1)
            assert abs(entry[token] - chosen) < tolerance
            if dtype == "float32":
                assert set(entry) == set(expected)
            logp = torch.log_softmax(logits.float(), dim=-1)
            for key, value in entry.items():
                assert abs(value - float(logp[key])) < tolerance
            total += entry[token]
            tokens.append(token)
        assert completion.cumulative_logprob == pytest.approx(total, abs=1e-4)


@pytest.mark.parametrize("name", ["llama", "wide"])
def test_decode_graphs_under_preemption_and_ids_used_again(name):
    """Long generations, a large token budget and few pages: prompts that wait one token short of
    their end are preempted by decoding requests that need their pages, come back, and decode in
    rows of graphs that showed other pages before; then the same ids are submitted again.  fp32 greedy tokens are the plain model's in
    both decode modes, and every kind of event is counted."""
    from kairyu_b200 import SamplingParams
    from kairyu_b200.config.engine_config import EngineConfig
    from kairyu_b200.engine.engine import Engine

    config, seed, page_size = TINY[name]
    prompts = prompts_of(config, [29, 31, 27, 30, 26], seed=150)
    new_tokens = [40, 55, 48, 36, 60]
    results = {}
    for mode in ("eager", "cuda_graph"):
        options = EngineConfig.from_kwargs(
            dtype="float32", seed=seed, page_size=page_size, num_pages=1 + 192 // page_size, max_num_seqs=4,
            max_num_batched_tokens=256, decode_mode=mode,
        )
        engine = Engine.from_random(config, seed, options)
        tokens = []
        for turn in range(2):  # the second turn uses the ids of the first again
            for index, prompt in enumerate(prompts):
                engine.add_request(f"request-{index}", prompt, SamplingParams(temperature=0.0, max_tokens=new_tokens[index]))
            finished = engine.run_to_completion()
            tokens.append([finished[f"request-{index}"].output_token_ids for index in range(len(prompts))])
            engine.cache.check()
            assert engine.cache.live_requests == 0
        engine.runner.check_errors()
        assert engine.scheduler.counters["preemptions"] > 0
        if mode == "cuda_graph":
            assert engine.runner.counters["graph_replays"] > 50
        results[mode] = tokens
        weights = engine_weights(type("Holder", (), {"engine": engine}))
    expected = [tuple(plain_generate(config, weights, prompt, count)) for prompt, count in zip(prompts, new_tokens)]
    for mode, turns in results.items():
        for turn in turns:
            assert turn == expected, mode


def test_warm_up_captures_every_decode_graph_ahead():
    """After ``warm_up`` a workload of every batch size up to the limit captures nothing more, and its
    fp32 greedy tokens are the plain model's."""
    from kairyu_b200 import SamplingParams
    from kairyu_b200.config.engine_config import EngineConfig
    from kairyu_b200.engine.engine import Engine

    config, seed, page_size = TINY["llama"]
    options = EngineConfig.from_kwargs(
        dtype="float32", seed=seed, page_size=page_size, num_pages=1 + 2048 // page_size, max_num_seqs=6,
        max_num_batched_tokens=256, decode_mode="cuda_graph",
    )
    engine = Engine.from_random(config, seed, options)
    captured = engine.warm_up(max_batch=6)
    # batch buckets 1, 2, 4 and 6 (the engine's limit); one context bucket (the model's 256 positions)
    assert captured == 4 and engine.runner.counters["graph_captures"] == 4
    assert engine.warm_up(max_batch=6) == 0
    prompts = prompts_of(config, [40, 3, 77, 150, 9, 61], seed=160)
    new_tokens = [30, 12, 40, 100, 25, 33]
    for index, prompt in enumerate(prompts):
        engine.add_request(f"request-{index}", prompt, SamplingParams(temperature=0.0, max_tokens=new_tokens[index]))
    finished = engine.run_to_completion()
    engine.runner.check_errors()
    assert engine.runner.counters["graph_captures"] == 4
    assert engine.runner.counters["graph_replays"] > 50
    weights = engine_weights(type("Holder", (), {"engine": engine}))
    for index, (prompt, count) in enumerate(zip(prompts, new_tokens)):
        assert finished[f"request-{index}"].output_token_ids == tuple(plain_generate(config, weights, prompt, count))
