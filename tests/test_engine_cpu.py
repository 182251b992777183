"""The engine loop (scheduler + step function + sampler + entry point) on the
CPU with the kernels replaced by their torch statements: host-side decisions
only.  The same workloads run on the GPU with the real kernels."""

import pytest

import plain_model
import torch_kernels
from test_engine_gpu import engine_weights, plain_generate, prompts_of
from tiny_configs import TINY

from kairyu_b200 import LLM, SamplingParams, TokensPrompt


@pytest.fixture(autouse=True)
def cpu_kernels(monkeypatch):
    torch_kernels.install(monkeypatch)


def make_llm(name, **kwargs):
    config, seed, page_size = TINY[name]
    kwargs.setdefault("page_size", page_size)
    return LLM.from_random(config, seed=seed, dtype="float32", device="cpu", **kwargs), config


def test_greedy_generation_matches_plain():
    llm, config = make_llm("llama", num_pages=32)
    weights = engine_weights(llm)
    prompts = prompts_of(config, [1, 7, 33, 50], seed=100)
    outputs = llm.generate([TokensPrompt(tuple(p)) for p in prompts], SamplingParams(temperature=0.0, max_tokens=8))
    for prompt, output in zip(prompts, outputs):
        assert list(output.outputs[0].token_ids) == plain_generate(config, weights, prompt, 8)
        assert output.outputs[0].finish_reason == "length"
        assert output.finished


def test_sampled_generation_matches_plain_and_repeats():
    llm, config = make_llm("qwen3", num_pages=64, prefill_chunk_size=24)
    weights = engine_weights(llm)
    prompts = prompts_of(config, [3, 50, 27], seed=101)
    params = [SamplingParams(temperature=0.8, top_p=0.9, seed=50 + i, max_tokens=6) for i in range(3)]
    outputs = llm.generate([TokensPrompt(tuple(p)) for p in prompts], params)
    for index, (prompt, output) in enumerate(zip(prompts, outputs)):
        expected = plain_generate(config, weights, prompt, 6, dict(temperature=0.8, top_p=0.9), request_seed=50 + index)
        assert list(output.outputs[0].token_ids) == expected
    again = llm.generate([TokensPrompt(tuple(p)) for p in prompts], params)
    assert [o.outputs[0].token_ids for o in again] == [o.outputs[0].token_ids for o in outputs]


def test_small_budget_few_pages_preempts_and_still_matches():
    llm, config = make_llm("odd", num_pages=9, max_num_batched_tokens=7, max_num_seqs=4)
    weights = engine_weights(llm)
    prompts = prompts_of(config, [30, 14, 46, 31, 15, 47], seed=102)
    outputs = llm.generate([TokensPrompt(tuple(p)) for p in prompts], SamplingParams(temperature=0.0, max_tokens=20))
    assert llm.engine.scheduler.counters["preemptions"] > 0
    llm.engine.cache.check()
    assert llm.engine.cache.live_requests == 0
    for prompt, output in zip(prompts, outputs):
        assert list(output.outputs[0].token_ids) == plain_generate(config, weights, prompt, 20)


def test_n_completions_and_param_lists():
    llm, config = make_llm("llama", num_pages=32)
    prompt = prompts_of(config, [6], seed=105)[0]
    out = llm.generate(TokensPrompt(tuple(prompt)), SamplingParams(temperature=1.0, seed=3, n=3, max_tokens=5))[0]
    assert len(out.outputs) == 3 and [c.index for c in out.outputs] == [0, 1, 2]
    assert len({c.token_ids for c in out.outputs}) > 1
    with pytest.raises(ValueError):
        llm.generate([TokensPrompt((1,)), TokensPrompt((2,))], [SamplingParams()])
    with pytest.raises(ValueError):
        llm.generate("text needs a tokenizer")
    with pytest.raises(ValueError):
        llm.generate(TokensPrompt((1,)), SamplingParams(prompt_logprobs=1))
    with pytest.raises(ValueError):
        llm.generate(TokensPrompt((1,) * 10), SamplingParams(max_tokens=100000))
    # vLLM-style dict prompts
    out = llm.generate({"prompt_token_ids": prompt}, SamplingParams(temperature=0.0, max_tokens=2))[0]
    assert len(out.outputs[0].token_ids) == 2


def test_llm_rejects_unknown_options_and_parallel_sizes():
    config, seed, _ = TINY["llama"]
    with pytest.raises(TypeError):
        LLM.from_random(config, seed=0, device="cpu", not_an_option=1)
    with pytest.raises(ValueError):
        LLM("/nonexistent", tensor_parallel_size=2)


# ------------------------------------------------------------------ schedule-ahead (pipeline_depth=2)


def test_pipeline_depth_two_gives_the_same_tokens_and_runs_ahead():
    prompts = None
    results = {}
    for depth in (1, 2):
        llm, config = make_llm("llama", num_pages=48, pipeline_depth=depth)
        prompts = prompts or prompts_of(config, [5, 21, 40, 9], seed=110)
        params = [SamplingParams(temperature=0.0, max_tokens=m) for m in (12, 3, 1, 7)]
        outputs = llm.generate([TokensPrompt(tuple(p)) for p in prompts], params)
        results[depth] = [(o.outputs[0].token_ids, o.outputs[0].finish_reason) for o in outputs]
        llm.engine.cache.check()
        assert llm.engine.cache.live_requests == 0 and not llm.engine._pending
        assert (llm.engine.runner.counters["future_tokens"] > 0) == (depth == 2)
        if depth == 2:
            weights = engine_weights(llm)
            for prompt, output, p in zip(prompts, outputs, params):
                assert list(output.outputs[0].token_ids) == plain_generate(config, weights, prompt, p.max_tokens)
    assert results[1] == results[2]


def test_pipeline_depth_two_drops_the_token_sampled_after_a_stop():
    llm, config = make_llm("qwen3", num_pages=64, pipeline_depth=2)
    weights = engine_weights(llm)
    prompts = prompts_of(config, [17, 30], seed=111)
    free = [plain_generate(config, weights, p, 10) for p in prompts]
    # stop request 0 at its 4th token and request 1 at its 7th: the step after each stop has
    # already been launched with a row for it
    stops = [free[0][3], free[1][6]]
    params = [SamplingParams(temperature=0.0, max_tokens=10, stop_token_ids=[stops[i]]) for i in range(2)]
    outputs = llm.generate([TokensPrompt(tuple(p)) for p in prompts], params)
    for i, output in enumerate(outputs):
        expected = free[i][: free[i].index(stops[i]) + 1]
        assert list(output.outputs[0].token_ids) == expected
        assert output.outputs[0].finish_reason == "stop" and output.outputs[0].stop_reason == stops[i]
    llm.engine.cache.check()
    assert llm.engine.cache.live_requests == 0


def test_pipeline_depth_two_under_page_pressure_and_with_sampling():
    llm, config = make_llm("odd", num_pages=9, max_num_batched_tokens=7, max_num_seqs=4, pipeline_depth=2)
    weights = engine_weights(llm)
    prompts = prompts_of(config, [30, 14, 46, 31, 15, 47], seed=102)
    outputs = llm.generate([TokensPrompt(tuple(p)) for p in prompts], SamplingParams(temperature=0.0, max_tokens=20))
    assert llm.engine.scheduler.counters["preemptions"] > 0
    llm.engine.cache.check()
    assert llm.engine.cache.live_requests == 0
    for prompt, output in zip(prompts, outputs):
        assert list(output.outputs[0].token_ids) == plain_generate(config, weights, prompt, 20)
    llm2, config2 = make_llm("qwen3", num_pages=64, pipeline_depth=2)
    weights2 = engine_weights(llm2)
    prompts2 = prompts_of(config2, [3, 50, 27], seed=101)
    params = [SamplingParams(temperature=0.8, top_p=0.9, seed=50 + i, max_tokens=6) for i in range(3)]
    outputs2 = llm2.generate([TokensPrompt(tuple(p)) for p in prompts2], params)
    for index, (prompt, output) in enumerate(zip(prompts2, outputs2)):
        expected = plain_generate(config2, weights2, prompt, 6, dict(temperature=0.8, top_p=0.9), request_seed=50 + index)
        assert list(output.outputs[0].token_ids) == expected


def test_pipeline_depth_two_falls_back_to_one_for_penalties():
    llm, config = make_llm("llama", num_pages=32, pipeline_depth=2)
    prompt = prompts_of(config, [12], seed=112)[0]
    one, _ = make_llm("llama", num_pages=32)
    params = SamplingParams(temperature=0.0, max_tokens=8, repetition_penalty=1.3, presence_penalty=0.4)
    a = llm.generate(TokensPrompt(tuple(prompt)), params)[0].outputs[0].token_ids
    b = one.generate(TokensPrompt(tuple(prompt)), params)[0].outputs[0].token_ids
    assert a == b


@pytest.mark.parametrize("seed", [0, 1, 2, 3, 7, 13, 21])
def test_pipeline_depth_two_equals_depth_one_on_random_workloads(seed):
    """Random prompt lengths, budgets, stop tokens and token limits on a pool so small that requests wait
    and are preempted: schedule-ahead must not change a token or a finish reason."""
    import random

    rng = random.Random(seed)
    count = rng.randint(3, 7)
    lengths = [rng.randint(1, 60) for _ in range(count)]
    limits = [rng.randint(1, 14) for _ in range(count)]
    options = dict(num_pages=rng.randint(10, 16), max_num_batched_tokens=rng.choice([5, 16, 64]), max_num_seqs=rng.choice([2, 4, 8]))
    results = {}
    stops = None
    for depth in (1, 2):
        llm, config = make_llm("llama", pipeline_depth=depth, **options)
        prompts = prompts_of(config, lengths, seed=200 + seed)
        if stops is None:  # tokens the free run produces, so that some requests stop early
            free = llm.generate([TokensPrompt(tuple(p)) for p in prompts], [SamplingParams(temperature=0.0, max_tokens=m) for m in limits])
            stops = [o.outputs[0].token_ids[len(o.outputs[0].token_ids) // 2] if i % 2 == 0 else None for i, o in enumerate(free)]
        params = [
            SamplingParams(temperature=0.0 if i % 3 else 0.7, seed=5 + i, max_tokens=limits[i], stop_token_ids=[stops[i]] if stops[i] is not None else [])
            for i in range(count)
        ]
        outputs = llm.generate([TokensPrompt(tuple(p)) for p in prompts], params)
        results[depth] = [(o.outputs[0].token_ids, o.outputs[0].finish_reason, o.outputs[0].stop_reason) for o in outputs]
        llm.engine.cache.check()
        assert llm.engine.cache.live_requests == 0 and not llm.engine._pending
    assert results[1] == results[2]
    assert any(reason == "stop" for _, reason, _ in results[2])


def check_logprobs(config, weights, prompt, completion, k):
    """Every generated token's entry against the plain log-softmax of the plain model's logits."""
    tokens = list(prompt)
    total = 0.0
    assert len(completion.logprobs) == len(completion.token_ids)
    for token, entry in zip(completion.token_ids, completion.logprobs):
        logits = plain_model.forward_logits(config, weights, tokens)[-1]
        expected, chosen = plain_model.logprob_entry(logits, token, k)
        assert set(entry) == set(expected) and len(entry) in (max(k, 1), k + 1)
        assert list(entry)[0] == token  # the chosen token comes first
        for key, value in expected.items():
            assert entry[key] == pytest.approx(value, abs=2e-4)
        total += chosen
        tokens.append(token)
    assert completion.cumulative_logprob == pytest.approx(total, abs=2e-3)


@pytest.mark.parametrize("depth", [1, 2])
def test_logprobs_of_generated_tokens_match_plain(depth):
    llm, config = make_llm("qwen3", num_pages=64, max_num_batched_tokens=24, pipeline_depth=depth)
    weights = engine_weights(llm)
    prompts = prompts_of(config, [9, 30, 4, 17], seed=140)
    params = [
        SamplingParams(temperature=0.0, max_tokens=6, logprobs=3),
        SamplingParams(temperature=0.9, top_k=12, seed=5, max_tokens=5, logprobs=0),
        SamplingParams(temperature=0.0, max_tokens=4),  # asks for none
        # penalties edit the logits; the report is of the raw ones
        SamplingParams(temperature=0.0, max_tokens=7, logprobs=5, repetition_penalty=1.4, presence_penalty=0.3),
    ]
    outputs = llm.generate([TokensPrompt(tuple(p)) for p in prompts], params)
    assert outputs[2].outputs[0].logprobs is None and outputs[2].outputs[0].cumulative_logprob is None
    for index in (0, 1, 3):
        check_logprobs(config, weights, prompts[index], outputs[index].outputs[0], params[index].logprobs)
    assert list(outputs[0].outputs[0].token_ids) == plain_generate(config, weights, prompts[0], 6)
    assert not llm.engine._logprobs


@pytest.mark.parametrize("depth", [1, 2])
def test_abort_in_the_middle_leaves_the_others_alone(depth):
    """A request aborted while its step is in flight: its pages and slot go back, its late token is
    dropped, the other requests' tokens are those of an undisturbed run."""
    from kairyu_b200.sampling.params import SamplingParams as Params

    llm, config = make_llm("llama", num_pages=40, max_num_batched_tokens=16, pipeline_depth=depth)
    prompts = prompts_of(config, [20, 9, 33], seed=150)
    params = Params(temperature=0.0, max_tokens=12, logprobs=1)
    undisturbed = llm.generate([TokensPrompt(tuple(p)) for p in prompts], params)
    engine = llm.engine
    for index, prompt in enumerate(prompts):
        engine.add_request(f"r{index}", tuple(prompt), params)
    for _ in range(4):
        engine.step()
    engine.abort("r1")
    engine.abort("r1")  # already gone
    engine.abort("nobody")
    finished = engine.run_to_completion()
    assert finished["r1"].finish_reason == "abort" and len(finished["r1"].output_token_ids) < 12
    for index in (0, 2):
        assert finished[f"r{index}"].output_token_ids == undisturbed[index].outputs[0].token_ids
        assert len(finished[f"r{index}"].logprobs) == 12
    engine.cache.check()
    assert engine.cache.live_requests == 0 and not engine._pending and not engine._logprobs


def test_priorities_through_the_entry_point():
    llm, config = make_llm("llama", num_pages=40, max_num_batched_tokens=8, max_num_partial_prefills=1, priority_scheduling=True)
    prompts = prompts_of(config, [8, 8, 8], seed=160)
    params = SamplingParams(temperature=0.0, max_tokens=2)
    started = []
    real = llm.engine.scheduler._admit

    def watch(request_id, *args, **kwargs):
        used = real(request_id, *args, **kwargs)
        if used is not None:
            started.append(request_id.rsplit("-", 1)[1])
        return used

    llm.engine.scheduler._admit = watch
    outputs = llm.generate([TokensPrompt(tuple(p)) for p in prompts], params, priority=[2, 0, 1])
    assert started == ["1", "2", "0"]
    assert [len(o.outputs[0].token_ids) for o in outputs] == [2, 2, 2]
    plain, _ = make_llm("llama", num_pages=40)
    with pytest.raises(ValueError, match="priority_scheduling"):
        plain.generate([TokensPrompt(tuple(p)) for p in prompts], params, priority=[2, 0, 1])
    with pytest.raises(ValueError, match="priority length"):
        llm.generate([TokensPrompt(tuple(p)) for p in prompts], params, priority=[1])
