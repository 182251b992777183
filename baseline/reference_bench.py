"""The reference arm of ``bench.py``: ytworks/kairyu, unmodified, measured through its own
public entry point on the same workload.

The package under ``baseline/_ref/kairyu`` is driven the way its users drive it:
``LLM(model=folder, backend=KairyuBackend(model_path=folder, ...)).generate(TokensPrompt...,
SamplingParams...)`` (kairyu/entrypoints/llm.py:70-85, 300-314; the backend assembles the engine
with ``build_engine_loop``, kairyu/engine/kairyu_backend.py:467, which loads the folder with
``load_model``, kairyu/models/loader.py:106).  The model folder is written here with torch and
safetensors alone: ``config.json`` as given, a ``tokenizer.json`` of one word per token id, every matrix ~N(0, 0.02) from a seeded generator,
norm weights 1 + N(0, 0.1), in bfloat16.  Nothing of this repository's engine is imported.

Decode tokens a second come from the difference between a generation of 1 + K tokens and a
generation of 1 token for the same prompts, so that the prompt's cost drops out: once between
CUDA events recorded around the two calls (``value``), once by the wall clock (``e2e``).
"""

from __future__ import annotations

import json
import os
import shutil
import sys
import tempfile
import time
from typing import Any, Mapping


def _write_model_folder(config: Mapping[str, Any], seed: int, folder: str) -> None:
    """config.json + model.safetensors of random bfloat16 weights, tensor names as the
    architecture's checkpoints have them (kairyu/models/llama.py, kairyu/models/loader.py:200-265)."""
    import torch
    from safetensors.torch import save_file

    hidden, inter, vocab = config["hidden_size"], config["intermediate_size"], config["vocab_size"]
    heads, kv_heads = config["num_attention_heads"], config.get("num_key_value_heads", config["num_attention_heads"])
    head_dim = config.get("head_dim") or hidden // heads
    qk_norm = config["architectures"][0] == "Qwen3ForCausalLM"
    generator = torch.Generator(device="cuda").manual_seed(int(seed))
    tensors: dict[str, Any] = {}

    def matrix(name: str, rows: int, cols: int) -> None:
        values = torch.randn((rows, cols), generator=generator, dtype=torch.float32, device="cuda") * 0.02
        tensors[name] = values.to(torch.bfloat16).cpu()

    def norm(name: str, size: int) -> None:
        values = 1.0 + 0.1 * torch.randn((size,), generator=generator, dtype=torch.float32, device="cuda")
        tensors[name] = values.to(torch.bfloat16).cpu()

    matrix("model.embed_tokens.weight", vocab, hidden)
    for layer in range(config["num_hidden_layers"]):
        p = f"model.layers.{layer}"
        matrix(f"{p}.self_attn.q_proj.weight", heads * head_dim, hidden)
        matrix(f"{p}.self_attn.k_proj.weight", kv_heads * head_dim, hidden)
        matrix(f"{p}.self_attn.v_proj.weight", kv_heads * head_dim, hidden)
        matrix(f"{p}.self_attn.o_proj.weight", hidden, heads * head_dim)
        if qk_norm:
            norm(f"{p}.self_attn.q_norm.weight", head_dim)
            norm(f"{p}.self_attn.k_norm.weight", head_dim)
        matrix(f"{p}.mlp.gate_proj.weight", inter, hidden)
        matrix(f"{p}.mlp.up_proj.weight", inter, hidden)
        matrix(f"{p}.mlp.down_proj.weight", hidden, inter)
        norm(f"{p}.input_layernorm.weight", hidden)
        norm(f"{p}.post_attention_layernorm.weight", hidden)
    norm("model.norm.weight", hidden)
    if not config.get("tie_word_embeddings", False):
        matrix("lm_head.weight", vocab, hidden)
    os.makedirs(folder, exist_ok=True)
    written = dict(config)
    written["torch_dtype"] = "bfloat16"
    with open(os.path.join(folder, "config.json"), "w") as handle:
        json.dump(written, handle, indent=2, sort_keys=True)
    save_file(tensors, os.path.join(folder, "model.safetensors"), metadata={"format": "pt"})
    # The reference wants a tokenizer beside the weights (it detokenises what it generates): one
    # word per token id, so that every id of the vocabulary is known to it.
    from tokenizers import Tokenizer, models, pre_tokenizers

    tokenizer = Tokenizer(models.WordLevel({f"t{index}": index for index in range(vocab)}, unk_token="t0"))
    tokenizer.pre_tokenizer = pre_tokenizers.Whitespace()
    tokenizer.save(os.path.join(folder, "tokenizer.json"))


def _random_tokens(count: int, vocab: int, seed: int) -> tuple[int, ...]:
    import torch

    generator = torch.Generator().manual_seed(seed)
    return tuple(torch.randint(0, vocab, (count,), generator=generator).tolist())


def run_reference(args: Any, model: Mapping[str, Any], workload: Mapping[str, Any]) -> dict:
    """One JSON line's worth of numbers for the reference on ``model`` (a config.json dict) and
    ``workload`` (prompt_len, gen_len, page_size, context_len, seed, ref_root, layers)."""
    import torch

    if not torch.cuda.is_available():
        return {"impl": "reference", "unavailable": "no CUDA device: the reference arm measures on a GPU"}
    ref_root = workload["ref_root"]
    if ref_root not in sys.path:
        sys.path.insert(0, ref_root)
    from kairyu.engine.kairyu_backend import KairyuBackend  # the reference
    from kairyu.engine.prompt import TokensPrompt
    from kairyu.entrypoints.llm import LLM
    from kairyu.sampling_params import SamplingParams

    config = dict(model)
    config["num_hidden_layers"] = workload["layers"]
    batch, steps = args.batch, min(args.steps, 64)
    prompt_len, gen_len, page_size = workload["prompt_len"], workload["gen_len"], workload["page_size"]
    vocab = config["vocab_size"]
    scratch = tempfile.mkdtemp(prefix="kairyu-reference-")
    try:
        _write_model_folder(config, workload["seed"], scratch)
        torch.cuda.empty_cache()
        max_batch = max(batch, 1 if args.no_points else 64)
        per_request = -(-(prompt_len + gen_len + 64) // page_size)
        options = dict(
            model_path=scratch, num_pages=max_batch * per_request + 1, page_size=page_size,
            max_num_batched_tokens=max(2048, 8 * prompt_len), max_num_seqs=max_batch, max_model_len=workload["context_len"],
            max_num_partial_prefills=1,
        )
        notes = []
        backend = None
        # its own fastest documented settings first; what it refuses is named and left out
        for extra in (dict(pipeline_depth=2, decode_mode="cuda_graph"), dict(decode_mode="cuda_graph"), dict()):
            try:
                backend = KairyuBackend(**options, **extra)
                notes.append("options: " + (", ".join(f"{k}={v}" for k, v in extra.items()) or "defaults"))
                break
            except Exception as error:  # an option this build of the reference does not take on this box
                notes.append(f"refused {sorted(extra)}: {type(error).__name__}: {str(error)[:120]}")
        if backend is None:
            return {"impl": "reference", "unavailable": "KairyuBackend could not be built: " + " | ".join(notes)[:300]}
        llm = LLM(model=scratch, backend=backend)
        attention = getattr(backend, "attention_backend_decision", None)

        def run(prompts, max_tokens: int) -> tuple[float, float]:
            params = SamplingParams(temperature=0.0, max_tokens=max_tokens, ignore_eos=True)
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            begin = time.perf_counter()
            start.record()
            outputs = llm.generate(list(prompts), params)
            stop.record()
            torch.cuda.synchronize()
            seconds = time.perf_counter() - begin
            if any(len(output.outputs[0].token_ids) != max_tokens for output in outputs):
                raise RuntimeError("the reference returned fewer tokens than asked for")
            return start.elapsed_time(stop) / 1e3, seconds

        def decode_rate(count: int, k: int) -> tuple[float, float, float]:
            prompts = [TokensPrompt(prompt_token_ids=_random_tokens(prompt_len, vocab, 200 + i)) for i in range(count)]
            run(prompts, 2)  # warm: graphs, libraries
            short = min(run(prompts, 1) for _ in range(2))
            long = min(run(prompts, 1 + k) for _ in range(2))
            device_s = max(long[0] - short[0], 1e-9)
            wall_s = max(long[1] - short[1], 1e-9)
            return count * k / device_s, count * k / wall_s, device_s / k * 1e3

        # warm-up is inside decode_rate: one untimed generation, then two timed of each length, the better kept
        sampler = workload["clock_sampler"]() if workload.get("clock_sampler") else None
        if sampler is not None:
            sampler.start()
        value, e2e, ms_per_step = decode_rate(batch, steps)
        clocks = sampler.stop() if sampler is not None else None
        line = {
            "metric": f"decode tok/s @bs{batch} ({workload['name']}, {prompt_len}-token prompts)",
            "value": value, "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": max(args.warmup, 3),
            "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic: seeded random token ids, seeded random weights (no checkpoint, no dataset)",
            "impl": "reference",
            "config": {
                "model": workload["name"], "layers": config["num_hidden_layers"], "layers_full": workload["layers_full"],
                "hidden": config["hidden_size"], "heads": config["num_attention_heads"], "kv_heads": config["num_key_value_heads"],
                "head_dim": config["head_dim"], "intermediate": config["intermediate_size"], "vocab": vocab,
                "global_batch": batch, "seq_len": prompt_len, "gen_len": gen_len, "context_len": workload["context_len"],
                "page_size": page_size, "parallelism": "single_gpu",
                "l2": "inputs>L2 (weights and cache exceed the 126 MB L2)",
                "entry": "kairyu LLM.generate over KairyuBackend", "notes": " | ".join(notes)[:200],
                "attention": str(attention)[:80] if attention is not None else "not reported",
            },
            "e2e": {"value": e2e, "unit": "tokens/s", "h2d_bytes_per_step": None, "d2h_bytes_per_step": None},
            "clocks": clocks,
            "gpu_launches": 0,  # none of this repository's kernels run in this arm
            "timing": "difference of a (1+K)-token and a 1-token generation of the same prompts; value between CUDA events, e2e by wall clock",
        }
        if not args.no_points:
            points = {}
            try:
                # a new prompt every time: the reference keeps the pages of a prompt it has seen
                # (its radix cache) and would not compute a repeated one again
                def fresh(index: int):
                    return [TokensPrompt(prompt_token_ids=_random_tokens(2048, vocab, 700 + index))]

                run(fresh(0), 1)
                seconds = min(run(fresh(1 + index), 1)[0] for index in range(3))
                line["prefill"] = {"value": 2048 / seconds, "tokens": 2048, "ms": seconds * 1e3}
                for count, key in ((1, "decode_b1"), (64, "decode_b64")):
                    points[key] = decode_rate(count, min(steps, 32))[0]
            except Exception as error:
                points["error"] = f"{type(error).__name__}: {str(error)[:160]}"
            line["points"] = points
        if getattr(args, "mixed", False):
            # The mixed workload of bench.py's own arm: 32 requests, prompt lengths uniform in [128, 4096] from
            # the same seeded draw, a token budget of 512 + 32 so that prompts are cut into portions that share
            # steps with the decodes of the others, 128 generated tokens each.  The warm-up prompts are others
            # than the timed ones: the reference keeps the pages of prompts it has seen.
            del llm, backend
            torch.cuda.empty_cache()
            generator = torch.Generator().manual_seed(int(workload["seed"]))
            lengths = torch.randint(128, 4097, (32,), generator=generator).tolist()
            mixed = KairyuBackend(
                model_path=scratch, num_pages=sum(-(-(n + 128 + 16) // page_size) for n in lengths) + 1, page_size=page_size,
                max_num_batched_tokens=512 + 32, max_num_seqs=32, max_model_len=workload["context_len"], max_num_partial_prefills=1,
                pipeline_depth=2, decode_mode="cuda_graph",
            )
            llm = LLM(model=scratch, backend=mixed)
            prompts = [TokensPrompt(prompt_token_ids=_random_tokens(n, vocab, 300 + i)) for i, n in enumerate(lengths)]
            warm = [TokensPrompt(prompt_token_ids=_random_tokens(600, vocab, 350 + i)) for i in range(4)]
            llm.generate(warm, SamplingParams(temperature=0.0, max_tokens=4, ignore_eos=True))
            torch.cuda.synchronize()
            begin = time.perf_counter()
            outputs = llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=128, ignore_eos=True))
            torch.cuda.synchronize()
            seconds = time.perf_counter() - begin
            generated = sum(len(output.outputs[0].token_ids) for output in outputs)
            line.setdefault("points", {}).update({
                "mixed_b32_total_tok_s": (sum(lengths) + generated) / seconds,
                "mixed_b32_generated_tok_s": generated / seconds,
                "mixed_b32_seconds": seconds,
            })
        return line
    finally:
        shutil.rmtree(scratch, ignore_errors=True)
