"""``LLM(model).generate(prompts, SamplingParams)``: the offline entry point, in
the reference's vLLM-compatible shape (kairyu/entrypoints/llm.py:70-85, 300-314).

``model`` is a folder with ``config.json`` and safetensors; the model class is
chosen by ``config.json``.  Text prompts need a ``tokenizer.json`` in the folder
(or in ``tokenizer``); ``TokensPrompt`` works without one.
"""

from __future__ import annotations

import json
import uuid
from collections.abc import Mapping, Sequence
from pathlib import Path
from typing import Any, Optional

from kairyu_b200.config.engine_config import EngineConfig
from kairyu_b200.engine.engine import Engine, FinishedRequest
from kairyu_b200.entrypoints.outputs import CompletionOutput, RequestOutput
from kairyu_b200.entrypoints.prompt import TextPrompt, TokensPrompt, normalize_prompt
from kairyu_b200.sampling.params import SamplingParams


def _eos_token_ids(model_dir: Optional[Path], model_config: Any) -> tuple[int, ...]:
    """generation_config.json wins over config.json (kairyu/models/generation.py:127-174)."""
    if model_dir is not None:
        path = model_dir / "generation_config.json"
        if path.exists():
            value = json.loads(path.read_text()).get("eos_token_id")
            if isinstance(value, int):
                return (value,)
            if isinstance(value, list) and all(isinstance(v, int) for v in value):
                return tuple(value)
    return tuple(getattr(model_config, "eos_token_ids", ()))


class LLM:
    def __init__(
        self,
        model: str,
        tokenizer: str | None = None,
        tensor_parallel_size: int = 1,
        dtype: str = "auto",
        seed: int | None = 0,
        gpu_memory_utilization: float = 0.9,
        enable_prefix_caching: bool | None = None,
        trust_remote_code: bool = False,
        **engine_kwargs: object,
    ) -> None:
        if tensor_parallel_size != 1:
            raise ValueError("this engine runs on one GPU: tensor_parallel_size must be 1")
        self.model = model
        self.seed = seed
        config = EngineConfig.from_kwargs(
            dtype=dtype,
            seed=seed or 0,
            gpu_memory_utilization=gpu_memory_utilization,
            enable_prefix_caching=bool(enable_prefix_caching),
            **engine_kwargs,
        )
        self._model_dir: Optional[Path] = Path(model)
        self.engine = Engine.from_model_dir(model, config)
        self._finish_init(tokenizer)

    @classmethod
    def from_random(cls, model_config: Mapping[str, Any], *, seed: int = 0, dtype: str = "auto", **engine_kwargs: object) -> "LLM":
        """An LLM over seeded random weights of the given config.json dict (no files)."""
        self = cls.__new__(cls)
        self.model = "random"
        self.seed = seed
        config = EngineConfig.from_kwargs(dtype=dtype, seed=seed, **engine_kwargs)
        self._model_dir = None
        self.engine = Engine.from_random(model_config, seed, config)
        self._finish_init(None)
        return self

    @classmethod
    def from_engine(cls, engine: Engine, *, model_dir: str | Path | None = None, tokenizer: str | None = None) -> "LLM":
        """An LLM over an engine that was built elsewhere (its model, cache and options as they are)."""
        self = cls.__new__(cls)
        self.model = str(model_dir) if model_dir is not None else "engine"
        self.seed = engine.config.seed
        self._model_dir = Path(model_dir) if model_dir is not None else None
        self.engine = engine
        self._finish_init(tokenizer)
        return self

    def _finish_init(self, tokenizer: str | None) -> None:
        self.eos_token_ids = _eos_token_ids(self._model_dir, self.engine.model_config)
        self._tokenizer = None
        source = Path(tokenizer) if tokenizer else self._model_dir
        if source is not None:
            path = source / "tokenizer.json" if source.is_dir() else source
            if path.exists():
                from tokenizers import Tokenizer

                self._tokenizer = Tokenizer.from_file(str(path))

    # ------------------------------------------------------------------ helpers
    def _encode(self, prompt: TextPrompt | TokensPrompt) -> tuple[tuple[int, ...], str | None]:
        if isinstance(prompt, TokensPrompt):
            return prompt.prompt_token_ids, prompt.prompt
        if self._tokenizer is None:
            raise ValueError(
                "a text prompt needs a tokenizer.json in the model folder; pass TokensPrompt(prompt_token_ids=...) instead"
            )
        return tuple(self._tokenizer.encode(prompt.prompt).ids), prompt.prompt

    def _decode(self, token_ids: Sequence[int], skip_special_tokens: bool) -> str:
        if self._tokenizer is None:
            return ""
        return self._tokenizer.decode(list(token_ids), skip_special_tokens=skip_special_tokens)

    def _normalize(
        self, prompts: object, sampling_params: SamplingParams | Sequence[SamplingParams] | None
    ) -> tuple[list[TextPrompt | TokensPrompt], list[SamplingParams]]:
        if isinstance(prompts, (str, TextPrompt, TokensPrompt, Mapping)):
            prompt_list = [normalize_prompt(prompts)]
        elif isinstance(prompts, Sequence):
            prompt_list = [normalize_prompt(prompt) for prompt in prompts]
        else:
            raise TypeError("prompts must be a prompt or a sequence of prompts")
        if sampling_params is None:
            params_list = [SamplingParams()] * len(prompt_list)
        elif isinstance(sampling_params, SamplingParams):
            params_list = [sampling_params] * len(prompt_list)
        else:
            params_list = list(sampling_params)
            if len(params_list) != len(prompt_list):
                raise ValueError(
                    f"sampling_params length {len(params_list)} does not match prompts length {len(prompt_list)}"
                )
        return prompt_list, params_list

    # ------------------------------------------------------------------ generate
    def generate(
        self,
        prompts: object,
        sampling_params: SamplingParams | Sequence[SamplingParams] | None = None,
        use_tqdm: bool = True,
        priority: Sequence[int] | None = None,
    ) -> list[RequestOutput]:
        prompt_list, params_list = self._normalize(prompts, sampling_params)
        if priority is not None and len(priority) != len(prompt_list):
            raise ValueError(f"priority length {len(priority)} does not match prompts length {len(prompt_list)}")
        batch = uuid.uuid4().hex[:12]
        submitted: list[tuple[str, list[str], tuple[int, ...], str | None, SamplingParams]] = []
        for index, (prompt, params) in enumerate(zip(prompt_list, params_list)):
            if params.prompt_logprobs is not None:
                raise ValueError("prompt_logprobs reporting is not implemented in this engine (logprobs of generated tokens is)")
            if params.best_of is not None and params.best_of != params.n:
                raise ValueError("best_of different from n is not implemented in this engine")
            if params.stop and self._tokenizer is None:
                raise ValueError("stop strings need a tokenizer; use stop_token_ids")
            token_ids, text = self._encode(prompt)
            request_id = f"{batch}-{index}"
            children: list[str] = []
            for sample in range(params.n):
                child_id = request_id if params.n == 1 else f"{request_id}.{sample}"
                child_params = params
                if params.n > 1 and params.seed is not None:
                    child_params = params.clone(seed=params.seed + sample)
                stop_check = None
                if params.stop:
                    stop_check = self._stop_checker(params)
                self.engine.add_request(
                    child_id, token_ids, child_params, eos_token_ids=self.eos_token_ids, stop_check=stop_check,
                    priority=priority[index] if priority is not None else 0,
                )
                children.append(child_id)
            submitted.append((request_id, children, tuple(token_ids), text, params))
        finished: dict[str, FinishedRequest] = {}
        while self.engine.has_unfinished():
            self.engine.step()
            finished.update(self.engine.take_finished())
        finished.update(self.engine.take_finished())
        results: list[RequestOutput] = []
        for request_id, children, token_ids, text, params in submitted:
            completions = []
            cached = 0
            for sample, child_id in enumerate(children):
                record = finished[child_id]
                cached = max(cached, record.num_cached_tokens)
                output_text = self._decode(record.output_token_ids, params.skip_special_tokens)
                if isinstance(record.stop_reason, str) and record.stop_reason in output_text:
                    output_text = output_text[: output_text.index(record.stop_reason)]
                completions.append(
                    CompletionOutput(
                        index=sample,
                        text=output_text,
                        token_ids=record.output_token_ids,
                        cumulative_logprob=record.cumulative_logprob,
                        logprobs=record.logprobs,
                        finish_reason=record.finish_reason,
                        stop_reason=record.stop_reason,
                    )
                )
            results.append(
                RequestOutput(
                    request_id=request_id,
                    prompt=text,
                    prompt_token_ids=token_ids,
                    outputs=tuple(completions),
                    metrics={"num_cached_tokens": cached},
                )
            )
        return results

    def _stop_checker(self, params: SamplingParams):
        stops = tuple(params.stop)

        def check(output_token_ids: Sequence[int]) -> str | None:
            text = self._decode(output_token_ids, params.skip_special_tokens)
            for stop in stops:
                if stop and stop in text:
                    return stop
            return None

        return check
