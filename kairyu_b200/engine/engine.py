"""The engine: model + cache + step function + scheduler + sampler, and the
synchronous loop ``schedule -> step -> sample -> update`` over them
(kairyu/engine/core/engine_core.py:57-103; assembly as in
kairyu/engine/kairyu_backend.py:467-1179, without tokenizer and server parts).
"""

from __future__ import annotations

import json
from dataclasses import dataclass
from pathlib import Path
from typing import Any, Callable, Mapping, Optional, Sequence

import torch

from kairyu_b200.cache.manager import CacheLayout, CacheManager
from kairyu_b200.cache.storage import CacheStorage
from kairyu_b200.config.engine_config import EngineConfig
from kairyu_b200.engine.runner import ModelRunner, StepEntry
from kairyu_b200.engine.scheduler import EngineRequest, Scheduler
from kairyu_b200.models.decoder import DecoderModel
from kairyu_b200.registry import architecture_of
from kairyu_b200.sampling.params import SamplingParams
from kairyu_b200.sampling.sampler import Sampler, SamplingRow
from kairyu_b200.weights.loading import load_into, read_config
from kairyu_b200.weights.random_init import init_random


@dataclass
class FinishedRequest:
    request_id: str
    prompt_token_ids: tuple[int, ...]
    output_token_ids: tuple[int, ...]
    finish_reason: str
    stop_reason: Optional[int | str] = None


def build_model(config: Mapping[str, Any], *, dtype: str, device: str) -> tuple[DecoderModel, Any]:
    """config.json dict -> (unloaded model, typed config), through the architecture registry."""
    architecture = architecture_of(config)
    model_config = architecture.parse_config(config)
    spec = architecture.build_spec(model_config)
    return DecoderModel(spec, dtype=dtype, device=device), model_config


def load_model(model_dir: str | Path, *, dtype: str, device: str) -> tuple[DecoderModel, Any]:
    """kairyu/models/loader.py:106-265: read config.json, build, bind tensors by name."""
    model, model_config = build_model(read_config(model_dir), dtype=dtype, device=device)
    load_into(model, model_dir)
    return model, model_config


def random_model(config: Mapping[str, Any], seed: int, *, dtype: str, device: str) -> tuple[DecoderModel, Any]:
    model, model_config = build_model(config, dtype=dtype, device=device)
    init_random(model, seed)
    return model, model_config


class Engine:
    def __init__(self, model: DecoderModel, model_config: Any, config: EngineConfig) -> None:
        self.model = model
        self.model_config = model_config
        self.config = config
        self.device = model.device
        max_positions = model.spec.max_position_embeddings
        self.max_model_len = min(config.max_model_len or max_positions, max_positions)
        layout = CacheLayout.from_slot_specs(model.cache_slot_specs())
        self.page_size = config.page_size
        element_size = torch.empty((), dtype=model.dtype).element_size()
        num_pages = config.num_pages
        if num_pages is None:
            num_pages = self._pages_that_fit(layout, element_size)
        self.num_pages = num_pages
        self.cache = CacheManager(
            layout, num_pages=num_pages, page_size=config.page_size, max_requests=config.max_num_seqs
        )
        self.storage = CacheStorage(
            layout,
            num_pages=num_pages,
            page_size=config.page_size,
            max_requests=config.max_num_seqs,
            dtype=model.dtype,
            device=self.device,
        )
        decode_mode = config.decode_mode
        if decode_mode is None:
            decode_mode = "cuda_graph" if str(self.device).startswith("cuda") else "eager"
        self.runner = ModelRunner(
            model,
            self.cache,
            self.storage,
            max_model_len=self.max_model_len,
            decode_mode=decode_mode,
            max_graph_batch=config.cuda_graph_max_batch or min(config.max_num_seqs, 256),
        )
        self.scheduler = Scheduler(
            self.cache,
            max_num_batched_tokens=config.max_num_batched_tokens,
            max_num_seqs=config.max_num_seqs,
            max_num_partial_prefills=config.max_num_partial_prefills,
            max_model_len=self.max_model_len,
            prefill_chunk_size=config.prefill_chunk_size,
        )
        self.sampler = Sampler(model.spec.vocab_size, self.device)
        self._finished: dict[str, FinishedRequest] = {}
        self._stop_checks: dict[str, Callable[[Sequence[int]], Optional[str]]] = {}
        self._steps_since_check = 0

    # ------------------------------------------------------------------ construction
    @classmethod
    def from_model_dir(cls, model_dir: str | Path, config: Optional[EngineConfig] = None) -> "Engine":
        config = config or EngineConfig()
        model, model_config = load_model(model_dir, dtype=config.dtype, device=config.device)
        return cls(model, model_config, config)

    @classmethod
    def from_random(cls, model_config: Mapping[str, Any], seed: int, config: Optional[EngineConfig] = None) -> "Engine":
        config = config or EngineConfig()
        model, parsed = random_model(model_config, seed, dtype=config.dtype, device=config.device)
        return cls(model, parsed, config)

    def _pages_that_fit(self, layout: CacheLayout, element_size: int) -> int:
        per_page = max(CacheStorage.bytes_per_page(layout, self.config.page_size, element_size), 1)
        wanted = self.config.max_num_seqs * -(-self.max_model_len // self.config.page_size) + 1
        if str(self.device).startswith("cuda"):
            free, total = torch.cuda.mem_get_info()
            # keep room for the step's scratch (activations, logits)
            reserve = 2 * 1024**3 + self.config.max_num_batched_tokens * self.model.spec.hidden_size * 64
            usable = int(total * self.config.gpu_memory_utilization) - (total - free) - reserve
            fit = max(usable // per_page, 2)
            return int(min(wanted, fit))
        return int(min(wanted, 4096))

    # ------------------------------------------------------------------ requests
    def add_request(
        self,
        request_id: str,
        prompt_token_ids: Sequence[int],
        params: SamplingParams,
        *,
        eos_token_ids: Sequence[int] = (),
        stop_check: Optional[Callable[[Sequence[int]], Optional[str]]] = None,
    ) -> None:
        prompt = tuple(int(token) for token in prompt_token_ids)
        vocab = self.model.spec.vocab_size
        if any(not 0 <= token < vocab for token in prompt):
            raise ValueError(f"prompt token ids must be in [0, {vocab})")
        max_new = params.max_tokens
        if max_new is None:  # kairyu/engine/engine_loop.py:611-628: the rest of the context
            max_new = self.max_model_len - len(prompt)
            if max_new < 1:
                raise ValueError(f"prompt of {len(prompt)} tokens leaves no room in max_model_len {self.max_model_len}")
        self.scheduler.add_request(
            EngineRequest(
                request_id=request_id,
                prompt_token_ids=prompt,
                max_new_tokens=max_new,
                eos_token_ids=tuple(eos_token_ids),
                stop_token_ids=tuple(params.stop_token_ids),
                min_tokens=params.min_tokens,
                ignore_eos=params.ignore_eos,
                params=params,
            )
        )
        if stop_check is not None:
            self._stop_checks[request_id] = stop_check

    def abort(self, request_id: str) -> None:
        self.scheduler.abort(request_id)
        self._collect(request_id)

    def has_unfinished(self) -> bool:
        return self.scheduler.has_unfinished()

    # ------------------------------------------------------------------ the loop
    def _collect(self, request_id: str, stop_reason: Optional[int | str] = None) -> None:
        state = self.scheduler.state(request_id)
        self._finished[request_id] = FinishedRequest(
            request_id,
            state.request.prompt_token_ids,
            tuple(state.outputs),
            state.finish_reason or "abort",
            stop_reason,
        )
        self._stop_checks.pop(request_id, None)
        self.scheduler.forget(request_id)

    def step(self) -> tuple[str, ...]:
        """One engine step; returns the ids of requests that finished in it."""
        plan = self.scheduler.schedule()
        done: list[str] = list(plan.rejected)
        for request_id in plan.rejected:
            self._collect(request_id)
        if not plan.scheduled:
            if self.scheduler.has_unfinished() and not plan.rejected and not plan.preempted:
                raise RuntimeError("the scheduler made no progress")
            return tuple(done)
        entries: list[StepEntry] = []
        rows: list[SamplingRow] = []
        for chunk in plan.scheduled:
            state = self.scheduler.state(chunk.request_id)
            held = self.cache.get(chunk.request_id).num_tokens if chunk.request_id in self.cache else 0
            if held != chunk.start:
                raise RuntimeError(
                    f"request {chunk.request_id!r}: the cache holds {held} tokens, the plan starts at {chunk.start}"
                )
            tokens = state.tokens(chunk.start, chunk.num_tokens)
            entries.append(StepEntry(chunk.request_id, tokens, want=(chunk.num_tokens - 1,) if chunk.samples else ()))
            if chunk.samples:
                request = state.request
                rows.append(
                    SamplingRow(
                        request_id=chunk.request_id,
                        params=request.params,
                        position=len(state.outputs),
                        prompt_token_ids=request.prompt_token_ids,
                        output_token_ids=state.outputs,
                        eos_token_ids=request.eos_token_ids,
                    )
                )
        logits = self.runner.step(entries)
        if rows:
            token_ids = self.sampler.sample(logits, rows).tolist()  # the step's one device->host read
            # The kernels' error word is sticky: reading it every few steps (and whenever a
            # request ends) reports the same faults with fewer round trips.
            self._steps_since_check += 1
            sampled = {row.request_id: int(token) for row, token in zip(rows, token_ids)}
            finished = list(self.scheduler.update(sampled))
            if finished or self._steps_since_check >= 16:
                self._steps_since_check = 0
                self.runner.check_errors()
            for request_id in finished:
                state = self.scheduler.state(request_id)
                last = state.outputs[-1] if state.outputs else None
                stop_reason = None
                if state.finish_reason == "stop" and last in state.request.stop_token_ids:
                    stop_reason = last
                self._collect(request_id, stop_reason)
            done.extend(finished)
            for request_id in sampled:
                check = self._stop_checks.get(request_id)
                if check is None or request_id in self._finished:
                    continue
                hit = check(self.scheduler.state(request_id).outputs)
                if hit is not None:
                    self.scheduler.finish_early(request_id, "stop")
                    self._collect(request_id, hit)
                    done.append(request_id)
        return tuple(done)

    def run_to_completion(self) -> dict[str, FinishedRequest]:
        while self.scheduler.has_unfinished():
            self.step()
        finished, self._finished = self._finished, {}
        return finished

    def take_finished(self) -> dict[str, FinishedRequest]:
        finished, self._finished = self._finished, {}
        return finished
