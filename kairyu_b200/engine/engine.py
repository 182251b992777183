"""The engine: model + cache + step function + scheduler + sampler, and the
synchronous loop ``schedule -> step -> sample -> update`` over them
(kairyu/engine/core/engine_core.py:57-103; assembly as in
kairyu/engine/kairyu_backend.py:467-1179, without tokenizer and server parts).
"""

from __future__ import annotations

import dataclasses
from collections import deque
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
    num_cached_tokens: int = 0  # prompt tokens found in the prefix tree at admission
    logprobs: Optional[tuple[dict[int, float], ...]] = None  # per output token, when the request asked for them
    cumulative_logprob: Optional[float] = None


class _PendingStep:
    """A launched step whose sampled ids have not been read yet."""

    __slots__ = ("request_ids", "index", "host", "event", "report", "report_host")

    def __init__(self, request_ids: list[str]) -> None:
        self.request_ids = request_ids
        self.index = {request_id: place for place, request_id in enumerate(request_ids)}  # row of each id in the sampled tensor
        self.host: Optional[torch.Tensor] = None
        self.event: Any = None
        self.report: Any = None  # the sampler's LogprobReport of the step, if a row asked for one
        self.report_host: Any = None  # (values, indices) on the host


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
            layout,
            num_pages=num_pages,
            page_size=config.page_size,
            max_requests=config.max_num_seqs,
            prefix_sharing=config.enable_prefix_caching,
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
            portion_graphs=config.portion_graphs,
        )
        self.scheduler = Scheduler(
            self.cache,
            max_num_batched_tokens=config.max_num_batched_tokens,
            max_num_seqs=config.max_num_seqs,
            max_num_partial_prefills=config.max_num_partial_prefills,
            max_model_len=self.max_model_len,
            prefill_chunk_size=config.prefill_chunk_size,
            priority_scheduling=config.priority_scheduling,
        )
        self.sampler = Sampler(model.spec.vocab_size, self.device)
        self._finished: dict[str, FinishedRequest] = {}
        self._stop_checks: dict[str, Callable[[Sequence[int]], Optional[str]]] = {}
        self._steps_since_check = 0
        self._pending: deque[_PendingStep] = deque()  # launched, not yet committed
        self._sampled: Optional[torch.Tensor] = None   # device ids of the step launched last
        self._host_ring: list[tuple[Optional[torch.Tensor], Any]] = [(None, None)] * 4
        self._next_host = 0
        self._logprobs: dict[str, list[dict[int, float]]] = {}  # per request that asked: one entry per output token

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

    def warm_up(self, max_batch: Optional[int] = None, max_context: Optional[int] = None) -> int:
        """Capture the decode graphs for up to ``max_batch`` rows (default: max_num_seqs) of up to
        ``max_context`` tokens (default: max_model_len) before the first request, so that no step of
        a serving engine pays for a capture.  Returns the number of graphs captured."""
        return self.runner.capture_decode_graphs(
            self.config.max_num_seqs if max_batch is None else max_batch,
            self.runner.max_model_len if max_context is None else max_context,
        )

    # ------------------------------------------------------------------ requests
    def add_request(
        self,
        request_id: str,
        prompt_token_ids: Sequence[int],
        params: SamplingParams,
        *,
        eos_token_ids: Sequence[int] = (),
        stop_check: Optional[Callable[[Sequence[int]], Optional[str]]] = None,
        priority: int = 0,
    ) -> None:
        if priority != 0 and not self.config.priority_scheduling:
            raise ValueError("a priority needs an engine built with priority_scheduling=True")
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
                priority=int(priority),
            )
        )
        if stop_check is not None:
            self._stop_checks[request_id] = stop_check

    def abort(self, request_id: str) -> None:
        """End a waiting or running request now (reason ``"abort"``); what it holds is given back, a
        token of its that is still in flight is dropped when its step commits.  An id that is not
        known, or has finished, is left alone."""
        if not self.scheduler.is_unfinished(request_id):
            return
        self.scheduler.abort(request_id)
        self._collect(request_id)

    def has_unfinished(self) -> bool:
        """Requests are waiting or running, or a launched step has not been committed yet."""
        return self.scheduler.has_unfinished() or bool(self._pending)

    # ------------------------------------------------------------------ the loop
    def _collect(self, request_id: str, stop_reason: Optional[int | str] = None) -> None:
        state = self.scheduler.state(request_id)
        self._finished[request_id] = FinishedRequest(
            request_id,
            state.request.prompt_token_ids,
            tuple(state.outputs),
            state.finish_reason or "abort",
            stop_reason,
            state.num_cached_tokens,
        )
        entries = self._logprobs.pop(request_id, None)
        if state.request.params.logprobs is not None:
            entries = entries or []
            chosen = [entry[token] for entry, token in zip(entries, state.outputs)]
            self._finished[request_id] = dataclasses.replace(
                self._finished[request_id], logprobs=tuple(entries), cumulative_logprob=float(sum(chosen))
            )
        self._stop_checks.pop(request_id, None)
        self.scheduler.forget(request_id)

    # A step is launched (planned, enqueued on the GPU, its sampled ids copied towards the host)
    # and later committed (ids read, requests updated and finished).  With pipeline_depth 2 the
    # next step is launched before the oldest is committed: its decode rows take their token
    # from the device tensor of sampled ids (kairyu/engine/engine_loop.py:1025-1136, 1282-1299).
    def _depth_now(self) -> int:
        if self.config.pipeline_depth < 2 or self._stop_checks:
            return 1  # stop strings are judged on committed text, between steps
        for request_id in self.scheduler.running_ids():
            params = self.scheduler.state(request_id).request.params
            if params.repetition_penalty != 1.0 or params.frequency_penalty != 0.0 or params.presence_penalty != 0.0:
                return 1  # penalties read the committed outputs
        return 2

    def _launch(self, done: list[str]) -> bool:
        """Plan one step and enqueue it; False when there was nothing to run."""
        plan = self.scheduler.schedule()
        done.extend(plan.rejected)
        for request_id in plan.rejected:
            self._collect(request_id)
        if not plan.scheduled:
            if self.scheduler.has_unfinished() and not plan.rejected and not plan.preempted and not self._pending:
                raise RuntimeError("the scheduler made no progress")
            return False
        previous = self._pending[-1] if self._pending else None
        entries: list[StepEntry] = []
        rows: list[SamplingRow] = []
        for chunk in plan.scheduled:
            state = self.scheduler.state(chunk.request_id)
            held = self.cache.get(chunk.request_id).num_tokens if chunk.request_id in self.cache else 0
            if held != chunk.start:
                raise RuntimeError(
                    f"request {chunk.request_id!r}: the cache holds {held} tokens, the plan starts at {chunk.start}"
                )
            known = state.total_tokens
            future = None
            if chunk.start + chunk.num_tokens > known:
                # the token it feeds was sampled by the step before and has not been read yet
                if chunk.num_tokens != 1 or previous is None or chunk.request_id not in previous.index:
                    raise RuntimeError(f"request {chunk.request_id!r}: a token in flight has no step to come from")
                future = previous.index[chunk.request_id]
                tokens: Sequence[int] = (0,)
            else:
                tokens = state.tokens(chunk.start, chunk.num_tokens)
            entries.append(StepEntry(chunk.request_id, tokens, want=(chunk.num_tokens - 1,) if chunk.samples else (), future=future))
            if chunk.samples:
                request = state.request
                rows.append(
                    SamplingRow(
                        request_id=chunk.request_id,
                        params=request.params,
                        position=len(state.outputs) + state.in_flight - 1,
                        prompt_token_ids=request.prompt_token_ids,
                        output_token_ids=state.outputs,
                        eos_token_ids=request.eos_token_ids,
                    )
                )
        logits = self.runner.step(entries, self._sampled if previous is not None else None)
        if not rows:
            return True
        if self._sampled is None or self._sampled.numel() < len(rows):
            self._sampled = torch.zeros(max(len(rows), self.config.max_num_seqs), dtype=torch.int32, device=self.device)
        out = self.sampler.sample(logits, rows, out=self._sampled[: len(rows)])
        pending = _PendingStep([row.request_id for row in rows])
        pending.report = self.sampler.take_report()
        if str(self.device).startswith("cuda"):
            slot = self._next_host
            self._next_host = (slot + 1) % len(self._host_ring)
            host, event = self._host_ring[slot]
            if host is None or host.numel() < len(rows):
                host = torch.empty(max(len(rows), self.config.max_num_seqs), dtype=torch.int32, pin_memory=True)
                event = torch.cuda.Event()
                self._host_ring[slot] = (host, event)
            host[: len(rows)].copy_(out, non_blocking=True)  # the step's one device->host read, awaited at commit
            if pending.report is not None:  # rare: its own pinned buffers, read after the same event
                report = pending.report
                pending.report_host = (
                    torch.empty(report.values.shape, dtype=torch.float32, pin_memory=True),
                    torch.empty(report.indices.shape, dtype=torch.int32, pin_memory=True),
                )
                pending.report_host[0].copy_(report.values, non_blocking=True)
                pending.report_host[1].copy_(report.indices, non_blocking=True)
            event.record()
            pending.host, pending.event = host, event
        else:
            pending.host = out.clone()
            if pending.report is not None:
                pending.report_host = (pending.report.values.clone(), pending.report.indices.clone())
        self._pending.append(pending)
        return True

    def _commit(self, pending: "_PendingStep", done: list[str]) -> None:
        if pending.event is not None:
            pending.event.synchronize()
        token_ids = pending.host[: len(pending.request_ids)].tolist()
        # The kernels' error word is sticky: reading it every few steps (and whenever a
        # request ends) reports the same faults with fewer round trips.
        self._steps_since_check += 1
        sampled = {request_id: int(token) for request_id, token in zip(pending.request_ids, token_ids)}
        if pending.report is not None:
            values, indices = (tensor.tolist() for tensor in pending.report_host)
            for row, entry, _ in pending.report.entries(values, indices, token_ids):
                request_id = pending.request_ids[row]
                if self.scheduler.is_unfinished(request_id):  # else the token is dropped, and its report with it
                    self._logprobs.setdefault(request_id, []).append(entry)
        alive = [request_id for request_id in sampled if request_id not in self._finished]
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
        for request_id in alive:
            check = self._stop_checks.get(request_id)
            if check is None or request_id in self._finished:
                continue
            hit = check(self.scheduler.state(request_id).outputs)
            if hit is not None:
                self.scheduler.finish_early(request_id, "stop")
                self._collect(request_id, hit)
                done.append(request_id)

    def step(self) -> tuple[str, ...]:
        """One engine step: launch until ``pipeline_depth`` steps are in flight, then commit the
        oldest.  Returns the ids of requests that finished in it."""
        done: list[str] = []
        while len(self._pending) < self._depth_now():
            before = len(self._pending)
            if not self._launch(done):
                break
            if len(self._pending) == before:
                break  # a step without sampling rows (prompt portions only): nothing to wait for
        if self._pending:
            self._commit(self._pending.popleft(), done)
        return tuple(done)

    def run_to_completion(self) -> dict[str, FinishedRequest]:
        while self.has_unfinished():
            self.step()
        finished, self._finished = self._finished, {}
        return finished

    def take_finished(self) -> dict[str, FinishedRequest]:
        finished, self._finished = self._finished, {}
        return finished
