"""The scheduler: admits requests, cuts prompts into portions under a token
budget, decodes, finishes and frees.  Pure policy over the cache manager; it
never touches a tensor (kairyu/engine/core/scheduler.py:404-1770 is the
reference; priority aging, scheduling classes and speculative reservations are
left out).

A request's work is ``prompt + outputs``; ``computed`` counts how many of those
tokens have been fed.  While more than one token is left to feed the request
is in prefill (portions, cut anywhere); when exactly one is left the request
decodes.  The step that feeds the last token samples the next one.  This view
makes recompute-preemption uniform: a victim's ``computed`` goes back to 0 and
its prompt *and* outputs are fed again.

Schedule-ahead (kairyu/engine/core/scheduler.py:1234-1242, engine_loop.py:1025-1136):
a chunk that samples puts one token ``in_flight``; until ``update`` commits it the
token counts as part of the request's work, so the next plan may already feed it
(the step takes its value from the device).  A request with a token in flight is
never preempted, and tokens that arrive for a request that has finished meanwhile
are dropped.

Prefix sharing, when the cache manager has it on: admission hands the request's tokens to
the cache, which may find their leading whole pages already computed; the request then
starts behind them (``computed`` and ``num_cached_tokens``), always leaving its last token
to compute (scheduler.py:1589-1593).  A request's whole pages are published when its first
token commits and again when it finishes (scheduler.py:1724-1729; radix_kv.py:815-889);
an aborted or preempted request publishes nothing more.

Order within a step (scheduler.py:1641-1657): decodes first (one token each),
then running prefills, then admissions from the head of the queue.

When pages run out:

* at admission, the head waits until the pages its whole prompt needs are
  free; while it waits and something runs, the one request right behind it may
  be admitted in its place, once per head (scheduler.py:28, 1543-1577); a
  prompt that could never fit, even in an empty cache, is rejected: finished,
  reason ``"length"``, no output (scheduler.py:1007-1019, 1479-1490);
* for a decode, the youngest running request that has no outputs yet is
  recompute-preempted (scheduler.py:1065-1110); if there is none, the youngest
  other running request is, outputs included (the reference raises here); the
  victim goes back to the front of the queue.  A request that is alone and
  still cannot grow is finished with reason ``"length"``;
* a prompt is kept one token short of its end while finishing it could leave requests that
  already decode without the pages they need to reach their limits: as long as it has not
  sampled it is the cheap victim (nothing of its outputs is lost), once it decodes it is not
  (scheduler.py:636-677, 719-730).  The spare pages are counted once a plan: free pages, plus
  what unfinished prompts hold, minus what decoding requests still lack up to
  ``prompt + max_new_tokens``; a prompt may finish if nothing decodes yet, if it will produce a
  single token, or if the pages of its own whole life fit in that count;
* a prefill portion that cannot get pages is skipped this step;
* if a step would be empty while requests are unfinished, the youngest running
  request is preempted, or the stuck head is rejected
  (kairyu/engine/core/engine_core.py:76-88).
"""

from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field
from enum import Enum
from typing import Mapping, Optional

from kairyu_b200.cache.manager import CacheManager
from kairyu_b200.cache.page_pool import OutOfPages
from kairyu_b200.sampling.params import SamplingParams


@dataclass(frozen=True)
class EngineRequest:
    """kairyu/engine/core/scheduler.py:31-57."""

    request_id: str
    prompt_token_ids: tuple[int, ...]
    max_new_tokens: int = 16
    eos_token_ids: tuple[int, ...] = ()
    stop_token_ids: tuple[int, ...] = ()
    min_tokens: int = 0
    ignore_eos: bool = False
    params: SamplingParams = field(default_factory=lambda: SamplingParams(temperature=0.0))
    priority: int = 0  # lower goes first when the scheduler orders by priority (scheduler.py:44, 191-199)


MAX_WAITING_BYPASSES = 1  # kairyu/engine/core/scheduler.py:28


class Status(Enum):
    WAITING = "waiting"
    RUNNING = "running"
    FINISHED = "finished"


class RequestState:
    __slots__ = (
        "request", "status", "computed", "outputs", "in_flight", "finish_reason", "preemptions", "arrival",
        "num_cached_tokens", "bypasses", "decoding",
    )

    def __init__(self, request: EngineRequest, arrival: int) -> None:
        self.request = request
        self.status = Status.WAITING
        self.computed = 0
        self.outputs: list[int] = []
        self.in_flight = 0  # sampled by a launched step, not yet committed by update()
        self.finish_reason: Optional[str] = None
        self.preemptions = 0
        self.arrival = arrival
        self.num_cached_tokens = 0  # tokens its first admission found in the prefix tree
        self.bypasses = 0  # times the request behind it was admitted while it waited for pages
        # Since it was last admitted, a step has fed its last known token and sampled: from then on it
        # is fed one token a step.  Until then it is a prompt (or a recomputation) under way.
        self.decoding = False

    @property
    def total_tokens(self) -> int:
        return len(self.request.prompt_token_ids) + len(self.outputs)

    @property
    def remaining(self) -> int:
        """Tokens left to feed, the ones in flight included (their values come later)."""
        return self.total_tokens + self.in_flight - self.computed

    def all_tokens(self) -> list[int]:
        return list(self.request.prompt_token_ids) + self.outputs

    def tokens(self, start: int, count: int) -> list[int]:
        prompt = self.request.prompt_token_ids
        end = start + count
        if end <= len(prompt):
            return list(prompt[start:end])
        if start >= len(prompt):
            return self.outputs[start - len(prompt) : end - len(prompt)]
        return list(prompt[start:]) + self.outputs[: end - len(prompt)]


@dataclass(frozen=True)
class ScheduledChunk:
    request_id: str
    start: int  # offset into prompt + outputs
    num_tokens: int
    is_prefill: bool
    samples: bool  # the chunk feeds the last known token, so its last logits pick the next


@dataclass(frozen=True)
class SchedulerOutput:
    scheduled: tuple[ScheduledChunk, ...]
    preempted: tuple[str, ...] = ()
    rejected: tuple[str, ...] = ()


class Scheduler:
    def __init__(
        self,
        cache: CacheManager,
        *,
        max_num_batched_tokens: int = 2048,
        max_num_seqs: int = 256,
        max_num_partial_prefills: int = 2,
        max_model_len: Optional[int] = None,
        prefill_chunk_size: Optional[int] = None,
        priority_scheduling: bool = False,
    ) -> None:
        self.cache = cache
        self.priority_scheduling = priority_scheduling
        self.budget = max_num_batched_tokens
        self.max_num_seqs = max_num_seqs
        self.max_num_partial_prefills = max_num_partial_prefills
        self.max_model_len = max_model_len
        self.prefill_chunk_size = prefill_chunk_size
        self._states: dict[str, RequestState] = {}
        self._waiting: deque[str] = deque()
        self._running: list[str] = []  # admission order; the last is the youngest
        self._arrivals = 0
        self.counters = {"preemptions": 0, "rejections": 0, "steps": 0, "prompt_tokens": 0, "cached_prompt_tokens": 0}

    # ------------------------------------------------------------------ intake
    def add_request(self, request: EngineRequest) -> None:
        if request.request_id in self._states:
            raise ValueError(f"request id {request.request_id!r} is already known")
        if not request.prompt_token_ids:
            raise ValueError("a request needs at least one prompt token")
        if request.max_new_tokens < 1:
            raise ValueError("max_new_tokens must be >= 1")
        if self.max_model_len is not None and len(request.prompt_token_ids) + request.max_new_tokens > self.max_model_len:
            # kairyu/engine/engine_loop.py:630-644
            raise ValueError(
                f"prompt ({len(request.prompt_token_ids)}) + max_tokens ({request.max_new_tokens}) "
                f"exceeds max_model_len ({self.max_model_len})"
            )
        self._states[request.request_id] = RequestState(request, self._arrivals)
        self._arrivals += 1
        self._enqueue(request.request_id)

    def _enqueue(self, request_id: str, front: bool = False) -> None:
        """Put a request on the waiting queue: first come, first served (a preempted request goes
        back to the front), or, with priority scheduling, by (priority, arrival), the lower first
        (kairyu/engine/core/scheduler.py:191-199; a preempted request keeps its place by its arrival)."""
        if not self.priority_scheduling:
            if front:
                self._waiting.appendleft(request_id)
            else:
                self._waiting.append(request_id)
            return
        key = self._queue_key(request_id)
        place = 0
        while place < len(self._waiting) and self._queue_key(self._waiting[place]) <= key:
            place += 1
        self._waiting.insert(place, request_id)

    def _queue_key(self, request_id: str) -> tuple[int, int]:
        state = self._states[request_id]
        return state.request.priority, state.arrival

    def abort(self, request_id: str) -> None:
        state = self._states.get(request_id)
        if state is None or state.status is Status.FINISHED:
            return
        if state.status is Status.WAITING:
            self._waiting.remove(request_id)
        else:
            self._running.remove(request_id)
        self._finish(state, "abort", in_running=False)

    def finish_early(self, request_id: str, reason: str) -> None:
        """End a running request between steps (a stop string was produced)."""
        state = self._states.get(request_id)
        if state is not None and state.status is Status.RUNNING:
            self._finish(state, reason)

    def forget(self, request_id: str) -> None:
        state = self._states.get(request_id)
        if state is not None and state.status is Status.FINISHED:
            del self._states[request_id]

    # ------------------------------------------------------------------ queries
    def has_unfinished(self) -> bool:
        return bool(self._waiting or self._running)

    def state(self, request_id: str) -> RequestState:
        return self._states[request_id]

    def is_unfinished(self, request_id: str) -> bool:
        state = self._states.get(request_id)
        return state is not None and state.status is not Status.FINISHED

    @property
    def prefix_hit_rate(self) -> float:
        """Prompt tokens found in the prefix tree over prompt tokens admitted
        (kairyu/engine/core/radix_kv.py:245-249)."""
        total = self.counters["prompt_tokens"]
        return self.counters["cached_prompt_tokens"] / total if total else 0.0

    def running_ids(self) -> tuple[str, ...]:
        return tuple(self._running)

    @property
    def num_waiting(self) -> int:
        return len(self._waiting)

    @property
    def num_running(self) -> int:
        return len(self._running)

    def output_tokens(self, request_id: str) -> tuple[int, ...]:
        return tuple(self._states[request_id].outputs)

    def finish_reason(self, request_id: str) -> Optional[str]:
        return self._states[request_id].finish_reason

    # ------------------------------------------------------------------ internals
    def _finish(self, state: RequestState, reason: str, *, in_running: bool = True) -> None:
        state.status = Status.FINISHED
        state.finish_reason = reason
        if in_running:
            self._running.remove(state.request.request_id)
        if state.request.request_id in self.cache:
            if reason in ("stop", "length"):
                self.cache.publish(state.request.request_id, state.all_tokens())
            self.cache.release(state.request.request_id)

    def _preempt(self, request_id: str) -> None:
        """Recompute-preemption: give everything back, start over from the front of the queue."""
        state = self._states[request_id]
        self._running.remove(request_id)
        if request_id in self.cache:
            self.cache.release(request_id)
        state.computed = 0
        state.decoding = False
        state.status = Status.WAITING
        state.preemptions += 1
        self._enqueue(request_id, front=True)
        self.counters["preemptions"] += 1

    def _pick_victim(self, needy: str, taken: set[str]) -> Optional[str]:
        fallback = None
        for candidate in reversed(self._running):
            if candidate == needy or candidate in taken or self._states[candidate].in_flight:
                continue
            if not self._states[candidate].outputs:
                return candidate
            if fallback is None:
                fallback = candidate
        return fallback

    def _grow(self, state: RequestState, count: int) -> bool:
        return self.cache.ensure_capacity(
            state.request.request_id, state.computed + count, query_start=state.computed
        )

    def _chunk_cap(self, budget: int, sharers: int) -> int:
        cap = -(-budget // max(sharers, 1))
        if self.prefill_chunk_size is not None:
            cap = min(cap, self.prefill_chunk_size)
        return cap

    def _largest_portion(self) -> int:
        return min(self.budget, self.prefill_chunk_size or self.budget)

    # -- completion safety (kairyu/engine/core/scheduler.py:636-677, 719-730)
    def _life_pages(self, state: RequestState) -> list[int]:
        """Pages per group the request holds when it has produced its last token."""
        return self.cache.peak_pages(len(state.request.prompt_token_ids) + state.request.max_new_tokens)

    def _spare_pages(self) -> tuple[int, list[int]]:
        """(requests that decode and will go on, pages per group that stay spare if each of them runs
        to its limit): what is free or can be taken back, what unfinished prompts hold, less what the
        decoding requests still lack."""
        spare = [self.cache.available_pages(group.index) for group in self.cache.layout.groups]
        decoders = 0
        for request_id in self._running:
            state = self._states[request_id]
            named, own = self.cache.held_pages(request_id) if request_id in self.cache else ([0] * len(spare), [0] * len(spare))
            if not state.decoding:
                spare = [total + pages for total, pages in zip(spare, own)]
            elif state.request.max_new_tokens > 1 and len(state.outputs) + state.in_flight < state.request.max_new_tokens:
                decoders += 1
                spare = [total - max(0, life - held) for total, life, held in zip(spare, self._life_pages(state), named)]
        return decoders, spare

    def _completion_cost(self, state: RequestState) -> list[int]:
        """Pages per group that stop being spare when this prompt finishes: the ones it holds (they
        can no longer be had back cheaply) and the ones it still lacks up to its limit."""
        request_id = state.request.request_id
        count = len(self.cache.layout.groups)
        named, own = self.cache.held_pages(request_id) if request_id in self.cache else ([0] * count, [0] * count)
        lacking = [max(0, life - held) for life, held in zip(self._life_pages(state), named)] if state.request.max_new_tokens > 1 else [0] * count
        return [mine + more for mine, more in zip(own, lacking)]

    def _may_complete(self, state: RequestState, safety: list) -> bool:
        decoders, spare = safety
        if state.request.max_new_tokens <= 1 or decoders < 1:
            return True  # the first request to decode can have every unfinished prompt's pages
        return all(cost <= room for cost, room in zip(self._completion_cost(state), spare))

    def _note_completion(self, state: RequestState, safety: list) -> None:
        safety[1] = [room - cost for room, cost in zip(safety[1], self._completion_cost(state))]
        if state.request.max_new_tokens > 1:
            safety[0] += 1
        state.decoding = True

    def _admit(self, request_id: str, budget: int, plan: list, taken: set, safety: list) -> Optional[int]:
        """Make a waiting request run if the pages its whole work needs are to be had: its first
        portion goes into ``plan``.  Returns the tokens it took from the budget, or None, with
        nothing changed, when it has to wait.  The caller takes it off the queue."""
        state = self._states[request_id]
        try:
            record = self.cache.admit(request_id, state.all_tokens())
        except OutOfPages:
            return None
        # every page of its work; a windowed group needs its window and one portion only
        needed = [pages - len(record.shared) for pages in self.cache.peak_pages(state.total_tokens, self._largest_portion())]
        if any(count > self.cache.available_pages(group) for group, count in enumerate(needed)):
            self.cache.release(request_id)
            return None
        state.computed = record.num_tokens  # the pages the prefix tree already holds
        count = min(state.remaining, budget, self._chunk_cap(budget, 1))
        if count == state.remaining and not self._may_complete(state, safety):
            count -= 1  # stays one token short until the decoding requests are safe
        if count < 1 or not self._grow(state, count):
            state.computed = 0
            self.cache.release(request_id)
            return None
        if state.preemptions == 0:
            state.num_cached_tokens = record.num_cached_tokens
            self.counters["prompt_tokens"] += state.total_tokens
            self.counters["cached_prompt_tokens"] += record.num_cached_tokens
        state.status = Status.RUNNING
        self._running.append(request_id)
        completes = count == state.remaining
        plan.append(ScheduledChunk(request_id, state.computed, count, count > 1 or not completes, completes))
        state.computed += count
        if completes:
            state.in_flight += 1
            self._note_completion(state, safety)
        taken.add(request_id)
        return count

    # ------------------------------------------------------------------ one plan
    def schedule(self) -> SchedulerOutput:
        self.counters["steps"] += 1
        plan, preempted, rejected = self._plan()
        if not plan and self.has_unfinished() and not any(self._states[r].in_flight for r in self._running):
            # Nothing can move (and nothing is merely waiting for a token in flight).  Free
            # something, or give up on the stuck head.
            if self._running:
                victim = self._running[-1]
                self._preempt(victim)
                preempted.append(victim)
                more, more_preempted, more_rejected = self._plan()
                plan, preempted, rejected = more, preempted + more_preempted, rejected + more_rejected
            if not plan and self._waiting and not self._running:
                head = self._waiting.popleft()
                self._finish(self._states[head], "length", in_running=False)
                self.counters["rejections"] += 1
                rejected.append(head)
        return SchedulerOutput(tuple(plan), tuple(preempted), tuple(rejected))

    def _plan(self) -> tuple[list[ScheduledChunk], list[str], list[str]]:
        plan: list[ScheduledChunk] = []
        preempted: list[str] = []
        rejected: list[str] = []
        budget = self.budget
        taken: set[str] = set()

        # 1. decodes: one token each, oldest first
        for request_id in list(self._running):
            if budget < 1:
                break
            state = self._states.get(request_id)
            if state is None or state.status is not Status.RUNNING or not state.decoding or state.remaining != 1:
                continue
            if len(state.outputs) + state.in_flight >= state.request.max_new_tokens:
                continue  # its last token is in flight
            while not self._grow(state, 1):
                victim = self._pick_victim(request_id, taken)
                if victim is None:
                    break
                self._preempt(victim)
                preempted.append(victim)
            else:
                plan.append(ScheduledChunk(request_id, state.computed, 1, False, True))
                state.computed += 1
                state.in_flight += 1
                taken.add(request_id)
                budget -= 1
                continue
            if len(self._running) == 1 and not state.in_flight:
                # alone and the cache is exhausted: it cannot go on
                self._finish(state, "length")
                rejected.append(request_id)

        # 2. running prefills share what is left of the budget.  Whether one may finish is judged
        # against the requests that decode now (step 1 may have ended or preempted some).
        safety = list(self._spare_pages())
        prefilling = [
            request_id
            for request_id in self._running
            if not self._states[request_id].decoding and self._states[request_id].remaining >= 1 and request_id not in taken
        ]
        for index, request_id in enumerate(prefilling):
            if budget < 1:
                break
            state = self._states[request_id]
            count = min(state.remaining, budget, self._chunk_cap(budget, len(prefilling) - index))
            if count == state.remaining and not self._may_complete(state, safety):
                count -= 1  # stays one token short until the decoding requests are safe
            if count < 1 or not self._grow(state, count):
                continue
            completes = count == state.remaining
            plan.append(ScheduledChunk(request_id, state.computed, count, count > 1 or not completes, completes))
            state.computed += count
            if completes:
                state.in_flight += 1
                self._note_completion(state, safety)
            taken.add(request_id)
            budget -= count

        # 3. admissions from the head of the queue
        while self._waiting and budget >= 1:
            if len(self._running) >= self.max_num_seqs:
                break
            partial = sum(1 for r in self._running if not self._states[r].decoding and r not in taken) + sum(
                1 for chunk in plan if chunk.is_prefill and not chunk.samples
            )
            if partial >= self.max_num_partial_prefills:
                break
            head = self._waiting[0]
            state = self._states[head]
            if not self.cache.can_hold(state.total_tokens, self._largest_portion()):
                self._waiting.popleft()
                self._finish(state, "length", in_running=False)
                self.counters["rejections"] += 1
                rejected.append(head)
                continue
            used = self._admit(head, budget, plan, taken, safety)
            if used is not None:
                self._waiting.popleft()
                budget -= used
                continue
            # The head waits for pages.  While something runs (and will free pages), the request
            # right behind it may go first, once per head (scheduler.py:28, 1543-1577).
            if not self._running or state.bypasses >= MAX_WAITING_BYPASSES or len(self._waiting) < 2:
                break
            successor = self._waiting[1]
            if not self.cache.can_hold(self._states[successor].total_tokens, self._largest_portion()):
                break
            used = self._admit(successor, budget, plan, taken, safety)
            if used is None:
                break
            state.bypasses += 1
            del self._waiting[1]
            budget -= used
        return plan, preempted, rejected

    # ------------------------------------------------------------------ results
    def update(self, sampled: Mapping[str, int]) -> tuple[str, ...]:
        """Commit one sampled token per request; return the ids that finished
        (kairyu/engine/core/scheduler.py:1688-1770)."""
        finished: list[str] = []
        for request_id, token in sampled.items():
            if isinstance(token, bool) or not isinstance(token, int):
                raise TypeError(f"request {request_id!r}: sampled tokens must be ints, got {token!r}")
            state = self._states.get(request_id)
            if state is None or state.status is Status.FINISHED:
                continue  # it ended while this token was in flight (scheduler.py:1712-1720)
            if state.in_flight < 1:
                raise ValueError(f"request {request_id!r} is not awaiting a sampled token")
            state.in_flight -= 1
            state.outputs.append(token)
            reason = self._terminal_reason(state, token)
            if reason is not None:
                self._finish(state, reason)
                finished.append(request_id)
            elif len(state.outputs) == 1 and request_id in self.cache:
                self.cache.publish(request_id, state.all_tokens())  # its prompt's pages become matchable
        return tuple(finished)

    @staticmethod
    def _terminal_reason(state: RequestState, token: int) -> Optional[str]:
        request = state.request
        is_eos = not request.ignore_eos and token in request.eos_token_ids
        is_stop = is_eos or token in request.stop_token_ids
        if is_stop and len(state.outputs) >= request.min_tokens:
            return "stop"
        if len(state.outputs) >= request.max_new_tokens:
            return "length"
        return None
