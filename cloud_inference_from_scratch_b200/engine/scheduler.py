"""Request lifecycle and the iteration-level scheduler above the step function.

Policy parity with the reference's packed scheduler (src/cloud_engine/scheduler.py):

* states ``waiting -> prefill -> decoding -> completed | cancelled | timed_out | failed``,
  terminal states are final (scheduler.py:29-46);
* submit refuses an empty prompt, ``prompt + max_output_tokens > max_model_len`` and a full
  queue (scheduler.py:233-254);
* admission is FIFO while fewer than ``max_active_sequences`` are active, with an empty block
  table; a request that was preempted waits until nothing else is active (scheduler.py:438-457);
* one plan per iteration under ``max_batched_tokens``: decoding requests first (one token each,
  FIFO inside a class because the sort is stable), then prompt portions of at most
  ``prefill_chunk_size`` tokens; ``sample`` is set when a portion ends at the end of the known
  sequence (scheduler.py:459-518);
* when the step reports that pages ran out, the active request with the largest
  ``(allocated_tokens, tokens_fed, arrival)`` is preempted: its pages are freed, it keeps its
  generated tokens, goes to the back of the queue and later recomputes prompt + generated
  tokens as prompt portions; with a single live request the plan's requests fail as rejected
  (scheduler.py:383-394, 527-553);
* EOS ends a request (the token is kept in ``generated_token_ids``), so does
  ``max_output_tokens`` (scheduler.py:581-607); every terminal path goes through one funnel
  that releases the cache (scheduler.py:640-668).

Unlike the reference this is a synchronous loop (``step()`` runs one iteration and the caller
owns the thread): no asyncio task, no worker thread, no stream queues or slow-consumer
watchdog.  Temperature sampling is allowed (the reference refuses it, scheduler.py:69-71).
"""

from __future__ import annotations

import time
from collections import deque
from collections.abc import Callable
from dataclasses import dataclass, field
from enum import Enum
from typing import Any


class RequestState(Enum):
    WAITING = "waiting"
    PREFILL = "prefill"
    DECODING = "decoding"
    COMPLETED = "completed"
    CANCELLED = "cancelled"
    TIMED_OUT = "timed_out"
    FAILED = "failed"


TERMINAL_STATES = frozenset(
    {RequestState.COMPLETED, RequestState.CANCELLED, RequestState.TIMED_OUT, RequestState.FAILED}
)


class RejectionReason(Enum):
    QUEUE_FULL = "queue_full"
    KV_CAPACITY = "capacity_exhausted"
    CONTEXT_OVERFLOW = "context_length_exceeded"


class RejectedError(RuntimeError):
    def __init__(self, reason: RejectionReason, detail: str = "") -> None:
        super().__init__(detail or reason.value)
        self.reason = reason


@dataclass
class GenerationConfig:
    """``temperature`` 0 is greedy; otherwise tokens are drawn from softmax(logits / temperature)
    with a draw that depends only on (``seed``, the request's stream number, the output index).
    ``eos_token_id`` None means no token ends the request early."""

    max_output_tokens: int
    temperature: float = 0.0
    eos_token_id: int | None = None
    seed: int = 0

    def __post_init__(self) -> None:
        if self.max_output_tokens < 1:
            raise ValueError("max_output_tokens must be positive")
        if self.temperature < 0:
            raise ValueError("temperature must be >= 0")


@dataclass
class StreamEvent:
    token_id: int | None
    finished: bool = False
    finish_reason: str = ""


@dataclass
class Request:
    request_id: str
    prompt_token_ids: list[int]
    config: GenerationConfig
    arrival_ns: int
    sequence_number: int = 0
    label: str = ""
    state: RequestState = RequestState.WAITING
    generated_token_ids: list[int] = field(default_factory=list)
    events: deque = field(default_factory=deque)
    tokens_fed: int = 0
    first_token_ns: int | None = None
    last_token_ns: int | None = None
    finish_ns: int | None = None
    finish_reason: str = ""
    error_detail: str = ""
    rejected: bool = False
    preemption_count: int = 0
    recomputed_tokens: int = 0
    recompute_until: int = 0

    @property
    def is_terminal(self) -> bool:
        return self.state in TERMINAL_STATES

    @property
    def generated_count(self) -> int:
        return len(self.generated_token_ids)

    @property
    def known_length(self) -> int:
        return len(self.prompt_token_ids) + len(self.generated_token_ids)


@dataclass(frozen=True)
class BatchItem:
    """One request's slice of tokens in a step."""

    request: Request
    token_ids: tuple[int, ...]
    start_pos: int
    sample: bool
    is_decode: bool

    @property
    def query_length(self) -> int:
        return len(self.token_ids)

    @property
    def end_pos(self) -> int:
        return self.start_pos + len(self.token_ids)


@dataclass(frozen=True)
class BatchPlan:
    items: tuple[BatchItem, ...]

    @property
    def token_count(self) -> int:
        return sum(item.query_length for item in self.items)

    @property
    def request_ids(self) -> tuple[str, ...]:
        return tuple(item.request.request_id for item in self.items)


@dataclass(frozen=True)
class SchedulingCandidate:
    request_id: str
    phase: str  # "decode" or "prefill"
    remaining_tokens: int
    prompt_tokens: int
    generated_tokens: int
    arrival_ns: int


@dataclass(frozen=True)
class PreemptionCandidate:
    request_id: str
    allocated_tokens: int
    tokens_fed: int
    generated_tokens: int
    arrival_ns: int


def decode_first_priority(candidate: SchedulingCandidate) -> tuple[int]:
    """Decoding requests before prompt portions; the stable sort keeps FIFO inside a class."""
    return (candidate.phase != "decode",)


def largest_sequence_preemption(candidate: PreemptionCandidate) -> tuple[int, int, int]:
    """The victim is the maximum of this key: most pages held, then most tokens fed."""
    return (candidate.allocated_tokens, candidate.tokens_fed, candidate.arrival_ns)


class Scheduler:
    def __init__(
        self,
        config: Any,
        runner: Any,
        metrics: Any,
        clock: Callable[[], int] = time.monotonic_ns,
        scheduling_priority: Callable[[SchedulingCandidate], tuple] = decode_first_priority,
        preemption_priority: Callable[[PreemptionCandidate], tuple] = largest_sequence_preemption,
    ) -> None:
        self.config = config
        self.runner = runner
        self.metrics = metrics
        self.clock = clock
        self.scheduling_priority = scheduling_priority
        self.preemption_priority = preemption_priority
        self.waiting: deque[Request] = deque()
        self.active: list[Request] = []
        self._counter = 0

    # ------------------------------------------------------------------ api
    def submit(self, prompt_token_ids: list[int], gen_config: GenerationConfig,
               label: str = "") -> Request:
        if len(prompt_token_ids) == 0:
            raise RejectedError(RejectionReason.CONTEXT_OVERFLOW, "empty prompt")
        if len(prompt_token_ids) + gen_config.max_output_tokens > self.config.max_model_len:
            raise RejectedError(RejectionReason.CONTEXT_OVERFLOW)
        if len(self.waiting) >= self.config.max_queue_size:
            raise RejectedError(RejectionReason.QUEUE_FULL)
        self._counter += 1
        request = Request(
            request_id=f"req-{self._counter:08d}",
            prompt_token_ids=[int(t) for t in prompt_token_ids],
            config=gen_config,
            arrival_ns=self.clock(),
            sequence_number=self._counter,
            label=label,
        )
        self.waiting.append(request)
        return request

    def cancel(self, request: Request) -> None:
        if request.is_terminal:
            return
        request.state = RequestState.CANCELLED
        request.finish_reason = "cancelled"
        self._finalize(request)

    @property
    def has_work(self) -> bool:
        return bool(self.waiting or self.active)

    def run_until_idle(self, max_iterations: int | None = None) -> int:
        iterations = 0
        while self.has_work:
            self.step()
            iterations += 1
            if max_iterations is not None and iterations >= max_iterations:
                break
        return iterations

    # ------------------------------------------------------------------ one iteration
    def step(self) -> bool:
        """reap -> admit -> plan -> execute -> account.  Returns whether anything happened."""
        progressed = self._reap(self.clock())
        progressed = self._admit_waiting() or progressed
        plan = self._build_batch_plan()
        if not plan.items:
            return progressed
        try:
            outputs = self.runner.execute_batch(plan)
        except Exception as exc:  # noqa: BLE001 - every failure must end in the funnel
            if bool(getattr(exc, "is_capacity_error", False)):
                if not self._preempt_for_capacity(plan):
                    for item in plan.items:
                        if not item.request.is_terminal:
                            self._fail(
                                item.request,
                                f"KV capacity cannot fit one runnable sequence: {exc}",
                                rejected=True,
                            )
                return True
            for item in plan.items:
                if not item.request.is_terminal:
                    self._fail(item.request, f"packed forward failed: {exc}")
            return True

        stamp = self.clock()
        self.metrics.record_input_tokens(plan.token_count)
        for item in plan.items:
            request = item.request
            if request.is_terminal:
                continue
            request.tokens_fed = item.end_pos
            recomputed = max(0, min(item.end_pos, request.recompute_until) - item.start_pos)
            if recomputed:
                request.recomputed_tokens += recomputed
                self.metrics.record_recomputed_tokens(recomputed)
            if item.sample:
                token_id = outputs.get(request.request_id)
                if token_id is None:
                    self._fail(request, "the step returned no token for a sampled request")
                    continue
                self._after_token(request, int(token_id), stamp)
            else:
                request.state = RequestState.PREFILL
        self.metrics.record_iteration(len(plan.items))
        return True

    # ------------------------------------------------------------------ internals
    def _admit_waiting(self) -> bool:
        progressed = False
        while self.waiting and len(self.active) < self.config.max_active_sequences:
            candidate = self.waiting[0]
            if candidate.preemption_count and self.active:
                break  # a preempted request waits for the residents to drain: no thrash
            self.waiting.popleft()
            try:
                self.runner.admit(candidate)
            except Exception as exc:  # noqa: BLE001
                capacity = bool(getattr(exc, "is_capacity_error", False))
                self._fail(candidate, f"admission refused: {exc}", rejected=capacity)
                continue
            candidate.state = RequestState.PREFILL
            self.active.append(candidate)
            progressed = True
        return progressed

    def _build_batch_plan(self) -> BatchPlan:
        budget = self.config.max_batched_tokens
        candidates: list[tuple[SchedulingCandidate, Request]] = []
        for request in self.active:
            if request.is_terminal:
                continue
            remaining = request.known_length - request.tokens_fed
            if remaining <= 0:
                continue
            phase = (
                "decode" if request.state is RequestState.DECODING and remaining == 1 else "prefill"
            )
            candidates.append(
                (
                    SchedulingCandidate(
                        request_id=request.request_id,
                        phase=phase,
                        remaining_tokens=remaining,
                        prompt_tokens=len(request.prompt_token_ids),
                        generated_tokens=request.generated_count,
                        arrival_ns=request.arrival_ns,
                    ),
                    request,
                )
            )
        items: list[BatchItem] = []
        for candidate, request in sorted(candidates, key=lambda pair: self.scheduling_priority(pair[0])):
            if budget <= 0:
                break
            limit = 1 if candidate.phase == "decode" else self.config.prefill_chunk_size
            length = min(candidate.remaining_tokens, limit, budget)
            start = request.tokens_fed
            end = start + length
            prompt_len = len(request.prompt_token_ids)
            if end <= prompt_len:
                tokens = tuple(request.prompt_token_ids[start:end])
            elif start >= prompt_len:
                tokens = tuple(request.generated_token_ids[start - prompt_len:end - prompt_len])
            else:
                tokens = tuple(request.prompt_token_ids[start:]) + tuple(
                    request.generated_token_ids[:end - prompt_len]
                )
            items.append(
                BatchItem(
                    request=request,
                    token_ids=tokens,
                    start_pos=start,
                    sample=end == request.known_length,
                    is_decode=length == 1 and start >= prompt_len,
                )
            )
            budget -= length
        return BatchPlan(tuple(items))

    def _preempt_for_capacity(self, plan: BatchPlan) -> bool:
        candidates = [request for request in self.active if not request.is_terminal]
        if len(candidates) <= 1:
            return False
        allocated = getattr(self.runner, "allocated_tokens", lambda _request: 0)
        victim = max(
            candidates,
            key=lambda request: self.preemption_priority(
                PreemptionCandidate(
                    request_id=request.request_id,
                    allocated_tokens=allocated(request),
                    tokens_fed=request.tokens_fed,
                    generated_tokens=request.generated_count,
                    arrival_ns=request.arrival_ns,
                )
            ),
        )
        self.active.remove(victim)
        self.runner.release(victim)
        victim.recompute_until = max(victim.recompute_until, victim.tokens_fed)
        victim.tokens_fed = 0
        victim.preemption_count += 1
        victim.state = RequestState.WAITING
        self.waiting.append(victim)
        self.metrics.inc_preempted()
        return True

    def _reap(self, now: int) -> bool:
        progressed = False
        timeout_ns = int(self.config.queue_timeout_seconds * 1_000_000_000)
        for request in list(self.waiting):
            if request.preemption_count == 0 and now - request.arrival_ns > timeout_ns:
                self.waiting.remove(request)
                request.state = RequestState.TIMED_OUT
                request.finish_reason = "timed_out"
                self._finalize(request)
                progressed = True
        return progressed

    def _after_token(self, request: Request, token_id: int, now: int) -> None:
        request.generated_token_ids.append(token_id)
        if request.first_token_ns is None:
            request.first_token_ns = now
            self.metrics.record_ttft_ms((now - request.arrival_ns) / 1e6)
        else:
            self.metrics.record_itl_ms((now - (request.last_token_ns or now)) / 1e6)
        request.last_token_ns = now
        self.metrics.record_output_token(1)
        eos = request.config.eos_token_id
        eos_hit = eos is not None and token_id == eos
        limit_hit = request.generated_count >= request.config.max_output_tokens
        if eos_hit:
            request.finish_reason = "eos_token_reached"
        elif limit_hit:
            request.finish_reason = "max_output_tokens_reached"
        request.events.append(StreamEvent(token_id=None if eos_hit else token_id))
        if eos_hit or limit_hit:
            request.state = RequestState.COMPLETED
            self._finalize(request)
        else:
            request.state = RequestState.DECODING

    def _fail(self, request: Request, detail: str, rejected: bool = False) -> None:
        if request.is_terminal:
            return
        request.rejected = rejected
        request.state = RequestState.FAILED
        request.error_detail = detail
        request.finish_reason = "failed"
        self._finalize(request)

    def _finalize(self, request: Request) -> None:
        """The single terminal funnel: out of the queues, cache released, stream closed."""
        if request in self.active:
            self.active.remove(request)
        if request in self.waiting:
            self.waiting.remove(request)
        try:
            self.runner.release(request)
        except Exception as exc:  # noqa: BLE001 - release must never break teardown
            request.error_detail = f"release error: {exc}"
        request.finish_ns = self.clock()
        request.events.append(
            StreamEvent(token_id=None, finished=True, finish_reason=request.finish_reason)
        )
        if request.state is RequestState.COMPLETED:
            self.metrics.record_e2e_ms((request.finish_ns - request.arrival_ns) / 1e6)
            self.metrics.inc_completed()
        elif request.state is RequestState.CANCELLED:
            self.metrics.inc_cancelled()
        elif request.state is RequestState.TIMED_OUT:
            self.metrics.inc_timed_out()
        elif request.rejected:
            self.metrics.inc_rejected()
        else:
            self.metrics.inc_failed()
