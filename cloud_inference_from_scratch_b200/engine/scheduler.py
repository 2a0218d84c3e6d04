"""Request lifecycle and the iteration-level scheduler above the step function.

The policy is the reference's packed scheduler (src/cloud_engine/scheduler.py); the code is laid
out for this engine's synchronous loop:

* a request is one growing token list (prompt followed by what was generated) and a cursor
  ``tokens_fed``; what a step feeds is the slice behind the cursor, whatever mix of prompt and
  generated tokens that is (which is all that recomputation after a preemption needs);
* one iteration = expire queued requests -> admit -> cut a plan -> run it -> account.  A plan is
  four parallel columns (request, start, length, sample), cut in two passes over the residents
  (single decoded tokens first, then prompt portions) without sorting or per-request objects;
  ``BatchItem`` views are built only for callers that ask for ``plan.items``;
* every way a request can end goes through ``_retire``.

Policy, with the reference's lines:

* states ``waiting -> prefill -> decoding -> completed | cancelled | timed_out | failed``
  (scheduler.py:29-46); submit refuses an empty prompt, ``prompt + max_output_tokens >
  max_model_len`` and a full queue (scheduler.py:233-254);
* admission in arrival order while fewer than ``max_active_sequences`` are resident; a request
  that was preempted comes back only into an empty house (scheduler.py:438-457);
* token budget ``max_batched_tokens`` per step: one token for every decoding request first, then
  prompt portions of at most ``prefill_chunk_size``; a portion that reaches the end of the known
  sequence is sampled (scheduler.py:459-518);
* pages run out -> the resident holding most (allocated tokens, tokens fed, arrival) gives back
  its pages, keeps its tokens, queues again and is recomputed; with one resident the plan's
  requests fail as rejected (scheduler.py:383-394, 527-553);
* EOS (token kept, event carries None) and ``max_output_tokens`` end a request
  (scheduler.py:581-607).

Not here: asyncio, the worker thread, stream queues and the slow-consumer watchdog.  Temperature
sampling is allowed (the reference refuses it, scheduler.py:69-71).
"""

from __future__ import annotations

import time
from collections import deque
from collections.abc import Callable, Sequence
from typing import Any

from .request import (  # noqa: F401  (re-exported: callers import these names from here)
    TERMINAL_STATES,
    BatchItem,
    BatchPlan,
    GenerationConfig,
    PreemptionCandidate,
    RejectedError,
    RejectionReason,
    Request,
    RequestState,
    SchedulingCandidate,
    StreamEvent,
    decode_first_priority,
    largest_sequence_preemption,
)


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
        self.active: list[Request] = []          # residents, in order of admission
        self._submitted = 0
        self._queue_timeout_ns = int(config.queue_timeout_seconds * 1e9)
        self._count_end = {
            RequestState.COMPLETED: metrics.inc_completed,
            RequestState.CANCELLED: metrics.inc_cancelled,
            RequestState.TIMED_OUT: metrics.inc_timed_out,
        }

    # ------------------------------------------------------------------ callers
    def submit(self, prompt_token_ids: Sequence[int], gen_config: GenerationConfig,
               label: str = "") -> Request:
        config = self.config
        if not len(prompt_token_ids):
            raise RejectedError(RejectionReason.CONTEXT_OVERFLOW, "empty prompt")
        if len(prompt_token_ids) + gen_config.max_output_tokens > config.max_model_len:
            raise RejectedError(RejectionReason.CONTEXT_OVERFLOW)
        if len(self.waiting) >= config.max_queue_size:
            raise RejectedError(RejectionReason.QUEUE_FULL)
        self._submitted += 1
        request = Request(f"req-{self._submitted:08d}", prompt_token_ids, gen_config, self.clock(),
                          sequence_number=self._submitted, label=label)
        self.waiting.append(request)
        return request

    def cancel(self, request: Request) -> None:
        if not request.is_terminal:
            self._retire(request, RequestState.CANCELLED, "cancelled")

    @property
    def has_work(self) -> bool:
        return bool(self.waiting) or bool(self.active)

    def run_until_idle(self, max_iterations: int | None = None) -> int:
        done = 0
        while self.has_work and (max_iterations is None or done < max_iterations):
            self.step()
            done += 1
        return done

    # ------------------------------------------------------------------ one iteration
    def step(self) -> bool:
        """Runs one iteration; returns whether anything moved."""
        moved = self._expire_queued(self.clock())
        moved = self._admit() or moved
        plan = self.plan_step()
        if not plan.requests:
            return moved
        try:
            sampled = self.runner.execute_batch(plan)
        except Exception as exc:  # noqa: BLE001 - whatever the step raises ends in _retire
            self._step_failed(plan, exc)
            return True
        self._account(plan, sampled, self.clock())
        return True

    def plan_step(self) -> BatchPlan:
        """Cuts the next step out of the residents under the token budget."""
        if self.scheduling_priority is decode_first_priority:
            order = self._decode_first_order()
        else:
            order = self._custom_order()
        budget = self.config.max_batched_tokens
        portion = self.config.prefill_chunk_size
        requests: list[Request] = []
        starts: list[int] = []
        lengths: list[int] = []
        samples: list[bool] = []
        for request, decoding in order:
            if budget <= 0:
                break
            fed = request.tokens_fed
            left = len(request.tokens) - fed
            take = 1 if decoding else min(left, portion, budget)
            requests.append(request)
            starts.append(fed)
            lengths.append(take)
            samples.append(take == left)
            budget -= take
        return BatchPlan(requests, starts, lengths, samples)

    def _decode_first_order(self) -> list[tuple[Request, bool]]:
        """(request, is a single decode token) for every resident with tokens to feed: the decoding
        ones, then the others, each class in order of admission."""
        decoding, DECODING = [], RequestState.DECODING
        others = []
        for request in self.active:
            left = len(request.tokens) - request.tokens_fed
            if left <= 0 or request.state in TERMINAL_STATES:
                continue
            if left == 1 and request.state is DECODING:
                decoding.append((request, True))
            else:
                others.append((request, False))
        return decoding + others

    def _custom_order(self) -> list[tuple[Request, bool]]:
        keyed = []
        for index, request in enumerate(self.active):
            left = len(request.tokens) - request.tokens_fed
            if left <= 0 or request.is_terminal:
                continue
            decoding = left == 1 and request.state is RequestState.DECODING
            seen = SchedulingCandidate(request.request_id, "decode" if decoding else "prefill", left,
                                       request.prompt_len, request.generated_count, request.arrival_ns)
            keyed.append((self.scheduling_priority(seen), index, request, decoding))
        keyed.sort(key=lambda entry: entry[:2])
        return [(request, decoding) for _, _, request, decoding in keyed]

    # ------------------------------------------------------------------ around the step
    def _expire_queued(self, now: int) -> bool:
        late = [r for r in self.waiting
                if not r.preemption_count and now - r.arrival_ns > self._queue_timeout_ns]
        for request in late:
            self._retire(request, RequestState.TIMED_OUT, "timed_out")
        return bool(late)

    def _admit(self) -> bool:
        admitted = False
        room = self.config.max_active_sequences
        while self.waiting and len(self.active) < room:
            head = self.waiting[0]
            if head.preemption_count and self.active:
                break      # a preempted request returns only when the residents have drained
            self.waiting.popleft()
            try:
                self.runner.admit(head)
            except Exception as exc:  # noqa: BLE001
                self._retire(head, RequestState.FAILED, "failed", f"admission refused: {exc}",
                             rejected=bool(getattr(exc, "is_capacity_error", False)))
                continue
            head.state = RequestState.PREFILL
            self.active.append(head)
            admitted = True
        return admitted

    def _account(self, plan: BatchPlan, sampled: dict[str, int], now: int) -> None:
        metrics = self.metrics
        metrics.record_input_tokens(plan.token_count)
        for request, start, length, sample in zip(plan.requests, plan.starts, plan.lengths, plan.samples):
            if request.is_terminal:     # cancelled while the step ran
                continue
            end = start + length
            request.tokens_fed = end
            again = min(end, request.recompute_until) - start
            if again > 0:
                request.recomputed_tokens += again
                metrics.record_recomputed_tokens(again)
            if not sample:
                request.state = RequestState.PREFILL
                continue
            token = sampled.get(request.request_id)
            if token is None:
                self._retire(request, RequestState.FAILED, "failed",
                             "the step returned no token for a sampled request")
                continue
            self._take_token(request, int(token), now)
        metrics.record_iteration(len(plan.requests))

    def _take_token(self, request: Request, token: int, now: int) -> None:
        metrics = self.metrics
        request.tokens.append(token)
        if request.first_token_ns is None:
            request.first_token_ns = now
            metrics.record_ttft_ms((now - request.arrival_ns) / 1e6)
        else:
            metrics.record_itl_ms((now - request.last_token_ns) / 1e6)
        request.last_token_ns = now
        metrics.record_output_token(1)
        limits = request.config
        if limits.eos_token_id is not None and token == limits.eos_token_id:
            request.events.append(StreamEvent(None))
            self._retire(request, RequestState.COMPLETED, "eos_token_reached")
        elif request.generated_count >= limits.max_output_tokens:
            request.events.append(StreamEvent(token))
            self._retire(request, RequestState.COMPLETED, "max_output_tokens_reached")
        else:
            request.events.append(StreamEvent(token))
            request.state = RequestState.DECODING

    def _step_failed(self, plan: BatchPlan, exc: Exception) -> None:
        out_of_pages = bool(getattr(exc, "is_capacity_error", False))
        if out_of_pages and self._evict_one():
            return                      # the next iteration plans again with the pages that came back
        if out_of_pages:
            detail, rejected = f"KV capacity cannot fit one runnable sequence: {exc}", True
        else:
            detail, rejected = f"packed forward failed: {exc}", False
        for request in plan.requests:
            if not request.is_terminal:
                self._retire(request, RequestState.FAILED, "failed", detail, rejected=rejected)

    def _evict_one(self) -> bool:
        """Takes the pages of one resident away (it keeps its tokens and queues again); False when
        there is nobody to take them from."""
        residents = [r for r in self.active if not r.is_terminal]
        if len(residents) < 2:
            return False
        held = getattr(self.runner, "allocated_tokens", None)
        rank = self.preemption_priority
        victim = max(residents, key=lambda r: rank(PreemptionCandidate(
            r.request_id, held(r) if held else 0, r.tokens_fed, r.generated_count, r.arrival_ns)))
        self.active.remove(victim)
        self.runner.release(victim)
        victim.recompute_until = max(victim.recompute_until, victim.tokens_fed)
        victim.tokens_fed = 0
        victim.preemption_count += 1
        victim.state = RequestState.WAITING
        self.waiting.append(victim)
        self.metrics.inc_preempted()
        return True

    def _retire(self, request: Request, state: RequestState, reason: str, detail: str = "",
                rejected: bool = False) -> None:
        """The one way out: the state becomes final, the request leaves both queues, its cache
        goes back, its stream is closed and the matching counter moves."""
        if request.is_terminal:
            return
        request.state = state
        request.finish_reason = reason
        request.rejected = rejected
        if detail:
            request.error_detail = detail
        for queue in (self.active, self.waiting):
            try:
                queue.remove(request)
            except ValueError:
                pass
        try:
            self.runner.release(request)
        except Exception as exc:  # noqa: BLE001 - a failing release must not stop the teardown
            request.error_detail = f"release error: {exc}"
        request.finish_ns = self.clock()
        request.events.append(StreamEvent(None, finished=True, finish_reason=reason))
        if state is RequestState.COMPLETED:
            self.metrics.record_e2e_ms((request.finish_ns - request.arrival_ns) / 1e6)
        count = self._count_end.get(state)
        if count is None:
            count = self.metrics.inc_rejected if rejected else self.metrics.inc_failed
        count()
