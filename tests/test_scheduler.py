"""The scheduler's decisions, with a fake step function that models the cache as a token budget
(the method of the reference's tests/test_ragged_scheduler.py: FakePackedRunner)."""

import pytest

from cloud_inference_from_scratch_b200 import InferenceEngine, build_config
from cloud_inference_from_scratch_b200.engine import (
    GenerationConfig,
    Metrics,
    RejectedError,
    RejectionReason,
    RequestState,
    Scheduler,
)


class CapacityError(Exception):
    is_capacity_error = True


class FakeRunner:
    """Next token = 100 + number of tokens generated so far; the cache is a count of tokens."""

    def __init__(self, capacity_tokens=10**9, fail_on=None):
        self.capacity = capacity_tokens
        self.held: dict[str, int] = {}
        self.plans = []
        self.fail_on = fail_on
        self.released = []

    def admit(self, request):
        self.held[request.request_id] = 0

    def release(self, request):
        self.held.pop(request.request_id, None)
        self.released.append(request.request_id)

    def allocated_tokens(self, request):
        return self.held.get(request.request_id, 0)

    def execute_batch(self, plan):
        self.plans.append([(i.request.request_id, i.start_pos, i.query_length, i.sample, i.is_decode)
                           for i in plan.items])
        if self.fail_on is not None and len(self.plans) == self.fail_on:
            raise RuntimeError("injected failure")
        wanted = dict(self.held)
        for item in plan.items:
            assert item.start_pos == item.request.tokens_fed
            wanted[item.request.request_id] = item.end_pos
        if sum(wanted.values()) > self.capacity:
            raise CapacityError("out of tokens")
        self.held = wanted
        return {i.request.request_id: 100 + i.request.generated_count for i in plan.items if i.sample}


def make(runner, **overrides):
    config = build_config("ragged", **{"max_model_len": 256, **overrides})
    return Scheduler(config, runner, Metrics()), config


def test_requests_share_one_step_and_decode_goes_first():
    runner = FakeRunner()
    sched, _ = make(runner, max_batched_tokens=64, prefill_chunk_size=64)
    a = sched.submit([1] * 5, GenerationConfig(max_output_tokens=3))
    sched.step()
    b = sched.submit([2] * 7, GenerationConfig(max_output_tokens=2))
    sched.step()
    assert runner.plans[0] == [(a.request_id, 0, 5, True, False)]
    assert runner.plans[1] == [(a.request_id, 5, 1, True, True), (b.request_id, 0, 7, True, False)]
    sched.run_until_idle()
    assert a.generated_token_ids == [100, 101, 102] and b.generated_token_ids == [100, 101]
    assert a.state is RequestState.COMPLETED and a.finish_reason == "max_output_tokens_reached"
    assert runner.held == {} and sorted(runner.released) == [a.request_id, b.request_id]


def test_prompt_is_cut_into_portions_under_the_budget():
    runner = FakeRunner()
    sched, _ = make(runner, max_batched_tokens=5, prefill_chunk_size=4)
    request = sched.submit(list(range(11)), GenerationConfig(max_output_tokens=1))
    sched.run_until_idle()
    assert [plan[0][2] for plan in runner.plans] == [4, 4, 3]
    assert [plan[0][3] for plan in runner.plans] == [False, False, True]
    assert request.generated_token_ids == [100]


def test_budget_is_shared_decode_first_then_portions():
    runner = FakeRunner()
    sched, _ = make(runner, max_batched_tokens=6, prefill_chunk_size=4)
    first = sched.submit([1] * 3, GenerationConfig(max_output_tokens=4))
    sched.step()
    second = sched.submit([2] * 9, GenerationConfig(max_output_tokens=1))
    third = sched.submit([3] * 9, GenerationConfig(max_output_tokens=1))
    sched.step()
    assert runner.plans[1] == [
        (first.request_id, 3, 1, True, True),
        (second.request_id, 0, 4, False, False),
        (third.request_id, 0, 1, False, False),
    ]


def test_active_limit_and_fifo_admission():
    runner = FakeRunner()
    sched, _ = make(runner, max_active_sequences=2)
    requests = [sched.submit([1, 2], GenerationConfig(max_output_tokens=2)) for _ in range(4)]
    sched.step()
    assert [r.state for r in requests[:2]] == [RequestState.DECODING] * 2
    assert [r.state for r in requests[2:]] == [RequestState.WAITING] * 2
    sched.run_until_idle()
    assert all(r.state is RequestState.COMPLETED for r in requests)
    first_seen = [min(i for i, plan in enumerate(runner.plans) if any(p[0] == r.request_id for p in plan))
                  for r in requests]
    assert first_seen == sorted(first_seen)


def test_submit_refusals():
    sched, _ = make(FakeRunner(), max_queue_size=1, max_model_len=16)
    with pytest.raises(RejectedError) as info:
        sched.submit([], GenerationConfig(max_output_tokens=1))
    assert info.value.reason is RejectionReason.CONTEXT_OVERFLOW
    with pytest.raises(RejectedError) as info:
        sched.submit([1] * 10, GenerationConfig(max_output_tokens=7))
    assert info.value.reason is RejectionReason.CONTEXT_OVERFLOW
    sched.submit([1], GenerationConfig(max_output_tokens=1))
    with pytest.raises(RejectedError) as info:
        sched.submit([1], GenerationConfig(max_output_tokens=1))
    assert info.value.reason is RejectionReason.QUEUE_FULL
    with pytest.raises(ValueError):
        GenerationConfig(max_output_tokens=0)
    with pytest.raises(ValueError):
        GenerationConfig(max_output_tokens=1, temperature=-1.0)


def test_eos_ends_a_request_and_keeps_the_token():
    runner = FakeRunner()
    sched, _ = make(runner)
    request = sched.submit([1, 2, 3], GenerationConfig(max_output_tokens=10, eos_token_id=102))
    sched.run_until_idle()
    assert request.generated_token_ids == [100, 101, 102]
    assert request.finish_reason == "eos_token_reached"
    events = list(request.events)
    assert [e.token_id for e in events] == [100, 101, None, None] and events[-1].finished


def test_pages_run_out_preempts_the_largest_and_recomputes_without_token_drift():
    runner = FakeRunner(capacity_tokens=30)
    sched, _ = make(runner, max_batched_tokens=64, prefill_chunk_size=64)
    metrics = sched.metrics
    a = sched.submit([1] * 12, GenerationConfig(max_output_tokens=8))
    b = sched.submit([2] * 10, GenerationConfig(max_output_tokens=8))
    sched.run_until_idle()
    for request in (a, b):
        assert request.state is RequestState.COMPLETED
        assert request.generated_token_ids == [100 + i for i in range(8)]
    assert metrics.counters["preempted_total"] >= 1
    assert metrics.counters["recomputed_total"] >= 12
    assert a.preemption_count + b.preemption_count == metrics.counters["preempted_total"]
    assert runner.held == {}
    # the victim was the one holding more tokens, and it came back only after the other finished
    assert a.preemption_count >= 1 and b.preemption_count == 0
    # a recomputed request samples only when its whole known sequence has been fed again
    resumed = [plan for plan in runner.plans if any(p[0] == a.request_id and p[1] == 0 for p in plan)]
    assert len(resumed) >= 2 and resumed[-1][0][2] > 12 and resumed[-1][0][3] is True


def test_single_request_that_cannot_fit_is_rejected_not_looped():
    runner = FakeRunner(capacity_tokens=8)
    sched, _ = make(runner)
    request = sched.submit([1] * 12, GenerationConfig(max_output_tokens=2))
    sched.run_until_idle(max_iterations=10)
    assert request.state is RequestState.FAILED and request.rejected
    assert "KV capacity" in request.error_detail and runner.held == {}
    assert sched.metrics.counters["rejected_total"] == 1


def test_step_failure_fails_the_plan_and_frees_everything():
    runner = FakeRunner(fail_on=2)
    sched, _ = make(runner)
    a = sched.submit([1, 2], GenerationConfig(max_output_tokens=5))
    sched.run_until_idle()
    assert a.state is RequestState.FAILED and "injected failure" in a.error_detail
    assert runner.held == {} and sched.metrics.counters["failed_total"] == 1
    c = sched.submit([1, 2], GenerationConfig(max_output_tokens=2))
    sched.run_until_idle()
    assert c.state is RequestState.COMPLETED


def test_cancel_is_idempotent_and_queue_timeout():
    now = [0]
    runner = FakeRunner()
    config = build_config("ragged", max_active_sequences=1, queue_timeout_seconds=1.0)
    sched = Scheduler(config, runner, Metrics(), clock=lambda: now[0])
    a = sched.submit([1], GenerationConfig(max_output_tokens=50))
    b = sched.submit([1], GenerationConfig(max_output_tokens=1))
    sched.step()
    now[0] = 2_000_000_000
    sched.step()
    assert b.state is RequestState.TIMED_OUT
    sched.cancel(a)
    sched.cancel(a)
    assert a.state is RequestState.CANCELLED and runner.held == {}
    assert sched.metrics.counters["cancelled_total"] == 1 and not sched.has_work


def test_custom_policies_are_used():
    runner = FakeRunner(capacity_tokens=30)
    config = build_config("ragged", max_batched_tokens=64, prefill_chunk_size=64)
    sched = Scheduler(
        config, runner, Metrics(),
        scheduling_priority=lambda c: (c.phase == "decode",),           # prompt portions first
        preemption_priority=lambda c: (-c.allocated_tokens,),           # smallest victim
    )
    a = sched.submit([1] * 12, GenerationConfig(max_output_tokens=8))
    sched.step()
    b = sched.submit([2] * 10, GenerationConfig(max_output_tokens=8))
    sched.step()
    assert runner.plans[1][0][0] == b.request_id
    sched.run_until_idle()
    assert b.preemption_count >= 1 and a.preemption_count == 0


def test_engine_facade_with_injected_runner_streams_and_waits():
    engine = InferenceEngine(build_config("ragged"), runner_factory=lambda config: FakeRunner())
    with engine:
        first = engine.submit([1, 2, 3], GenerationConfig(max_output_tokens=3))
        second = engine.submit([4], GenerationConfig(max_output_tokens=2))
        streamed = [event.token_id for event in first.stream()]
        assert streamed == [100, 101, 102]
        result = second.wait()
        assert result.token_ids == [100, 101] and result.input_tokens == 1
        assert result.finish_reason == "max_output_tokens_reached" and result.ttft_ms is not None
        snapshot = engine.snapshot_metrics()
        assert snapshot["requests"]["completed_total"] == 2
        assert snapshot["requests"]["output_tokens_total"] == 5
        cancelled = engine.submit([1], GenerationConfig(max_output_tokens=9))
        cancelled.cancel()
        with pytest.raises(RuntimeError, match="cancelled"):
            cancelled.wait()
