"""Counters and latency windows of the engine (trimmed from src/cloud_engine/metrics.py:52-200:
the same counters and percentiles, bounded windows, no wall-clock pruning)."""

from __future__ import annotations

import time
from collections import deque
from typing import Any


def _percentile(values: list[float], fraction: float) -> float | None:
    if not values:
        return None
    ordered = sorted(values)
    index = min(len(ordered) - 1, max(0, int(round(fraction * (len(ordered) - 1)))))
    return ordered[index]


class Metrics:
    def __init__(self, window: int = 4096) -> None:
        self._ttft = deque(maxlen=window)
        self._itl = deque(maxlen=window)
        self._e2e = deque(maxlen=window)
        self.counters = dict(
            completed_total=0, cancelled_total=0, timed_out_total=0, failed_total=0,
            rejected_total=0, preempted_total=0, recomputed_total=0, input_tokens_total=0,
            output_tokens_total=0, iterations_total=0, batched_requests_total=0,
        )
        self.started_ns = time.monotonic_ns()

    def now(self) -> int:
        return time.monotonic_ns()

    def record_ttft_ms(self, value: float) -> None:
        self._ttft.append(value)

    def record_itl_ms(self, value: float) -> None:
        self._itl.append(value)

    def record_e2e_ms(self, value: float) -> None:
        self._e2e.append(value)

    def record_input_tokens(self, count: int) -> None:
        self.counters["input_tokens_total"] += count

    def record_output_token(self, count: int) -> None:
        self.counters["output_tokens_total"] += count

    def record_recomputed_tokens(self, count: int) -> None:
        self.counters["recomputed_total"] += count

    def record_iteration(self, requests: int) -> None:
        self.counters["iterations_total"] += 1
        self.counters["batched_requests_total"] += requests

    def inc_completed(self) -> None:
        self.counters["completed_total"] += 1

    def inc_cancelled(self) -> None:
        self.counters["cancelled_total"] += 1

    def inc_timed_out(self) -> None:
        self.counters["timed_out_total"] += 1

    def inc_failed(self) -> None:
        self.counters["failed_total"] += 1

    def inc_rejected(self) -> None:
        self.counters["rejected_total"] += 1

    def inc_preempted(self) -> None:
        self.counters["preempted_total"] += 1

    def snapshot(self) -> dict[str, Any]:
        def window(values: deque) -> dict[str, Any]:
            data = list(values)
            return dict(count=len(data), p50=_percentile(data, 0.5), p95=_percentile(data, 0.95))

        return dict(
            requests=dict(self.counters),
            latency_ms=dict(ttft=window(self._ttft), itl=window(self._itl), e2e=window(self._e2e)),
            scheduler={},
            kv_cache={},
            uptime_seconds=(time.monotonic_ns() - self.started_ns) / 1e9,
        )
