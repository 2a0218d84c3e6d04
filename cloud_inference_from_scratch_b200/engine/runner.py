"""The scheduler's runner: turns a batch plan into one step, samples on the device, returns ids.

Interface towards the scheduler (duck-typed, as in the reference, src/cloud_engine/scheduler.py:287-290,
449, 523, 531): ``admit``, ``release``, ``allocated_tokens``, ``execute_batch(plan) -> {request id:
token id}``.  Counterpart of ``RaggedRunner`` (src/cloud_engine/engine.py:193-488).

A plan made only of single decoded tokens is replayed from a CUDA graph captured per
power-of-two batch size (engine.py:320-408): the step's metadata goes into the graph's fixed
buffers with one copy, rows beyond the real batch repeat the last real row (they rewrite the
same cache slot with the same values and their tokens are dropped; ``request_active`` is 0 for
them).  Graphs are not used when a mixer keeps per-request state and has not declared that it
honours that flag (``state_in_graphs``), because a repeated row would advance the state twice.
Sampling parameters (temperature and draw key per row) ride in the same metadata copy; only
the sampled token ids and the device error word come back to the host.
"""

from __future__ import annotations

from typing import Any

import numpy as np

from ..sampling.keys import as_signed, draw_key
from .profiling import nvtx_range
from .step import MetadataBuffer, StepEntry


class _DecodeGraph:
    """One captured decode step for one batch size: its metadata buffers, its result buffers."""

    def __init__(self, bucket: int, meta: MetadataBuffer, graph: Any, result_dev: Any, ctx: Any,
                 torch: Any) -> None:
        self.bucket = bucket
        self.meta = meta
        self.graph = graph
        self.result_dev = result_dev
        self.result_host = torch.zeros(1 + bucket, dtype=torch.int32, pin_memory=True)
        self.token_ids = ctx.token_ids          # device view: where the step reads its token ids
        self.event = torch.cuda.Event()
        self.logits: Any = None                 # the float32 logits buffer the captured step writes


class _InFlight:
    """A decode step that has been launched and whose tokens have not been read yet."""

    def __init__(self, graph: _DecodeGraph, request_ids: list[str], spans: dict, real: int,
                 committed: bool, logits: Any = None) -> None:
        self.graph = graph
        self.request_ids = request_ids
        self.spans = spans
        self.real = real
        self.committed = committed
        self.logits = logits     # a copy of the step's logits rows, only while logits are traced


class EngineRunner:
    def __init__(self, core: Any, config: Any) -> None:
        import torch

        self.torch = torch
        self.core = core
        self.config = config
        self.step = core.step
        self.ops = core.runtime.ops
        self.max_rows = max(1, config.max_active_sequences)
        self.result_dev = torch.zeros(1 + self.max_rows, dtype=torch.int32, device=core.runtime.device)
        self.result_host = torch.zeros(1 + self.max_rows, dtype=torch.int32, pin_memory=True)
        self.ops.error_word = self.result_dev[0:1]
        # Steps are captured in CUDA graphs (and decode batches padded by repeating their last row)
        # unless a part keeps per-request state and has not declared ``state_in_graphs``: that its
        # forward runs on the device alone and leaves the state of rows with request_active == 0 alone.
        keepers = [layer.cache_part for layer in core.model.layers
                   if layer.cache_part is not None and getattr(layer.cache_part, "state_spec", lambda: None)() is not None]
        self.use_graphs = bool(config.cuda_graph_decode) and all(
            getattr(part, "state_in_graphs", False) for part in keepers)
        self.stateful = bool(keepers)
        if self.use_graphs:
            core.step.enable_graphs(config.max_model_len)
        self.table_width = -(-config.max_model_len // core.page_size)
        self._graphs: dict[tuple[int, int], _DecodeGraph] = {}
        self._parity = 0
        self._ahead: _InFlight | None = None   # the next decode step, launched before it was asked for
        # The next decode step is launched before the host knows whether it will be asked for; if it
        # is not, it is dropped.  What a dropped step wrote to pages lies beyond every committed
        # length and is written again, but per-request state would have been advanced for good: no
        # steps ahead when a part keeps state.
        self.pipeline_decode = not self.stateful
        self.steps_launched_ahead = 0
        self.steps_ahead_adopted = 0
        self.steps_ahead_dropped = 0
        # For tests and self-checks: with ``trace_logits`` on, every step leaves (request ids,
        # position of each sampled row's token, a device copy of the float32 logits rows) in
        # ``logit_trace``.  A decode step's rows are copied on the stream right behind the step,
        # before the step launched ahead of the host can overwrite the shared logits buffer.
        self.trace_logits = False
        self.logit_trace: list[tuple[list[str], list[int], Any]] = []
        self.forward_invocations = 0
        self.max_forward_request_count = 0
        self.cuda_graph_captures = 0
        self.cuda_graph_replays = 0
        self.forward_plans: list[tuple[tuple[str, int, int, bool], ...]] = []
        self.launches_per_graph: dict[int, int] = {}  # kernels of ours inside each captured graph
        self.d2h_bytes = 0

    # ------------------------------------------------------------------ scheduler interface
    def admit(self, request: Any) -> None:
        self.step.admit(request.request_id)

    def release(self, request: Any) -> None:
        self.step.release(request.request_id)

    def allocated_tokens(self, request: Any) -> int:
        return self.core.cache.allocated_tokens(request.request_id)

    def execute_batch(self, plan: Any) -> dict[str, int]:
        requests, starts, lengths, samples = plan.requests, plan.starts, plan.lengths, plan.samples
        entries = [
            StepEntry(request.request_id, request.tokens[start:start + length],
                      want=(length - 1,) if sample else (), start_pos=start)
            for request, start, length, sample in zip(requests, starts, lengths, samples)
        ]
        sampled = [request for request, sample in zip(requests, samples) if sample]
        self.forward_invocations += 1
        self.max_forward_request_count = max(self.max_forward_request_count, len(requests))
        self.forward_plans.append(
            tuple(zip((r.request_id for r in requests), starts, lengths, samples))
        )
        if len(self.forward_plans) > 256:
            del self.forward_plans[:128]
        decode_only = plan.decode_only
        phase = "decode" if decode_only else "mixed"
        with nvtx_range(f"ragged.forward.{phase}.requests_{len(requests)}.tokens_{plan.token_count}"):
            if decode_only and self.use_graphs and len(requests) <= self.max_rows:
                tokens = self._pipelined_decode(requests, starts, entries)
            else:
                self._drop_ahead()   # a step launched ahead committed nothing
                tokens = self._eager(entries, sampled)
        return {request.request_id: int(tokens[i]) for i, request in enumerate(sampled)}

    def _drop_ahead(self) -> None:
        if self._ahead is not None:
            self.steps_ahead_dropped += 1
            self._ahead = None

    # ------------------------------------------------------------------ sampling parameters
    @staticmethod
    def _sampling_arrays(sampled: list[Any], rows: int, ahead: int = 0) -> dict[str, np.ndarray]:
        """Temperature and draw key per sampled row; ``ahead`` = 1 for the step after the current
        one (its output index is one further).  Rows beyond the real ones repeat the last real row,
        so that a padded row samples what the row it repeats samples."""
        temperature = np.zeros(rows, dtype=np.float32)
        keys = np.zeros(rows, dtype=np.int64)
        for index, request in enumerate(sampled):
            temperature[index] = request.config.temperature
            if request.config.temperature > 0:
                keys[index] = as_signed(
                    draw_key(request.config.seed, request.sequence_number, request.generated_count + ahead)
                )
        if sampled and rows > len(sampled):
            temperature[len(sampled):] = temperature[len(sampled) - 1]
            keys[len(sampled):] = keys[len(sampled) - 1]
        return {"temperature": temperature.view(np.int32), "keys": keys.view(np.int32)}

    def _launch_sampling(self, logits: Any, ctx: Any, result_dev: Any, rows: int) -> None:
        torch = self.torch
        params = ctx.extras["sampling"]
        self.ops.sample(logits, params["temperature"].view(torch.float32),
                        params["keys"].view(torch.int64), result_dev[1:1 + rows])

    def _read_back(self, result_dev: Any, rows: int) -> np.ndarray:
        with nvtx_range("ragged.sample.readback"):
            self.result_host[:1 + rows].copy_(result_dev[:1 + rows], non_blocking=True)
            self.torch.cuda.current_stream().synchronize()
        self.d2h_bytes = 4 * (1 + rows)
        values = self.result_host[:1 + rows].numpy()
        if values[0]:
            self.ops.error_word = result_dev[0:1]
            self.ops.check_errors()
        return values[1:].copy()

    # ------------------------------------------------------------------ eager (mixed) step
    def _eager(self, entries: list[StepEntry], sampled: list[Any]) -> np.ndarray:
        step = self.step
        with nvtx_range("ragged.kv.ensure_capacity"):
            host, _, spans = step.prepare(entries)
        rows = len(sampled)
        host.extras["sampling"] = self._sampling_arrays(sampled, rows)
        self.ops.error_word = self.result_dev[0:1]
        ctx, logits = step.forward_host(host)
        with nvtx_range("ragged.kv.commit"):
            self.core.cache.commit_lengths({rid: end for rid, (_, end) in spans.items()})
        step.steps_run += 1
        step.tokens_run += host.num_tokens
        if rows:
            self._launch_sampling(logits, ctx, self.result_dev, rows)
            if self.trace_logits:
                ids = [request.request_id for request in sampled]
                self.logit_trace.append((ids, [spans[rid][1] - 1 for rid in ids], logits[:rows].clone()))
        return self._read_back(self.result_dev, rows)

    # ------------------------------------------------------------------ graphed decode
    @staticmethod
    def _bucket(batch: int) -> int:
        return 1 << (batch - 1).bit_length()

    def _pad(self, host: Any, bucket: int) -> None:
        """Repeats the last row until the batch has ``bucket`` requests of one token each."""
        real = host.num_requests
        extra = bucket - real
        if extra <= 0:
            return

        def grow(array: np.ndarray) -> np.ndarray:
            return np.concatenate([array, np.repeat(array[-1:], extra, axis=0)])

        host.token_ids = grow(host.token_ids)
        host.positions = grow(host.positions)
        host.context_lens = grow(host.context_lens)
        host.query_lens = grow(host.query_lens)
        host.slots = grow(host.slots)
        host.request_active = np.concatenate([host.request_active, np.zeros(extra, dtype=np.int32)])
        host.request_of_token = np.arange(bucket, dtype=np.int32)
        host.query_start = np.arange(bucket + 1, dtype=np.int32)
        host.logit_rows = np.arange(bucket, dtype=np.int32)
        host.num_single = bucket
        host.tables = [grow(table) for table in host.tables]

    def _launch_decode(self, entries: list[StepEntry], sampled: list[Any], ahead: int,
                       feed: _DecodeGraph | None) -> _InFlight:
        """Prepares and launches one decode step from its CUDA graph (captured on first use).

        ``feed``: take the token ids from the tokens the step in ``feed`` is sampling, on the
        device, instead of from ``entries`` (whose ids are placeholders then)."""
        torch = self.torch
        step = self.step
        real = len(entries)
        bucket = self._bucket(real)
        with nvtx_range("ragged.kv.ensure_capacity"):
            host, _, spans = step.prepare(entries, table_width=self.table_width)
        self._pad(host, bucket)
        host.extras["sampling"] = self._sampling_arrays(sampled, bucket, ahead)
        for key, mixer in step.planners.items():
            host.extras[key] = mixer.plan(host, self.core.cache)
        self._parity ^= 1
        cached = self._graphs.get((bucket, self._parity))
        if cached is None:
            if feed is not None:
                raise RuntimeError("a decode graph is captured by a step that has its token ids")
            meta = MetadataBuffer(self.core.runtime.device, words=1 << 12)
            result_dev = torch.zeros(1 + bucket, dtype=torch.int32, device=self.core.runtime.device)
            # the launches run once before they are captured and replayed: with per-request state
            # that first run sees every row as inactive, so that the state moves once, not twice
            active = host.request_active
            if self.stateful:
                host.request_active = np.zeros_like(active)
            ctx = step.upload(host, meta)
            self.ops.error_word = result_dev[0:1]
            # once eagerly (allocates workspace, loads kernels), then capture the same launches
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                logits = self.core.model.forward(ctx)
                self._launch_sampling(logits, ctx, result_dev, bucket)
            torch.cuda.current_stream().wait_stream(side)
            torch.cuda.synchronize()
            if self.stateful:
                host.request_active = active
                ctx = step.upload(host, meta)      # the same addresses, the real flags
            graph = torch.cuda.CUDAGraph()
            self.core.runtime.workspace.frozen = True
            self.ops.freeze_scratch()
            launches_before = self.ops.launches
            with torch.cuda.graph(graph):
                logits = self.core.model.forward(ctx)
                self._launch_sampling(logits, ctx, result_dev, bucket)
            self.launches_per_graph[bucket] = self.ops.launches - launches_before
            cached = _DecodeGraph(bucket, meta, graph, result_dev, ctx, torch)
            cached.logits = logits
            self._graphs[(bucket, self._parity)] = cached
            self.cuda_graph_captures += 1
        else:
            step.upload(host, cached.meta)
            if feed is not None:
                # row i reads the token that row i of the step before it is sampling (pad rows the last one's)
                self.ops.feed_tokens(feed.result_dev[1:], cached.token_ids, real)
        cached.graph.replay()
        self.cuda_graph_replays += 1
        step.steps_run += 1
        step.tokens_run += real
        kept = cached.logits[:real].clone() if self.trace_logits else None
        return _InFlight(cached, [entry.request_id for entry in entries], spans, real, committed=False,
                         logits=kept)

    def _commit(self, flight: _InFlight) -> None:
        if not flight.committed:
            with nvtx_range("ragged.kv.commit"):
                self.core.cache.commit_lengths({rid: end for rid, (_, end) in flight.spans.items()})
            flight.committed = True

    def _launch_ahead(self, requests: list[Any], ends: list[int], current: _InFlight) -> _InFlight | None:
        """Launches the decode step that will most likely be asked for next: the same requests,
        one position further (``ends``), their token ids taken on the device from what ``current``
        samples.  It commits nothing; if the next plan turns out different it is simply dropped
        (what it wrote lies beyond every committed length and is written again before it is read)."""
        if not self.pipeline_decode or (current.graph.bucket, self._parity ^ 1) not in self._graphs:
            return None
        for request, end in zip(requests, ends):
            if request.generated_count + 1 >= request.config.max_output_tokens:
                return None    # this request ends with the token being sampled now
            if end + 1 > self.config.max_model_len:
                return None
        entries = [StepEntry(request.request_id, (0,), want=(0,), start_pos=end)
                   for request, end in zip(requests, ends)]
        try:
            flight = self._launch_decode(entries, requests, ahead=1, feed=current.graph)
        except Exception as exc:  # noqa: BLE001 - no pages (or anything else): run the step when asked
            if not bool(getattr(exc, "is_capacity_error", False)):
                raise
            return None    # pages ran out while preparing: nothing was launched, nothing flipped
        self.steps_launched_ahead += 1
        return flight

    def _pipelined_decode(self, requests: list[Any], starts: list[int], entries: list[StepEntry]) -> np.ndarray:
        ahead, self._ahead = self._ahead, None
        current = None
        if ahead is not None:
            same = ahead.request_ids == [request.request_id for request in requests] and all(
                ahead.spans[request.request_id][0] == start for request, start in zip(requests, starts)
            )
            if same:
                current = ahead
                self.steps_ahead_adopted += 1
            else:
                self.steps_ahead_dropped += 1
        if current is None:
            current = self._launch_decode(entries, requests, ahead=0, feed=None)
        self._commit(current)
        graph = current.graph
        with nvtx_range("ragged.sample.readback"):
            graph.result_host.copy_(graph.result_dev, non_blocking=True)
            graph.event.record()
        # while the device works on the current step, the next one is prepared and queued
        self._ahead = self._launch_ahead(requests, [start + 1 for start in starts], current)
        graph.event.synchronize()
        self.d2h_bytes = 4 * (1 + graph.bucket)
        values = graph.result_host.numpy()
        if values[0]:
            self._ahead = None
            self.ops.error_word = graph.result_dev[0:1]
            self.ops.check_errors()
        if current.logits is not None:
            self.logit_trace.append(([request.request_id for request in requests], list(starts), current.logits))
        return values[1:1 + current.real].copy()
