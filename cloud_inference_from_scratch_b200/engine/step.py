"""The step function: one flat batch of (request, its next tokens) through the model, from the cache.

Contract (the reference's ``RaggedRunner._pack`` + ``execute_batch``,
src/cloud_engine/engine.py:231-301, 439-488): a step holds any mix of prompt portions and
single decoded tokens, no request twice; the cache tables of all its requests grow in one
all-or-nothing transaction BEFORE anything is launched, so running out of pages is a host
exception and nothing has changed; keys and values of every token are written; lengths are
committed after the launch sequence was issued; float32 logits come back only for the rows
that were asked for.

Differences: all integer metadata of the step is laid out in one pinned buffer and copied to
the device once (the reference makes seven tensors plus one copy per request row,
engine.py:264-300); positions and request indices are built with vectorised numpy, not
per-token Python loops; a step made only of single tokens can be replayed from a CUDA graph
(``GraphedDecode``), padded to a power-of-two batch by repeating its last row, as the reference
pads (engine.py:320-356).
"""

from __future__ import annotations

from collections import OrderedDict

from collections.abc import Hashable, Sequence
from dataclasses import dataclass, field
from typing import Any

import numpy as np

from ..cache.manager import CacheManager
from .context import StepContext


@dataclass
class StepEntry:
    request_id: Hashable
    token_ids: Sequence[int]
    want: Sequence[int] = ()          # places among token_ids whose logits are wanted
    start_pos: int | None = None      # default: the request's committed length


@dataclass
class HostBatch:
    """The integer arrays of one step on the host (numpy int32)."""

    token_ids: np.ndarray
    positions: np.ndarray
    request_of_token: np.ndarray
    query_start: np.ndarray
    context_lens: np.ndarray
    query_lens: np.ndarray
    slots: np.ndarray
    request_active: np.ndarray   # 1 per request; 0 for a row that only pads a captured batch
    logit_rows: np.ndarray
    tables: list[np.ndarray]
    extras: dict[Any, dict[str, np.ndarray]] = field(default_factory=dict)
    # requests that bring exactly one token come first in a step; this many lead the batch (their
    # token row equals their request index, which is what the decode kernels count on)
    num_single: int = 0

    @property
    def num_tokens(self) -> int:
        return int(self.token_ids.shape[0])

    @property
    def num_requests(self) -> int:
        return int(self.query_lens.shape[0])


@dataclass
class StepResult:
    logits: Any                                   # float32 [R, vocab] on the device, or None
    rows: list[tuple[Hashable, int]]              # (request id, place in its entry) per logits row


def _align(n: int, to: int = 4) -> int:
    return (n + to - 1) // to * to


class MetadataBuffer:
    """A pinned host buffer and its device twin; ``upload`` lays the arrays out and copies once."""

    def __init__(self, device: Any, words: int = 1 << 16) -> None:
        import torch

        self.torch = torch
        self.device = device
        self.capacity = 0
        self.host = None
        self.dev = None
        self.event = torch.cuda.Event()
        self.pending = False
        self.reserve(words)

    def reserve(self, words: int) -> None:
        if words <= self.capacity:
            return
        torch = self.torch
        if self.pending:
            self.event.synchronize()
            self.pending = False
        self.capacity = max(words, 2 * self.capacity)
        self.host = torch.empty(self.capacity, dtype=torch.int32, pin_memory=True)
        self.host_np = self.host.numpy()
        self.dev = torch.empty(self.capacity, dtype=torch.int32, device=self.device)

    def upload(self, arrays: list[np.ndarray]) -> list[Any]:
        """Copies the arrays (any shape, int32) and returns device views of the same shapes."""
        offsets = []
        total = 0
        for array in arrays:
            offsets.append(total)
            total += _align(array.size)
        self.reserve(max(total, 4))
        if self.pending:
            self.event.synchronize()  # the previous copy must have left the pinned buffer
        for array, offset in zip(arrays, offsets, strict=True):
            if array.size:
                self.host_np[offset:offset + array.size] = array.reshape(-1)
        if total:
            self.dev[:total].copy_(self.host[:total], non_blocking=True)
            self.event.record()
            self.pending = True
        return [
            self.dev[offset:offset + array.size].view(array.shape)
            for array, offset in zip(arrays, offsets, strict=True)
        ]


class _StepGraph:
    """One captured forward pass for one shape of step: its own metadata buffer, whose device
    addresses the captured kernels hold, and the logits it leaves."""

    def __init__(self, meta: MetadataBuffer, graph: Any, logits: Any, stamp: Any) -> None:
        self.meta, self.graph, self.logits, self.stamp = meta, graph, logits, stamp


MAX_STEP_GRAPHS = 8          # captured shapes kept (least recently used goes first)
# A capture costs about two runs of the step plus the instantiation of the graph, and pays only
# where the host issues launches more slowly than the device runs them: wait for a shape to prove
# that it recurs.
CAPTURE_AT_OCCURRENCE = 3    # a shape is captured when it is seen for the third time


class StepFunction:
    def __init__(self, model: Any, runtime: Any, cache: CacheManager, pools: Any) -> None:
        self.model = model
        self.runtime = runtime
        self.cache = cache
        self.pools = pools
        self.vocab_size = model.spec.vocab_size
        self.num_groups = len(cache.groups)
        self.meta = MetadataBuffer(runtime.device)
        self.planners = self._collect_planners()
        self.steps_run = 0
        self.tokens_run = 0
        self.h2d_bytes = 0
        # CUDA graphs by shape of step (the lengths of the requests' portions, the number of
        # wanted rows, the sizes of every metadata array): a prompt portion of a common length is
        # many hundred kernel launches that the host would otherwise issue one by one, slower
        # than the device runs them.  Off until ``enable_graphs`` is called.
        self.graphs_enabled = False
        self.fixed_table_width: int | None = None   # block-table columns of every step, if set
        self._graphs: "OrderedDict[Any, _StepGraph]" = OrderedDict()
        self._seen: dict[Any, int] = {}
        self.graph_captures = 0
        self.graph_replays = 0

    def _collect_planners(self) -> dict[Any, Any]:
        """Mixers may add integer work lists of their own to a step's metadata: a mixer with
        ``plan_key`` and ``plan(host, cache)`` is asked once per distinct key."""
        planners: dict[Any, Any] = {}
        for layer in self.model.layers:
            for part in layer.parts.values():
                key = getattr(part, "plan_key", None)
                if key is not None and key not in planners:
                    planners[key] = part
        return planners

    def enable_graphs(self, max_model_len: int) -> None:
        """Steps of a shape seen before run from a captured CUDA graph.  Block tables of such
        steps always have the columns of the longest request the engine admits, so that the
        shape does not depend on how long the requests have grown."""
        self.graphs_enabled = True
        self.fixed_table_width = -(-int(max_model_len) // self.cache.page_size)

    # ------------------------------------------------------------------ admission
    def admit(self, request_id: Hashable) -> int:
        return self.cache.admit(request_id)

    def release(self, request_id: Hashable) -> None:
        self.cache.release(request_id)

    # ------------------------------------------------------------------ packing
    def build_host_batch(self, entries: Sequence[StepEntry], table_width: int | None = None
                         ) -> tuple[HostBatch, list[tuple[Hashable, int]], dict[Hashable, tuple[int, int]]]:
        """Checks the entries and lays the step out.  Inside the step, requests that bring a single
        token are placed before the others (each class in the order given), so that the kernels for
        single queries can take the leading rows of a mixed step; the wanted rows keep the order of
        the entries and of ``want``."""
        cache = self.cache
        seen: set[Hashable] = set()
        starts: list[int] = []
        lens: list[int] = []
        for entry in entries:
            if entry.request_id in seen:
                raise ValueError(f"request {entry.request_id!r} appears twice in one step")
            seen.add(entry.request_id)
            if not cache.is_admitted(entry.request_id):
                raise KeyError(f"request {entry.request_id!r} is not admitted")
            committed = cache.committed_length(entry.request_id)
            start = committed if entry.start_pos is None else int(entry.start_pos)
            if start != committed:
                raise ValueError(
                    f"request {entry.request_id!r}: tokens start at position {start} but the "
                    f"cache holds {committed}"
                )
            if len(entry.token_ids) == 0:
                raise ValueError(f"request {entry.request_id!r} brings no tokens")
            starts.append(start)
            lens.append(len(entry.token_ids))
        count = len(entries)
        singles = [i for i in range(count) if lens[i] == 1]
        order = singles + [i for i in range(count) if lens[i] != 1] if 0 < len(singles) < count else list(range(count))
        place_of = [0] * count
        for placed, index in enumerate(order):
            place_of[index] = placed
        query_lens = np.asarray([lens[i] for i in order], dtype=np.int32)
        context_lens = np.asarray([starts[i] for i in order], dtype=np.int32)
        query_start = np.zeros(count + 1, dtype=np.int32)
        np.cumsum(query_lens, out=query_start[1:])
        total = int(query_start[-1])
        token_ids = np.fromiter(
            (t for i in order for t in entries[i].token_ids), dtype=np.int64, count=total
        )
        if total and (token_ids.min() < 0 or token_ids.max() >= self.vocab_size):
            raise ValueError(f"token id outside the vocabulary of {self.vocab_size}")
        request_of_token = np.repeat(np.arange(count, dtype=np.int32), query_lens)
        positions = (
            np.arange(total, dtype=np.int32)
            - np.repeat(query_start[:-1] - context_lens, query_lens)
        ).astype(np.int32)
        rows: list[tuple[Hashable, int]] = []
        logit_rows: list[int] = []
        for index, entry in enumerate(entries):
            first = int(query_start[place_of[index]])
            for place in entry.want:
                if not 0 <= place < lens[index]:
                    raise ValueError(
                        f"request {entry.request_id!r}: wanted place {place} is outside its "
                        f"{lens[index]} tokens"
                    )
                rows.append((entry.request_id, int(place)))
                logit_rows.append(first + int(place))
        spans = {
            entry.request_id: (starts[i], starts[i] + lens[i]) for i, entry in enumerate(entries)
        }
        slots = np.asarray([cache.slot(entries[i].request_id) for i in order], dtype=np.int32)
        host = HostBatch(
            token_ids=token_ids.astype(np.int32),
            positions=positions,
            request_of_token=request_of_token,
            query_start=query_start,
            context_lens=context_lens,
            query_lens=query_lens,
            slots=slots,
            request_active=np.ones(count, dtype=np.int32),
            logit_rows=np.asarray(logit_rows, dtype=np.int32),
            tables=[],
            num_single=len(singles),
        )
        host._table_width = table_width  # type: ignore[attr-defined]
        return host, rows, spans

    def _fill_tables(self, host: HostBatch, spans: dict[Hashable, tuple[int, int]]) -> None:
        width = getattr(host, "_table_width", None)
        if width is None:
            width = self.cache.width_for(max(end for _, end in spans.values()))
        host.tables = [
            np.ascontiguousarray(self.cache.table_rows(group, host.slots, width))
            for group in range(self.num_groups)
        ]
        for key, mixer in self.planners.items():
            host.extras[key] = mixer.plan(host, self.cache)

    def upload(self, host: HostBatch, meta: MetadataBuffer | None = None) -> StepContext:
        meta = meta or self.meta
        extra_items = [(key, name, array) for key, arrays in host.extras.items()
                       for name, array in arrays.items()]
        arrays = [
            host.token_ids, host.positions, host.request_of_token, host.query_start,
            host.context_lens, host.query_lens, host.slots, host.request_active, host.logit_rows,
            *host.tables, *[array for _, _, array in extra_items],
        ]
        views = meta.upload(arrays)
        self.h2d_bytes = sum(_align(a.size) for a in arrays) * 4
        extras: dict[Any, dict[str, Any]] = {}
        for (key, name, _), view in zip(extra_items, views[9 + len(host.tables):], strict=True):
            extras.setdefault(key, {})[name] = view
        return StepContext(
            num_tokens=host.num_tokens,
            num_requests=host.num_requests,
            num_logit_rows=int(host.logit_rows.shape[0]),
            token_ids=views[0],
            positions=views[1],
            request_of_token=views[2],
            query_start=views[3],
            context_lens=views[4],
            query_lens=views[5],
            slots=views[6],
            request_active=views[7],
            logit_rows=views[8],
            block_tables=list(views[9:9 + len(host.tables)]),
            host=host,
            bindings=self.pools.bindings,
            all_decode=host.num_single == host.num_requests,
            num_single=host.num_single,
            extras=extras,
        )

    # ------------------------------------------------------------------ the step
    def prepare(self, entries: Sequence[StepEntry], table_width: int | None = None
                ) -> tuple[HostBatch, list[tuple[Hashable, int]], dict[Hashable, tuple[int, int]]]:
        """Everything that can fail on the host: checks the entries, grows the tables
        (``CacheCapacityFull`` leaves the cache untouched) and builds the host arrays."""
        if table_width is None:
            table_width = self.fixed_table_width
        host, rows, spans = self.build_host_batch(entries, table_width)
        self.cache.ensure_capacity_batch(spans)
        dirty = self.cache.take_dirty_slots()
        if dirty:
            self.pools.zero_slots(dirty)
        self._fill_tables(host, spans)
        return host, rows, spans

    def _graph_key(self, host: HostBatch) -> Any:
        extras = tuple((key, name, array.shape) for key, arrays in host.extras.items()
                       for name, array in arrays.items())
        return (tuple(host.query_lens.tolist()), int(host.logit_rows.shape[0]),
                tuple(table.shape for table in host.tables), extras,
                self.runtime.ops.error_word.data_ptr())

    def _buffer_stamp(self) -> tuple[int, int]:
        return (self.runtime.workspace.generation, self.runtime.ops.scratch_generation)

    def forward_host(self, host: HostBatch) -> tuple[StepContext, Any]:
        """Uploads the step's metadata and runs the model on it: from the captured graph of this
        shape of step if there is one, else kernel by kernel (and, the third time a shape comes
        by, capturing it).  Returns the context and the logits (None if no row was wanted)."""
        if not self.graphs_enabled:
            ctx = self.upload(host)
            return ctx, self.model.forward(ctx)
        key = self._graph_key(host)
        held = self._graphs.get(key)
        if held is not None and held.stamp != self._buffer_stamp():
            # a workspace or scratch buffer has been replaced by a larger one since the capture:
            # the graph holds the address of the old one
            del self._graphs[key]
            held = None
        if held is not None:
            self._graphs.move_to_end(key)
            ctx = self.upload(host, held.meta)
            held.graph.replay()
            self.graph_replays += 1
            return ctx, held.logits
        seen = self._seen.get(key, 0) + 1
        if len(self._seen) > 4096:
            self._seen.clear()
        self._seen[key] = seen
        if seen < CAPTURE_AT_OCCURRENCE:
            ctx = self.upload(host)
            return ctx, self.model.forward(ctx)
        import torch

        meta = MetadataBuffer(self.runtime.device, words=1 << 10)
        ctx = self.upload(host, meta)
        torch.cuda.synchronize()
        # the same shape ran kernel by kernel before, so every buffer it needs exists; should one be
        # replaced later, the stamp tells (see above)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            logits = self.model.forward(ctx)
        graph.replay()
        self.graph_captures += 1
        self._graphs[key] = _StepGraph(meta, graph, logits, self._buffer_stamp())
        while len(self._graphs) > MAX_STEP_GRAPHS:
            self._graphs.popitem(last=False)
        return ctx, logits

    def run(self, entries: Sequence[StepEntry]) -> StepResult:
        if not entries:
            return StepResult(None, [])
        host, rows, spans = self.prepare(entries)
        _, logits = self.forward_host(host)
        self.cache.commit_lengths({request_id: end for request_id, (_, end) in spans.items()})
        self.steps_run += 1
        self.tokens_run += host.num_tokens
        return StepResult(logits, rows)
