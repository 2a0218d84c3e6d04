"""Per-step metadata of a flat batch, as the parts see it.

The reference's counterpart is ``PackedContext`` (src/cloud_engine/attention.py:36-49: positions,
query_start_loc, block_tables, slot_mapping, query_seq_ids as separate device tensors built from
Python lists, src/cloud_engine/engine.py:231-301).  Here every integer array of a step lives in
ONE pinned host buffer that goes to the device in ONE copy; the fields below are views into the
device copy.  There is no slot mapping: kernels derive a token's cache slot from its position and
its request's block-table row.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any


@dataclass
class KVLayerView:
    """Keys and values of one cache-owning schedule entry: [pages, kv_heads, page_size, head_dim]."""

    group: int
    k: Any
    v: Any
    num_pages: int
    page_size: int


@dataclass
class LayerBinding:
    """What one schedule entry sees of the cache.  ``owns_cache`` False: it reads what an earlier
    entry wrote and must write nothing.  ``state``: [request slots, *state shape] or None."""

    entry: int
    owns_cache: bool
    kv: KVLayerView | None
    state: Any = None


@dataclass
class StepContext:
    num_tokens: int
    num_requests: int
    num_logit_rows: int
    # device int32 views -----------------------------------------------------------------
    token_ids: Any            # [T]
    positions: Any            # [T] absolute position of each token in its request
    request_of_token: Any     # [T] index into this step's requests
    query_start: Any          # [B + 1] first flat token of each request
    context_lens: Any         # [B] tokens already in the cache before this step
    query_lens: Any           # [B]
    slots: Any                # [B] per-request state slot
    request_active: Any       # [B] 1; 0 for a row that only pads a captured batch (it repeats a real
                              #     row: what it writes to pages is the same again, but per-request
                              #     state must not be advanced for it)
    logit_rows: Any           # [R] flat token rows whose logits are wanted
    block_tables: list[Any]   # per cache group: [B, W_g], -1 where no page
    # host side ----------------------------------------------------------------------------
    host: Any                 # HostBatch (numpy) the device views were copied from
    bindings: list[LayerBinding] = field(default_factory=list)
    all_decode: bool = False  # every request brings exactly one token
    num_single: int = 0       # the first this many requests bring one token each (token row == request index)
    extras: dict[Any, dict[str, Any]] = field(default_factory=dict)
    # The float32 residual stream [T, H] when every norm of the model accepts an ``Accumulated``
    # update, else None.  A mixer or feed-forward may hand it to ``ops.linear(..., residual=...)``
    # for its last projection, whose kernel then adds the result into the stream itself.
    residual_sink: Any = None
