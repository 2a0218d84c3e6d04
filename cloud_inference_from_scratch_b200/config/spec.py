"""The data description of a decoder: which parts each layer has, and in what order layers run.

An architecture module turns its typed configuration into a ``ModelSpec``.  Nothing
below ``ModelSpec`` knows which architecture it came from: a layer is a block kind
plus a norm, a mixer and a feed-forward, each a ``PartSpec`` (a registered kind and
its constants).  The run order is a list of ``ScheduleEntry``: it may name a layer
more than once (the weights are shared, each run has a cache of its own unless it
says otherwise) and an entry may read the cache that an earlier entry wrote instead
of writing one.

The reference hard-codes this arrangement in ``Qwen2CausalLM.forward``
(src/cloud_engine/model.py:211-220); here it is data so that another arrangement
needs no change to the engine.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any


@dataclass(frozen=True)
class PartSpec:
    """One part: the kind it is registered under, the constants it is built with, and the
    tensor-name prefix (relative to its layer's prefix) under which its weights are stored."""

    kind: str
    params: dict[str, Any] = field(default_factory=dict)
    prefix: str = ""


@dataclass(frozen=True)
class LayerSpec:
    """One decoder layer: how its parts are arranged (``block``) and what they are.

    ``prefix`` is the tensor-name prefix of the layer in the weight files.
    """

    prefix: str
    block: PartSpec
    mixer: PartSpec
    feed_forward: PartSpec
    mixer_norm: PartSpec
    feed_forward_norm: PartSpec


@dataclass(frozen=True)
class ScheduleEntry:
    """One run of a layer.

    ``layer``      index into ``ModelSpec.layers``.
    ``reads_cache_of``  index of an EARLIER schedule entry whose cache (pages and
                   per-request state) this run reads instead of owning one; then it
                   writes nothing to a cache.
    """

    layer: int
    reads_cache_of: int | None = None


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    vocab_size: int
    hidden_size: int
    embedding_tensor: str
    layers: tuple[LayerSpec, ...]
    schedule: tuple[ScheduleEntry, ...]
    final_norm: PartSpec
    final_norm_prefix: str
    head_tensor: str  # equals embedding_tensor when the head is tied
    max_positions: int
    eos_token_id: int | None = None
    # tensors that may be present in the files and are ignored (e.g. a tied head stored twice)
    optional_tensors: tuple[str, ...] = ()

    def validate(self) -> None:
        if not self.layers:
            raise ValueError("a model needs at least one layer")
        for index, entry in enumerate(self.schedule):
            if not 0 <= entry.layer < len(self.layers):
                raise ValueError(f"schedule entry {index} names layer {entry.layer}, which does not exist")
            if entry.reads_cache_of is not None:
                if not 0 <= entry.reads_cache_of < index:
                    raise ValueError(
                        f"schedule entry {index} reads the cache of entry {entry.reads_cache_of}; "
                        "it must be an earlier entry"
                    )
                if self.schedule[entry.reads_cache_of].reads_cache_of is not None:
                    raise ValueError(
                        f"schedule entry {index} reads the cache of entry {entry.reads_cache_of}, "
                        "which owns none itself"
                    )
