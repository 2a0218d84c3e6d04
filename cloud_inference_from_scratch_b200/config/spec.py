"""The data description of a decoder: which parts each layer has, and in what order layers run.

An architecture module turns its typed configuration into a ``ModelSpec``.  Nothing
below ``ModelSpec`` knows which architecture it came from: a layer is a block kind
plus a named map of parts (norms, mixers, feed-forwards), each a ``PartSpec`` (the
family it belongs to, a registered kind and its constants); which names a block
expects is the block's own business.  The run order is a list of ``ScheduleEntry``: it may name a layer
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
    tensor-name prefix (relative to its layer's prefix) under which its weights are stored.
    ``family`` is the registry it is looked up in ("norm", "mixer", "feed_forward", "position",
    "block"); empty means "what the slot's name says" (see ``LayerSpec``)."""

    kind: str
    params: dict[str, Any] = field(default_factory=dict)
    prefix: str = ""
    family: str = ""


def _family_of(slot: str, spec: PartSpec) -> str:
    if spec.family:
        return spec.family
    if slot.endswith("norm"):
        return "norm"
    if slot in ("mixer", "feed_forward"):
        return slot
    raise ValueError(f"slot {slot!r} does not say which family its part belongs to; give PartSpec.family")


@dataclass(frozen=True, init=False, eq=True)
class LayerSpec:
    """One decoder layer: how its parts are arranged (``block``) and what they are (``parts``, by
    slot name).  ``prefix`` is the tensor-name prefix of the layer in the weight files.

    The pre-norm residual block expects the slots ``mixer``, ``feed_forward``, ``mixer_norm`` and
    ``feed_forward_norm``, which may also be given as keyword arguments (and read as attributes);
    another block kind names the slots it wants: a post-norm, a second feed-forward, no
    feed-forward at all.  ``dataclasses.replace(layer, mixer=...)`` swaps one part."""

    prefix: str
    block: PartSpec
    parts: dict[str, PartSpec]

    def __init__(self, prefix: str, block: PartSpec, parts: dict[str, PartSpec] | None = None,
                 **named: PartSpec) -> None:
        merged = dict(parts or {})
        merged.update(named)
        for slot, spec in merged.items():
            if not isinstance(spec, PartSpec):
                raise TypeError(f"layer {prefix!r}: slot {slot!r} is not a PartSpec")
        object.__setattr__(self, "prefix", prefix)
        object.__setattr__(self, "block", block)
        object.__setattr__(self, "parts", {
            slot: spec if spec.family else PartSpec(spec.kind, spec.params, spec.prefix, _family_of(slot, spec))
            for slot, spec in merged.items()
        })

    def __getattr__(self, name: str) -> PartSpec:
        # mixer, feed_forward, mixer_norm, feed_forward_norm (or any other slot) by name
        parts = self.__dict__.get("parts")
        if parts is not None and name in parts:
            return parts[name]
        raise AttributeError(f"layer {self.__dict__.get('prefix')!r} has no part {name!r}")


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
    embedding_scale: float = 1.0      # the gathered embedding rows are multiplied by this
    logit_scale: float = 1.0          # logits = softcap * tanh(head(x) * scale / softcap), or head(x) * scale
    logit_softcap: float = 0.0        # 0: no soft cap

    def validate(self) -> None:
        if not self.layers:
            raise ValueError("a model needs at least one layer")
        if self.logit_softcap < 0:
            raise ValueError("logit_softcap must be >= 0")
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
