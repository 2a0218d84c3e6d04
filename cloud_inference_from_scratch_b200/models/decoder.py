"""A decoder put together from a ``ModelSpec``: embedding (times a constant), scheduled layers,
final norm, head, logits (times a constant, softly capped).

This is the only model class of the framework; an architecture contributes a
description, not a class.  The forward pass is the reference's
``Qwen2CausalLM.forward`` (src/cloud_engine/model.py:194-228) restated over parts:
gather embeddings into the float32 residual stream, run the schedule, normalise only
the rows whose logits are wanted (the reference normalises all rows and then selects,
model.py:221-225), multiply by the head and return float32 logits.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any

from ..config.spec import ModelSpec
from ..parts.base import (
    Block,
    CacheSpec,
    Norm,
    Part,
    StateSpec,
    TensorSpec,
    build_part,
    part_class,
)


@dataclass
class LayerParts:
    """The built parts of one layer by slot name, their arrangement, and the tensor-name prefix of
    each part in the weight files."""

    prefix: str
    parts: dict[str, Part]
    families: dict[str, str]
    block: Block
    prefixes: dict[str, str]

    def named_parts(self):
        for slot, part in self.parts.items():
            yield self.prefixes[slot], part

    @property
    def cache_part(self) -> Part | None:
        """The part whose cache the layer's binding belongs to (at most one part of a layer keeps one)."""
        return self.parts.get(self.block.cache_slot)

    def __getattr__(self, name: str) -> Part:      # layer.mixer, layer.feed_forward, ...
        try:
            return self.__dict__["parts"][name]
        except KeyError:
            raise AttributeError(name) from None


@dataclass(frozen=True)
class CacheNeed:
    """What one schedule entry needs of the cache manager (``owner`` is the entry whose
    cache it uses: itself, or the earlier entry it reads)."""

    entry: int
    owner: int
    pages: CacheSpec | None
    state: StateSpec | None


class DecoderModel:
    def __init__(self, spec: ModelSpec) -> None:
        spec.validate()
        self.spec = spec
        self.layers: list[LayerParts] = []
        for layer in spec.layers:
            parts = {slot: build_part(part.family, part) for slot, part in layer.parts.items()}
            block = part_class("block", layer.block.kind)(parts, **layer.block.params)
            keepers = [slot for slot, part in parts.items()
                       if getattr(part, "cache_spec", None) and (part.cache_spec() or part.state_spec())]
            if any(slot != block.cache_slot for slot in keepers):
                raise ValueError(
                    f"layer {layer.prefix!r}: the parts {keepers} keep a cache, but the block binds only "
                    f"{block.cache_slot!r} to one"
                )
            self.layers.append(
                LayerParts(
                    prefix=layer.prefix, parts=parts, block=block,
                    families={slot: part.family for slot, part in layer.parts.items()},
                    prefixes={slot: layer.prefix + part.prefix for slot, part in layer.parts.items()},
                )
            )
        self.final_norm: Norm = build_part("norm", spec.final_norm)
        # a projection may add itself into the residual stream only if whoever normalises next
        # understands that the sum is already there
        norms = [self.final_norm] + [part for layer in self.layers for slot, part in layer.parts.items()
                                     if layer.families[slot] == "norm"]
        self.norms_accept_accumulated = all(getattr(norm, "accepts_accumulated", False) for norm in norms)
        # A decode step may be recorded and run as one persistent kernel only if every kernel of every
        # part is a method of ``Ops`` (which then keeps the order of recorded and launched work); a part
        # says so itself, and a part that launches anything of its own (torch ops included) does not.
        self.records_programs = all(
            getattr(part, "kernels_through_ops", False)
            for layer in self.layers for part in [layer.block, *layer.parts.values()])
        self.embedding: Any = None
        self.head: Any = None
        self.runtime: Any = None

    # ------------------------------------------------------------------ tensors
    def tensor_table(self) -> dict[str, TensorSpec]:
        """Every tensor the model reads, by its name in the weight files."""
        spec = self.spec
        table: dict[str, TensorSpec] = {
            spec.embedding_tensor: TensorSpec((spec.vocab_size, spec.hidden_size))
        }
        if spec.head_tensor != spec.embedding_tensor:
            table[spec.head_tensor] = TensorSpec((spec.vocab_size, spec.hidden_size))
        for layer in self.layers:
            for prefix, part in layer.named_parts():
                for name, tensor in part.tensor_specs().items():
                    table[prefix + name] = tensor
        for name, tensor in self.final_norm.tensor_specs().items():
            table[spec.final_norm_prefix + name] = tensor
        return table

    def cache_needs(self) -> list[CacheNeed]:
        needs: list[CacheNeed] = []
        for index, entry in enumerate(self.spec.schedule):
            keeper = self.layers[entry.layer].cache_part
            owner = index if entry.reads_cache_of is None else entry.reads_cache_of
            pages = keeper.cache_spec() if keeper is not None and hasattr(keeper, "cache_spec") else None
            state = keeper.state_spec() if keeper is not None and hasattr(keeper, "state_spec") else None
            needs.append(CacheNeed(index, owner, pages, state))
        for need in needs:
            if need.owner != need.entry:
                owner = needs[need.owner]
                if (owner.pages, owner.state) != (need.pages, need.state):
                    raise ValueError(
                        f"schedule entry {need.entry} reads the cache of entry {need.owner}, "
                        "whose mixer keeps a different kind of cache"
                    )
        return needs

    # ------------------------------------------------------------------ binding
    def bind(self, tensors: Any, runtime: Any) -> None:
        """``tensors(name)`` returns the tensor on the device in the dtype its role asks for."""
        self.runtime = runtime
        spec = self.spec
        self.embedding = runtime.ops.prepare_weight(tensors(spec.embedding_tensor))
        self.head = (
            self.embedding
            if spec.head_tensor == spec.embedding_tensor
            else runtime.ops.prepare_weight(tensors(spec.head_tensor))
        )
        for layer in self.layers:
            for prefix, part in layer.named_parts():
                part.bind({name: tensors(prefix + name) for name in part.tensor_specs()}, runtime)
        self.final_norm.bind(
            {name: tensors(spec.final_norm_prefix + name) for name in self.final_norm.tensor_specs()},
            runtime,
        )

    # ------------------------------------------------------------------ forward
    def forward(self, ctx: Any) -> Any:
        """Runs the tokens of ``ctx`` and returns float32 logits [wanted rows, vocab]."""
        import torch

        rt = self.runtime
        spec = self.spec
        residual = rt.workspace.get("residual", ctx.num_tokens, spec.hidden_size, torch.float32)
        rt.ops.embedding(ctx.token_ids, self.embedding, residual, spec.embedding_scale)
        sink = rt.ops.residual_sink(residual) if self.norms_accept_accumulated else None
        ctx.residual_sink = sink
        pending = None
        recorded = self.records_programs and sink is not None and rt.ops.begin_program(ctx)
        for index, entry in enumerate(spec.schedule):
            if sink is not None:
                # what the block after this layer wants to know of its first norm (the final norm
                # takes plain rows)
                sink.following_gain = None
                if index + 1 < len(spec.schedule):
                    sink.following_gain = self.layers[spec.schedule[index + 1].layer].block.entry_gain()
            pending = self.layers[entry.layer].block.forward(
                residual, pending, ctx, ctx.bindings[index]
            )
        if recorded:
            rt.ops.end_program()
        if ctx.num_logit_rows == 0:
            return None
        x = self.final_norm.forward(residual, pending, ctx, rows=ctx.logit_rows)
        logits = rt.workspace.get("logits", ctx.num_logit_rows, spec.vocab_size, torch.float32,
                                  per_request=True)
        rt.ops.linear(x, self.head, None, logits)
        rt.ops.shape_logits(logits, spec.logit_scale, spec.logit_softcap)
        return logits
