"""A decoder put together from a ``ModelSpec``: embedding, scheduled layers, final norm, head.

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
from ..native.ops import ResidualSink
from ..parts.base import (
    Block,
    CacheSpec,
    FeedForward,
    Mixer,
    Norm,
    StateSpec,
    TensorSpec,
    build_part,
    part_class,
)


@dataclass
class LayerParts:
    prefix: str
    mixer: Mixer
    feed_forward: FeedForward
    mixer_norm: Norm
    feed_forward_norm: Norm
    block: Block
    prefixes: dict[str, str]

    def named_parts(self):
        yield self.prefixes["mixer"], self.mixer
        yield self.prefixes["feed_forward"], self.feed_forward
        yield self.prefixes["mixer_norm"], self.mixer_norm
        yield self.prefixes["feed_forward_norm"], self.feed_forward_norm


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
            mixer = build_part("mixer", layer.mixer)
            feed_forward = build_part("feed_forward", layer.feed_forward)
            mixer_norm = build_part("norm", layer.mixer_norm)
            feed_forward_norm = build_part("norm", layer.feed_forward_norm)
            block = part_class("block", layer.block.kind)(
                mixer, feed_forward, mixer_norm, feed_forward_norm, **layer.block.params
            )
            self.layers.append(
                LayerParts(
                    prefix=layer.prefix,
                    mixer=mixer,
                    feed_forward=feed_forward,
                    mixer_norm=mixer_norm,
                    feed_forward_norm=feed_forward_norm,
                    block=block,
                    prefixes={
                        "mixer": layer.prefix + layer.mixer.prefix,
                        "feed_forward": layer.prefix + layer.feed_forward.prefix,
                        "mixer_norm": layer.prefix + layer.mixer_norm.prefix,
                        "feed_forward_norm": layer.prefix + layer.feed_forward_norm.prefix,
                    },
                )
            )
        self.final_norm: Norm = build_part("norm", spec.final_norm)
        # a projection may add itself into the residual stream only if whoever normalises next
        # understands that the sum is already there
        norms = [self.final_norm] + [n for layer in self.layers for n in (layer.mixer_norm, layer.feed_forward_norm)]
        self.norms_accept_accumulated = all(getattr(norm, "accepts_accumulated", False) for norm in norms)
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
            mixer = self.layers[entry.layer].mixer
            owner = index if entry.reads_cache_of is None else entry.reads_cache_of
            needs.append(CacheNeed(index, owner, mixer.cache_spec(), mixer.state_spec()))
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
        rt.ops.embedding(ctx.token_ids, self.embedding, residual)
        sink = ResidualSink(residual) if self.norms_accept_accumulated else None
        ctx.residual_sink = sink
        pending = None
        for index, entry in enumerate(spec.schedule):
            if sink is not None:
                # who normalises after this layer: the next layer's first norm, if its mixer can
                # finish a pre-scaled norm; the final norm takes the plain kernel
                sink.following_gain = None
                if index + 1 < len(spec.schedule):
                    following = self.layers[spec.schedule[index + 1].layer].block
                    if getattr(following.mixer, "takes_normed_input", False) and hasattr(following.mixer_norm, "forward_lazy"):
                        sink.following_gain = getattr(following.mixer_norm, "lazy_gain", None)
            pending = self.layers[entry.layer].block.forward(
                residual, pending, ctx, ctx.bindings[index]
            )
        if ctx.num_logit_rows == 0:
            return None
        x = self.final_norm.forward(residual, pending, ctx, rows=ctx.logit_rows)
        logits = rt.workspace.get("logits", ctx.num_logit_rows, spec.vocab_size, torch.float32,
                                  per_request=True)
        rt.ops.linear(x, self.head, None, logits)
        return logits
