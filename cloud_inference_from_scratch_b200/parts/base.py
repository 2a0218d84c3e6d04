"""Interfaces of the parts a layer is put together from, and the registries they are chosen from.

A part is built from constants only (its ``PartSpec.params``); it never sees a model
configuration.  Each part says which tensors it needs (``tensor_specs``), takes them
(``bind``) and runs on a flat batch of tokens (``forward``).  Five kinds exist:

* ``Norm``              normalises the residual stream (after adding a pending update to it)
* ``PositionEncoding``  owned by a mixer; gives the constants its kernels rotate with
* ``Mixer``             mixes information between the tokens of a request; may own pages of
                        a cache (``cache_spec``) and/or per-request state of fixed size
                        (``state_spec``)
* ``FeedForward``       acts on each token alone
* ``Block``             the arrangement of the above inside one layer

Registering a new kind is ``register_part("mixer", "name", cls)``; a model description
then names it in a ``PartSpec``.  The reference builds the same parts as fixed
``nn.Module`` classes taking the whole ``ModelDims`` (src/cloud_engine/model.py:86-160).
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import TYPE_CHECKING, Any

from ..config.spec import PartSpec

if TYPE_CHECKING:  # pragma: no cover
    import torch

    from ..engine.context import LayerBinding, StepContext
    from ..engine.runtime import Runtime


@dataclass(frozen=True)
class TensorSpec:
    """A tensor a part reads from the weight files.

    ``init`` is how the random-weights mode fills it: "normal" N(0, std), "gain"
    1 + N(0, std), "zeros".  ``role`` "matrix" tensors are held in the compute dtype
    (bfloat16 unless the whole run is 32-bit); "vector" tensors (norm gains, biases)
    are held in float32, which keeps a 32-bit stored tensor as it is and widens a
    bfloat16 one without loss; "table" tensors are integer tables held as int32.
    """

    shape: tuple[int, ...]
    init: str = "normal"
    role: str = "matrix"


@dataclass(frozen=True)
class CacheSpec:
    """What a mixer needs of the page manager: keys and values for ``kv_heads`` heads of
    ``head_dim`` per token, for all earlier tokens (``window == 0``) or the last ``window``."""

    kv_heads: int
    head_dim: int
    window: int = 0

    @property
    def group_key(self) -> tuple[int, int, int]:
        return (self.window, self.kv_heads, self.head_dim)


@dataclass(frozen=True)
class StateSpec:
    """Per-request state of fixed size, one tensor of ``shape`` per live request."""

    shape: tuple[int, ...]
    dtype: str = "float32"


class Part:
    """Common protocol: declare tensors, take them, run."""

    # True says: every kernel this part launches is a method of ``runtime.ops`` (no torch operation, no
    # library of its own).  A decode step of a model whose parts all say so may be recorded and run
    # as one persistent kernel (``Ops.begin_program``); one part that does not keeps every step on
    # separate launches.
    kernels_through_ops = False

    def tensor_specs(self) -> dict[str, TensorSpec]:
        return {}

    def bind(self, tensors: dict[str, "torch.Tensor"], runtime: "Runtime") -> None:
        self.runtime = runtime


class Norm(Part):
    def forward(
        self,
        residual: "torch.Tensor",
        update: "torch.Tensor | None",
        ctx: "StepContext",
        rows: "torch.Tensor | None" = None,
    ) -> "torch.Tensor":
        """``residual`` is the float32 stream [T, H].  Adds ``update`` to it in place (32-bit
        sum) when given, and returns the normalised rows in the compute dtype.  ``update`` is a
        tensor [T, H] or the ``Partials`` a split matrix product returned (a norm that cannot
        add those up itself calls ``runtime.ops.resolve``).  With ``rows``
        only those rows are normalised and returned, and ``residual`` is left as it was."""
        raise NotImplementedError


class PositionEncoding(Part):
    """Constants of a position encoding; the mixer's kernels consume them."""


class Mixer(Part):
    # A mixer with per-request state sets this to True to say: my forward runs on the device alone
    # (it reads this step's numbers from the device views of ``ctx``, never from ``ctx.host``) and
    # leaves the state of requests with ``ctx.request_active == 0`` as it is.  Steps with such a
    # mixer may then run from captured CUDA graphs, padded decode batches included.
    state_in_graphs = False

    def cache_spec(self) -> CacheSpec | None:
        return None

    def state_spec(self) -> StateSpec | None:
        return None

    def forward(
        self, x: "torch.Tensor", ctx: "StepContext", binding: "LayerBinding"
    ) -> "torch.Tensor":
        """x: normalised input [T, H] in the compute dtype; returns the update [T, H]."""
        raise NotImplementedError


class FeedForward(Part):
    def forward(self, x: "torch.Tensor", ctx: "StepContext") -> "torch.Tensor":
        raise NotImplementedError


class Block:
    """Arrangement of the parts of one layer around the residual stream.

    A block is built from the layer's parts by slot name (``parts["mixer"]``, ...; every part is
    also an attribute of that name) and its own constants.  ``slots`` names what it needs; the
    model checks a layer's description against it.  ``cache_slot`` names the part whose cache
    (pages and/or per-request state) the layer's binding belongs to."""

    slots: tuple[str, ...] = ()
    cache_slot: str = "mixer"
    kernels_through_ops = False   # as for a part: True if the block launches nothing but methods of ``Ops``

    def __init__(self, parts: "dict[str, Part]", **params: Any) -> None:
        missing = [name for name in self.slots if name not in parts]
        if missing:
            raise ValueError(f"{type(self).__name__} needs the parts {list(self.slots)}; missing {missing}")
        self.parts = dict(parts)
        for name, part in parts.items():
            setattr(self, name, part)

    def forward(
        self,
        residual: "torch.Tensor",
        pending: "torch.Tensor | None",
        ctx: "StepContext",
        binding: "LayerBinding",
    ) -> "torch.Tensor | None":
        """Runs the layer.  ``pending`` is an update not yet added to ``residual``; the
        returned tensor is this layer's last update, again pending."""
        raise NotImplementedError

    def entry_gain(self) -> Any:
        """What the layer BEFORE this one may know about this block's first norm: the gain vector
        its last projection may multiply the new residual rows with, if this block's first
        consumer finishes that norm itself; None (the default) if the block wants plain rows."""
        return None


_KINDS = ("norm", "position", "mixer", "feed_forward", "block")
_REGISTRY: dict[str, dict[str, type]] = {kind: {} for kind in _KINDS}


def register_part(kind: str, name: str, cls: type, *, replace: bool = False) -> None:
    if kind not in _REGISTRY:
        raise ValueError(f"unknown part kind {kind!r}; expected one of {_KINDS}")
    if name in _REGISTRY[kind] and not replace:
        raise ValueError(f"{kind} {name!r} is already registered")
    _REGISTRY[kind][name] = cls


def part_class(kind: str, name: str) -> type:
    try:
        return _REGISTRY[kind][name]
    except KeyError:
        known = ", ".join(sorted(_REGISTRY.get(kind, {}))) or "none"
        raise KeyError(f"no {kind} registered under {name!r} (known: {known})") from None


def build_part(kind: str, spec: PartSpec) -> Any:
    return part_class(kind, spec.kind)(**spec.params)


def registered_parts(kind: str) -> tuple[str, ...]:
    return tuple(sorted(_REGISTRY[kind]))
