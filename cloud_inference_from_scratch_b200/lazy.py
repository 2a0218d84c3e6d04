"""Values that travel between parts instead of tensors.

A part hands the next one a tensor, or one of these: a product whose last additions are left to
its consumer (``Partials``), a product that has already added itself into the residual stream
(``Accumulated``), rows of a norm that its consumer finishes (``NormedInput``).  ``ResidualSink`` is
how a block tells a projection where the residual stream is; ``GateUpWeight`` is a stacked weight
with its layout.  A part that knows none of this gets tensors (``Ops.resolve``, ``materialize``);
the kernels behind ``Ops`` produce and consume them.
"""

from __future__ import annotations

from typing import Any


class Partials:
    """A projection whose last additions are left to the kernel that consumes it.

    ``splits`` > 0: ``data`` holds float32 partial sums [splits, rows, width] of a matrix product
    that was cut along K.  ``splits`` == 0: ``data`` is the product itself [rows, width] in the
    compute dtype.  In both cases ``bias`` (or None) is still to be added.  The consumers
    (residual-add + RMSNorm, rotary + cache write) add everything up in float32, parts in
    ascending split order."""

    def __init__(self, data: Any, splits: int, rows: int, width: int, bias: Any) -> None:
        self.data, self.splits, self.rows, self.width, self.bias = data, splits, rows, width, bias

    @property
    def shape(self) -> tuple[int, int]:
        return (self.rows, self.width)


class ResidualSink:
    """The float32 residual stream [T, H] as a target: a projection handed this (``Ops.linear(...,
    residual=sink)``) may add its result into ``tensor`` itself.  ``gain`` is the gain vector of the
    norm that will read the stream next, when that norm can take its input pre-scaled (else None);
    whoever arranges the layers sets it before each projection."""

    def __init__(self, tensor: Any) -> None:
        self.tensor = tensor
        self.gain: Any = None
        self.following_gain: Any = None   # for the last projection of the current layer
        # Whoever arranges the layers may set this when it knows that the kernel after such a
        # projection touches, before its own dependency wait, only what no kernel of the same step
        # writes: the projection then lets that kernel start beside the kernel before itself.
        self.early_trigger = False


class Accumulated:
    """A projection that its own kernel has already added into the float32 residual stream.

    ``sq`` holds, for every token row, the sums of squares of the new residual row per block of 32
    columns ([rows, tiles] float32): a norm that follows needs no pass over the row to know its
    mean square.  ``scaled`` (or None) is bfloat16(new row * ``gain``) for the norm whose gain
    vector ``gain`` is.  A consumer that only wants the sum treats this as "nothing left to add"."""

    def __init__(self, residual: Any, sq: Any, tiles: int, scaled: Any = None, gain: Any = None) -> None:
        self.residual, self.sq, self.tiles, self.scaled, self.gain = residual, sq, tiles, scaled, gain

    @property
    def shape(self) -> tuple[int, ...]:
        return tuple(self.residual.shape)


class NormedInput:
    """RMSNorm of the residual rows, not yet divided by the root mean square: ``accumulated.scaled``
    holds bfloat16(row * gain) and the matrix product that takes this (``Ops.linear``,
    ``Ops.gate_up``) multiplies its result rows by rstd, which it forms from ``accumulated.sq``.
    ``materialize()`` runs the ordinary norm kernel and returns a plain tensor for anyone else."""

    def __init__(self, accumulated: Accumulated, eps: float, materialize: Any) -> None:
        self.accumulated, self.eps, self.materialize = accumulated, eps, materialize

    @property
    def shape(self) -> tuple[int, ...]:
        return tuple(self.accumulated.scaled.shape)


class GateUpWeight:
    """Stacked gate and up matrices [2I, H].  ``block`` == I: all gate rows, then all up rows.
    ``block`` < I: rows interleaved in blocks (``block`` gate rows, the matching ``block`` up
    rows, ...), which lets one CTA of the streaming kernel finish SiLU(gate) * up by itself."""

    def __init__(self, weight: Any, inter: int, block: int) -> None:
        self.weight, self.inter, self.block = weight, inter, block
