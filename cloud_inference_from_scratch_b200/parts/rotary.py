"""Rotary position encoding: the constants the attention kernels use.

Formula (src/cloud_engine/attention.py:60-85): ``inv_freq[j] = theta^(-2j/R)`` for
j < R/2, angle = position * inv_freq[j]; element j pairs with element j + R/2:
``x'[j] = x[j] cos - x[j+R/2] sin``, ``x'[j+R/2] = x[j+R/2] cos + x[j] sin``.  The
reference builds a cos/sin table of 32768 rows (model.py:190-192) and rotates in the
model dtype; here the kernel computes the angle and the rotation in float32 from
``inv_freq`` and rounds once.  ``rotary_dim`` may be smaller than ``head_dim`` (the rest
of the head passes through).

Beyond the reference (which has exactly the above):

* ``pairing="interleaved"`` pairs element 2j with element 2j + 1 instead.  The kernels keep the
  one pairing they have: the mixer permutes the q and k rows of its weights at load time
  (``row_order``) so that element 2j lands at j and element 2j + 1 at j + R/2.  Scores are dot
  products of q and k, which the same permutation of both leaves unchanged, and nobody else
  reads q or k.
* ``position_scale`` divides positions (linear position scaling); ``attention_factor`` multiplies
  the softmax scale of the mixer that owns this encoding.
"""

from __future__ import annotations

from .base import PositionEncoding, register_part


class RopeNeox(PositionEncoding):
    style = "neox"

    def __init__(self, head_dim: int, rotary_dim: int, theta: float, max_positions: int,
                 pairing: str = "half", position_scale: float = 1.0, attention_factor: float = 1.0) -> None:
        if rotary_dim % 2 or rotary_dim > head_dim or rotary_dim < 2:
            raise ValueError(f"rotary_dim {rotary_dim} must be even and within head_dim {head_dim}")
        if pairing not in ("half", "interleaved"):
            raise ValueError(f"pairing must be 'half' or 'interleaved', got {pairing!r}")
        if position_scale <= 0 or attention_factor <= 0:
            raise ValueError("position_scale and attention_factor must be positive")
        self.head_dim = int(head_dim)
        self.rotary_dim = int(rotary_dim)
        self.theta = float(theta)
        self.max_positions = int(max_positions)
        self.pairing = pairing
        self.position_scale = float(position_scale)
        self.attention_factor = float(attention_factor)

    def row_order(self) -> list[int] | None:
        """For a mixer: the order in which the elements of a q or k head are to be stored so that
        this encoding's pairs are (j, j + rotary_dim/2) for the kernels; None if they are already."""
        if self.pairing == "half":
            return None
        half = self.rotary_dim // 2
        order = [2 * j for j in range(half)] + [2 * j + 1 for j in range(half)]
        return order + list(range(self.rotary_dim, self.head_dim))

    def bind(self, tensors, runtime) -> None:
        import torch

        self.runtime = runtime
        exponent = torch.arange(0, self.rotary_dim, 2, dtype=torch.float32) / self.rotary_dim
        inv_freq = 1.0 / (self.theta ** exponent) / self.position_scale
        self.inv_freq = inv_freq.to(runtime.device).contiguous()


register_part("position", "rope_neox", RopeNeox, replace=True)
