"""NeoX-style (rotate-half) rotary position encoding: the constants the attention kernels use.

Formula (src/cloud_engine/attention.py:60-85): ``inv_freq[j] = theta^(-2j/R)`` for
j < R/2, angle = position * inv_freq[j]; element j pairs with element j + R/2:
``x'[j] = x[j] cos - x[j+R/2] sin``, ``x'[j+R/2] = x[j+R/2] cos + x[j] sin``.  The
reference builds a cos/sin table of 32768 rows (model.py:190-192) and rotates in the
model dtype; here the kernel computes the angle and the rotation in float32 from
``inv_freq`` and rounds once.  ``rotary_dim`` may be smaller than ``head_dim`` (the rest
of the head passes through).
"""

from __future__ import annotations

from .base import PositionEncoding, register_part


class RopeNeox(PositionEncoding):
    style = "neox"

    def __init__(self, head_dim: int, rotary_dim: int, theta: float, max_positions: int) -> None:
        if rotary_dim % 2 or rotary_dim > head_dim or rotary_dim < 2:
            raise ValueError(f"rotary_dim {rotary_dim} must be even and within head_dim {head_dim}")
        self.head_dim = int(head_dim)
        self.rotary_dim = int(rotary_dim)
        self.theta = float(theta)
        self.max_positions = int(max_positions)

    def bind(self, tensors, runtime) -> None:
        import torch

        self.runtime = runtime
        exponent = torch.arange(0, self.rotary_dim, 2, dtype=torch.float32) / self.rotary_dim
        self.inv_freq = (1.0 / (self.theta ** exponent)).to(runtime.device).contiguous()


register_part("position", "rope_neox", RopeNeox, replace=True)
