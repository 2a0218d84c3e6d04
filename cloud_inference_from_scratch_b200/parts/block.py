"""Pre-norm residual arrangement of one layer.

``h = h + mixer(norm1(h)); h = h + feed_forward(norm2(h))`` (src/cloud_engine/model.py:212-220).
The residual stream is float32 and each add is fused into the norm that follows it, so
a layer leaves its last update pending for whoever normalises next.
"""

from __future__ import annotations

from .base import Block, register_part


class PreNormResidual(Block):
    def forward(self, residual, pending, ctx, binding):
        x = self.mixer_norm.forward(residual, pending, ctx)
        update = self.mixer.forward(x, ctx, binding)
        x = self.feed_forward_norm.forward(residual, update, ctx)
        return self.feed_forward.forward(x, ctx)


register_part("block", "prenorm_residual", PreNormResidual, replace=True)
