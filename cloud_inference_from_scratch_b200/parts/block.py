"""Pre-norm residual arrangement of one layer.

``h = h + mixer(norm1(h)); h = h + feed_forward(norm2(h))`` (src/cloud_engine/model.py:212-220).
The residual stream is float32 and each add is fused into the norm that follows it, so
a layer leaves its last update pending for whoever normalises next.
"""

from __future__ import annotations

from .base import Block, register_part


def _normalise(norm, consumer, residual, pending, ctx):
    """A consumer that declares ``takes_normed_input`` may get the norm un-computed (see
    ``Norm.forward_lazy``); every other pairing runs the norm's kernel."""
    lazy = getattr(norm, "forward_lazy", None)
    if lazy is not None and getattr(consumer, "takes_normed_input", False):
        return lazy(residual, pending, ctx)
    return norm.forward(residual, pending, ctx)


def _lazy_gain(norm, consumer):
    """The gain a projection may pre-multiply with for ``norm``, if ``consumer`` can finish it."""
    if getattr(consumer, "takes_normed_input", False) and hasattr(norm, "forward_lazy"):
        return getattr(norm, "lazy_gain", None)
    return None


class PreNormResidual(Block):
    slots = ("mixer", "feed_forward", "mixer_norm", "feed_forward_norm")
    kernels_through_ops = True   # the block itself launches nothing

    def entry_gain(self):
        return _lazy_gain(self.mixer_norm, self.mixer)

    def forward(self, residual, pending, ctx, binding):
        sink = getattr(ctx, "residual_sink", None)
        if sink is not None:
            # after a projection of this block comes a product of this engine (the feed-forward's, or
            # the next layer's first) or a norm kernel: before their dependency wait they ask for
            # weights only, so the projection may let them start early
            sink.early_trigger = True
        x = _normalise(self.mixer_norm, self.mixer, residual, pending, ctx)
        if sink is not None:   # the mixer's sum is read next by this layer's second norm
            sink.gain = _lazy_gain(self.feed_forward_norm, self.feed_forward)
        update = self.mixer.forward(x, ctx, binding)
        x = _normalise(self.feed_forward_norm, self.feed_forward, residual, update, ctx)
        if sink is not None:   # the feed-forward's sum by whoever comes after this layer
            sink.gain = sink.following_gain
        return self.feed_forward.forward(x, ctx)


register_part("block", "prenorm_residual", PreNormResidual, replace=True)
