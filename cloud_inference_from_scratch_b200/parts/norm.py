"""RMSNorm over the float32 residual stream, fused with the pending residual add.

Formula (src/cloud_engine/attention.py:52-57): ``w * (x * rsqrt(mean(x^2) + eps))`` with
the statistics in float32.  The reference keeps the residual in float16 and adds in
float16 (model.py:217-220); here the stream is float32, the add is a 32-bit sum inside
the same kernel, and the result is rounded once to the compute dtype.
"""

from __future__ import annotations

from ..lazy import Accumulated, NormedInput
from .base import Norm, TensorSpec, register_part


class RMSNorm(Norm):
    def __init__(self, hidden_size: int, eps: float) -> None:
        self.hidden_size = int(hidden_size)
        self.eps = float(eps)

    def tensor_specs(self) -> dict[str, TensorSpec]:
        return {"weight": TensorSpec((self.hidden_size,), init="gain", role="vector")}

    def bind(self, tensors, runtime) -> None:
        self.runtime = runtime
        self.weight = tensors["weight"]

    accepts_accumulated = True   # ``update`` may be an ``Accumulated``: the sum is already in the stream
    kernels_through_ops = True  # every kernel of this part is a method of ``Ops``: a decode step may be recorded

    def forward(self, residual, update, ctx, rows=None):
        rt = self.runtime
        count = residual.shape[0] if rows is None else rows.shape[0]
        out = rt.workspace.get("norm.out" if rows is None else "norm.rows", count,
                               self.hidden_size, rt.dtype, per_request=rows is not None)
        rt.ops.add_rmsnorm(residual, update, self.weight, self.eps, out, rows)
        return out

    @property
    def lazy_gain(self):
        """The gain vector a projection may pre-multiply the new residual rows with for this norm
        (see ``forward_lazy``)."""
        return self.weight

    def forward_lazy(self, residual, update, ctx):
        """For a consumer that finishes the norm itself (``takes_normed_input``): when the sum is
        already in the stream, scaled by this norm's gain, and its sums of squares are known,
        nothing runs here."""
        if isinstance(update, Accumulated) and update.scaled is not None and update.gain is self.weight:
            return NormedInput(update, self.eps, materialize=lambda: self.forward(residual, None, ctx))
        return self.forward(residual, update, ctx)


register_part("norm", "rmsnorm", RMSNorm, replace=True)
