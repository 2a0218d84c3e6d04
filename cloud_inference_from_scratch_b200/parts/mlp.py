"""SwiGLU feed-forward: ``down(silu(gate(x)) * up(x))``, no biases.

Reference: ``Qwen2MLP.forward`` (src/cloud_engine/model.py:86-100) runs gate and up as
two matrix products and three elementwise kernels.  Here gate and up are stacked into
one weight [2I, H] and one product; SiLU and the multiply run in float32 registers in
one kernel that writes [T, I].
"""

from __future__ import annotations

from .base import FeedForward, TensorSpec, register_part


class SwiGLU(FeedForward):
    def __init__(self, hidden_size: int, intermediate_size: int) -> None:
        self.hidden_size = int(hidden_size)
        self.intermediate_size = int(intermediate_size)

    def tensor_specs(self) -> dict[str, TensorSpec]:
        return {
            "gate_proj.weight": TensorSpec((self.intermediate_size, self.hidden_size)),
            "up_proj.weight": TensorSpec((self.intermediate_size, self.hidden_size)),
            "down_proj.weight": TensorSpec((self.hidden_size, self.intermediate_size)),
        }

    def bind(self, tensors, runtime) -> None:
        self.runtime = runtime
        self.w_gate_up = runtime.ops.prepare_gate_up(tensors["gate_proj.weight"], tensors["up_proj.weight"])
        self.w_down = runtime.ops.prepare_weight(tensors["down_proj.weight"])

    takes_normed_input = True   # x goes to ops.gate_up only
    kernels_through_ops = True  # every kernel of this part is a method of ``Ops``: a decode step may be recorded

    def forward(self, x, ctx):
        rt = self.runtime
        tokens = x.shape[0]
        hidden = rt.workspace.get("swiglu.hidden", tokens, self.intermediate_size, rt.dtype)
        rt.ops.gate_up(x, self.w_gate_up, hidden, rt.workspace)
        update = rt.workspace.get("feed_forward.update", tokens, self.hidden_size, rt.dtype)
        return rt.ops.linear(hidden, self.w_down, None, update, allow_partials=True,
                             tag="feed_forward.update", residual=getattr(ctx, "residual_sink", None))


register_part("feed_forward", "swiglu", SwiGLU, replace=True)
