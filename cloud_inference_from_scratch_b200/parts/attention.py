"""Grouped-query causal attention over the paged cache.

Reference formulas: projections with bias, head-major split (src/cloud_engine/model.py:132-137);
rotary on q and k (attention.py:83-85); keys and values written to the pages before
attention so that a portion attends to itself through the cache (attention.py:193,225;
cache.py:398-425); per q head h the kv head h // (Hq/Hkv), keys 0..pos inclusive,
scale 1/sqrt(head_dim), float32 softmax (kernel.py:356-405; attention.py:88-112,129);
output projection without bias (model.py:128-130).

Here q, k and v come from ONE matrix product with the three weights stacked, the
rotation is fused with the write of k and v into the pages, and attention reads the
pages directly through the block table.  ``window`` > 0 limits a query at position p
to keys p-window+1..p.
"""

from __future__ import annotations

import math

from ..config.spec import PartSpec
from .base import CacheSpec, Mixer, TensorSpec, build_part, register_part


class Attention(Mixer):
    def __init__(
        self,
        hidden_size: int,
        num_heads: int,
        num_kv_heads: int,
        head_dim: int,
        qkv_bias: bool,
        position: PartSpec | None,
        window: int = 0,
        scale: float | None = None,
    ) -> None:
        if num_heads % num_kv_heads:
            raise ValueError("num_heads must be a multiple of num_kv_heads")
        self.hidden_size = int(hidden_size)
        self.num_heads = int(num_heads)
        self.num_kv_heads = int(num_kv_heads)
        self.head_dim = int(head_dim)
        self.qkv_bias = bool(qkv_bias)
        self.window = int(window)
        self.position = build_part("position", position) if position is not None else None
        self.scale = float(scale) if scale is not None else 1.0 / math.sqrt(self.head_dim)
        self.scale *= float(getattr(self.position, "attention_factor", 1.0))
        self.q_width = self.num_heads * self.head_dim
        self.kv_width = self.num_kv_heads * self.head_dim
        self.qkv_width = self.q_width + 2 * self.kv_width

    @property
    def plan_key(self):
        return ("attention", self.num_heads // self.num_kv_heads)

    def plan(self, host, cache):
        """Work lists for this step's attention kernels, added to the step's metadata copy."""
        return self.runtime.ops.plan_attention(host, self.num_heads // self.num_kv_heads)

    def cache_spec(self) -> CacheSpec:
        return CacheSpec(kv_heads=self.num_kv_heads, head_dim=self.head_dim, window=self.window)

    def tensor_specs(self) -> dict[str, TensorSpec]:
        specs = {
            "q_proj.weight": TensorSpec((self.q_width, self.hidden_size)),
            "k_proj.weight": TensorSpec((self.kv_width, self.hidden_size)),
            "v_proj.weight": TensorSpec((self.kv_width, self.hidden_size)),
            "o_proj.weight": TensorSpec((self.hidden_size, self.q_width)),
        }
        if self.qkv_bias:
            specs["q_proj.bias"] = TensorSpec((self.q_width,), role="vector")
            specs["k_proj.bias"] = TensorSpec((self.kv_width,), role="vector")
            specs["v_proj.bias"] = TensorSpec((self.kv_width,), role="vector")
        return specs

    def bind(self, tensors, runtime) -> None:
        import torch

        self.runtime = runtime
        ops = runtime.ops
        # With a rotary encoding whose sizes allow it, the q and k rows are kept in the paired
        # layout: a decode step then rotates and stores inside the projection's kernel, and the
        # separate rotary kernel (prompt portions) reads the same layout.
        rotary = self.position.rotary_dim if self.position is not None else 0
        self.paired = bool(self.position is not None and getattr(ops, "can_pair_rotary", None)
                           and ops.can_pair_rotary(self.head_dim, rotary))

        # an encoding may want the elements of every q and k head stored in another order (its
        # pairs side by side for the kernels); scores do not change when q and k move together
        order = getattr(self.position, "row_order", lambda: None)()

        def reorder(rows, heads):
            index = (torch.arange(heads).view(-1, 1) * self.head_dim + torch.tensor(order).view(1, -1)).reshape(-1)
            return rows.index_select(0, index.to(rows.device)).contiguous()

        def stacked(suffix):
            q, k, v = (tensors[f"{name}_proj.{suffix}"] for name in "qkv")
            if order is not None:
                q, k = reorder(q, self.num_heads), reorder(k, self.num_kv_heads)
            if self.paired:
                q = ops.pair_rotary_rows(q, self.num_heads, self.head_dim, rotary)
                k = ops.pair_rotary_rows(k, self.num_kv_heads, self.head_dim, rotary)
            return torch.cat([q, k, v]).contiguous()

        self.w_qkv = ops.prepare_weight(stacked("weight"))
        self.b_qkv = stacked("bias") if self.qkv_bias else None
        self.w_o = runtime.ops.prepare_weight(tensors["o_proj.weight"])
        if self.position is not None:
            self.position.bind({}, runtime)
        runtime.ops.require_attention(self.head_dim)

    takes_normed_input = True   # x goes to ops.linear only
    kernels_through_ops = True  # every kernel of this part is a method of ``Ops``: a decode step may be recorded

    def forward(self, x, ctx, binding):
        rt = self.runtime
        tokens = x.shape[0]
        kv = binding.kv
        q_buffer = rt.workspace.get("attention.q", tokens, self.q_width, rt.dtype)
        q = None
        if self.paired:   # a few decode tokens: projection, rotation and cache write in one kernel
            q = rt.ops.qkv_rope(x, self.w_qkv, self.b_qkv, ctx, kv, self.position, self.num_heads,
                                self.num_kv_heads, self.head_dim, binding.owns_cache, q_buffer)
        if q is None:
            qkv = rt.workspace.get("attention.qkv", tokens, self.qkv_width, rt.dtype)
            # for few tokens the projection may come back as partial sums that the next kernel adds up
            qkv = rt.ops.linear(x, self.w_qkv, self.b_qkv, qkv, allow_partials=True, tag="attention.qkv",
                                defer_bias=True)
            q = rt.ops.rope_kv_write(
                qkv, ctx, kv, self.position, self.num_heads, self.num_kv_heads, self.head_dim,
                write_cache=binding.owns_cache, q_buffer=q_buffer, paired=self.paired,
            )
        mixed = rt.workspace.get("attention.out", tokens, self.q_width, rt.dtype)
        rt.ops.attention(
            q, mixed, ctx, kv, self.num_heads, self.num_kv_heads, self.head_dim,
            self.scale, self.window,
        )
        update = rt.workspace.get("mixer.update", tokens, self.hidden_size, rt.dtype)
        return rt.ops.linear(mixed, self.w_o, None, update, allow_partials=True, tag="mixer.update",
                             residual=getattr(ctx, "residual_sink", None))


register_part("mixer", "attention", Attention, replace=True)
