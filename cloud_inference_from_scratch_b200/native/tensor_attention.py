"""Python side of the tensor-core attention kernels (csrc/attention_tensor.cu), one build per head size.

``plan`` turns a step's request lengths into the tile list of the prefill kernel (on the host,
with numpy; it rides in the step's single metadata copy).  ``run`` picks the kernel: a step in
which every request brings exactly one token goes to the split-key decode kernel, any other
step to the prefill kernel.
"""

from __future__ import annotations

from ctypes import c_float, c_int, c_void_p
from typing import Any

import numpy as np

from .build import load_library

BM = 64            # query rows of a prefill tile (must match the kernel)
SM_COUNT = 148
MIN_KEYS_PER_SPLIT = 256


def supports(head_dim: int) -> bool:
    return head_dim % 16 == 0 and 16 <= head_dim <= 256


def heads_per_tile(group: int) -> int:
    return min(group, BM)


def plan_tiles(query_lens: np.ndarray, group: int) -> dict[str, np.ndarray]:
    """Tile list of the prefill kernel: (request, first token of the tile), longest work first."""
    tokens_per_tile = BM // heads_per_tile(group)
    counts = -(-query_lens.astype(np.int64) // tokens_per_tile)
    total = int(counts.sum())
    request = np.repeat(np.arange(len(query_lens), dtype=np.int32), counts)
    first = np.cumsum(counts) - counts
    within = np.arange(total, dtype=np.int64) - np.repeat(first, counts)
    q0 = (within * tokens_per_tile).astype(np.int32)
    return {"tile_request": request[::-1].copy(), "tile_q0": q0[::-1].copy()}


class TensorAttention:
    def __init__(self, ops: Any, head_dim: int) -> None:
        from .ops import _Lib

        if not supports(head_dim):
            raise ValueError(f"tensor-core attention takes head sizes 16..256 in steps of 16, not {head_dim}")
        self.ops = ops
        self.head_dim = head_dim
        lib = _Lib(load_library("attention_tensor.cu", {"HEAD_DIM": head_dim}))
        v, i, f = c_void_p, c_int, c_float
        self._prefill = lib.function(
            "cie_attention_prefill",
            [v, i, v, i, v, v, v, i, i, v, v, i, v, v, v, i, i, i, i, f, i, v, v],
        )
        self._decode = lib.function(
            "cie_attention_decode",
            [v, i, v, i, v, v, v, i, i, v, i, i, i, i, i, f, i, v, v, v, v],
        )

    def _buffer(self, name: str, per_slot: int, requests: int, q_heads: int, splits: int) -> Any:
        # requests * splits never exceeds 2 * SM_COUNT + requests; reserve for 256 requests
        reserve = (2 * SM_COUNT + max(requests, 256)) * q_heads * per_slot
        return self.ops.scratch(f"attention.{name}.d{self.head_dim}",
                                requests * q_heads * splits * per_slot, reserve=reserve)

    @staticmethod
    def splits_for(requests: int, kv_heads: int, group: int, max_keys: int) -> int:
        ctas = requests * kv_heads * -(-group // 16)
        wanted = -(-2 * SM_COUNT // ctas)
        return max(1, min(wanted, max_keys // MIN_KEYS_PER_SPLIT))

    def run(self, qkv: Any, out: Any, ctx: Any, kv: Any, q_heads: int, kv_heads: int,
            scale: float, window: int, plan: dict[str, Any] | None = None) -> bool:
        ops = self.ops
        torch = ops.torch
        if qkv.dtype != torch.bfloat16:
            return False
        table = ctx.block_tables[kv.group]
        group = q_heads // kv_heads
        if ctx.all_decode:
            requests = ctx.num_requests
            max_keys = table.shape[1] * kv.page_size
            if window > 0:
                max_keys = min(max_keys, window)
            splits = self.splits_for(requests, kv_heads, group, max_keys)
            partial_o = partial_ml = None
            if splits > 1:
                partial_o = self._buffer("o", self.head_dim, requests, q_heads, splits)
                partial_ml = self._buffer("ml", 2, requests, q_heads, splits)
            ops.launches += 2 if splits > 1 else 1
            self._decode(qkv.data_ptr(), qkv.shape[1], out.data_ptr(), out.shape[1], kv.k.data_ptr(),
                         kv.v.data_ptr(), table.data_ptr(), table.shape[1], kv.num_pages,
                         ctx.context_lens.data_ptr(), requests, q_heads, kv_heads, kv.page_size,
                         splits, scale, window,
                         None if partial_o is None else partial_o.data_ptr(),
                         None if partial_ml is None else partial_ml.data_ptr(),
                         ops.error_word.data_ptr(), ops.stream)
            return True
        if plan is None:
            tiles = plan_tiles(ctx.host.query_lens, group)
            plan = {name: torch.from_numpy(array).to(ops.device) for name, array in tiles.items()}
        num_tiles = plan["tile_request"].shape[0]
        ops.launches += 1
        self._prefill(qkv.data_ptr(), qkv.shape[1], out.data_ptr(), out.shape[1], kv.k.data_ptr(),
                      kv.v.data_ptr(), table.data_ptr(), table.shape[1], kv.num_pages,
                      plan["tile_request"].data_ptr(), plan["tile_q0"].data_ptr(), num_tiles,
                      ctx.context_lens.data_ptr(), ctx.query_lens.data_ptr(),
                      ctx.query_start.data_ptr(), q_heads, kv_heads, kv.page_size,
                      heads_per_tile(group), scale, window, ops.error_word.data_ptr(), ops.stream)
        return True
