"""Python side of the weight-streaming tcgen05 product for 17 to 256 tokens (csrc/gemm_skinny.cu):
the plan of a launch and the call."""

from __future__ import annotations

import os
from ctypes import c_int, c_longlong, c_void_p
from typing import Any, Callable

from .build import load_library

OUT_BF16, OUT_F32, OUT_SILU_MUL = 0, 1, 3
MIN_ROWS, MAX_ROWS = 17, 256        # token rows the kernel is used for (fewer go to the streaming kernel)
TOKEN_TILE = 128
BLOCK_K = 64
MAX_STAGES = 12
STAGE_ALIGN = 1024
# what a cluster's exchange of sums costs, in bytes a CTA could have streamed meanwhile
EXCHANGE_BYTES = 48 * 1024
# a K range shorter than this many blocks of 64 is not worth a CTA of its own
MIN_K_BLOCKS = 4
# "rows,k_parts,stages" for every launch, whatever the sizes (for measurements)
FORCE_PLAN = tuple(int(n) for n in os.environ["CIE_SKINNY_PLAN"].split(",")) if os.environ.get("CIE_SKINNY_PLAN") else None


def smem_bytes(m: int, rows: int, stages: int) -> int:
    """Dynamic shared memory of a launch: the ring and the slack to align it (as the kernel counts)."""
    tiles_m = 2 if m > TOKEN_TILE else 1
    return stages * (tiles_m * TOKEN_TILE * BLOCK_K * 2 + rows * BLOCK_K * 2) + STAGE_ALIGN


def plan(m: int, n: int, k: int, silu: bool, sm_count: int, clusters_at_once: Callable[[int, int, int], int],
         smem_limit: int) -> tuple[int, int, int] | None:
    """(weight rows a CTA takes, K ranges of a cluster, stages of the ring) for a product of ``m``
    tokens with ``n`` weight rows over ``k``, or None if no launch fits.

    Every CTA streams ``rows`` weight rows over its K range; what decides is the most bytes any CTA
    has to bring into shared memory (its weights once, the token rows once per block of K: the copy
    engine of an SM moves about 50 KB a microsecond wherever the bytes come from), times the rounds the launch takes on the device, plus what a cluster's exchange costs.
    ``clusters_at_once(rows, k_parts, stages)`` says how many clusters the device runs at one time."""
    tiles_m = 2 if m > TOKEN_TILE else 1
    k_blocks = -(-k // BLOCK_K)
    step = 32 if silu else 16
    token_bytes = (tiles_m * TOKEN_TILE if tiles_m > 1 else -(-m // 16) * 16) * BLOCK_K * 2
    best, best_cost = None, None
    for k_parts in (1, 2, 4, 8):
        if k_parts > 1 and k_blocks // k_parts < MIN_K_BLOCKS:
            break
        longest = -(-k_blocks // k_parts)
        for rows in range(step, 256 + 1, step):
            stages = min(MAX_STAGES, longest, (smem_limit - STAGE_ALIGN) // (tiles_m * TOKEN_TILE * BLOCK_K * 2 + rows * BLOCK_K * 2))
            if stages < 2:
                continue
            if k_parts > 1 and tiles_m * TOKEN_TILE * (rows + 4) * 4 > smem_bytes(m, rows, stages) - STAGE_ALIGN:
                continue
            at_once = sm_count if k_parts == 1 else clusters_at_once(rows, k_parts, stages)
            if at_once < 1:
                continue
            row_parts = -(-n // rows)
            rounds = -(-row_parts // at_once)
            cost = rounds * (longest * (rows * BLOCK_K * 2 + token_bytes) + (EXCHANGE_BYTES if k_parts > 1 else 0))
            if best_cost is None or cost < best_cost:
                best, best_cost = (rows, k_parts, stages), cost
    return best


class SkinnyGemm:
    def __init__(self, ops: Any) -> None:
        from .ops import _Lib

        self.ops = ops
        lib = _Lib(load_library("gemm_skinny.cu"))
        v, i = c_void_p, c_int
        self._gemm = lib.function("cie_gemm_skinny", [v, v, v, v, i, i, i, i, i, i, i, v, v])
        self._clusters = lib.handle.cie_gemm_skinny_clusters
        self._clusters.argtypes = [i, i, i, i]
        self._clusters.restype = c_int
        self._smem = lib.handle.cie_gemm_skinny_smem
        self._smem.argtypes = [i, i, i]
        self._smem.restype = c_longlong
        self.smem_limit = int(lib.handle.cie_gemm_skinny_smem_limit())
        self.sm_count = ops.torch.cuda.get_device_properties(ops.device).multi_processor_count
        self._room: dict[tuple[int, int, int, int], int] = {}
        self._plans: dict[tuple[int, int, int, bool], tuple[int, int, int] | None] = {}

    def clusters_at_once(self, m: int, rows: int, k_parts: int, stages: int) -> int:
        key = (2 if m > TOKEN_TILE else 1, rows, k_parts, stages)
        if key not in self._room:
            self._room[key] = int(self._clusters(m, rows, k_parts, stages))
        return self._room[key]

    def plan(self, m: int, n: int, k: int, silu: bool) -> tuple[int, int, int] | None:
        key = (m, n, k, silu)
        if key not in self._plans:
            self._plans[key] = plan(m, n, k, silu, self.sm_count,
                                    lambda rows, k_parts, stages: self.clusters_at_once(m, rows, k_parts, stages),
                                    self.smem_limit)
        return self._plans[key]

    def supports(self, x: Any, weight: Any, m: int, n: int, k: int, silu: bool, out: Any = None) -> bool:
        if not MIN_ROWS <= m <= MAX_ROWS or k % 8 or k < 8:
            return False
        if x.data_ptr() % 16 or weight.data_ptr() % 16 or not x.is_contiguous() or not weight.is_contiguous():
            return False
        if out is not None and (out.data_ptr() % 16 or not out.is_contiguous()):
            return False   # the epilogues write whole rows of [M, N] (or [M, N / 2]) in 8- and 16-byte pieces
        if silu and n % 32:
            return False
        return (FORCE_PLAN or self.plan(m, n, k, silu)) is not None

    def launch(self, x: Any, weight: Any, bias: Any, out: Any, mode: int) -> None:
        ops = self.ops
        m, k = x.shape
        n = weight.shape[0]
        rows, k_parts, stages = FORCE_PLAN or self.plan(m, n, k, mode == OUT_SILU_MUL)
        ops.launches += 1
        self._gemm(x.data_ptr(), weight.data_ptr(), None if bias is None else bias.data_ptr(), out.data_ptr(),
                   m, n, k, mode, rows, k_parts, stages, ops.error_word.data_ptr(), ops.stream)
