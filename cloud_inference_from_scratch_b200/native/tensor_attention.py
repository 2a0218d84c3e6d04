"""Python side of the tensor-core attention kernels (csrc/attention_tensor.cu and
csrc/attention_prefill_tc.cu), one build per head size.

``plan`` turns a step's request lengths into the tile list of the prefill kernels (on the host,
with numpy; it rides in the step's single metadata copy).  ``run`` picks the kernels: requests
that bring exactly one token (they lead the batch) go to the split-key decode kernel; the
others to the tcgen05 prefill kernel where it exists (head size 64 or 128, no window, pages of a
multiple of 16 tokens), else to the mma.sync prefill kernel.  A mixed step therefore launches
two attention kernels, each on its own rows.
"""

from __future__ import annotations

import os

from ctypes import c_float, c_int, c_void_p
from typing import Any

import numpy as np

from .build import load_library

BM = 128           # query rows of a prefill tile (must match the kernel)
SM_COUNT = 148     # only where the device cannot be asked (the planners take the device's own count)
MIN_KEYS_PER_SPLIT = 128
# the split decode kernel: a CTA keeps at least this many keys (four stages of 64), so that its
# set-up and the hand-over of its share stay small beside the keys it streams
MIN_KEYS_PER_SPLIT_CTA = int(os.environ.get("CIE_DECODE_SPLIT_KEYS", "256"))
# "CTAs per unit,stages[,cluster]" to launch the split decode kernel with whatever the sizes (for measurements)
FORCE_SPLIT_PLAN = tuple(int(n) for n in os.environ["CIE_DECODE_SPLIT_PLAN"].split(",")) if os.environ.get("CIE_DECODE_SPLIT_PLAN") else None
# several clusters per request only while each CTA keeps this many keys: handing the shares over
# through global memory costs about as much as streaming a thousand keys
MIN_KEYS_PER_CHUNKED_CTA = int(os.environ.get("CIE_DECODE_CHUNK_KEYS", "1024"))
# CTAs of clusters that can be counted on to run at one time when the device cannot be asked: a
# cluster stays inside one of the 8 GPCs, and with one CTA an SM the device reports room for 15
# clusters of 8 (a 16th waits for a second round, which costs more than the cut brings)
CLUSTERED_CTAS = 112
MAX_CHUNKS = 16                  # must match DECODE_MAX_CHUNKS of the kernel
# the split decode kernel: from this many keys a CTA on, the CTAs of a unit form no cluster (8 requests of
# 32,000 keys: 3.42 ms a step with 18 CTAs a unit and tickets against 3.85 with two clusters of 8)
LONG_RANGE_KEYS = 1024


def supports(head_dim: int) -> bool:
    return head_dim % 16 == 0 and 16 <= head_dim <= 256


def heads_per_tile(group: int) -> int:
    return min(group, BM)


def plan_tiles(query_lens: np.ndarray, group: int, skip: int = 0) -> dict[str, np.ndarray]:
    """Tile list of the prefill kernel: (request, first token of the tile), longest work first.
    The first ``skip`` requests get no tile (single tokens that the decode kernel takes)."""
    tokens_per_tile = BM // heads_per_tile(group)
    counts = -(-query_lens.astype(np.int64) // tokens_per_tile)
    counts[:skip] = 0
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
            [v, i, v, i, v, v, v, i, i, v, i, i, i, i, i, i, i, v, v, f, i, i, v, v],
        )
        self._decode_clusters = lib.handle.cie_attention_decode_clusters
        self._decode_clusters.argtypes = [i, i]
        self._decode_clusters.restype = c_int
        self._cluster_room: dict[int, int] = {}
        # the split decode kernel (no clusters; shares merged by whoever draws the last ticket): for
        # pools TMA can read.  Its scratch is sized once for the most CTAs a launch with more than
        # one CTA per unit can have: four per SM.
        # where clusters of one request leave their shares (at most one CTA an SM takes part), and
        # the tickets that tell the last one; the kernel leaves the tickets at zero
        torch = ops.torch
        self.sm_count = ops.torch.cuda.get_device_properties(ops.device).multi_processor_count
        self._chunk_shares = torch.zeros(self.sm_count * 16 * (head_dim + 2), dtype=torch.float32, device=ops.device)
        self._chunk_tickets = torch.zeros(self.sm_count, dtype=torch.int32, device=ops.device)
        self._decode_split = None
        if head_dim % 64 == 0 and os.environ.get("CIE_DECODE_SPLIT", "1") != "0":
            self._decode_split = lib.function(
                "cie_attention_decode_split",
                [v, i, v, i, v, v, v, i, i, v, i, i, i, i, i, i, i, i, v, v, f, i, v, v],
            )
            self.split_max = int(lib.handle.cie_attention_decode_split_max())
            self.split_tile = int(lib.handle.cie_attention_decode_split_tile())
            per_sm = lib.handle.cie_attention_decode_split_ctas_per_sm
            per_sm.argtypes = [i, i, i]
            per_sm.restype = c_int
            self._split_per_sm = per_sm
            self.split_cluster_max = int(os.environ.get("CIE_DECODE_SPLIT_CLUSTER", "8"))
            self._split_rings: dict[tuple[int, int], dict[int, int]] = {}
            if not self.split_rings(1, 1):
                raise RuntimeError(f"the split decode kernel does not fit this device at head size {head_dim}")
            self.split_cta_limit = 4 * self.sm_count
            self._split_shares = ops.torch.zeros(self.split_cta_limit * 16 * (head_dim + 4), dtype=ops.torch.float32,
                                                 device=ops.device)
            self._split_tickets = ops.torch.zeros(self.split_cta_limit, dtype=ops.torch.int32, device=ops.device)

        self.use_tma = 0 if os.environ.get("CIE_DECODE_TMA", "1") == "0" else 1
        # prompt portions on tcgen05 where the kernel exists: head size 64 or 128, no window,
        # pages of a multiple of 16 tokens; everything else stays on the mma.sync kernel
        self._prefill_tc = None
        if head_dim in (64, 128) and os.environ.get("CIE_PREFILL_TC", "1") != "0":
            defines = {"HEAD_DIM": head_dim}
            for name in ("TC_BN", "TC_STAGES", "TC_KEY_PRODUCERS", "TC_VALUE_PRODUCERS"):
                if os.environ.get("CIE_" + name):
                    defines[name] = int(os.environ["CIE_" + name])
            tc = _Lib(load_library("attention_prefill_tc.cu", defines))
            self._prefill_tc = tc.function(
                "cie_attention_prefill_tc",
                [v, i, v, i, v, v, v, i, i, v, v, i, v, v, v, i, i, i, i, f, v, v],
            )

    def cluster_room(self, splits: int) -> int:
        """CTAs in clusters of ``splits`` that run at one time, one cluster held back for whatever
        still runs beside them (asked of the device once per cluster size)."""
        room = self._cluster_room.get(splits)
        if room is None:
            clusters = int(self._decode_clusters(splits, self.use_tma))
            room = CLUSTERED_CTAS if clusters < 2 else min(self.sm_count, (clusters - 1) * splits)
            self._cluster_room[splits] = room
        return room

    def split_rings(self, cluster: int, rows: int) -> dict[int, int]:
        """Ring depths the split decode kernel can be launched with for clusters of ``cluster`` CTAs
        and ``rows`` head rows a unit, and how many CTAs an SM then holds (a CTA of a cluster keeps
        room for its peers' shares of the rows it owns); asked of the device once."""
        key = (cluster, min(16, rows))
        if key not in self._split_rings:
            rings = {stages: int(self._split_per_sm(stages, key[0], key[1])) for stages in range(1, 9)}
            self._split_rings[key] = {stages: ctas for stages, ctas in rings.items() if ctas >= 1}
        return self._split_rings[key]

    def cluster_for(self, ctas: int) -> int:
        """CTAs of a unit that form one thread-block cluster: the largest of 8, 4, 2 that the unit's
        CTAs fill at least once (and the device has a ring for), else no cluster."""
        for cluster in (8, 4, 2):
            if cluster <= min(ctas, self.split_cluster_max):
                return cluster
        return 1

    @staticmethod
    def split_plan(units: int, max_keys: int, sm_count: int, rings: dict[int, int], limit: int, most: int,
                   tile: int = 64, min_keys: int = MIN_KEYS_PER_SPLIT_CTA) -> tuple[int, int]:
        """(CTAs per unit, stages of the ring) for the split decode kernel.  ``units``: (request, kv
        head, 16 heads) triples; ``rings``: ring depth -> CTAs an SM holds with it.

        Few units (half the SMs or fewer): one CTA an SM with the deepest ring, so that a CTA can ask
        for its whole range of keys at once, even before the kernel before it has finished; unless
        two CTAs an SM let a unit have more CTAs that each still keep ``min_keys`` keys (long
        contexts).  More units: two CTAs an SM with the deepest ring that allows it (a CTA is four warps, and four
        warps alone do not keep an SM's tensor pipe and copy engine busy), every CTA of the launch
        resident at one time.  Every CTA keeps at least ``min_keys`` keys of the longest context the
        tables hold; a launch stays within ``limit`` CTAs (the scratch is sized for that) and a unit
        within ``most``.  Measured on a B200 at head size 128: 8 requests of 2,048 keys 9.8 us with
        (9, 6) against 10.4 with (8, 3); 64 requests 26.8 us with (2, 3) against 37 with (1, 6)."""
        depths = sorted(rings, reverse=True)
        paired = [depth for depth in depths if rings[depth] >= 2]
        by_keys = max(1, max_keys // min_keys)
        alone = max(1, min(by_keys, sm_count // max(1, units), most))          # CTAs a unit gets at one CTA an SM
        doubled = max(1, min(by_keys, 2 * sm_count // max(1, units), most))    # ... at two
        if units * 2 <= sm_count and paired and doubled > alone:
            # long contexts: more CTAs a unit, each still with its keys, stream more than a deep ring
            # does (8 requests of 32,000 keys: 3.42 ms a step with (18, 3) against 4.25 with (9, 6))
            stages, slots = paired[0], 2 * sm_count
        elif units * 2 <= sm_count or not paired:
            stages, slots = depths[0], sm_count
        else:
            stages, slots = paired[0], 2 * sm_count
        splits = max(1, min(by_keys, slots // max(1, units), most))
        while splits > 1 and units * splits > limit:
            splits -= 1
        # no deeper than the longest range a CTA can get
        wanted = max(min(depths), min(stages, -(-(-(-max_keys // splits)) // tile)))
        stages = min(depth for depth in depths if depth >= wanted)
        return splits, stages

    @staticmethod
    def splits_for(requests: int, kv_heads: int, group: int, max_keys: int, sm_count: int = SM_COUNT) -> int:
        """CTAs (of one cluster) that share a request's keys: enough to put work on every SM,
        at least MIN_KEYS_PER_SPLIT keys each, a power of two up to 8."""
        ctas = requests * kv_heads * -(-group // 16)
        limit = max(1, max_keys // MIN_KEYS_PER_SPLIT)
        splits = 1
        while splits < 8 and ctas * splits * 2 <= sm_count and splits * 2 <= limit:
            splits *= 2
        if splits == 8 and ctas * splits > sm_count // 2:
            splits = 4   # big clusters cost more than they bring once half the SMs have work
        return splits

    @staticmethod
    def chunks_for(requests: int, kv_heads: int, group: int, max_keys: int, splits: int,
                   room: int = CLUSTERED_CTAS) -> int:
        """Clusters per request: long contexts at small batches leave most SMs without work
        even with clusters of 8, so the keys are cut once more, as long as every SM gets at
        most one CTA (``room`` CTAs run at one time) and every CTA keeps MIN_KEYS_PER_CHUNKED_CTA keys."""
        ctas = requests * kv_heads * -(-group // 16) * splits
        if ctas * 4 > room:
            return 1   # half the SMs have work already: measured, a second cluster brings nothing
        by_sms = room // ctas
        by_keys = max_keys // (splits * MIN_KEYS_PER_CHUNKED_CTA)
        return max(1, min(by_sms, by_keys, MAX_CHUNKS))

    def _run_decode(self, qkv: Any, out: Any, ctx: Any, kv: Any, table: Any, requests: int, q_heads: int,
                    kv_heads: int, scale: float, window: int) -> None:
        """One query token for each of the first ``requests`` requests of the step (their token row
        is their request index)."""
        ops = self.ops
        group = q_heads // kv_heads
        max_keys = table.shape[1] * kv.page_size
        if window > 0:
            max_keys = min(max_keys, window)
        page = kv.page_size
        ops.launches += 1
        if (self._decode_split is not None and page >= 16 and page & (page - 1) == 0
                and (kv.k.data_ptr() | kv.v.data_ptr()) % 16 == 0):
            units = requests * kv_heads * -(-group // 16)
            ctas, stages = self.split_plan(units, max_keys, self.sm_count, self.split_rings(1, group), self.split_cta_limit,
                                           self.split_max, self.split_tile, MIN_KEYS_PER_SPLIT_CTA)
            cluster = self.cluster_for(ctas)
            if max_keys // max(1, ctas) >= LONG_RANGE_KEYS:
                cluster = 1   # ranges this long hide the hand-over through global memory; clusters only bind the placement
            if cluster > 1:
                # Neighbouring CTAs of a unit in one cluster: whole clusters, and the deepest ring with
                # which an SM still holds two CTAs.  (A cluster starts only when all its CTAs find room in
                # one part of the device; with one CTA an SM the 16th cluster of 8 waits for a second
                # round, which costs more than the exchange through shared memory saves.)
                ctas -= ctas % cluster
                rings = self.split_rings(cluster, group)
                paired = [depth for depth in rings if rings[depth] >= 2]
                if paired:
                    stages = max(paired)
                else:
                    cluster = 1
            if FORCE_SPLIT_PLAN:
                ctas, stages = FORCE_SPLIT_PLAN[:2]
                cluster = FORCE_SPLIT_PLAN[2] if len(FORCE_SPLIT_PLAN) > 2 else self.cluster_for(ctas)
            self._decode_split(qkv.data_ptr(), qkv.shape[1], out.data_ptr(), out.shape[1], kv.k.data_ptr(),
                               kv.v.data_ptr(), table.data_ptr(), table.shape[1], kv.num_pages,
                               ctx.context_lens.data_ptr(), requests, q_heads, kv_heads, page, ctas,
                               MIN_KEYS_PER_SPLIT_CTA, stages, cluster, self._split_shares.data_ptr(),
                               self._split_tickets.data_ptr(), scale, window, ops.error_word.data_ptr(),
                               ops.stream)
            return
        splits = self.splits_for(requests, kv_heads, group, max_keys, self.sm_count)
        chunks = self.chunks_for(requests, kv_heads, group, max_keys, splits, self.cluster_room(splits))
        self._decode(qkv.data_ptr(), qkv.shape[1], out.data_ptr(), out.shape[1], kv.k.data_ptr(),
                     kv.v.data_ptr(), table.data_ptr(), table.shape[1], kv.num_pages,
                     ctx.context_lens.data_ptr(), requests, q_heads, kv_heads, kv.page_size,
                     splits, chunks, MIN_KEYS_PER_CHUNKED_CTA, self._chunk_shares.data_ptr(), self._chunk_tickets.data_ptr(),
                     scale, window, self.use_tma, ops.error_word.data_ptr(), ops.stream)

    def run(self, qkv: Any, out: Any, ctx: Any, kv: Any, q_heads: int, kv_heads: int,
            scale: float, window: int, plan: dict[str, Any] | None = None) -> bool:
        ops = self.ops
        torch = ops.torch
        if qkv.dtype != torch.bfloat16:
            return False
        table = ctx.block_tables[kv.group]
        group = q_heads // kv_heads
        singles = ctx.num_single
        program = ops.program
        if (program is not None and singles == ctx.num_requests
                and program.can_attend(self.head_dim, kv.page_size, singles, kv.k, kv.v)):
            # a decode step that is being recorded: a phase of its program, not a launch
            program.attention(qkv, out, kv.k, kv.v, table, kv.num_pages, ctx.context_lens, singles, q_heads,
                              kv_heads, self.head_dim, kv.page_size, scale, window)
            return True
        ops._flush()
        if singles:
            self._run_decode(qkv, out, ctx, kv, table, singles, q_heads, kv_heads, scale, window)
            if singles == ctx.num_requests:
                return True
        if plan is None:
            tiles = plan_tiles(ctx.host.query_lens, group, skip=singles)
            plan = {name: torch.from_numpy(array).to(ops.device) for name, array in tiles.items()}
        num_tiles = plan["tile_request"].shape[0]
        ops.launches += 1
        if (self._prefill_tc is not None and window <= 0 and kv.page_size % 16 == 0
                and qkv.shape[1] % 8 == 0 and out.shape[1] % 8 == 0):
            self._prefill_tc(qkv.data_ptr(), qkv.shape[1], out.data_ptr(), out.shape[1], kv.k.data_ptr(),
                             kv.v.data_ptr(), table.data_ptr(), table.shape[1], kv.num_pages,
                             plan["tile_request"].data_ptr(), plan["tile_q0"].data_ptr(), num_tiles,
                             ctx.context_lens.data_ptr(), ctx.query_lens.data_ptr(),
                             ctx.query_start.data_ptr(), q_heads, kv_heads, kv.page_size,
                             heads_per_tile(group), scale, ops.error_word.data_ptr(), ops.stream)
            return True
        self._prefill(qkv.data_ptr(), qkv.shape[1], out.data_ptr(), out.shape[1], kv.k.data_ptr(),
                      kv.v.data_ptr(), table.data_ptr(), table.shape[1], kv.num_pages,
                      plan["tile_request"].data_ptr(), plan["tile_q0"].data_ptr(), num_tiles,
                      ctx.context_lens.data_ptr(), ctx.query_lens.data_ptr(),
                      ctx.query_start.data_ptr(), q_heads, kv_heads, kv.page_size,
                      heads_per_tile(group), scale, window, ops.error_word.data_ptr(), ops.stream)
        return True
