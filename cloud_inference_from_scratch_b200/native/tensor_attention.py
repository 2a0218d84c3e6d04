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
# the split decode kernel: where several shares of a unit meet in global memory, a CTA keeps at
# least this many keys (four tiles of 64), so that its set-up and the hand-over stay small beside
# the keys it streams; None: the plan's own figure
MIN_KEYS_PER_SPLIT_CTA = 256
FORCE_SPLIT_KEYS = int(os.environ["CIE_DECODE_SPLIT_KEYS"]) if os.environ.get("CIE_DECODE_SPLIT_KEYS") else None
# ... and where the CTAs of a unit are one thread-block cluster, whose shares meet in shared memory
MIN_KEYS_PER_CLUSTERED_CTA = 128
# a unit stays one cluster while a CTA's range stays within this many keys of the longest context
# (16 units in a whole step: clusters of 8 win at 3,800 keys, 1.91 against 1.96 ms, and lose at
# 6,000, 2.08 against 2.06)
ONE_CLUSTER_KEYS = 640
# this many shares of a unit the CTA with the last ticket adds up by itself; a unit that has room
# for twice as many CTAs gets clusters of 8 that add up eight of them each first (2 units of
# 32,000 keys: 21.8 us with 64 CTAs in clusters of 8 against 30.7 without; 16 units of 8,192: a
# step of 2.16 ms with 16 CTAs and no clusters, 2.21 with 18, 2.27 with one cluster of 8)
MOST_TICKETS = 16
# the tcgen05 prompt kernel: a key range of a query tile keeps at least this many tiles of 128 keys
MAX_KEY_RANGES = 4   # must match MAX_RANGES of the kernel
MIN_KEY_TILES_PER_RANGE = int(os.environ.get("CIE_PREFILL_RANGE_TILES", "4"))
# "CTAs per unit,stages,cluster" to launch the split decode kernel with whatever the sizes (for measurements)
FORCE_SPLIT_PLAN = tuple(int(n) for n in os.environ["CIE_DECODE_SPLIT_PLAN"].split(",")) if os.environ.get("CIE_DECODE_SPLIT_PLAN") else None
# several clusters per request only while each CTA keeps this many keys: handing the shares over
# through global memory costs about as much as streaming a thousand keys
MIN_KEYS_PER_CHUNKED_CTA = int(os.environ.get("CIE_DECODE_CHUNK_KEYS", "1024"))
# CTAs of clusters that can be counted on to run at one time when the device cannot be asked: a
# cluster stays inside one of the 8 GPCs, and with one CTA an SM the device reports room for 15
# clusters of 8 (a 16th waits for a second round, which costs more than the cut brings)
CLUSTERED_CTAS = 112
MAX_CHUNKS = 16                  # must match DECODE_MAX_CHUNKS of the kernel


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
        # the cluster decode kernel: where clusters of one request leave their shares (at most one
        # CTA an SM takes part), and the tickets that tell the last one; the kernel leaves the
        # tickets at zero
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
            at_once = lib.handle.cie_attention_decode_split_clusters
            at_once.argtypes = [i, i, i]
            at_once.restype = c_int
            self._split_at_once = at_once
            self.split_cluster_max = int(os.environ.get("CIE_DECODE_SPLIT_CLUSTER", "16"))
            self._split_rings: dict[tuple[int, int], dict[int, int]] = {}
            self._split_plans: dict[int, tuple[dict[int, dict[int, int]], dict[int, int]]] = {}
            if not self.split_rings(1, 1):
                raise RuntimeError(f"the split decode kernel does not fit this device at head size {head_dim}")
            # shares that meet in global memory (several clusters, or CTAs without a cluster, on one
            # unit) and their tickets: sized once for the most shares a launch can have
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
                [v, i, v, i, v, v, v, i, i, v, v, i, v, v, v, i, i, i, i, f, i, i, v, v, v, v],
            )
            # key ranges of a query tile (few query tiles over a long context): where the CTAs of a
            # tile leave their shares, and the tickets that tell the last one; a launch with key
            # ranges has at most one CTA an SM
            self.prefill_key_tile = int(tc.handle.cie_attention_prefill_tc_key_tile())
            self.prefill_ranges = os.environ.get("CIE_PREFILL_RANGES", "1") != "0"
            self._prefill_shares = torch.zeros(self.sm_count * BM * (head_dim + 2), dtype=torch.float32, device=ops.device)
            self._prefill_tickets = torch.zeros(self.sm_count, dtype=torch.int32, device=ops.device)

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

    def split_choices(self, rows: int) -> tuple[dict[int, dict[int, int]], dict[int, int]]:
        """What the split decode kernel can be launched with for ``rows`` head rows a unit, asked of
        the device once: cluster size -> (ring depth -> CTAs an SM holds), and cluster size -> how
        many such clusters run at one time with the deepest ring with which an SM still holds two CTAs."""
        rows = min(16, rows)
        if rows not in self._split_plans:
            rings = {1: self.split_rings(1, rows)}
            room: dict[int, int] = {}
            for cluster in (2, 4, 8, 16):
                if cluster > self.split_cluster_max:
                    continue
                paired = [depth for depth, ctas in self.split_rings(cluster, rows).items() if ctas >= 2]
                at_once = int(self._split_at_once(max(paired), cluster, rows)) if paired else 0
                if at_once >= 1:
                    rings[cluster] = self.split_rings(cluster, rows)
                    room[cluster] = at_once
            self._split_plans[rows] = (rings, room)
        return self._split_plans[rows]

    @staticmethod
    def split_plan(units: int, max_keys: int, sm_count: int, rings: dict[int, dict[int, int]], room: dict[int, int],
                   limit: int, most: int, tile: int = 64) -> tuple[int, int, int, int]:
        """(CTAs per unit, stages of the ring, CTAs of a cluster, least keys of a CTA) for the split
        decode kernel.  ``units``: (request, kv head, 16 heads) triples; ``rings``: cluster size ->
        (ring depth -> CTAs an SM holds with it), 1 for no clusters; ``room``: cluster size -> how
        many such clusters the device runs at one time.

        The CTAs of a unit are one thread-block cluster wherever that works out: the largest of 16,
        8, 4, 2 of which the device runs one per unit at one time, since shares that meet in shared
        memory cost a few hundred cycles and shares that meet in global memory a few microseconds.
        Only where a CTA's range of the longest context then passes ``ONE_CLUSTER_KEYS`` and the
        device has room for twice as many CTAs does a unit get more of them (each with
        ``MIN_KEYS_PER_SPLIT_CTA`` keys at least, all resident at one time, at most two an SM): up to
        ``MOST_TICKETS`` without clusters, or, with room for twice that, clusters of 8.  The ring is the deepest that leaves an SM two
        CTAs (the kernel before this one still holds its own shared memory when this one starts),
        but no deeper than the longest range a CTA can get.  A launch stays within ``limit`` shares
        (the scratch is sized for that) and a unit within ``most`` CTAs.

        Measured on a B200 at head size 128, 8 head rows a unit, in microseconds a launch
        (units x keys: this plan against the best other):
        2 x 2,100: 5.9 with (16, 3, 16) against 7.6 with (8, 3, 8);  2 x 4,000: 7.1 against 11.2;
        8 x 4,000: 9.0 with (16, 3, 16) against 11.5 with (8, 3, 8);
        16 x 4,000: 12.8 with (8, 3, 8) against 18.1 with (16, 3, 8) and 17.7 with (16, 3, 16);
        16 x 8,000: 19.1 with (16, 3, 1) against 22.2 with (8, 3, 8);
        32 x 4,000: 16.7 with (8, 3, 8) against 21.3 with (4, 3, 4);
        64 x 4,000: 25.0 with (4, 3, 4) against 32.3 with (8, 3, 8) and 38.2 with (2, 3, 2)."""
        plain = rings[1]
        paired = [depth for depth in plain if plain[depth] >= 2]
        slots = (2 if paired else 1) * sm_count
        one = 1
        for cluster in (16, 8, 4, 2):
            if (cluster <= most and units <= room.get(cluster, 0) and cluster in rings
                    and max_keys // cluster >= MIN_KEYS_PER_CLUSTERED_CTA):
                one = cluster
                break
        ctas, cluster, min_keys = one, one, MIN_KEYS_PER_CLUSTERED_CTA
        many = max(1, min(max_keys // MIN_KEYS_PER_SPLIT_CTA, slots // max(1, units), most))
        if max_keys // one > ONE_CLUSTER_KEYS and many >= 2 * one:
            min_keys = MIN_KEYS_PER_SPLIT_CTA
            clusters = min(many // 8, room.get(8, 0) // max(1, units))
            if many >= 2 * MOST_TICKETS and clusters >= 3:
                ctas, cluster = 8 * clusters, 8
            else:
                ctas, cluster = min(many, MOST_TICKETS), 1
            while ctas > cluster and units * ctas // cluster > limit:
                ctas -= cluster
        depths = rings[cluster]
        if cluster > 1 or paired:
            stages = max(depth for depth in depths if depths[depth] >= 2)
        else:
            stages = max(depths)
        # no deeper than the longest range a CTA can get
        wanted = max(min(depths), min(stages, -(-(-(-max_keys // ctas)) // tile)))
        stages = min(depth for depth in depths if depth >= wanted)
        return ctas, stages, cluster, min_keys

    @staticmethod
    def key_ranges(ctas: int, max_keys: int, sm_count: int, key_tile: int) -> int:
        """Key ranges per query tile of the tcgen05 prompt kernel: a launch of ``ctas`` query tiles
        (times kv heads) that leaves most SMs idle cuts the keys of a tile over up to 4 CTAs, as
        long as the launch stays within one CTA an SM and every range keeps
        ``MIN_KEY_TILES_PER_RANGE`` key tiles of the longest context the tables hold (a tile of
        128 keys takes a CTA about a microsecond, setting a CTA up and adding its share up several)."""
        if ctas < 1 or ctas * 2 > sm_count:
            return 1
        return max(1, min(MAX_KEY_RANGES, sm_count // ctas, max_keys // (key_tile * MIN_KEY_TILES_PER_RANGE)))

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
            rings, room = self.split_choices(group)
            ctas, stages, cluster, min_keys = self.split_plan(units, max_keys, self.sm_count, rings, room,
                                                              self.split_cta_limit, self.split_max, self.split_tile)
            if FORCE_SPLIT_PLAN:
                ctas, stages, cluster = FORCE_SPLIT_PLAN
            if FORCE_SPLIT_KEYS:
                min_keys = FORCE_SPLIT_KEYS
            self._decode_split(qkv.data_ptr(), qkv.shape[1], out.data_ptr(), out.shape[1], kv.k.data_ptr(),
                               kv.v.data_ptr(), table.data_ptr(), table.shape[1], kv.num_pages,
                               ctx.context_lens.data_ptr(), requests, q_heads, kv_heads, page, ctas,
                               min_keys, stages, cluster, self._split_shares.data_ptr(),
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
            ranges = 1
            if self.prefill_ranges:
                ctas = num_tiles * kv_heads * -(-group // heads_per_tile(group))
                ranges = self.key_ranges(ctas, table.shape[1] * kv.page_size, self.sm_count, self.prefill_key_tile)
            self._prefill_tc(qkv.data_ptr(), qkv.shape[1], out.data_ptr(), out.shape[1], kv.k.data_ptr(),
                             kv.v.data_ptr(), table.data_ptr(), table.shape[1], kv.num_pages,
                             plan["tile_request"].data_ptr(), plan["tile_q0"].data_ptr(), num_tiles,
                             ctx.context_lens.data_ptr(), ctx.query_lens.data_ptr(),
                             ctx.query_start.data_ptr(), q_heads, kv_heads, kv.page_size,
                             heads_per_tile(group), scale, ranges, MIN_KEY_TILES_PER_RANGE,
                             self._prefill_shares.data_ptr(), self._prefill_tickets.data_ptr(),
                             ops.error_word.data_ptr(), ops.stream)
            return True
        self._prefill(qkv.data_ptr(), qkv.shape[1], out.data_ptr(), out.shape[1], kv.k.data_ptr(),
                      kv.v.data_ptr(), table.data_ptr(), table.shape[1], kv.num_pages,
                      plan["tile_request"].data_ptr(), plan["tile_q0"].data_ptr(), num_tiles,
                      ctx.context_lens.data_ptr(), ctx.query_lens.data_ptr(),
                      ctx.query_start.data_ptr(), q_heads, kv_heads, kv.page_size,
                      heads_per_tile(group), scale, window, ops.error_word.data_ptr(), ops.stream)
        return True
