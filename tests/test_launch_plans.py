"""Host-side launch plans of the attention kernels: pure arithmetic, checked without a GPU."""

import numpy as np
import pytest

from cloud_inference_from_scratch_b200.native import tensor_attention as ta
from cloud_inference_from_scratch_b200.native.tensor_attention import TensorAttention

SHAPES = [(requests, kv_heads, group, keys)
          for requests in (1, 2, 3, 8, 16, 64, 200)
          for kv_heads, group in ((2, 8), (1, 4), (4, 7), (8, 1), (1, 20))
          for keys in (16, 100, 2304, 9008, 33024)]


@pytest.mark.parametrize("requests,kv_heads,group,keys", SHAPES)
def test_decode_splits_are_a_power_of_two_that_leaves_every_cta_keys(requests, kv_heads, group, keys):
    splits = TensorAttention.splits_for(requests, kv_heads, group, keys)
    assert splits in (1, 2, 4, 8)
    assert splits == 1 or keys // splits >= ta.MIN_KEYS_PER_SPLIT
    ctas = requests * kv_heads * -(-group // 16)
    # a cut is made only while it does not ask for more CTAs than there are SMs
    assert splits == 1 or ctas * splits <= ta.SM_COUNT


@pytest.mark.parametrize("room", [112, 128, 147])
@pytest.mark.parametrize("requests,kv_heads,group,keys", SHAPES)
def test_decode_clusters_fit_the_room_and_keep_their_keys(requests, kv_heads, group, keys, room):
    splits = TensorAttention.splits_for(requests, kv_heads, group, keys)
    chunks = TensorAttention.chunks_for(requests, kv_heads, group, keys, splits, room)
    ctas = requests * kv_heads * -(-group // 16) * splits
    assert 1 <= chunks <= ta.MAX_CHUNKS
    if chunks > 1:
        assert ctas * chunks <= room
        assert ctas * 4 <= room                       # only when most SMs would be idle otherwise
        assert keys // (splits * chunks) >= ta.MIN_KEYS_PER_CHUNKED_CTA


def test_the_headline_batch_keeps_one_cluster_a_request():
    for keys in (2304, 4096, 32768):
        splits = TensorAttention.splits_for(8, 2, 8, keys)
        assert TensorAttention.chunks_for(8, 2, 8, keys, splits) == 1


# what a device may answer: cluster size -> (ring depth -> CTAs an SM holds), and cluster size -> clusters at one time
CHOICES = [
    ({1: {1: 3, 2: 3, 3: 2, 4: 1, 5: 1, 6: 1}, 2: {1: 3, 2: 3, 3: 2, 4: 1}, 4: {1: 3, 2: 2, 3: 2, 4: 1},
      8: {1: 3, 2: 2, 3: 2, 4: 1}, 16: {1: 3, 2: 2, 3: 2}}, {2: 148, 4: 72, 8: 32, 16: 8}),
    ({1: {1: 1, 2: 1, 3: 1}}, {}),                                   # no room for two CTAs an SM, no clusters
    ({1: {2: 6, 4: 3, 6: 2, 8: 1}, 8: {2: 4, 4: 2}}, {8: 30}),       # clusters of 8 only
]


@pytest.mark.parametrize("rings,room", CHOICES)
@pytest.mark.parametrize("sm_count", [148, 132, 16])
@pytest.mark.parametrize("requests,kv_heads,group,keys", SHAPES)
def test_split_decode_plan_fills_the_device_and_keeps_every_cta_keys(requests, kv_heads, group, keys, sm_count, rings, room):
    units = requests * kv_heads * -(-group // 16)
    limit, most = 4 * sm_count, 64
    room = {cluster: min(at_once, 2 * sm_count // cluster) for cluster, at_once in room.items()}
    ctas, stages, cluster, min_keys = TensorAttention.split_plan(units, keys, sm_count, rings, room, limit, most, 64)
    assert 1 <= ctas <= most and cluster in rings and stages in rings[cluster]
    assert ctas % cluster == 0
    assert ctas == 1 or keys // ctas >= min_keys                   # every CTA keeps its keys
    if cluster > 1:
        assert units * (ctas // cluster) <= room[cluster]          # every cluster runs at once
        assert rings[cluster][stages] >= 2
    if ctas > cluster:                                             # shares that meet in global memory
        assert min_keys == ta.MIN_KEYS_PER_SPLIT_CTA
        assert units * ctas // cluster <= limit                    # the scratch holds every share
        assert units * ctas <= sm_count * min(2, rings[cluster][stages])   # one wave
        assert ctas <= ta.MOST_TICKETS if cluster == 1 else cluster == 8 and ctas >= 24
    else:
        assert ctas == cluster
    # a ring is no deeper than the longest range a CTA can get (but a ring the kernel can be launched with)
    longest = -(-(-(-keys // ctas)) // 64)
    depths = rings[cluster]
    assert stages == min(d for d in depths if d >= max(min(depths), min(stages, longest)))


def test_split_decode_plan_of_the_measured_batches():
    rings, room = CHOICES[0]
    plan = lambda units, keys: TensorAttention.split_plan(units, keys, 148, rings, room, 592, 64)
    assert plan(2, 4096) == (16, 3, 16, 128)      # batch 1, two kv heads: one cluster of 16 a unit
    assert plan(8, 4096) == (16, 3, 16, 128)      # batch 4
    assert plan(16, 4096) == (8, 3, 8, 128)       # batch 8: 16 clusters of 16 would not run at one time
    assert plan(16, 2048) == (8, 3, 8, 128)
    assert plan(16, 5120) == (8, 3, 8, 128)
    assert plan(16, 8192) == (16, 3, 1, 256)      # ... longer contexts: more CTAs, shares through global memory
    assert plan(16, 32768) == (16, 3, 1, 256)
    assert plan(32, 8192) == (8, 3, 8, 128)       # batch 16: no room for twice the CTAs
    assert plan(64, 4096) == (4, 3, 4, 128)       # batch 32
    assert plan(128, 4096) == (2, 3, 2, 128)      # batch 64
    assert plan(300, 4096) == (1, 3, 1, 128)
    assert plan(2, 32768) == (64, 3, 8, 256)      # one long request: 8 clusters of 8 a unit
    assert plan(8, 32768) == (32, 3, 8, 256)
    assert plan(2, 512) == (4, 2, 4, 128)         # short tables: no more CTAs than have 128 keys, no deeper ring than their range


@pytest.mark.parametrize("group", [1, 2, 7, 8, 16, 40, 128, 200])
def test_prefill_tiles_cover_every_token_once(group):
    lens = np.asarray([1, 130, 0, 64, 999], dtype=np.int32)
    plan = ta.plan_tiles(lens, group)
    skipping = ta.plan_tiles(lens, group, skip=2)      # the first two requests go to the decode kernel
    assert set(skipping["tile_request"].tolist()) == {3, 4}
    per_tile = ta.BM // ta.heads_per_tile(group)
    covered = {r: np.zeros(n, dtype=np.int32) for r, n in enumerate(lens)}
    for request, q0 in zip(plan["tile_request"], plan["tile_q0"]):
        n = int(lens[request])
        assert 0 <= q0 < n
        covered[int(request)][q0:min(n, q0 + per_tile)] += 1
    for r, marks in covered.items():
        assert (marks == 1).all(), (r, marks)


# ------------------------------------------------------------------ weight-streaming tcgen05 product
@pytest.mark.parametrize("m", [17, 64, 128, 129, 256])
@pytest.mark.parametrize("n,k,silu", [(2560, 2048, False), (2048, 2048, False), (22016, 2048, True), (2048, 11008, False),
                                      (151936, 2048, False), (331, 96, False), (64, 4096, True), (37888, 3584, True)])
def test_skinny_plan_fits_the_kernel(m, n, k, silu):
    from cloud_inference_from_scratch_b200.native import skinny

    room = {2: 74, 4: 36, 8: 15}
    limit = 232448
    rows, k_parts, stages = skinny.plan(m, n, k, silu, 148, lambda rows, k_parts, stages: room[k_parts], limit)
    assert rows % (32 if silu else 16) == 0 and 16 <= rows <= 256 and k_parts in (1, 2, 4, 8)
    assert 2 <= stages <= skinny.MAX_STAGES and skinny.smem_bytes(m, rows, stages) <= limit
    k_blocks = -(-k // 64)
    assert k_parts == 1 or k_blocks // k_parts >= skinny.MIN_K_BLOCKS
    assert stages <= -(-k_blocks // k_parts)                     # no deeper than the K range of a CTA
    if k_parts > 1:                                              # the ring holds the sums a cluster exchanges
        assert (2 if m > 128 else 1) * 128 * (rows + 4) * 4 <= skinny.smem_bytes(m, rows, stages) - 1024
        assert -(-n // rows) <= room[k_parts] or n > 256 * room[k_parts]


def test_skinny_plan_deals_the_weight_rows_out_evenly():
    from cloud_inference_from_scratch_b200.native import skinny

    room = {2: 74, 4: 36, 8: 15}
    at_once = lambda rows, k_parts, stages: room[k_parts]
    rows, k_parts, _ = skinny.plan(64, 22016, 2048, True, 148, at_once, 232448)
    assert k_parts == 1 and -(-22016 // rows) <= 148 and rows * 148 < 22016 * 1.1   # one round, within a tenth of even
    rows, k_parts, _ = skinny.plan(64, 2048, 11008, False, 148, at_once, 232448)
    assert k_parts > 1                                                              # few rows, long K: cut along K
    assert skinny.plan(64, 2048, 64, False, 148, lambda *a: 0, 232448) is None      # one block of K cannot fill a ring of two


def test_prompt_attention_key_ranges():
    key_ranges = TensorAttention.key_ranges
    assert key_ranges(256, 4096, 148, 128) == 1            # a whole prompt fills the device by itself
    assert key_ranges(32, 4096, 148, 128) == 4             # 256 tokens of the 3B shape: 32 query tiles
    assert key_ranges(64, 4096, 148, 128) == 2             # 512 tokens
    assert key_ranges(8, 1024, 148, 128) == 2              # tables that hold few keys: no more ranges than have four tiles
    assert key_ranges(8, 256, 148, 128) == 1 and key_ranges(0, 4096, 148, 128) == 1
    for ctas in range(1, 200):
        for keys in (128, 4096, 1 << 20):
            ranges = key_ranges(ctas, keys, 148, 128)
            assert 1 <= ranges <= ta.MAX_KEY_RANGES and (ranges == 1 or ctas * ranges <= 148)
