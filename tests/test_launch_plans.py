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


RINGS = [{1: 3, 2: 3, 3: 2, 4: 1, 5: 1, 6: 1}, {1: 1, 2: 1, 3: 1}, {2: 6, 4: 3, 6: 2, 8: 1}]


@pytest.mark.parametrize("rings", RINGS)
@pytest.mark.parametrize("sm_count", [148, 132, 16])
@pytest.mark.parametrize("requests,kv_heads,group,keys", SHAPES)
def test_split_decode_plan_fills_the_device_and_keeps_every_cta_keys(requests, kv_heads, group, keys, sm_count, rings):
    units = requests * kv_heads * -(-group // 16)
    limit, most = 4 * sm_count, 64
    splits, stages = TensorAttention.split_plan(units, keys, sm_count, rings, limit, most, 64, 256)
    assert 1 <= splits <= most and stages in rings
    assert splits == 1 or keys // splits >= 256                    # every CTA keeps its keys
    assert splits == 1 or units * splits <= limit                  # the scratch holds every share
    assert splits == 1 or units * splits <= sm_count * min(2, rings[stages])   # one wave
    # a ring is no deeper than the longest range a CTA can get (but a ring the kernel can be launched with)
    longest = -(-(-(-keys // splits)) // 64)
    assert stages == min(d for d in rings if d >= max(min(rings), min(stages, longest)))


def test_split_decode_plan_of_the_measured_batches():
    rings = {1: 3, 2: 3, 3: 2, 4: 1, 5: 1, 6: 1}
    assert TensorAttention.split_plan(16, 4096, 148, rings, 592, 64) == (16, 3)    # batch 8, two kv heads: two clusters of 8
    assert TensorAttention.split_plan(16, 2048, 148, rings, 592, 64) == (8, 4)     # ... tables that end at 2,048 keys
    assert TensorAttention.split_plan(16, 32768, 148, rings, 592, 64) == (18, 3)   # ... and long contexts
    assert TensorAttention.split_plan(64, 4096, 148, rings, 592, 64) == (4, 3)     # batch 32
    assert TensorAttention.split_plan(128, 4096, 148, rings, 592, 64) == (2, 3)    # batch 64
    assert TensorAttention.split_plan(2, 4096, 148, rings, 592, 64) == (16, 4)     # batch 1
    assert TensorAttention.split_plan(2, 32768, 148, rings, 592, 64) == (64, 6)    # one long request


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
