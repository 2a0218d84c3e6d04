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


@pytest.mark.parametrize("group", [1, 2, 7, 8, 16, 40, 128, 200])
def test_prefill_tiles_cover_every_token_once(group):
    lens = np.asarray([1, 130, 0, 64, 999], dtype=np.int32)
    plan = ta.plan_tiles(lens, group)
    per_tile = ta.BM // ta.heads_per_tile(group)
    covered = {r: np.zeros(n, dtype=np.int32) for r, n in enumerate(lens)}
    for request, q0 in zip(plan["tile_request"], plan["tile_q0"]):
        n = int(lens[request])
        assert 0 <= q0 < n
        covered[int(request)][q0:min(n, q0 + per_tile)] += 1
    for r, marks in covered.items():
        assert (marks == 1).all(), (r, marks)
