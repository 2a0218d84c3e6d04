"""Each kernel alone against a plain float32 reference, at sizes other than the models' own."""

import math
from types import SimpleNamespace

import numpy as np
import pytest
import torch

import plain_model
from cloud_inference_from_scratch_b200.sampling import as_signed, draw_key, uniform_from_key

pytestmark = pytest.mark.gpu
DTYPES = [torch.float32, torch.bfloat16]


def tol(dtype):
    return dict(rtol=2e-5, atol=2e-5) if dtype == torch.float32 else dict(rtol=2e-2, atol=2e-2)


@pytest.fixture(scope="module")
def ops():
    from cloud_inference_from_scratch_b200.native import Ops

    made = {dtype: Ops("cuda:0", dtype) for dtype in DTYPES}
    yield made
    for item in made.values():
        item.check_errors()


def rand(*shape, dtype=torch.float32, scale=1.0, seed=0):
    generator = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=generator) * scale).to(dtype).cuda()


@pytest.mark.parametrize("dtype", DTYPES)
def test_embedding(ops, dtype):
    table = rand(1000, 200, dtype=dtype)
    ids = torch.tensor([0, 999, 5, 5, 123], dtype=torch.int32).cuda()
    out = torch.empty(5, 200, dtype=torch.float32).cuda()
    ops[dtype].embedding(ids, table, out)
    torch.testing.assert_close(out, plain_model.embedding(table.float().cpu(), ids.cpu().tolist()).cuda())


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("hidden", [96, 200, 2048, 5000])
def test_add_rmsnorm(ops, dtype, hidden):
    residual = rand(7, hidden, seed=1)
    update = rand(7, hidden, dtype=dtype, seed=2)
    gain = 1 + rand(hidden, scale=0.1, seed=3)
    eps = 1e-5
    expect_res = residual + update.float()
    expect = plain_model.rms_norm(expect_res.cpu(), gain.cpu(), eps).cuda()
    out = torch.empty(7, hidden, dtype=dtype).cuda()
    work = residual.clone()
    ops[dtype].add_rmsnorm(work, update, gain, eps, out)
    torch.testing.assert_close(work, expect_res)                 # 32-bit sum, written back
    torch.testing.assert_close(out.float(), expect, **tol(dtype))
    out2 = torch.empty(7, hidden, dtype=dtype).cuda()            # no update: residual untouched
    work = residual.clone()
    ops[dtype].add_rmsnorm(work, None, gain, eps, out2)
    assert torch.equal(work, residual)
    torch.testing.assert_close(out2.float(), plain_model.rms_norm(residual.cpu(), gain.cpu(), eps).cuda(), **tol(dtype))
    rows = torch.tensor([6, 0, 3], dtype=torch.int32).cuda()     # selected rows: nothing written back
    out3 = torch.empty(3, hidden, dtype=dtype).cuda()
    work = residual.clone()
    ops[dtype].add_rmsnorm(work, update, gain, eps, out3, rows)
    assert torch.equal(work, residual)
    torch.testing.assert_close(out3.float(), expect[rows.long()], **tol(dtype))


def paged_setup(lengths, page, heads, dim, dtype, seed=0, extra_pages=3, pages="shuffled"):
    """Random keys/values scattered over a page pool; returns pools, tables, dense copies.
    ``pages``: "shuffled" (every page anywhere), "consecutive" (a request's pages follow each other,
    as a fresh allocator hands them out) or "runs" (consecutive except that every fifth page is
    swapped with its neighbour)."""
    generator = torch.Generator().manual_seed(seed)
    pages_per = [-(-n // page) for n in lengths]
    total = sum(pages_per) + extra_pages
    order = torch.randperm(total, generator=generator).tolist()
    if pages != "shuffled":
        order = list(range(total))
        if pages == "runs":
            for i in range(4, total - 1, 5):
                order[i], order[i + 1] = order[i + 1], order[i]
    width = max(pages_per) + 1
    table = torch.full((len(lengths), width), -1, dtype=torch.int32)
    k_pool = torch.zeros(total, heads, page, dim)
    v_pool = torch.zeros(total, heads, page, dim)
    dense = []
    cursor = 0
    for r, n in enumerate(lengths):
        k = torch.randn(n, heads, dim, generator=generator)
        v = torch.randn(n, heads, dim, generator=generator)
        dense.append((k, v))
        for p in range(pages_per[r]):
            page_id = order[cursor]
            cursor += 1
            table[r, p] = page_id
            count = min(page, n - p * page)
            k_pool[page_id, :, :count] = k[p * page:p * page + count].transpose(0, 1)
            v_pool[page_id, :, :count] = v[p * page:p * page + count].transpose(0, 1)
    return k_pool.to(dtype).cuda(), v_pool.to(dtype).cuda(), table.cuda(), dense, total


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("page,dim,rot", [(4, 48, 32), (16, 128, 128), (32, 16, 16)])
def test_rope_kv_write(ops, dtype, page, dim, rot):
    q_heads, kv_heads = 6, 3
    starts, lens = [0, 37, 5], [9, 2, 20]
    width = (q_heads + 2 * kv_heads) * dim
    tokens = sum(lens)
    qkv = rand(tokens, width, dtype=dtype, seed=4)
    positions = torch.cat([torch.arange(s, s + n) for s, n in zip(starts, lens)]).int().cuda()
    request = torch.cat([torch.full((n,), i) for i, n in enumerate(lens)]).int().cuda()
    k_pool, v_pool, table, _, total = paged_setup([s + n for s, n in zip(starts, lens)], page, kv_heads, dim, dtype)
    before_k, before_v = k_pool.clone(), v_pool.clone()
    theta = 50000.0
    inv_freq = (1.0 / (theta ** (torch.arange(0, rot, 2, dtype=torch.float32) / rot))).cuda()
    position = SimpleNamespace(rotary_dim=rot, inv_freq=inv_freq)
    ctx = SimpleNamespace(positions=positions, request_of_token=request, block_tables=[table])
    kv = SimpleNamespace(group=0, k=k_pool, v=v_pool, num_pages=total, page_size=page)
    original = qkv.clone()
    ops[dtype].rope_kv_write(qkv, ctx, kv, position, q_heads, kv_heads, dim, write_cache=True)
    torch.cuda.synchronize()
    src = original.float().cpu().view(tokens, q_heads + 2 * kv_heads, dim)
    cos, sin = plain_model.rope_tables(rot, positions.cpu().tolist(), theta)
    want_q = plain_model.apply_rope(src[:, :q_heads], cos, sin)
    want_k = plain_model.apply_rope(src[:, q_heads:q_heads + kv_heads], cos, sin)
    want_v = src[:, q_heads + kv_heads:]
    got = qkv.float().cpu().view(tokens, q_heads + 2 * kv_heads, dim)
    torch.testing.assert_close(got[:, :q_heads], want_q, **tol(dtype))
    assert torch.equal(got[:, q_heads:], src[:, q_heads:])      # k and v stay as they were in qkv
    touched = torch.zeros_like(k_pool, dtype=torch.bool)
    for t in range(tokens):
        r, pos = int(request[t]), int(positions[t])
        page_id = int(table[r, pos // page])
        torch.testing.assert_close(k_pool[page_id, :, pos % page].float().cpu(), want_k[t], **tol(dtype))
        assert torch.equal(v_pool[page_id, :, pos % page].float().cpu(), want_v[t])
        touched[page_id, :, pos % page] = True
    assert torch.equal(k_pool[~touched], before_k[~touched])   # nothing else was written
    assert torch.equal(v_pool[~touched], before_v[~touched])
    k2, v2 = before_k.clone(), before_v.clone()                 # a run that reads another's cache
    kv2 = SimpleNamespace(group=0, k=k2, v=v2, num_pages=total, page_size=page)
    again = original.clone()
    ops[dtype].rope_kv_write(again, ctx, kv2, position, q_heads, kv_heads, dim, write_cache=False)
    assert torch.equal(k2, before_k) and torch.equal(v2, before_v)
    assert torch.equal(again, qkv)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("m", [1, 3, 8, 9, 64, 65, 130])
def test_gemm_simt_any_shape(ops, dtype, m):
    n, k = 331, 100
    x, w = rand(m, k, dtype=dtype, seed=5), rand(n, k, dtype=dtype, scale=0.1, seed=6)
    bias = rand(n, seed=7)
    want = plain_model.linear(x.float().cpu(), w.float().cpu(), bias.cpu()).cuda()
    item = ops[dtype]
    out = torch.empty(m, n, dtype=dtype).cuda()
    item._gemm_simt(x.data_ptr(), w.data_ptr(), bias.data_ptr(), out.data_ptr(), m, n, k,
                    item._code_of(x), item._code_of(out), 1, item.stream)
    torch.testing.assert_close(out.float(), want, **tol(dtype))
    wide = torch.empty(m, n, dtype=torch.float32).cuda()        # float32 output (logits)
    item._gemm_simt(x.data_ptr(), w.data_ptr(), None, wide.data_ptr(), m, n, k, item._code_of(x), 0, 0,
                    item.stream)
    torch.testing.assert_close(wide, plain_model.linear(x.float().cpu(), w.float().cpu()).cuda(),
                               rtol=2e-5, atol=2e-5)


def test_gemm_float32_rows_do_not_depend_on_the_batch(ops):
    item = ops[torch.float32]
    x, w = rand(70, 300, seed=8), rand(200, 300, scale=0.1, seed=9)
    full = torch.empty(70, 200).cuda()
    item.linear(x, w, None, full)
    for rows in (1, 2, 33):
        part = torch.empty(rows, 200).cuda()
        item.linear(x[:rows].contiguous(), w, None, part)
        assert torch.equal(part, full[:rows])


@pytest.mark.parametrize("dtype", DTYPES)
def test_linear_of_the_engine(ops, dtype):
    """Whatever kernel ``linear`` picks for the dtype: bias, float32 output, odd sizes."""
    item = ops[dtype]
    for m, n, k in [(1, 331, 96), (5, 64, 200), (130, 1000, 128), (64, 2048, 2048)]:
        x, w = rand(m, k, dtype=dtype, seed=m), item.prepare_weight(rand(n, k, scale=0.05, seed=n))
        bias = rand(n, seed=k)
        out = torch.empty(m, n, dtype=dtype).cuda()
        item.linear(x, w, bias, out)
        want = plain_model.linear(x.float().cpu(), w.float().cpu(), bias.cpu()).cuda()
        torch.testing.assert_close(out.float(), want, **tol(dtype))
        logits = torch.empty(m, n, dtype=torch.float32).cuda()
        item.linear(x, w, None, logits)
        torch.testing.assert_close(logits, plain_model.linear(x.float().cpu(), w.float().cpu()).cuda(),
                                   rtol=1e-3 if dtype == torch.bfloat16 else 2e-5, atol=1e-3 if dtype == torch.bfloat16 else 2e-5)


@pytest.mark.parametrize("dtype", DTYPES)
def test_silu_mul(ops, dtype):
    gate_up = rand(9, 2 * 208, dtype=dtype, scale=3.0, seed=10)
    out = torch.empty(9, 208, dtype=dtype).cuda()
    ops[dtype].silu_mul(gate_up, out)
    g, u = gate_up.float()[:, :208], gate_up.float()[:, 208:]
    torch.testing.assert_close(out.float(), torch.nn.functional.silu(g) * u, **tol(dtype))


def attention_case(ops, dtype, contexts, query_lens, q_heads, kv_heads, dim, page, window=0, seed=0,
                   plant=None, fn="attention_generic", pages="shuffled"):
    lengths = [c + q for c, q in zip(contexts, query_lens)]
    k_pool, v_pool, table, dense, total = paged_setup(lengths, page, kv_heads, dim, dtype, seed=seed, pages=pages)
    tokens = sum(query_lens)
    q = rand(tokens, q_heads * dim, dtype=dtype, seed=seed + 1)
    if plant is not None:   # make one far key the only one that matters for the last query
        request, key_pos, strength = plant
        row = sum(query_lens[:request + 1]) - 1
        key = dense[request][0][key_pos, 0]
        q[row, :dim] = (key * strength).to(dtype).cuda()
    positions = torch.cat([torch.arange(c, c + n) for c, n in zip(contexts, query_lens)]).int().cuda()
    request_of = torch.cat([torch.full((n,), i) for i, n in enumerate(query_lens)]).int().cuda()
    host = SimpleNamespace(query_lens=np.asarray(query_lens, dtype=np.int32),
                           context_lens=np.asarray(contexts, dtype=np.int32),
                           query_start=np.concatenate([[0], np.cumsum(query_lens)]).astype(np.int32))
    ctx = SimpleNamespace(positions=positions, request_of_token=request_of, block_tables=[table],
                          host=host, all_decode=all(n == 1 for n in query_lens), extras={},
                          num_single=next((i for i, n in enumerate(query_lens) if n != 1), len(query_lens)),
                          num_tokens=tokens, num_requests=len(query_lens),
                          context_lens=torch.tensor(contexts, dtype=torch.int32).cuda(),
                          query_lens=torch.tensor(query_lens, dtype=torch.int32).cuda(),
                          query_start=torch.tensor(host.query_start).cuda())
    kv = SimpleNamespace(group=0, k=k_pool, v=v_pool, num_pages=total, page_size=page)
    out = torch.zeros(tokens, q_heads * dim, dtype=dtype).cuda()
    scale = 1.0 / math.sqrt(dim)
    getattr(ops[dtype], fn)(q, out, ctx, kv, q_heads, kv_heads, dim, scale, window)
    torch.cuda.synchronize()
    ops[dtype].check_errors()
    start = 0
    worst = 0.0
    for r, (context, n) in enumerate(zip(contexts, query_lens)):
        k = k_pool_dense(dense[r][0], dtype)
        v = k_pool_dense(dense[r][1], dtype)
        full_q = torch.zeros(context + n, q_heads, dim)
        full_q[context:] = q[start:start + n].float().cpu().view(n, q_heads, dim)
        want = plain_model.attention(full_q, k, v, scale, window=window)[context:]
        got = out[start:start + n].float().cpu()
        worst = max(worst, float((got - want).abs().max()))
        torch.testing.assert_close(got, want, **tol(dtype))
        start += n
    return worst


def k_pool_dense(values, dtype):
    return values.to(dtype).float()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("query_len", [1, 2, 7, 16])
def test_attention_generic_context_matrix(ops, dtype, query_len):
    contexts = [0, 15, 16, 17, 127, 128, 511, 1024]
    attention_case(ops, dtype, contexts, [query_len] * len(contexts), q_heads=4, kv_heads=2, dim=64, page=16)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("dim,page,q_heads,kv_heads", [(16, 4, 6, 3), (48, 8, 5, 5), (128, 32, 8, 1), (256, 16, 2, 1), (80, 5, 3, 1)])
def test_attention_generic_sizes(ops, dtype, dim, page, q_heads, kv_heads):
    attention_case(ops, dtype, [3, 0, 200, 61], [5, 1, 1, 40], q_heads, kv_heads, dim, page, seed=3)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("window", [1, 5, 16, 100])
def test_attention_generic_window(ops, dtype, window):
    attention_case(ops, dtype, [0, 33, 150], [20, 9, 1], 4, 2, 32, 8, window=window, seed=5)


@pytest.mark.parametrize("dtype", DTYPES)
def test_attention_generic_far_key(ops, dtype):
    """The last query is aligned with key 3 of 900: its output must be that key's value."""
    attention_case(ops, dtype, [899, 10], [1, 4], 2, 1, 64, 16, seed=6, plant=(0, 3, 4.0))


def test_sampling_greedy_ties_take_the_lowest_index(ops):
    item = ops[torch.float32]
    logits = torch.full((3, 5003), -1.0).cuda()
    logits[0, 4000] = 2.0
    logits[0, 77] = 2.0
    logits[1, 5002] = 0.5
    logits[2, 0] = -0.5
    out = torch.zeros(3, dtype=torch.int32).cuda()
    item.sample(logits, None, None, out)
    assert out.tolist() == [77, 5002, 0]
    temperature = torch.zeros(3).cuda()
    keys = torch.zeros(3, dtype=torch.int64).cuda()
    item.sample(logits, temperature, keys, out)      # temperature 0 rows are greedy too
    assert out.tolist() == [77, 5002, 0]


@pytest.mark.parametrize("vocab", [331, 1000, 151936])
def test_sampling_temperature_is_the_inverse_cdf_of_the_keyed_draw(ops, vocab):
    item = ops[torch.float32]
    rows = 24
    logits = rand(rows, vocab, scale=2.0, seed=11)
    temps = torch.tensor([0.8 if r % 3 else 1.7 for r in range(rows)]).cuda()
    keys_int = [draw_key(5, r // 2, r) for r in range(rows)]
    keys = torch.tensor([as_signed(k) for k in keys_int], dtype=torch.int64).cuda()
    out = torch.zeros(rows, dtype=torch.int32).cuda()
    item.sample(logits, temps, keys, out)
    again = torch.zeros(rows, dtype=torch.int32).cuda()
    item.sample(logits, temps, keys, again)
    assert torch.equal(out, again)
    for r in range(rows):
        probs = plain_model.temperature_probs(logits[r].cpu().double(), float(temps[r])).double()
        cdf = torch.cumsum(probs, 0)
        u = uniform_from_key(keys_int[r])
        token = int(out[r])
        low = float(cdf[token - 1]) if token else 0.0
        assert low - 1e-5 <= u <= float(cdf[token]) + 1e-5, (r, token, low, u, float(cdf[token]))
    picks = {int(t) for t in out}
    assert len(picks) > rows // 2


def test_sampling_draws_follow_the_distribution(ops):
    item = ops[torch.float32]
    logits = torch.tensor([[0.0, math.log(2.0), math.log(5.0), -30.0]]).repeat(4000, 1).cuda()
    temps = torch.ones(4000).cuda()
    keys = torch.tensor([as_signed(draw_key(9, 1, i)) for i in range(4000)], dtype=torch.int64).cuda()
    out = torch.zeros(4000, dtype=torch.int32).cuda()
    item.sample(logits, temps, keys, out)
    counts = torch.bincount(out.long().cpu(), minlength=4).float() / 4000
    torch.testing.assert_close(counts, torch.tensor([0.125, 0.25, 0.625, 0.0]), atol=0.03, rtol=0)


# ------------------------------------------------------------------ tensor-core attention (bfloat16)
def tensor_case(ops, dim, *args, **kwargs):
    item = ops[torch.bfloat16]
    item.require_attention(dim)
    assert dim in item._tensor_attention, "the tensor-core attention library was not loaded"
    before = item.launches
    worst = attention_case(ops, torch.bfloat16, *args, **kwargs, fn="attention")
    assert item.launches > before
    return worst


@pytest.mark.parametrize("query_len", [1, 2, 7, 16])
@pytest.mark.parametrize("batch", [1, 2, 4, 8, 16])
def test_tensor_attention_context_matrix(ops, query_len, batch):
    """The reference's kernel matrix (tests/remote_ragged_gpu_tests.py:118-121): batches of 1..16,
    contexts across page edges up to 4000, query lengths 1, 2, 7, 16."""
    contexts = [0, 15, 16, 17, 127, 128, 511, 1024, 2047, 4000]
    chosen = [contexts[(i * 3 + batch) % len(contexts)] for i in range(batch)]
    tensor_case(ops, 128, chosen, [query_len] * batch, 16, 2, 128, 16, seed=batch)


@pytest.mark.parametrize("dim,page,q_heads,kv_heads", [
    (16, 4, 4, 2), (48, 8, 5, 5), (64, 8, 2, 1), (128, 32, 8, 1), (256, 16, 2, 1), (80, 5, 3, 1),
    (32, 16, 14, 2), (64, 16, 20, 1), (128, 16, 28, 4),
])
def test_tensor_attention_sizes(ops, dim, page, q_heads, kv_heads):
    tensor_case(ops, dim, [3, 0, 200, 61, 0], [5, 1, 1, 40, 130], q_heads, kv_heads, dim, page, seed=3)
    tensor_case(ops, dim, [3, 0, 700, 61], [1, 1, 1, 1], q_heads, kv_heads, dim, page, seed=4)


@pytest.mark.parametrize("window", [1, 5, 16, 100])
def test_tensor_attention_window(ops, window):
    tensor_case(ops, 32, [0, 33, 150], [20, 9, 1], 4, 2, 32, 8, window=window, seed=5)
    tensor_case(ops, 32, [10, 33, 450], [1, 1, 1], 4, 2, 32, 8, window=window, seed=6)


def test_tensor_attention_far_key(ops):
    """The last query is aligned with key 3 of 900 (prefill kernel) and of 4000 (split decode
    kernel): its output must be that key's value, wherever its page lies."""
    tensor_case(ops, 64, [899, 10], [1, 4], 2, 1, 64, 16, seed=6, plant=(0, 3, 4.0))
    tensor_case(ops, 64, [3999, 10], [1, 1], 2, 1, 64, 16, seed=7, plant=(0, 3, 4.0))
    tensor_case(ops, 128, [2047], [1], 16, 2, 128, 16, seed=8, plant=(0, 2040, 4.0))


def test_tensor_attention_decode_of_a_long_context_in_several_clusters(ops, monkeypatch):
    """Few requests with thousands of keys: the keys of a request go to several clusters, whose
    shares the CTA that delivers last merges.  A planted key near the start, in the middle and at
    the end of the context; a short request beside a long one (it uses one cluster of those
    launched for it); a cluster count that is no power of two; the cp.async variant; and the same
    object again and again (the tickets must be back at zero after every launch)."""
    from cloud_inference_from_scratch_b200.native import tensor_attention
    from cloud_inference_from_scratch_b200.native.tensor_attention import TensorAttention

    # the device says how many clusters run at one time; the plan keeps one of them back
    ops[torch.bfloat16].require_attention(128)
    room = ops[torch.bfloat16]._tensor_attention[128].cluster_room(8)
    assert room % 8 == 0 and 64 <= room <= 148, room
    # the threshold as it ships: 20,000 keys of one request make two clusters
    assert TensorAttention.chunks_for(1, 2, 8, 20016, TensorAttention.splits_for(1, 2, 8, 20016)) == 2
    assert TensorAttention.chunks_for(8, 2, 8, 32768, TensorAttention.splits_for(8, 2, 8, 32768)) == 1
    tensor_case(ops, 128, [20000], [1], 16, 2, 128, 16, seed=10, plant=(0, 11000, 4.0))
    # a lower one, so that shorter contexts reach every case
    monkeypatch.setattr(tensor_attention, "MIN_KEYS_PER_CHUNKED_CTA", 256)
    assert TensorAttention.chunks_for(1, 2, 8, 9008, TensorAttention.splits_for(1, 2, 8, 9008)) == 4
    tensor_case(ops, 128, [9000], [1], 16, 2, 128, 16, seed=11)
    tensor_case(ops, 128, [9000], [1], 16, 2, 128, 16, seed=12, plant=(0, 5, 4.0))
    tensor_case(ops, 128, [8999], [1], 16, 2, 128, 16, seed=13, plant=(0, 8990, 4.0))
    tensor_case(ops, 64, [6000, 37], [1, 1], 4, 1, 64, 16, seed=14, plant=(0, 3000, 4.0))
    tensor_case(ops, 32, [7000], [1], 4, 2, 32, 8, seed=15, plant=(0, 6100, 4.0))
    tensor_case(ops, 128, [20000], [1], 28, 4, 128, 32, seed=16)
    tensor_case(ops, 128, [700, 9000], [1, 1], 16, 2, 128, 16, seed=17, plant=(1, 4500, 4.0))
    # a window: the clusters share the last 5,000 keys only, and a key before them must not count
    tensor_case(ops, 32, [7000], [1], 4, 2, 32, 8, window=5000, seed=18, plant=(0, 2500, 4.0))
    tensor_case(ops, 32, [7000], [1], 4, 2, 32, 8, window=5000, seed=19, plant=(0, 1500, 4.0))


def test_split_decode_kernel(ops):
    """The decode kernel that cuts a request's keys over CTAs, in clusters or without (head sizes that
    are multiples of 64, pages of a power of two >= 16): 64 requests of very different lengths in one
    launch; a window whose first key lies inside a page; more than 16 heads on a kv head; head size
    192; planted keys in the first, a middle and the last CTA's range; and the same object again and
    again (the tickets must be back at zero after every launch)."""
    item = ops[torch.bfloat16]
    item.require_attention(128)
    assert item._tensor_attention[128]._decode_split is not None
    contexts = [(i * 379) % 4001 for i in range(64)]
    contexts[5], contexts[17], contexts[40] = 0, 15, 16
    tensor_case(ops, 128, contexts, [1] * 64, 16, 2, 128, 16, seed=20, plant=(63, contexts[63] // 2, 4.0))
    tensor_case(ops, 128, contexts[:33], [1] * 33, 16, 2, 128, 16, seed=21)
    tensor_case(ops, 128, [2047] * 8, [1] * 8, 16, 2, 128, 16, seed=22, plant=(3, 1, 4.0))
    tensor_case(ops, 128, [2047] * 8, [1] * 8, 16, 2, 128, 16, seed=23, plant=(7, 2046, 4.0))
    tensor_case(ops, 128, [30000], [1], 16, 2, 128, 16, seed=24, plant=(0, 17000, 4.0))
    tensor_case(ops, 64, [7000, 100, 16, 40], [1, 1, 1, 1], 4, 1, 64, 16, window=5000, seed=25, plant=(0, 2100, 4.0))
    tensor_case(ops, 64, [7000, 100, 16, 40], [1, 1, 1, 1], 4, 1, 64, 16, window=5000, seed=26, plant=(0, 1900, 4.0))
    tensor_case(ops, 64, [700, 100, 16, 40], [1, 1, 1, 1], 4, 1, 64, 32, window=33, seed=27)
    tensor_case(ops, 64, [900, 3], [1, 1], 20, 1, 64, 16, seed=28, plant=(0, 450, 4.0))
    tensor_case(ops, 192, [1000, 77], [1, 1], 3, 1, 192, 32, seed=29, plant=(0, 999, 4.0))
    tensor_case(ops, 256, [5000], [1], 2, 1, 256, 16, seed=30, plant=(0, 2500, 4.0))
    # a mixed step: single tokens lead, a prompt portion follows (two launches)
    tensor_case(ops, 128, [1500, 16, 700, 40], [1, 1, 1, 300], 16, 2, 128, 16, seed=31, plant=(0, 750, 4.0))


@pytest.mark.parametrize("plan,min_keys", [
    ((16, 3, 16), 128), ((16, 2, 16), 64), ((32, 3, 16), 128), ((8, 3, 8), 128), ((24, 3, 8), 256),
    ((4, 3, 4), 128), ((2, 3, 2), 128), ((16, 3, 1), 256), ((5, 6, 1), 64), ((1, 3, 1), 128),
])
def test_split_decode_kernel_with_every_kind_of_plan(ops, monkeypatch, plan, min_keys):
    """Whatever (CTAs a unit, ring depth, cluster size, least keys of a CTA) the planner may pick:
    one cluster of 16 a unit (more CTAs than head rows, so some own no row), several clusters whose
    shares meet in global memory, no clusters; requests so short that only some CTAs of a cluster
    work, or one, beside long ones; 1, 7 and 20 head rows on a kv head; a planted key in the first,
    a middle and the last range; one launch after the other on the same object (tickets and
    inboxes are left clean)."""
    from cloud_inference_from_scratch_b200.native import tensor_attention

    item = ops[torch.bfloat16]
    item.require_attention(128)
    fast = item._tensor_attention[128]
    rings, room = fast.split_choices(8)
    ctas, stages, cluster = plan
    if cluster > 1 and (cluster not in rings or stages not in rings[cluster]):
        pytest.skip(f"this device does not run clusters of {cluster} with a ring of {stages}")
    monkeypatch.setattr(tensor_attention, "FORCE_SPLIT_PLAN", plan)
    monkeypatch.setattr(tensor_attention, "FORCE_SPLIT_KEYS", min_keys)
    contexts = [4000, 0, 130, 700, 2047, 63, 1029]
    for seed, planted in enumerate([(0, 5, 4.0), (0, 2200, 4.0), (0, 3999, 4.0), (4, 1100, 4.0)]):
        tensor_case(ops, 128, contexts, [1] * len(contexts), 16, 2, 128, 16, seed=40 + seed, plant=planted)
    tensor_case(ops, 128, [3000, 77], [1, 1], 7, 7, 128, 16, seed=45, plant=(0, 1500, 4.0))      # one head row a unit
    tensor_case(ops, 128, [3000, 300], [1, 1], 14, 2, 128, 32, seed=46, plant=(0, 2999, 4.0))    # seven
    tensor_case(ops, 64, [2500, 9], [1, 1], 20, 1, 64, 16, seed=47, plant=(0, 1250, 4.0))        # twenty: two units a kv head


def test_split_decode_plans_of_this_device(ops):
    """What the planner picks from the device's own answers can be launched: every cluster it names
    has a ring for it and runs at one time."""
    item = ops[torch.bfloat16]
    item.require_attention(128)
    fast = item._tensor_attention[128]
    rings, room = fast.split_choices(8)
    assert 1 in rings and all(cluster in rings and at_once >= 1 for cluster, at_once in room.items())
    for units in (1, 2, 3, 8, 14, 15, 16, 31, 32, 33, 64, 128, 147, 300, 1000):
        for keys in (16, 128, 500, 2048, 4096, 5120, 8192, 40000, 131072):
            ctas, stages, cluster, min_keys = fast.split_plan(units, keys, fast.sm_count, rings, room,
                                                              fast.split_cta_limit, fast.split_max, fast.split_tile)
            assert stages in rings[cluster] and ctas % cluster == 0 and 1 <= ctas <= fast.split_max
            assert cluster == 1 or units * (ctas // cluster) <= room[cluster]
            assert ctas == cluster or units * ctas // cluster <= fast.split_cta_limit


@pytest.mark.parametrize("min_tiles", [1, 2, 4])
def test_prompt_attention_with_key_ranges(ops, monkeypatch, min_tiles):
    """A prompt portion over a long context makes few query tiles: the keys of a tile are then cut
    into ranges, one CTA each, whose shares the CTA with the last ticket adds up.  A planted key in
    the first, a middle and the last range; a short request beside a long one (its tiles use one
    range of those launched); head size 64; seven heads on a kv head; single tokens beside the
    portion; and one launch after the other on the same object (the tickets are left at zero)."""
    from cloud_inference_from_scratch_b200.native import tensor_attention
    from cloud_inference_from_scratch_b200.native.tensor_attention import TensorAttention

    monkeypatch.setattr(tensor_attention, "MIN_KEY_TILES_PER_RANGE", min_tiles)
    assert TensorAttention.key_ranges(26, 2048, 148, 128) == min(4, 2048 // (128 * min_tiles))
    assert TensorAttention.key_ranges(80, 8192, 148, 128) == 1 and TensorAttention.key_ranges(8, 65536, 148, 128) == 4
    item = ops[torch.bfloat16]
    item.require_attention(128)
    assert item._tensor_attention[128]._prefill_tc is not None
    for seed, planted in enumerate([(0, 3, 4.0), (0, 900, 4.0), (0, 1699, 4.0)]):
        tensor_case(ops, 128, [1500], [200], 16, 2, 128, 16, seed=50 + seed, plant=planted)
    tensor_case(ops, 128, [1800, 0, 40], [150, 100, 30], 16, 2, 128, 16, seed=54, plant=(0, 1000, 4.0))
    tensor_case(ops, 128, [3000, 700, 16, 1200], [1, 1, 1, 64], 14, 2, 128, 32, seed=55, plant=(3, 600, 4.0))
    tensor_case(ops, 64, [2500], [90], 4, 1, 64, 16, seed=56, plant=(0, 1250, 4.0))
    tensor_case(ops, 128, [4000], [17], 16, 2, 128, 16, seed=57, plant=(0, 2047, 4.0))
    tensor_case(ops, 128, [9000, 500], [40, 300], 16, 2, 128, 16, seed=58, plant=(0, 8999, 4.0))
    assert int(item._tensor_attention[128]._prefill_tickets.abs().sum()) == 0


def test_tensor_attention_long_prompt_whole(ops):
    tensor_case(ops, 128, [0], [1500], 16, 2, 128, 16, seed=9)
    tensor_case(ops, 64, [300, 0], [700, 64], 14, 2, 64, 16, seed=10)


# ------------------------------------------------------------------ weight-streaming tcgen05 product (17 to 256 rows)
@pytest.mark.parametrize("m,n,k,mode,plan", [
    (64, 256, 256, 1, (32, 1, 2)), (17, 200, 136, 1, (48, 1, 2)), (100, 1000, 1000, 0, (112, 4, 3)),
    (33, 331, 96, 0, (16, 1, 2)), (128, 2560, 2048, 0, (176, 8, 4)), (64, 2048, 1408, 3, (64, 2, 6)),
    (200, 1000, 520, 1, (160, 2, 4)), (256, 704, 2048, 3, (160, 1, 4)), (130, 1000, 520, 1, (256, 1, 2)),
    (64, 2048, 11008, 0, None), (48, 22016, 2048, 3, None), (129, 2560, 2048, 0, None), (256, 3000, 136, 1, None),
])
def test_gemm_skinny(ops, monkeypatch, m, n, k, mode, plan):
    """The tcgen05 product whose CTAs take a chosen number of weight rows each and, in clusters, a K
    range each: one and two token tiles, rows and K that are no multiple of anything but 8, the last
    CTA ragged, bias, float32 and bfloat16 rows and the SiLU epilogue, with 1, 2, 4 and 8 K ranges;
    and the plans the planner picks for this device."""
    from cloud_inference_from_scratch_b200.native import skinny

    item = ops[torch.bfloat16]
    gemm = item._skinny_gemm()
    x = rand(m, k, dtype=torch.bfloat16, scale=0.5, seed=m)
    w = rand(n, k, dtype=torch.bfloat16, scale=0.05, seed=n)
    bias = rand(n, seed=k) if mode != 3 else None
    want = plain_model.linear(x.float().cpu(), w.float().cpu(), None if bias is None else bias.cpu())
    if mode == 3:
        blocks = want.view(m, n // 32, 2, 16)
        want = (torch.nn.functional.silu(blocks[:, :, 0]) * blocks[:, :, 1]).reshape(m, n // 2)
    out = torch.full(tuple(want.shape), 7.0, dtype=torch.float32 if mode == 1 else torch.bfloat16).cuda()
    monkeypatch.setattr(skinny, "FORCE_PLAN", plan)
    assert gemm.supports(x, w, m, n, k, mode == 3)
    before = item.launches
    gemm.launch(x, w, bias, out, mode)
    torch.cuda.synchronize()
    item.check_errors()
    assert item.launches == before + 1
    scale = float(want.abs().max())
    if mode == 1:
        torch.testing.assert_close(out.cpu(), want, rtol=2e-3, atol=2e-3 * max(1.0, scale))
    else:
        torch.testing.assert_close(out.float().cpu(), want, rtol=2e-2, atol=2e-2 * max(1.0, scale / 4))


def test_gemm_skinny_refuses_what_it_cannot_run(ops):
    from cloud_inference_from_scratch_b200.native import skinny
    from cloud_inference_from_scratch_b200.native.ops import KernelError

    item = ops[torch.bfloat16]
    gemm = item._skinny_gemm()
    x = rand(64, 256, dtype=torch.bfloat16)
    w = rand(256, 256, dtype=torch.bfloat16)
    out = torch.empty(64, 256, dtype=torch.bfloat16).cuda()
    for plan in [(24, 1, 2), (272, 1, 2), (32, 3, 2), (32, 8, 2), (32, 1, 1), (256, 1, 12), (256, 4, 2)]:
        with pytest.raises(KernelError):
            gemm._gemm(x.data_ptr(), w.data_ptr(), None, out.data_ptr(), 64, 256, 256, 0, *plan,
                       item.error_word.data_ptr(), item.stream)
    assert not gemm.supports(x, w, 300, 256, 256, False) and not gemm.supports(x, w, 16, 256, 256, False)
    assert gemm._smem(64, 160, 6) == skinny.smem_bytes(64, 160, 6) and gemm._smem(200, 96, 3) == skinny.smem_bytes(200, 96, 3)


# ------------------------------------------------------------------ streaming matrix product (decode)
@pytest.mark.parametrize("m", [1, 2, 8, 9, 16])
@pytest.mark.parametrize("n,k", [(331, 96), (2560, 2048), (2048, 11008), (1000, 136)])
def test_gemm_stream_outputs(ops, m, n, k):
    item = ops[torch.bfloat16]
    x = rand(m, k, dtype=torch.bfloat16, seed=m)
    w = rand(n, k, dtype=torch.bfloat16, scale=0.05, seed=n)
    bias = rand(n, seed=k)
    want = plain_model.linear(x.float().cpu(), w.float().cpu(), bias.cpu()).cuda()
    scale = float(want.abs().max())
    out = torch.empty(m, n, dtype=torch.bfloat16).cuda()
    assert item.stream_plan(m, n, k, False) is not None
    assert item.linear(x, w, bias, out) is out
    torch.testing.assert_close(out.float(), want, rtol=2e-2, atol=2e-2 * max(1.0, scale / 4))
    logits = torch.empty(m, n, dtype=torch.float32).cuda()
    item.linear(x, w, bias, logits)
    torch.testing.assert_close(logits, want, rtol=2e-3, atol=2e-3 * max(1.0, scale))
    parts = item.linear(x, w, bias, out, allow_partials=True, tag=f"test{n}")
    if item.stream_plan(m, n, k, True)[1] > 1:
        from cloud_inference_from_scratch_b200.native.ops import Partials

        assert isinstance(parts, Partials) and parts.splits > 1
        total = torch.empty(m, n, dtype=torch.float32).cuda()
        item.resolve(parts, total)
        torch.testing.assert_close(total, want, rtol=2e-3, atol=2e-3 * max(1.0, scale))
        # the consumers add the parts up themselves
        residual = rand(m, n, seed=3)
        gain = 1 + rand(n, scale=0.1, seed=4)
        normed = torch.empty(m, n, dtype=torch.bfloat16).cuda()
        work = residual.clone()
        item.add_rmsnorm(work, parts, gain, 1e-6, normed)
        torch.testing.assert_close(work, residual + want, rtol=2e-3, atol=2e-3 * max(1.0, scale))
        expect = plain_model.rms_norm((residual + want).cpu(), gain.cpu(), 1e-6).cuda()
        torch.testing.assert_close(normed.float(), expect, rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("m", [1, 8, 16])
@pytest.mark.parametrize("inter", [208, 11008, 408])
def test_gate_up_fused_silu(ops, m, inter):
    item = ops[torch.bfloat16]
    hidden = 256
    gate = rand(inter, hidden, dtype=torch.bfloat16, scale=0.1, seed=1)
    up = rand(inter, hidden, dtype=torch.bfloat16, scale=0.1, seed=2)
    weight = item.prepare_gate_up(gate, up)
    assert weight.block == (16 if inter % 16 == 0 else inter)
    for rows in (m, 100):      # few rows: streaming kernel; many rows: product + SiLU kernel
        x = rand(rows, hidden, dtype=torch.bfloat16, seed=rows)
        out = torch.empty(rows, inter, dtype=torch.bfloat16).cuda()
        from cloud_inference_from_scratch_b200.engine.runtime import Workspace

        item.gate_up(x, weight, out, Workspace("cuda:0"))
        xf = x.float().cpu()
        want = torch.nn.functional.silu(xf @ gate.float().cpu().t()) * (xf @ up.float().cpu().t())
        torch.testing.assert_close(out.float().cpu(), want, rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("splits_case", ["partials", "tensor"])
def test_rope_from_partial_sums(ops, splits_case):
    item = ops[torch.bfloat16]
    q_heads, kv_heads, dim, page = 16, 2, 128, 16
    width = (q_heads + 2 * kv_heads) * dim
    tokens, hidden = 5, 2048
    x = rand(tokens, hidden, dtype=torch.bfloat16, seed=1)
    w = rand(width, hidden, dtype=torch.bfloat16, scale=0.03, seed=2)
    bias = rand(width, seed=3)
    qkv_buf = torch.empty(tokens, width, dtype=torch.bfloat16).cuda()
    qkv = item.linear(x, w, bias, qkv_buf, allow_partials=splits_case == "partials", tag="ropetest")
    positions = torch.tensor([0, 7, 15, 16, 300], dtype=torch.int32).cuda()
    request = torch.arange(tokens, dtype=torch.int32).cuda()
    k_pool, v_pool, table, _, total = paged_setup([1, 8, 16, 17, 301], page, kv_heads, dim, torch.bfloat16)
    inv_freq = (1.0 / (1e6 ** (torch.arange(0, dim, 2, dtype=torch.float32) / dim))).cuda()
    ctx = SimpleNamespace(positions=positions, request_of_token=request, block_tables=[table])
    kv = SimpleNamespace(group=0, k=k_pool, v=v_pool, num_pages=total, page_size=page)
    q_buffer = torch.zeros(tokens, q_heads * dim, dtype=torch.bfloat16).cuda()
    q = item.rope_kv_write(qkv, ctx, kv, SimpleNamespace(rotary_dim=dim, inv_freq=inv_freq),
                           q_heads, kv_heads, dim, q_buffer=q_buffer)
    full = plain_model.linear(x.float().cpu(), w.float().cpu(), bias.cpu()).view(tokens, -1, dim)
    cos, sin = plain_model.rope_tables(dim, positions.cpu().tolist(), 1e6)
    want_q = plain_model.apply_rope(full[:, :q_heads], cos, sin)
    want_k = plain_model.apply_rope(full[:, q_heads:q_heads + kv_heads], cos, sin)
    got_q = q.float().cpu()[:, :q_heads * dim].view(tokens, q_heads, dim)
    torch.testing.assert_close(got_q, want_q, rtol=2e-2, atol=2e-2)
    for t in range(tokens):
        pos = int(positions[t])
        page_id = int(table[t, pos // page])
        torch.testing.assert_close(k_pool[page_id, :, pos % page].float().cpu(), want_k[t], rtol=2e-2, atol=2e-2)
        torch.testing.assert_close(v_pool[page_id, :, pos % page].float().cpu(), full[t, q_heads + kv_heads:], rtol=2e-2, atol=2e-2)


# ------------------------------------------------------------------ tcgen05 matrix product
@pytest.fixture(scope="module")
def tensor_ops():
    from cloud_inference_from_scratch_b200.native import Ops

    item = Ops("cuda:0", torch.bfloat16, gemm="tensor")
    yield item
    item.check_errors()


@pytest.mark.parametrize("m,n,k", [
    (128, 128, 64), (128, 128, 128), (256, 384, 512), (2048, 2560, 2048), (200, 331, 96),
    (65, 1000, 136), (1000, 64, 2048), (130, 2048, 11008), (300, 777, 1024),
    (1, 128, 64), (8, 256, 512), (16, 2560, 2048), (17, 331, 96), (33, 1000, 136), (64, 2048, 11008),
    (3, 151936, 256),
])
def test_gemm_tcgen05(tensor_ops, m, n, k):
    item = tensor_ops
    x = rand(m, k, dtype=torch.bfloat16, seed=m)
    w = rand(n, k, dtype=torch.bfloat16, scale=0.05, seed=n)
    bias = rand(n, seed=k)
    want = plain_model.linear(x.float().cpu(), w.float().cpu(), bias.cpu()).cuda()
    scale = max(1.0, float(want.abs().max()))
    out = torch.full((m, n), float("nan"), dtype=torch.bfloat16).cuda()
    assert item._tensor_gemm.run(x, w, bias, out)
    item.check_errors()
    torch.testing.assert_close(out.float(), want, rtol=2e-2, atol=2e-2 * scale / 4)
    logits = torch.full((m, n), float("nan"), dtype=torch.float32).cuda()
    assert item._tensor_gemm.run(x, w, None, logits)
    item.check_errors()
    torch.testing.assert_close(logits, plain_model.linear(x.float().cpu(), w.float().cpu()).cuda(),
                               rtol=2e-3, atol=2e-3 * scale)


@pytest.mark.parametrize("m", [1, 8, 30, 64])
@pytest.mark.parametrize("n,k,splits", [(2560, 2048, 4), (2048, 11008, 8), (384, 192, 3)])
def test_gemm_tcgen05_partials(tensor_ops, m, n, k, splits):
    item = tensor_ops
    x = rand(m, k, dtype=torch.bfloat16, seed=m)
    w = rand(n, k, dtype=torch.bfloat16, scale=0.05, seed=n)
    parts = torch.full((splits, m, n), float("nan"), dtype=torch.float32).cuda()
    item._tensor_gemm.launch(x, w, None, parts, 2, splits)
    item.check_errors()
    want = plain_model.linear(x.float().cpu(), w.float().cpu()).cuda()
    torch.testing.assert_close(parts.sum(0), want, rtol=2e-3, atol=2e-3 * max(1.0, float(want.abs().max())))


@pytest.mark.parametrize("m", [1, 8, 40])
def test_gemm_tcgen05_silu_epilogue(tensor_ops, m):
    item = tensor_ops
    hidden, inter = 256, 11008
    gate = rand(inter, hidden, dtype=torch.bfloat16, scale=0.1, seed=1)
    up = rand(inter, hidden, dtype=torch.bfloat16, scale=0.1, seed=2)
    weight = item.prepare_gate_up(gate, up)
    assert weight.block == 16
    x = rand(m, hidden, dtype=torch.bfloat16, seed=m)
    out = torch.full((m, inter), float("nan"), dtype=torch.bfloat16).cuda()
    item._tensor_gemm.launch(x, weight.weight, None, out, 3, 1)
    item.check_errors()
    xf = x.float().cpu()
    want = torch.nn.functional.silu(xf @ gate.float().cpu().t()) * (xf @ up.float().cpu().t())
    torch.testing.assert_close(out.float().cpu(), want, rtol=2e-2, atol=2e-2)


# ------------------------------------------------------------------ prompt attention on tcgen05
@pytest.mark.parametrize("dim,page,q_heads,kv_heads", [
    (128, 16, 16, 2), (128, 48, 7, 1), (64, 16, 14, 2), (64, 128, 3, 3), (128, 64, 40, 8), (64, 32, 24, 2),
])
def test_prefill_attention_tcgen05(ops, dim, page, q_heads, kv_heads):
    """Prompt portions whose keys cross several 128-key tiles, with and without a cached prefix,
    beside short ones; lengths around the tile and page edges."""
    item = ops[torch.bfloat16]
    item.require_attention(dim)
    assert item._tensor_attention[dim]._prefill_tc is not None, "the tcgen05 prefill kernel was not loaded"
    tensor_case(ops, dim, [0, 127, 128, 300, 0], [129, 2, 256, 77, 1], q_heads, kv_heads, dim, page, seed=11)
    tensor_case(ops, dim, [1000, 0], [3, 640], q_heads, kv_heads, dim, page, seed=12)


def test_prefill_attention_tcgen05_far_key(ops):
    """The last query of a 300-token portion behind 1,700 cached keys is aligned with key 5, then
    with key 1,663 (the last key of a tile): the output must be that key's value."""
    tensor_case(ops, 128, [1700, 10], [300, 4], 16, 2, 128, 16, seed=13, plant=(0, 5, 4.0))
    tensor_case(ops, 128, [1700, 10], [300, 4], 16, 2, 128, 16, seed=14, plant=(0, 1663, 4.0))
    tensor_case(ops, 64, [0], [513], 4, 1, 64, 16, seed=15, plant=(0, 384, 4.0))


# ------------------------------------------------------------------ residual epilogue and normed input
@pytest.mark.parametrize("m", [1, 5, 8, 13, 16])
@pytest.mark.parametrize("n,k", [(2048, 2048), (2048, 11008), (331, 96), (1000, 520)])
def test_gemm_stream_adds_into_the_residual_and_feeds_the_next_product(ops, m, n, k):
    """A projection adds itself into the float32 residual stream (its K slices are one cluster) and
    leaves the sums of squares and the rows times the next norm's gain; the next product divides
    its result rows by the root mean square."""
    from cloud_inference_from_scratch_b200.engine.runtime import Workspace
    from cloud_inference_from_scratch_b200.native.ops import Accumulated, NormedInput, ResidualSink

    item = ops[torch.bfloat16]
    x = rand(m, k, dtype=torch.bfloat16, seed=m)
    w = rand(n, k, dtype=torch.bfloat16, scale=0.05, seed=n)
    bias = rand(n, seed=k)
    before = rand(m, n, seed=5)
    residual = before.clone()
    gain = 1 + rand(n, scale=0.1, seed=4)
    sink = ResidualSink(residual)
    sink.gain = gain
    out = torch.empty(m, n, dtype=torch.bfloat16).cuda()
    got = item.linear(x, w, bias, out, allow_partials=True, tag=f"residual{n}x{k}", residual=sink)
    assert isinstance(got, Accumulated) and got.residual is residual
    want = before + plain_model.linear(x.float().cpu(), w.float().cpu(), bias.cpu()).cuda()
    scale = float(want.abs().max())
    torch.testing.assert_close(residual, want, rtol=2e-3, atol=2e-3 * max(1.0, scale))
    squares = got.sq[: m * got.tiles].view(m, got.tiles).sum(-1)
    torch.testing.assert_close(squares, residual.pow(2).sum(-1), rtol=1e-4, atol=1e-4)
    if n % 8:
        assert got.scaled is None      # rows of the next product's input would not be 16-byte aligned
        return
    assert got.gain is gain
    torch.testing.assert_close(got.scaled.float(), (residual * gain).to(torch.bfloat16).float(), rtol=0, atol=0)

    # the same rows as the input of a product that finishes the RMSNorm itself
    eps = 1e-5
    lazy = NormedInput(got, eps, materialize=None)
    normed = plain_model.rms_norm(residual.cpu(), gain.cpu(), eps)
    w2 = rand(200, n, dtype=torch.bfloat16, scale=0.05, seed=7)
    logits = torch.empty(m, 200, dtype=torch.float32).cuda()
    assert item.linear(lazy, w2, None, logits) is logits
    want2 = normed @ w2.float().cpu().t()
    torch.testing.assert_close(logits.cpu(), want2, rtol=2e-2, atol=2e-2 * max(1.0, float(want2.abs().max()) / 4))
    inter = 208
    gate = rand(inter, n, dtype=torch.bfloat16, scale=0.05, seed=8)
    up = rand(inter, n, dtype=torch.bfloat16, scale=0.05, seed=9)
    hidden = torch.empty(m, inter, dtype=torch.bfloat16).cuda()
    item.gate_up(lazy, item.prepare_gate_up(gate, up), hidden, Workspace("cuda:0"))
    want3 = torch.nn.functional.silu(normed @ gate.float().cpu().t()) * (normed @ up.float().cpu().t())
    torch.testing.assert_close(hidden.float().cpu(), want3, rtol=2e-2, atol=2e-2 * max(1.0, float(want3.abs().max()) / 4))
    # and as partial sums for a consumer that adds them up
    parts = item.linear(lazy, w2, None, torch.empty(m, 200, dtype=torch.bfloat16).cuda(), allow_partials=True, tag="lazy.parts")
    total = torch.empty(m, 200, dtype=torch.float32).cuda()
    torch.testing.assert_close(item.resolve(parts, total).float().cpu(), want2, rtol=2e-2,
                               atol=2e-2 * max(1.0, float(want2.abs().max()) / 4))


def test_a_projection_of_more_rows_leaves_the_sum_to_the_norm(ops):
    """Above the row limit of the residual epilogue the same call returns partial sums (or the
    product) and the residual is untouched."""
    from cloud_inference_from_scratch_b200.native.ops import Accumulated, FUSED_RESIDUAL_MAX_ROWS, ResidualSink

    item = ops[torch.bfloat16]
    m, n, k = FUSED_RESIDUAL_MAX_ROWS + 1, 2048, 2048
    x = rand(m, k, dtype=torch.bfloat16, seed=1)
    w = rand(n, k, dtype=torch.bfloat16, scale=0.05, seed=2)
    residual = rand(m, n, seed=3)
    before = residual.clone()
    out = torch.empty(m, n, dtype=torch.bfloat16).cuda()
    got = item.linear(x, w, None, out, allow_partials=True, tag="rows9", residual=ResidualSink(residual))
    assert not isinstance(got, Accumulated)
    torch.cuda.synchronize()
    assert torch.equal(residual, before)


# ------------------------------------------------------------------ rotary epilogue of the q/k/v product
def paired_projection(item, q_heads, kv_heads, dim, rot, hidden, seed):
    """A stacked q/k/v weight and bias, natural and in the paired layout."""
    width = (q_heads + 2 * kv_heads) * dim
    w = rand(width, hidden, dtype=torch.bfloat16, scale=0.03, seed=seed)
    bias = rand(width, seed=seed + 1)
    q_rows, k_rows = q_heads * dim, kv_heads * dim

    def pair(t):
        return torch.cat([item.pair_rotary_rows(t[:q_rows], q_heads, dim, rot),
                          item.pair_rotary_rows(t[q_rows:q_rows + k_rows], kv_heads, dim, rot),
                          t[q_rows + k_rows:]]).contiguous()

    return w, bias, pair(w), pair(bias)


def rotary_want(x, w, bias, positions, q_heads, kv_heads, dim, rot, theta):
    tokens = x.shape[0]
    full = plain_model.linear(x.float().cpu(), w.float().cpu(), bias.cpu()).view(tokens, -1, dim)
    cos, sin = plain_model.rope_tables(rot, positions.cpu().tolist(), theta)
    return (plain_model.apply_rope(full[:, :q_heads], cos, sin),
            plain_model.apply_rope(full[:, q_heads:q_heads + kv_heads], cos, sin),
            full[:, q_heads + kv_heads:])


@pytest.mark.parametrize("q_heads,kv_heads,dim,rot,page", [(16, 2, 128, 128, 16), (6, 3, 64, 32, 8), (4, 4, 96, 64, 32)])
@pytest.mark.parametrize("tokens", [1, 5, 8, 11, 16])
def test_qkv_projection_rotates_and_stores_in_its_own_kernel(ops, q_heads, kv_heads, dim, rot, page, tokens):
    """Decode tokens: q comes back rotated in the natural order, k and v land in the right slot of
    the right page, nothing else in the pools changes; with write_cache off the pools stay as
    they were.  The same paired weight through the separate rotary kernel gives the same."""
    item = ops[torch.bfloat16]
    hidden, theta = 1024, 1e6
    assert item.can_pair_rotary(dim, rot)
    w, bias, w_paired, bias_paired = paired_projection(item, q_heads, kv_heads, dim, rot, hidden, seed=tokens)
    x = rand(tokens, hidden, dtype=torch.bfloat16, seed=9)
    lengths = [1, 8, 16, 17, 301, 64, 33, 100, 2, 129, 48, 257, 31, 32, 5, 77][:tokens]
    positions = torch.tensor([n - 1 for n in lengths], dtype=torch.int32).cuda()
    request = torch.arange(tokens, dtype=torch.int32).cuda()
    k_pool, v_pool, table, _, total = paged_setup(lengths, page, kv_heads, dim, torch.bfloat16)
    before_k, before_v = k_pool.clone(), v_pool.clone()
    inv_freq = (1.0 / (theta ** (torch.arange(0, rot, 2, dtype=torch.float32) / rot))).cuda()
    position = SimpleNamespace(rotary_dim=rot, inv_freq=inv_freq)
    ctx = SimpleNamespace(positions=positions, request_of_token=request, block_tables=[table])
    kv = SimpleNamespace(group=0, k=k_pool, v=v_pool, num_pages=total, page_size=page)
    want_q, want_k, want_v = rotary_want(x, w, bias, positions, q_heads, kv_heads, dim, rot, theta)

    q_buffer = torch.zeros(tokens, q_heads * dim, dtype=torch.bfloat16).cuda()
    got = item.qkv_rope(x, w_paired, bias_paired, ctx, kv, position, q_heads, kv_heads, dim, True, q_buffer)
    assert got is q_buffer
    torch.cuda.synchronize()
    torch.testing.assert_close(q_buffer.float().cpu().view(tokens, q_heads, dim), want_q, rtol=2e-2, atol=2e-2)
    touched = torch.zeros_like(k_pool, dtype=torch.bool)
    for t in range(tokens):
        pos = int(positions[t])
        page_id = int(table[t, pos // page])
        torch.testing.assert_close(k_pool[page_id, :, pos % page].float().cpu(), want_k[t], rtol=2e-2, atol=2e-2)
        torch.testing.assert_close(v_pool[page_id, :, pos % page].float().cpu(), want_v[t], rtol=2e-2, atol=2e-2)
        touched[page_id, :, pos % page] = True
    assert torch.equal(k_pool[~touched], before_k[~touched])
    assert torch.equal(v_pool[~touched], before_v[~touched])

    # a layer that reads another layer's cache writes nothing
    k2, v2 = before_k.clone(), before_v.clone()
    kv2 = SimpleNamespace(group=0, k=k2, v=v2, num_pages=total, page_size=page)
    q2 = torch.zeros_like(q_buffer)
    item.qkv_rope(x, w_paired, bias_paired, ctx, kv2, position, q_heads, kv_heads, dim, False, q2)
    torch.cuda.synchronize()
    assert torch.equal(k2, before_k) and torch.equal(v2, before_v) and torch.equal(q2, q_buffer)

    # the separate kernel on the same paired layout (as prompt portions use it)
    k3, v3 = before_k.clone(), before_v.clone()
    kv3 = SimpleNamespace(group=0, k=k3, v=v3, num_pages=total, page_size=page)
    qkv = torch.empty(tokens, w.shape[0], dtype=torch.bfloat16).cuda()
    qkv = item.linear(x, w_paired, bias_paired, qkv, allow_partials=True, tag="pairedrope", defer_bias=True)
    q3 = item.rope_kv_write(qkv, ctx, kv3, position, q_heads, kv_heads, dim, q_buffer=torch.zeros_like(q_buffer),
                            paired=True)
    torch.cuda.synchronize()
    torch.testing.assert_close(q3.float().cpu().view(tokens, q_heads, dim), want_q, rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(k3.float(), k_pool.float(), rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(v3.float(), v_pool.float(), rtol=2e-2, atol=2e-2)


def test_paired_rotary_kernel_on_a_prompt_portion(ops):
    """Many tokens: the library product leaves q/k/v in the paired layout in the compute dtype with
    the bias still to add; the rotary kernel reads it and writes q in the natural order."""
    item = ops[torch.bfloat16]
    q_heads, kv_heads, dim, rot, page, hidden, theta = 14, 2, 64, 64, 16, 896, 1e6
    w, bias, w_paired, bias_paired = paired_projection(item, q_heads, kv_heads, dim, rot, hidden, seed=21)
    tokens = 150
    x = rand(tokens, hidden, dtype=torch.bfloat16, seed=22)
    positions = torch.arange(40, 40 + tokens, dtype=torch.int32).cuda()
    request = torch.zeros(tokens, dtype=torch.int32).cuda()
    k_pool, v_pool, table, _, total = paged_setup([40 + tokens], page, kv_heads, dim, torch.bfloat16)
    inv_freq = (1.0 / (theta ** (torch.arange(0, rot, 2, dtype=torch.float32) / rot))).cuda()
    position = SimpleNamespace(rotary_dim=rot, inv_freq=inv_freq)
    ctx = SimpleNamespace(positions=positions, request_of_token=request, block_tables=[table])
    kv = SimpleNamespace(group=0, k=k_pool, v=v_pool, num_pages=total, page_size=page)
    qkv = torch.empty(tokens, w.shape[0], dtype=torch.bfloat16).cuda()
    qkv = item.linear(x, w_paired, bias_paired, qkv, allow_partials=True, tag="pairedprompt", defer_bias=True)
    q = item.rope_kv_write(qkv, ctx, kv, position, q_heads, kv_heads, dim,
                           q_buffer=torch.zeros(tokens, q_heads * dim, dtype=torch.bfloat16).cuda(), paired=True)
    torch.cuda.synchronize()
    want_q, want_k, want_v = rotary_want(x, w, bias, positions, q_heads, kv_heads, dim, rot, theta)
    torch.testing.assert_close(q.float().cpu().view(tokens, q_heads, dim), want_q, rtol=2e-2, atol=2e-2)
    for t in (0, 7, 149):
        pos = int(positions[t])
        page_id = int(table[0, pos // page])
        torch.testing.assert_close(k_pool[page_id, :, pos % page].float().cpu(), want_k[t], rtol=2e-2, atol=2e-2)
        torch.testing.assert_close(v_pool[page_id, :, pos % page].float().cpu(), want_v[t], rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("dim,rot,page", [(128, 128, 16), (128, 64, 16), (48, 16, 4), (64, 32, 32)])
def test_rope_kv_write_many_tokens_in_place(ops, dim, rot, page):
    """More than 64 bfloat16 tokens take the 16-byte-wide kernel: q rotated in place (natural
    layout), the part of a head beyond the rotary dims untouched, k and v in their slots."""
    q_heads, kv_heads = 5, 2
    starts, lens = [3, 0], [90, 33]
    width = (q_heads + 2 * kv_heads) * dim
    tokens = sum(lens)
    qkv = rand(tokens, width, dtype=torch.bfloat16, seed=31)
    positions = torch.cat([torch.arange(s, s + n) for s, n in zip(starts, lens)]).int().cuda()
    request = torch.cat([torch.full((n,), i) for i, n in enumerate(lens)]).int().cuda()
    k_pool, v_pool, table, _, total = paged_setup([s + n for s, n in zip(starts, lens)], page, kv_heads, dim, torch.bfloat16)
    theta = 10000.0
    inv_freq = (1.0 / (theta ** (torch.arange(0, rot, 2, dtype=torch.float32) / rot))).cuda()
    ctx = SimpleNamespace(positions=positions, request_of_token=request, block_tables=[table])
    kv = SimpleNamespace(group=0, k=k_pool, v=v_pool, num_pages=total, page_size=page)
    original = qkv.clone()
    got = ops[torch.bfloat16].rope_kv_write(qkv, ctx, kv, SimpleNamespace(rotary_dim=rot, inv_freq=inv_freq),
                                            q_heads, kv_heads, dim)
    assert got is qkv
    torch.cuda.synchronize()
    src = original.float().cpu().view(tokens, q_heads + 2 * kv_heads, dim)
    cos, sin = plain_model.rope_tables(rot, positions.cpu().tolist(), theta)
    want_q = plain_model.apply_rope(src[:, :q_heads], cos, sin)
    want_k = plain_model.apply_rope(src[:, q_heads:q_heads + kv_heads], cos, sin)
    out = qkv.float().cpu().view(tokens, q_heads + 2 * kv_heads, dim)
    torch.testing.assert_close(out[:, :q_heads], want_q, **tol(torch.bfloat16))
    assert torch.equal(out[:, :q_heads, rot:], src[:, :q_heads, rot:])
    assert torch.equal(out[:, q_heads:], src[:, q_heads:])
    for t in range(tokens):
        r, pos = int(request[t]), int(positions[t])
        page_id = int(table[r, pos // page])
        torch.testing.assert_close(k_pool[page_id, :, pos % page].float().cpu(), want_k[t], **tol(torch.bfloat16))
        assert torch.equal(v_pool[page_id, :, pos % page].float().cpu(), src[t, q_heads + kv_heads:])


@pytest.mark.parametrize("m,n,k", [(2048, 2048, 2048), (300, 1000, 520), (129, 331 * 32, 96)])
def test_gemm_tcgen05_persistent_folds_norm_activation_and_residual(tensor_ops, m, n, k):
    """More than 64 rows: the residual epilogue leaves new residual rows, their sums of squares and
    the rows times a gain; the next product scales its result rows by rstd, with a plain output and
    with SiLU(gate) * up."""
    item = tensor_ops
    gemm = item._tensor_gemm
    x = rand(m, k, dtype=torch.bfloat16, seed=m)
    w = rand(n, k, dtype=torch.bfloat16, scale=0.05, seed=n)
    bias = rand(n, seed=3)
    before = rand(m, n, seed=5)
    residual = before.clone()
    gain = 1 + rand(n, scale=0.1, seed=4)
    tiles = -(-n // 32)
    sq = torch.full((m, tiles), float("nan"), dtype=torch.float32).cuda()
    scaled = torch.full((m, n), float("nan"), dtype=torch.bfloat16).cuda() if n % 8 == 0 else None
    gemm.launch_fused(x, w, bias, None, 4, residual=residual, sq=sq, scaled=scaled,
                      next_gain=gain if scaled is not None else None)
    item.check_errors()
    want = before + plain_model.linear(x.float().cpu(), w.float().cpu(), bias.cpu()).cuda()
    top = max(1.0, float(want.abs().max()))
    torch.testing.assert_close(residual, want, rtol=2e-3, atol=2e-3 * top)
    torch.testing.assert_close(sq.sum(-1), residual.pow(2).sum(-1), rtol=1e-4, atol=1e-4)
    if scaled is None:
        return
    torch.testing.assert_close(scaled.float(), (residual * gain).to(torch.bfloat16).float(), rtol=0, atol=0)
    eps = 1e-5
    normed = plain_model.rms_norm(residual.cpu(), gain.cpu(), eps)
    w2 = rand(416, n, dtype=torch.bfloat16, scale=0.05, seed=7)
    out = torch.full((m, 416), float("nan"), dtype=torch.float32).cuda()
    gemm.launch_fused(scaled, w2, None, out, 1, row_sq=sq, row_tiles=tiles, eps=eps)
    item.check_errors()
    want2 = normed @ w2.float().cpu().t()
    torch.testing.assert_close(out.cpu(), want2, rtol=2e-2, atol=2e-2 * max(1.0, float(want2.abs().max()) / 4))
    inter = 208
    gate = rand(inter, n, dtype=torch.bfloat16, scale=0.05, seed=8)
    up = rand(inter, n, dtype=torch.bfloat16, scale=0.05, seed=9)
    stacked = item.prepare_gate_up(gate, up)
    assert stacked.block == 16
    hidden = torch.full((m, inter), float("nan"), dtype=torch.bfloat16).cuda()
    gemm.launch_fused(scaled, stacked.weight, None, hidden, 3, row_sq=sq, row_tiles=tiles, eps=eps)
    item.check_errors()
    want3 = torch.nn.functional.silu(normed @ gate.float().cpu().t()) * (normed @ up.float().cpu().t())
    torch.testing.assert_close(hidden.float().cpu(), want3, rtol=2e-2, atol=2e-2 * max(1.0, float(want3.abs().max()) / 4))


@pytest.mark.parametrize("pages", ["consecutive", "runs"])
@pytest.mark.parametrize("dim,page,q_heads,kv_heads", [(128, 16, 16, 2), (64, 16, 14, 2), (128, 64, 8, 8), (64, 256, 4, 1), (128, 32, 7, 1)])
def test_prefill_attention_tcgen05_with_pages_in_a_row(ops, dim, page, q_heads, kv_heads, pages):
    """Where the pages of a 128-key tile follow each other in the pool the kernel fetches the tile
    with one copy (also past the keys in use and past the pool's end); where they do not, page by
    page.  Both in one launch: some tiles of "runs" are in a row, some are not."""
    tensor_case(ops, dim, [0, 127, 128, 300, 0], [129, 2, 256, 77, 1], q_heads, kv_heads, dim, page, seed=21, pages=pages)
    tensor_case(ops, dim, [1000, 0], [3, 640], q_heads, kv_heads, dim, page, seed=22, pages=pages)
    tensor_case(ops, dim, [1700, 10], [300, 4], q_heads, kv_heads, dim, page, seed=23, plant=(0, 1663, 4.0), pages=pages)
