"""The persistent decode kernel (csrc/decode_program.cu) phase by phase and as a chain, against plain
float32 references: products with each epilogue, products cut along K with their finish phase, the
q/k/v product with rotation and cache write, attention over pages with its merge phase, and two
layers' worth of phases in one launch against the same work launched kernel by kernel."""

import math
from contextlib import contextmanager
from types import SimpleNamespace

import pytest
import torch

import plain_model
from test_gpu_kernels import attention_case, paged_setup, paired_projection, rand, rotary_want

pytestmark = pytest.mark.gpu
BF16 = torch.bfloat16


@pytest.fixture(scope="module")
def item():
    from cloud_inference_from_scratch_b200.native import Ops

    made = Ops("cuda:0", BF16)
    yield made
    made.check_errors()


@contextmanager
def recorded(item):
    """What ``Ops`` would launch inside is written down and runs as one program at the end."""
    from cloud_inference_from_scratch_b200.native.program import DecodeProgram

    if item.program is None:
        item.program = DecodeProgram(item)
    before = item.program.programs_run
    item.program.begin()
    yield item.program
    item.program.end()
    torch.cuda.synchronize()
    item.check_errors()
    assert item.program.programs_run > before, "nothing was recorded"


def test_splits_of_a_product():
    from cloud_inference_from_scratch_b200.native.program import product_splits

    assert product_splits(80, 8, 148) == 1        # q/k/v of the 3B shape: finished where it is streamed
    assert product_splits(64, 8, 148) == 1
    assert product_splits(688, 8, 148) == 1
    assert product_splits(64, 43, 148) == 9       # the down projection: K cut, a finish phase
    assert product_splits(4748, 8, 148) == 1
    assert product_splits(3, 2, 148) == 1


@pytest.mark.parametrize("m", [1, 2, 8, 9, 16])
@pytest.mark.parametrize("n,k", [(331, 96), (2560, 2048), (2048, 11008), (1000, 136), (64, 4096)])
def test_products_with_plain_outputs(item, m, n, k):
    x = rand(m, k, dtype=BF16, seed=m)
    w = rand(n, k, dtype=BF16, scale=0.05, seed=n)
    bias = rand(n, seed=k)
    want = plain_model.linear(x.float().cpu(), w.float().cpu(), bias.cpu()).cuda()
    scale = float(want.abs().max())
    out = torch.empty(m, n, dtype=BF16).cuda()
    logits = torch.empty(m, n, dtype=torch.float32).cuda()
    with recorded(item) as program:
        assert item.linear(x, w, bias, out) is out
        assert item.linear(x, w, None, logits) is logits
        assert len(program.calls) == 2
    torch.testing.assert_close(out.float(), want, rtol=2e-2, atol=2e-2 * max(1.0, scale / 4))
    torch.testing.assert_close(logits, want - bias, rtol=2e-3, atol=2e-3 * max(1.0, scale))


@pytest.mark.parametrize("m", [1, 8, 16])
@pytest.mark.parametrize("inter", [208, 11008, 416])
def test_gate_up_with_silu(item, m, inter):
    from cloud_inference_from_scratch_b200.engine.runtime import Workspace

    hidden = 256
    gate = rand(inter, hidden, dtype=BF16, scale=0.1, seed=1)
    up = rand(inter, hidden, dtype=BF16, scale=0.1, seed=2)
    weight = item.prepare_gate_up(gate, up)
    x = rand(m, hidden, dtype=BF16, seed=m)
    out = torch.empty(m, inter, dtype=BF16).cuda()
    with recorded(item):
        item.gate_up(x, weight, out, Workspace("cuda:0"))
    xf = x.float().cpu()
    want = torch.nn.functional.silu(xf @ gate.float().cpu().t()) * (xf @ up.float().cpu().t())
    torch.testing.assert_close(out.float().cpu(), want, rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("m", [1, 5, 8, 13, 16])
@pytest.mark.parametrize("n,k", [(2048, 2048), (2048, 11008), (331, 96), (1000, 520)])
def test_residual_epilogue_feeds_the_next_product(item, m, n, k):
    """A projection adds itself into the residual stream (directly, or through the finish phase when
    K was cut), leaves sums of squares and rows times the next gain; the products that follow IN THE
    SAME PROGRAM divide by the root mean square they form from those sums."""
    from cloud_inference_from_scratch_b200.engine.runtime import Workspace
    from cloud_inference_from_scratch_b200.native.ops import Accumulated, NormedInput, ResidualSink

    x = rand(m, k, dtype=BF16, seed=m)
    w = rand(n, k, dtype=BF16, scale=0.05, seed=n)
    bias = rand(n, seed=k)
    before = rand(m, n, seed=5)
    residual = before.clone()
    gain = 1 + rand(n, scale=0.1, seed=4)
    sink = ResidualSink(residual)
    sink.gain = gain
    eps = 1e-5
    w2 = rand(200, n, dtype=BF16, scale=0.05, seed=7)
    logits = torch.empty(m, 200, dtype=torch.float32).cuda()
    inter = 208
    gate = rand(inter, n, dtype=BF16, scale=0.05, seed=8)
    up = rand(inter, n, dtype=BF16, scale=0.05, seed=9)
    hidden = torch.empty(m, inter, dtype=BF16).cuda()
    gate_up = item.prepare_gate_up(gate, up)
    with recorded(item) as program:
        got = item.linear(x, w, bias, torch.empty(m, n, dtype=BF16).cuda(), allow_partials=True,
                          tag=f"program{n}x{k}", residual=sink)
        assert isinstance(got, Accumulated) and got.residual is residual
        if n % 8 == 0:
            lazy = NormedInput(got, eps, materialize=None)
            assert item.linear(lazy, w2, None, logits) is logits
            item.gate_up(lazy, gate_up, hidden, Workspace("cuda:0"))
            assert len(program.calls) == 3
    want = before + plain_model.linear(x.float().cpu(), w.float().cpu(), bias.cpu()).cuda()
    scale = float(want.abs().max())
    torch.testing.assert_close(residual, want, rtol=2e-3, atol=2e-3 * max(1.0, scale))
    squares = got.sq[: m * got.tiles].view(m, got.tiles).sum(-1)
    torch.testing.assert_close(squares, residual.pow(2).sum(-1), rtol=1e-4, atol=1e-4)
    if n % 8:
        assert got.scaled is None
        return
    torch.testing.assert_close(got.scaled.float(), (residual * gain).to(BF16).float(), rtol=0, atol=0)
    normed = plain_model.rms_norm(residual.cpu(), gain.cpu(), eps)
    want2 = normed @ w2.float().cpu().t()
    torch.testing.assert_close(logits.cpu(), want2, rtol=2e-2, atol=2e-2 * max(1.0, float(want2.abs().max()) / 4))
    want3 = torch.nn.functional.silu(normed @ gate.float().cpu().t()) * (normed @ up.float().cpu().t())
    torch.testing.assert_close(hidden.float().cpu(), want3, rtol=2e-2, atol=2e-2 * max(1.0, float(want3.abs().max()) / 4))


@pytest.mark.parametrize("q_heads,kv_heads,dim,rot,page", [(16, 2, 128, 128, 16), (6, 3, 64, 32, 8), (4, 4, 96, 64, 32)])
@pytest.mark.parametrize("tokens", [1, 5, 8, 11, 16])
def test_qkv_phase_rotates_and_stores(item, q_heads, kv_heads, dim, rot, page, tokens):
    hidden, theta = 1024, 1e6
    w, bias, w_paired, bias_paired = paired_projection(item, q_heads, kv_heads, dim, rot, hidden, seed=tokens)
    x = rand(tokens, hidden, dtype=BF16, seed=9)
    lengths = [1, 8, 16, 17, 301, 64, 33, 100, 2, 129, 48, 257, 31, 32, 5, 77][:tokens]
    positions = torch.tensor([n - 1 for n in lengths], dtype=torch.int32).cuda()
    request = torch.arange(tokens, dtype=torch.int32).cuda()
    k_pool, v_pool, table, _, total = paged_setup(lengths, page, kv_heads, dim, BF16)
    before_k, before_v = k_pool.clone(), v_pool.clone()
    inv_freq = (1.0 / (theta ** (torch.arange(0, rot, 2, dtype=torch.float32) / rot))).cuda()
    position = SimpleNamespace(rotary_dim=rot, inv_freq=inv_freq)
    ctx = SimpleNamespace(positions=positions, request_of_token=request, block_tables=[table])
    kv = SimpleNamespace(group=0, k=k_pool, v=v_pool, num_pages=total, page_size=page)
    want_q, want_k, want_v = rotary_want(x, w, bias, positions, q_heads, kv_heads, dim, rot, theta)
    q_buffer = torch.zeros(tokens, q_heads * dim, dtype=BF16).cuda()
    with recorded(item):
        assert item.qkv_rope(x, w_paired, bias_paired, ctx, kv, position, q_heads, kv_heads, dim, True, q_buffer) is q_buffer
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
    k2, v2 = before_k.clone(), before_v.clone()
    kv2 = SimpleNamespace(group=0, k=k2, v=v2, num_pages=total, page_size=page)
    q2 = torch.zeros_like(q_buffer)
    with recorded(item):
        item.qkv_rope(x, w_paired, bias_paired, ctx, kv2, position, q_heads, kv_heads, dim, False, q2)
    assert torch.equal(k2, before_k) and torch.equal(v2, before_v) and torch.equal(q2, q_buffer)


class Recording:
    """``attention`` of an ``Ops`` as one recorded program (for ``attention_case``)."""

    def __init__(self, item):
        self.item = item

    def require_attention(self, head_dim):
        self.item.require_attention(head_dim)

    def attention(self, *args):
        with recorded(self.item) as program:
            self.item.attention(*args)
            assert len(program.calls) == 1, "the attention was launched, not recorded"

    def check_errors(self):
        self.item.check_errors()


def program_attention(item, dim, contexts, q_heads, kv_heads, page, **kwargs):
    wrapped = Recording(item)
    wrapped.require_attention(dim)
    return attention_case({BF16: wrapped}, BF16, contexts, [1] * len(contexts), q_heads, kv_heads, dim, page,
                          fn="attention", **kwargs)


def test_attention_phase_and_merge(item):
    """Requests of very different lengths; one CTA per request and many; a window whose first key
    lies inside a page; more than 16 heads on a kv head; planted keys in the first, a middle and the
    last CTA's range; head size 64; pages of 64 tokens; and the same object again and again."""
    contexts = [(i * 379) % 4001 for i in range(16)]
    contexts[5], contexts[9], contexts[12] = 0, 15, 16
    program_attention(item, 128, contexts, 16, 2, 16, seed=20, plant=(15, contexts[15] // 2, 4.0))
    program_attention(item, 128, contexts[:7], 16, 2, 16, seed=21)
    program_attention(item, 128, [2047] * 8, 16, 2, 16, seed=22, plant=(3, 1, 4.0))
    program_attention(item, 128, [2047] * 8, 16, 2, 16, seed=23, plant=(7, 2046, 4.0))
    program_attention(item, 128, [2047] * 8, 16, 2, 16, seed=32, plant=(5, 1000, 4.0))
    program_attention(item, 128, [30000], 16, 2, 16, seed=24, plant=(0, 17000, 4.0))
    program_attention(item, 128, [30000], 16, 2, 16, seed=33, plant=(0, 29999, 4.0))
    program_attention(item, 64, [7000, 100, 16, 40], 4, 1, 16, window=5000, seed=25, plant=(0, 2100, 4.0))
    program_attention(item, 64, [7000, 100, 16, 40], 4, 1, 16, window=5000, seed=26, plant=(0, 1900, 4.0))
    program_attention(item, 64, [700, 100, 16, 40], 4, 1, 32, window=33, seed=27)
    program_attention(item, 64, [900, 3], 20, 1, 16, seed=28, plant=(0, 450, 4.0))
    program_attention(item, 128, [900, 3, 64, 63], 8, 8, 64, seed=29, plant=(0, 899, 4.0))


def test_two_layers_in_one_launch(item):
    """q/k/v with rotation and cache write -> attention (reads the key just written) -> output
    projection into the stream -> gate/up -> down projection (cut along K), twice, as ONE launch;
    the same calls launched kernel by kernel give the same stream, up to the order of the sums."""
    from cloud_inference_from_scratch_b200.engine.runtime import Workspace
    from cloud_inference_from_scratch_b200.native.ops import NormedInput, ResidualSink

    q_heads, kv_heads, dim, page, hidden, inter, tokens = 16, 2, 128, 16, 2048, 11008, 8
    theta, eps = 1e6, 1e-6
    lengths = [2048, 1, 17, 300, 1999, 64, 1024, 33]
    weights = []
    for layer in range(2):
        _, _, w_qkv, b_qkv = paired_projection(item, q_heads, kv_heads, dim, dim, hidden, seed=40 + layer)
        weights.append(dict(
            qkv=w_qkv, bias=b_qkv,
            o=rand(hidden, q_heads * dim, dtype=BF16, scale=0.02, seed=50 + layer),
            gate_up=item.prepare_gate_up(rand(inter, hidden, dtype=BF16, scale=0.02, seed=60 + layer),
                                         rand(inter, hidden, dtype=BF16, scale=0.02, seed=70 + layer)),
            down=rand(hidden, inter, dtype=BF16, scale=0.02, seed=80 + layer),
            gain1=1 + rand(hidden, scale=0.1, seed=90 + layer), gain2=1 + rand(hidden, scale=0.1, seed=95 + layer)))
    inv_freq = (1.0 / (theta ** (torch.arange(0, dim, 2, dtype=torch.float32) / dim))).cuda()
    position = SimpleNamespace(rotary_dim=dim, inv_freq=inv_freq)
    positions = torch.tensor([n - 1 for n in lengths], dtype=torch.int32).cuda()
    request = torch.arange(tokens, dtype=torch.int32).cuda()
    start = rand(tokens, hidden, seed=1)
    item.require_attention(dim)

    def run(record):
        pools = [paged_setup(lengths, page, kv_heads, dim, BF16, seed=30 + layer) for layer in range(2)]
        table = pools[0][2]
        ctx = SimpleNamespace(positions=positions, request_of_token=request, block_tables=[table], extras={},
                              num_single=tokens, num_requests=tokens, num_tokens=tokens,
                              context_lens=(positions.clone()), host=None)
        residual = start.clone()
        workspace = Workspace("cuda:0")
        # the first norm as a kernel; everything after it may be recorded
        first = torch.empty(tokens, hidden, dtype=BF16).cuda()
        item.add_rmsnorm(residual, None, weights[0]["gain1"], eps, first)
        if record:
            item.program.begin()
        x = first
        for layer in range(2):
            w = weights[layer]
            k_pool, v_pool, _, _, total = pools[layer]
            kv = SimpleNamespace(group=0, k=k_pool, v=v_pool, num_pages=total, page_size=page)
            q = torch.zeros(tokens, q_heads * dim, dtype=BF16).cuda()
            assert item.qkv_rope(x, w["qkv"], w["bias"], ctx, kv, position, q_heads, kv_heads, dim, True, q) is q
            mixed = torch.zeros(tokens, q_heads * dim, dtype=BF16).cuda()
            item.attention(q, mixed, ctx, kv, q_heads, kv_heads, dim, 1.0 / math.sqrt(dim), 0)
            sink = ResidualSink(residual)
            sink.gain = w["gain2"]
            acc = item.linear(mixed, w["o"], None, torch.empty(tokens, hidden, dtype=BF16).cuda(),
                              allow_partials=True, tag="chain.o", residual=sink)
            act = torch.empty(tokens, inter, dtype=BF16).cuda()
            item.gate_up(NormedInput(acc, eps, materialize=None), w["gate_up"], act, workspace)
            sink.gain = weights[1]["gain1"] if layer == 0 else w["gain1"]
            acc = item.linear(act, w["down"], None, torch.empty(tokens, hidden, dtype=BF16).cuda(),
                              allow_partials=True, tag="chain.down", residual=sink)
            x = NormedInput(acc, eps, materialize=None)
        if record:
            assert len(item.program.calls) == 10
            before = item.program.programs_run
            item.program.end()
            assert item.program.programs_run == before + 1, "the chain was not one launch"
        torch.cuda.synchronize()
        item.check_errors()
        return residual, pools

    from cloud_inference_from_scratch_b200.native.program import DecodeProgram

    if item.program is None:
        item.program = DecodeProgram(item)
    separate, pools_a = run(False)
    together, pools_b = run(True)
    spread = float(separate.std())
    assert float((together - separate).abs().max()) < 0.02 * spread, (float((together - separate).abs().max()), spread)
    for (ka, va, *_), (kb, vb, *_) in zip(pools_a, pools_b):
        torch.testing.assert_close(kb.float(), ka.float(), rtol=2e-2, atol=2e-2)
        torch.testing.assert_close(vb.float(), va.float(), rtol=2e-2, atol=2e-2)
    again, _ = run(True)
    assert torch.equal(again, together), "the same program twice gives the same bits"


@pytest.mark.parametrize("name", ["B", "D"])
def test_generation_with_recorded_decode_steps(sharp_models, name, monkeypatch):
    """The whole path with the switch on: decode steps of the scheduler's runner (CUDA graphs, padded
    buckets, steps launched ahead and dropped, a request joining, a small pool) run as programs, and
    every sampled row's logits are the plain model's."""
    from helpers import check_trace_rows
    from test_gpu_runner import _drive

    monkeypatch.setenv("CIE_PROGRAM", "1")
    folder = sharp_models.get(name, "bfloat16")
    programs = []
    from cloud_inference_from_scratch_b200.native import program as program_module

    launched = program_module.DecodeProgram.flush

    def counting(self):
        before = self.programs_run
        launched(self)
        programs.append(self.programs_run - before)

    monkeypatch.setattr(program_module.DecodeProgram, "flush", counting)
    requests, trace, counters, most_pages = _drive(folder, name, "bfloat16", blocks=64)
    check_trace_rows(folder, requests, trace, "bfloat16", f"{name} runner")
    assert sum(programs) > 0, "no decode step was recorded"
    assert counters["replays"] > 0 and counters["adopted"] > 0
    requests, trace, counters, _ = _drive(folder, name, "bfloat16", blocks=most_pages - 2)
    check_trace_rows(folder, requests, trace, "bfloat16", f"{name} runner")
    assert counters["preempted"] >= 1
