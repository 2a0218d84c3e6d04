"""Each part of a layer alone against the plain implementation, and the generality of the layer
machinery: a toy mixer with state of its own that is defined HERE, registered, built and stepped
without a change to the package; a layer that runs twice; a run that reads another run's cache;
windowed attention beside full attention (two cache groups with pools of their own)."""

import math
from dataclasses import dataclass
from types import SimpleNamespace

import numpy as np
import pytest
import torch

import plain_model
from helpers import random_tokens, record, relative_error, replay, sharpen, tolerance, trace_mixed, trace_portions, trace_whole
from tiny_configs import TINY

pytestmark = pytest.mark.gpu


def runtime(dtype):
    from cloud_inference_from_scratch_b200.engine.runtime import Runtime

    return Runtime("cuda:0", dtype)


def rand(*shape, scale=1.0, seed=0):
    generator = torch.Generator().manual_seed(seed)
    return torch.randn(*shape, generator=generator) * scale


def close(got, want, dtype):
    error = record("a part alone", dtype, relative_error(got.float().cpu().numpy(), want.float().cpu().numpy()))
    assert error <= tolerance(dtype, "a part alone"), error


# ------------------------------------------------------------------ parts alone
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_rmsnorm_part(dtype):
    from cloud_inference_from_scratch_b200.parts import build_part
    from cloud_inference_from_scratch_b200.config import PartSpec

    rt = runtime(dtype)
    norm = build_part("norm", PartSpec("rmsnorm", dict(hidden_size=200, eps=1e-5)))
    assert norm.tensor_specs()["weight"].shape == (200,) and norm.tensor_specs()["weight"].role == "vector"
    gain = 1 + rand(200, scale=0.1, seed=1)
    norm.bind({"weight": gain.cuda()}, rt)
    residual = rand(9, 200, seed=2).cuda()
    update = rand(9, 200, seed=3).to(rt.dtype).cuda()
    before = residual.clone()
    out = norm.forward(residual, update, None)
    want_residual = before + update.float()
    torch.testing.assert_close(residual, want_residual)
    close(out, plain_model.rms_norm(want_residual.cpu(), gain, 1e-5), dtype)
    rows = torch.tensor([8, 2], dtype=torch.int32).cuda()
    picked = norm.forward(residual, None, None, rows=rows)
    close(picked, plain_model.rms_norm(want_residual.cpu()[[8, 2]], gain, 1e-5), dtype)


def test_rotary_part_constants():
    from cloud_inference_from_scratch_b200.parts import build_part
    from cloud_inference_from_scratch_b200.config import PartSpec

    rope = build_part("position", PartSpec("rope_neox", dict(head_dim=64, rotary_dim=32, theta=5e5, max_positions=128)))
    rope.bind({}, runtime("float32"))
    want = 1.0 / (5e5 ** (torch.arange(0, 32, 2, dtype=torch.float32) / 32))
    torch.testing.assert_close(rope.inv_freq.cpu(), want)
    with pytest.raises(ValueError):
        build_part("position", PartSpec("rope_neox", dict(head_dim=64, rotary_dim=66, theta=1e4, max_positions=8)))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_swiglu_part(dtype):
    from cloud_inference_from_scratch_b200.parts import build_part
    from cloud_inference_from_scratch_b200.config import PartSpec

    rt = runtime(dtype)
    part = build_part("feed_forward", PartSpec("swiglu", dict(hidden_size=96, intermediate_size=208)))
    assert set(part.tensor_specs()) == {"gate_proj.weight", "up_proj.weight", "down_proj.weight"}
    gate, up, down = rand(208, 96, scale=0.1, seed=1), rand(208, 96, scale=0.1, seed=2), rand(96, 208, scale=0.1, seed=3)
    cast = lambda t: t.to(rt.dtype).cuda()  # noqa: E731
    part.bind({"gate_proj.weight": cast(gate), "up_proj.weight": cast(up), "down_proj.weight": cast(down)}, rt)
    for tokens in (3, 70):
        x = cast(rand(tokens, 96, seed=tokens))
        update = rt.ops.resolve(part.forward(x, None),
                                torch.empty(tokens, 96, dtype=torch.float32, device="cuda"))
        want = plain_model.swiglu(x.float().cpu(), cast(gate).float().cpu(), cast(up).float().cpu(),
                                  cast(down).float().cpu())
        close(update, want, dtype)


def one_layer_core(config, dtype, pages=64, page=16, seed=3, sharp=None, tmp=None):
    from cloud_inference_from_scratch_b200.engine.core import build_core
    from cloud_inference_from_scratch_b200.weights import write_random_model

    folder = write_random_model(tmp / "plain", config, seed)
    if sharp:
        folder = sharpen(folder, tmp / "sharp", score_std=sharp)
    core = build_core(folder, dtype=dtype, page_size=page, num_pages=pages, max_requests=4, max_model_len=pages * page)
    return core, folder


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_attention_mixer_and_block_alone(dtype, tmp_path):
    """One layer, its mixer and its block called directly with a hand-made residual stream."""
    config = dict(TINY["B"], num_hidden_layers=1)
    core, folder = one_layer_core(config, dtype, sharp=1.5, tmp=tmp_path)
    cfg, weights = plain_model.read_model_folder(folder)
    layer = core.model.layers[0]
    tokens = random_tokens(cfg["vocab_size"], 21, 5)
    core.step.admit("r")
    hidden = plain_model.embedding(weights["model.embed_tokens.weight"], tokens)
    ref_h, _ = plain_model.decoder_layer(hidden, weights, 0, cfg, list(range(21)))
    x_in = plain_model.rms_norm(hidden, weights["model.layers.0.input_layernorm.weight"], cfg["rms_norm_eps"])
    ref_update, _ = plain_model.attention_layer(x_in, weights, "model.layers.0.self_attn.", cfg, list(range(21)))
    rt = core.runtime
    got_update, got_h = [], []
    position = 0
    from cloud_inference_from_scratch_b200.engine.step import StepEntry

    for size in (13, 2, 6):
        entries = [StepEntry("r", tokens[position:position + size])]
        host, _, spans = core.step.prepare(entries)
        ctx = core.step.upload(host)
        binding = ctx.bindings[0]
        x = x_in[position:position + size].to(rt.dtype).cuda()
        update = rt.ops.resolve(layer.mixer.forward(x, ctx, binding),
                                torch.empty(size, cfg["hidden_size"], dtype=torch.float32, device="cuda"))
        got_update.append(update.float().cpu())
        residual = hidden[position:position + size].clone().cuda()
        pending = layer.block.forward(residual, None, ctx, binding)   # writes the same K/V again
        pending = rt.ops.resolve(pending, torch.empty(size, cfg["hidden_size"], dtype=torch.float32, device="cuda"))
        got_h.append((residual + pending.float()).cpu())
        core.cache.commit_lengths({"r": spans["r"][1]})
        position += size
    core.runtime.ops.check_errors()
    close(torch.cat(got_update), ref_update, dtype)
    close(torch.cat(got_h), ref_h, dtype)


# ------------------------------------------------------------------ a toy mixer with state
def register_toy():
    from cloud_inference_from_scratch_b200.config import LayerSpec, ModelSpec, PartSpec, ScheduleEntry, register_architecture
    from cloud_inference_from_scratch_b200.parts import Mixer, StateSpec, TensorSpec, register_part

    class RunningMean(Mixer):
        """update[t] = W * mean(x[0..t]) over the request's tokens so far; the state is the running
        sum of x and the token count (float32), one row per request slot.  Everything runs on the
        device from the device views of the step's metadata, and a row that only pads a captured
        batch (request_active == 0) adds nothing to the state: steps may be captured in CUDA graphs."""

        state_in_graphs = True

        def __init__(self, hidden_size):
            self.hidden_size = hidden_size

        def state_spec(self):
            return StateSpec((self.hidden_size + 1,), "float32")

        def tensor_specs(self):
            return {"mix.weight": TensorSpec((self.hidden_size, self.hidden_size))}

        def bind(self, tensors, runtime):
            self.runtime = runtime
            self.weight = tensors["mix.weight"]

        def forward(self, x, ctx, binding):
            rows = x.double()
            tokens = rows.shape[0]
            before = torch.cat([torch.zeros_like(rows[:1]), torch.cumsum(rows, 0)])   # before[i]: sum of rows < i
            start, end = ctx.query_start[:-1].long(), ctx.query_start[1:].long()
            request = ctx.request_of_token.long()
            slots = ctx.slots.long()
            prior = binding.state[slots].double()                                      # [requests, hidden + 1]
            sums = prior[request, :-1] + before[1:] - before[start][request]
            counts = prior[request, -1] + (torch.arange(tokens, device=x.device) - start[request] + 1)
            mean = (sums / counts[:, None]).to(x.dtype)
            out = mean @ self.weight.t()
            gained = torch.cat([before[end] - before[start], (end - start).double()[:, None]], 1)
            gained = gained * ctx.request_active.double()[:, None]
            binding.state.index_add_(0, slots, gained.float())
            return out

    register_part("mixer", "toy_running_mean", RunningMean, replace=True)

    @dataclass(frozen=True)
    class ToyConfig:
        hidden_size: int
        intermediate_size: int
        vocab_size: int
        eps: float
        heads: int

        @classmethod
        def from_dict(cls, raw):
            return cls(raw["hidden_size"], raw["intermediate_size"], raw["vocab_size"], raw["eps"], raw["heads"])

        def to_dict(self):
            return dict(architectures=["ToyForCausalLM"], model_type="toy", hidden_size=self.hidden_size,
                        intermediate_size=self.intermediate_size, vocab_size=self.vocab_size, eps=self.eps,
                        heads=self.heads)

    def toy_spec(config):
        norm = PartSpec("rmsnorm", dict(hidden_size=config.hidden_size, eps=config.eps))
        ffn = PartSpec("swiglu", dict(hidden_size=config.hidden_size, intermediate_size=config.intermediate_size), prefix="mlp.")
        head_dim = config.hidden_size // config.heads
        attention = PartSpec("attention", dict(
            hidden_size=config.hidden_size, num_heads=config.heads, num_kv_heads=1, head_dim=head_dim, qkv_bias=False,
            position=PartSpec("rope_neox", dict(head_dim=head_dim, rotary_dim=head_dim, theta=1e4, max_positions=512)),
        ), prefix="self_attn.")
        toy = PartSpec("toy_running_mean", dict(hidden_size=config.hidden_size), prefix="toy.")

        def layer(index, mixer):
            return LayerSpec(prefix=f"model.layers.{index}.", block=PartSpec("prenorm_residual"), mixer=mixer,
                             feed_forward=ffn, mixer_norm=PartSpec("rmsnorm", norm.params, prefix="input_layernorm."),
                             feed_forward_norm=PartSpec("rmsnorm", norm.params, prefix="post_attention_layernorm."))

        return ModelSpec(
            architecture="ToyForCausalLM", vocab_size=config.vocab_size, hidden_size=config.hidden_size,
            embedding_tensor="model.embed_tokens.weight", layers=(layer(0, toy), layer(1, attention)),
            schedule=(ScheduleEntry(0), ScheduleEntry(1)), final_norm=norm, final_norm_prefix="model.norm.",
            head_tensor="model.embed_tokens.weight", max_positions=512,
        )

    register_architecture("ToyForCausalLM", "toy", ToyConfig.from_dict, toy_spec, replace=True)
    return ToyConfig(hidden_size=64, intermediate_size=96, vocab_size=300, eps=1e-5, heads=2)


def toy_plain_forward(folder, tokens):
    """The toy model, plainly: layer 0 mixes with the running mean, layer 1 with attention."""
    _, weights = plain_model.read_model_folder(folder)
    eps = 1e-5
    h = plain_model.embedding(weights["model.embed_tokens.weight"], tokens)
    x = plain_model.rms_norm(h, weights["model.layers.0.input_layernorm.weight"], eps)
    mean = torch.cumsum(x, 0) / torch.arange(1, len(tokens) + 1)[:, None]
    h = h + mean @ weights["model.layers.0.toy.mix.weight"].t()
    x = plain_model.rms_norm(h, weights["model.layers.0.post_attention_layernorm.weight"], eps)
    h = h + plain_model.swiglu(x, weights["model.layers.0.mlp.gate_proj.weight"],
                               weights["model.layers.0.mlp.up_proj.weight"], weights["model.layers.0.mlp.down_proj.weight"])
    config = dict(num_attention_heads=2, num_key_value_heads=1, hidden_size=64, rope_theta=1e4)
    x = plain_model.rms_norm(h, weights["model.layers.1.input_layernorm.weight"], eps)
    update, _ = plain_model.attention_layer(x, weights, "model.layers.1.self_attn.", config, list(range(len(tokens))))
    h = h + update
    x = plain_model.rms_norm(h, weights["model.layers.1.post_attention_layernorm.weight"], eps)
    h = h + plain_model.swiglu(x, weights["model.layers.1.mlp.gate_proj.weight"],
                               weights["model.layers.1.mlp.up_proj.weight"], weights["model.layers.1.mlp.down_proj.weight"])
    h = plain_model.rms_norm(h, weights["model.norm.weight"], eps)
    return h @ weights["model.embed_tokens.weight"].t()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_mixer_with_state_is_registered_built_and_stepped(dtype, tmp_path):
    from cloud_inference_from_scratch_b200.engine.core import build_core
    from cloud_inference_from_scratch_b200.weights import write_random_model

    config = register_toy()
    folder = write_random_model(tmp_path / "toy", config.to_dict(), 9)
    core = build_core(folder, dtype=dtype, page_size=8, num_pages=40, max_requests=4, max_model_len=128)
    assert core.architecture == "ToyForCausalLM"
    needs = core.model.cache_needs()
    assert needs[0].state is not None and needs[0].pages is None      # the toy mixer: state, no pages
    assert needs[1].pages is not None and needs[1].state is None      # attention: pages, no state
    assert list(core.pools.states) == [0]
    requests = {f"t{i}": random_tokens(300, n, 70 + i) for i, n in enumerate((37, 5, 64, 18, 29))}
    for steps in (trace_whole(requests), trace_portions(requests), trace_mixed(requests, seed=4)):
        got = replay(core, steps)      # slots are reused: state must have been zeroed on admission
        for rid, tokens in requests.items():
            ref = toy_plain_forward(folder, tokens).numpy()
            mine = np.stack([got[rid][p] for p in range(len(tokens))])
            assert record("toy models", dtype, relative_error(mine, ref)) <= tolerance(dtype, "toy models"), (rid, relative_error(mine, ref))
    # through the public entry point.  The mixer has declared that padded rows leave its state alone
    # (state_in_graphs), so decode steps run from captured graphs: three requests make a batch of
    # four with one padded row, and they end at different steps.
    from cloud_inference_from_scratch_b200 import GenerationConfig, InferenceEngine, build_config

    prompts = [requests["t1"], requests["t3"], requests["t0"][:9]]
    config = build_config("ragged", dtype=dtype, block_size=8, kv_cache_blocks=40, prefill_chunk_size=7,
                          max_batched_tokens=16, max_model_len=128, max_active_sequences=4)
    with InferenceEngine(config, folder) as engine:
        assert engine.runner.use_graphs
        handles = [engine.submit(p, GenerationConfig(max_output_tokens=5 + 2 * i)) for i, p in enumerate(prompts)]
        results = [h.wait() for h in handles]
        # captured and padded, but never launched ahead of the host: a dropped step would have moved the state
        assert engine.runner.cuda_graph_replays > 0 and engine.runner.steps_launched_ahead == 0
    for prompt, result in zip(prompts, results):
        tokens = list(prompt)
        for produced in result.token_ids:
            logits = toy_plain_forward(folder, tokens)[-1]
            best = int(torch.argmax(logits))
            assert produced == best or float(logits[best] - logits[produced]) < (1e-4 if dtype == "float32" else 3e-2)
            tokens.append(produced)


# ------------------------------------------------------------------ run order and windows are data
def register_variant(name, schedule, windows):
    from cloud_inference_from_scratch_b200.config import Qwen2Config, ScheduleEntry, register_architecture
    from cloud_inference_from_scratch_b200.models.qwen2 import qwen2_spec
    from dataclasses import replace

    def build(config):
        spec = qwen2_spec(config)
        layers = []
        for index, layer in enumerate(spec.layers):
            params = dict(layer.mixer.params, window=windows[index])
            layers.append(replace(layer, mixer=replace(layer.mixer, params=params)))
        return replace(spec, architecture=name, layers=tuple(layers),
                       schedule=tuple(ScheduleEntry(layer, reads) for layer, reads in schedule))

    def parse(raw):
        return Qwen2Config.from_dict(dict(raw, architectures=[name]))

    register_architecture(name, "qwen2-variant", parse, build, replace=True)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_layer_run_twice_and_cache_read_by_a_later_run(dtype, tmp_path):
    from cloud_inference_from_scratch_b200.engine.core import build_core
    from cloud_inference_from_scratch_b200.weights import write_random_model

    schedule = [(0, None), (1, None), (0, None), (1, 1)]
    register_variant("Qwen2TwiceForCausalLM", schedule, windows=[0, 0])
    folder = write_random_model(tmp_path / "m", dict(TINY["A"], architectures=["Qwen2TwiceForCausalLM"]), 4)
    folder = sharpen(folder, tmp_path / "s", score_std=3.0 if dtype == "float32" else 1.5)
    core = build_core(folder, dtype=dtype, page_size=4, num_pages=80, max_requests=4, max_model_len=160)
    needs = core.model.cache_needs()
    assert [n.owner for n in needs] == [0, 1, 2, 1]
    assert core.pools.pools[0].shape[0] == 3                 # three runs own a cache, one only reads
    assert core.pools.bindings[3].owns_cache is False
    assert core.pools.bindings[3].kv.k.data_ptr() == core.pools.bindings[1].kv.k.data_ptr()
    cfg, weights = plain_model.read_model_folder(folder)
    requests = {f"q{i}": random_tokens(cfg["vocab_size"], n, 30 + i) for i, n in enumerate((23, 50, 9, 41))}
    for steps in (trace_whole(requests), trace_mixed(requests, seed=2)):
        got = replay(core, steps)
        for rid, tokens in requests.items():
            ref = plain_model.forward(cfg, weights, tokens, schedule=schedule).numpy()
            mine = np.stack([got[rid][p] for p in range(len(tokens))])
            assert record("toy models", dtype, relative_error(mine, ref)) <= tolerance(dtype, "toy models"), (rid, relative_error(mine, ref))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "D"])
def test_windowed_and_full_attention_in_one_model(dtype, name, tmp_path):
    """Layer 0 sees the last 11 keys, layer 1 all of them: two cache groups, each with pages of its
    own; the windowed group's pool is so small that pages are given back as the window passes."""
    from cloud_inference_from_scratch_b200.engine.core import build_core
    from cloud_inference_from_scratch_b200.cache import CacheManager
    from cloud_inference_from_scratch_b200.cache.pools import CachePools, plan_groups
    from cloud_inference_from_scratch_b200.engine.step import StepFunction
    from cloud_inference_from_scratch_b200.weights import write_random_model

    arch = f"Qwen2Window{name}ForCausalLM"
    register_variant(arch, [(0, None), (1, None)], windows=[11, 0])
    folder = write_random_model(tmp_path / "m", dict(TINY[name], architectures=[arch]), 8)
    folder = sharpen(folder, tmp_path / "s", score_std=3.0 if dtype == "float32" else 1.5)
    page = 4 if name == "A" else 16
    core = build_core(folder, dtype=dtype, page_size=page, num_pages=64, max_requests=4, max_model_len=64 * page)
    assert len(core.cache.groups) == 2 and sorted(g.spec.window for g in core.cache.groups) == [0, 11]
    # rebuild the cache side with a window pool that only fits what the window needs
    needs = core.model.cache_needs()
    groups, place = plan_groups(needs, 4 if dtype == "float32" else 2)
    window_group = [i for i, g in enumerate(groups) if g.window][0]
    per_group = [64, 64]
    per_group[window_group] = 4 * (-(-(11 + 13) // page) + 1)
    core.cache = CacheManager(groups, page, per_group, 4, 64 * page)
    core.pools = CachePools(needs, groups, place, per_group, page, 4, core.runtime.dtype, core.runtime.device)
    core.step = StepFunction(core.model, core.runtime, core.cache, core.pools)
    cfg, weights = plain_model.read_model_folder(folder)
    requests = {f"w{i}": random_tokens(cfg["vocab_size"], n, 50 + i) for i, n in enumerate((60, 33, 90, 17, 45))}
    steps = trace_mixed(requests, seed=6)   # portions of at most 21 tokens, then single tokens
    got = replay(core, steps)
    for rid, tokens in requests.items():
        ref = plain_model.forward(cfg, weights, tokens, window=[11, 0]).numpy()
        mine = np.stack([got[rid][p] for p in range(len(tokens))])
        assert record("toy models", dtype, relative_error(mine, ref)) <= tolerance(dtype, "toy models"), (rid, relative_error(mine, ref))
    assert core.cache.groups[window_group].allocator.allocations_total > per_group[window_group]
    assert core.cache.free_pages(0) == core.cache.total_pages(0)
    assert core.cache.free_pages(1) == core.cache.total_pages(1)


# ------------------------------------------------------------------ a routed feed-forward and another position encoding
def register_toy_routed():
    """A model whose first layer has a feed-forward with top-1 routing over two experts and an
    attention with linearly scaled rotary positions; both parts are defined here, not in the package."""
    from cloud_inference_from_scratch_b200.config import LayerSpec, ModelSpec, PartSpec, ScheduleEntry, register_architecture
    from cloud_inference_from_scratch_b200.parts import FeedForward, PositionEncoding, TensorSpec, register_part

    class TopOneExperts(FeedForward):
        """update = expert_e(x) with e = argmax(router(x)) in float32; every expert is a SwiGLU."""

        def __init__(self, hidden_size, intermediate_size, experts):
            self.hidden_size, self.intermediate_size, self.experts = hidden_size, intermediate_size, experts

        def tensor_specs(self):
            specs = {"router.weight": TensorSpec((self.experts, self.hidden_size))}
            for e in range(self.experts):
                specs[f"experts.{e}.gate_proj.weight"] = TensorSpec((self.intermediate_size, self.hidden_size))
                specs[f"experts.{e}.up_proj.weight"] = TensorSpec((self.intermediate_size, self.hidden_size))
                specs[f"experts.{e}.down_proj.weight"] = TensorSpec((self.hidden_size, self.intermediate_size))
            return specs

        def bind(self, tensors, runtime):
            self.runtime, self.tensors = runtime, tensors

        def forward(self, x, ctx):
            logits = x.float() @ self.tensors["router.weight"].float().t()      # router in float32
            choice = logits.argmax(-1)
            out = torch.zeros_like(x)
            for e in range(self.experts):
                rows = (choice == e).nonzero().flatten()
                if rows.numel() == 0:
                    continue
                xe = x[rows]
                gate = xe @ self.tensors[f"experts.{e}.gate_proj.weight"].t()
                up = xe @ self.tensors[f"experts.{e}.up_proj.weight"].t()
                hidden = (torch.nn.functional.silu(gate.float()) * up.float()).to(x.dtype)
                out[rows] = hidden @ self.tensors[f"experts.{e}.down_proj.weight"].t()
            return out

    class RopeLinear(PositionEncoding):
        """Rotate-half rotary with positions divided by ``factor``: the attention part and its
        kernels only read ``rotary_dim`` and ``inv_freq``."""

        def __init__(self, head_dim, theta, factor):
            self.head_dim, self.rotary_dim, self.theta, self.factor = head_dim, head_dim, theta, factor

        def bind(self, tensors, runtime):
            exponent = torch.arange(0, self.rotary_dim, 2, dtype=torch.float32) / self.rotary_dim
            self.inv_freq = (1.0 / (self.theta ** exponent) / self.factor).to(runtime.device).contiguous()

    register_part("feed_forward", "toy_top_one_experts", TopOneExperts, replace=True)
    register_part("position", "toy_rope_linear", RopeLinear, replace=True)

    @dataclass(frozen=True)
    class RoutedConfig:
        hidden_size: int
        intermediate_size: int
        vocab_size: int
        heads: int

        @classmethod
        def from_dict(cls, raw):
            return cls(raw["hidden_size"], raw["intermediate_size"], raw["vocab_size"], raw["heads"])

        def to_dict(self):
            return dict(architectures=["ToyRoutedForCausalLM"], model_type="toy_routed", hidden_size=self.hidden_size,
                        intermediate_size=self.intermediate_size, vocab_size=self.vocab_size, heads=self.heads)

    def spec(config):
        eps = 1e-5
        head_dim = config.hidden_size // config.heads
        norm = dict(hidden_size=config.hidden_size, eps=eps)

        def attention(position):
            return PartSpec("attention", dict(hidden_size=config.hidden_size, num_heads=config.heads, num_kv_heads=1,
                                              head_dim=head_dim, qkv_bias=False, position=position), prefix="self_attn.")

        def layer(index, mixer, feed_forward):
            return LayerSpec(prefix=f"model.layers.{index}.", block=PartSpec("prenorm_residual"), mixer=mixer,
                             feed_forward=feed_forward, mixer_norm=PartSpec("rmsnorm", norm, prefix="input_layernorm."),
                             feed_forward_norm=PartSpec("rmsnorm", norm, prefix="post_attention_layernorm."))

        scaled = PartSpec("toy_rope_linear", dict(head_dim=head_dim, theta=1e4, factor=4.0))
        plain_rope = PartSpec("rope_neox", dict(head_dim=head_dim, rotary_dim=head_dim, theta=1e4, max_positions=512))
        routed = PartSpec("toy_top_one_experts", dict(hidden_size=config.hidden_size,
                                                      intermediate_size=config.intermediate_size, experts=2), prefix="moe.")
        dense = PartSpec("swiglu", dict(hidden_size=config.hidden_size, intermediate_size=config.intermediate_size), prefix="mlp.")
        return ModelSpec(
            architecture="ToyRoutedForCausalLM", vocab_size=config.vocab_size, hidden_size=config.hidden_size,
            embedding_tensor="model.embed_tokens.weight",
            layers=(layer(0, attention(scaled), routed), layer(1, attention(plain_rope), dense)),
            schedule=(ScheduleEntry(0), ScheduleEntry(1)), final_norm=PartSpec("rmsnorm", norm),
            final_norm_prefix="model.norm.", head_tensor="model.embed_tokens.weight", max_positions=512,
        )

    register_architecture("ToyRoutedForCausalLM", "toy_routed", RoutedConfig.from_dict, spec, replace=True)
    return RoutedConfig(hidden_size=64, intermediate_size=80, vocab_size=257, heads=2)


def toy_routed_plain_forward(folder, tokens):
    _, w = plain_model.read_model_folder(folder)
    eps = 1e-5
    config = dict(num_attention_heads=2, num_key_value_heads=1, hidden_size=64, rope_theta=1e4)
    positions = list(range(len(tokens)))
    h = plain_model.embedding(w["model.embed_tokens.weight"], tokens)
    x = plain_model.rms_norm(h, w["model.layers.0.input_layernorm.weight"], eps)
    update, _ = plain_model.attention_layer(x, w, "model.layers.0.self_attn.", config, [p / 4.0 for p in positions])
    h = h + update
    x = plain_model.rms_norm(h, w["model.layers.0.post_attention_layernorm.weight"], eps)
    choice = (x @ w["model.layers.0.moe.router.weight"].t()).argmax(-1)
    routed = torch.zeros_like(x)
    for e in range(2):
        p = f"model.layers.0.moe.experts.{e}."
        full = plain_model.swiglu(x, w[p + "gate_proj.weight"], w[p + "up_proj.weight"], w[p + "down_proj.weight"])
        routed[choice == e] = full[choice == e]
    h = h + routed
    x = plain_model.rms_norm(h, w["model.layers.1.input_layernorm.weight"], eps)
    update, _ = plain_model.attention_layer(x, w, "model.layers.1.self_attn.", config, positions)
    h = h + update
    x = plain_model.rms_norm(h, w["model.layers.1.post_attention_layernorm.weight"], eps)
    h = h + plain_model.swiglu(x, w["model.layers.1.mlp.gate_proj.weight"], w["model.layers.1.mlp.up_proj.weight"],
                               w["model.layers.1.mlp.down_proj.weight"])
    return plain_model.rms_norm(h, w["model.norm.weight"], eps) @ w["model.embed_tokens.weight"].t(), choice


def test_toy_routed_feed_forward_and_another_position_encoding(tmp_path):
    """Registered, built from a folder and stepped through every cutting without a change to the
    package.  32-bit only: a router's argmax over near-equal logits would make a bfloat16 run and
    the plain model pick different experts, which says nothing about the engine."""
    from cloud_inference_from_scratch_b200.engine.core import build_core
    from cloud_inference_from_scratch_b200.weights import write_random_model

    config = register_toy_routed()
    folder = write_random_model(tmp_path / "routed", config.to_dict(), 5)
    core = build_core(folder, dtype="float32", page_size=8, num_pages=48, max_requests=4, max_model_len=128)
    assert core.architecture == "ToyRoutedForCausalLM"
    requests = {f"r{i}": random_tokens(257, n, 40 + i) for i, n in enumerate((33, 6, 50, 21))}
    used = set()
    for steps in (trace_whole(requests), trace_portions(requests), trace_mixed(requests, seed=2)):
        got = replay(core, steps)
        for rid, tokens in requests.items():
            ref, choice = toy_routed_plain_forward(folder, tokens)
            used.update(choice.tolist())
            mine = np.stack([got[rid][p] for p in range(len(tokens))])
            assert record("toy routed", "float32", relative_error(mine, ref.numpy())) <= tolerance("float32", "toy routed"), (rid, relative_error(mine, ref.numpy()))
    assert used == {0, 1}      # both experts took tokens


# ------------------------------------------------------------------ another block, another pairing, scaled ends
def register_toy_sandwich():
    """A fourth toy architecture, registered from here alone: rotary pairs side by side (interleaved),
    positions divided by a factor and a factor on the softmax scale, a partial rotary size; a block
    with a norm on the mixer's output (its parts are data of the layer: one slot more); embeddings
    times a constant; logits times a constant and softly capped."""
    from cloud_inference_from_scratch_b200.config import LayerSpec, ModelSpec, PartSpec, ScheduleEntry, register_architecture
    from cloud_inference_from_scratch_b200.parts import register_part
    from cloud_inference_from_scratch_b200.parts.base import Block

    class Sandwich(Block):
        """h += post_norm(mixer(norm(h))); h += feed_forward(norm(h))"""

        slots = ("mixer", "feed_forward", "mixer_norm", "mixer_post_norm", "feed_forward_norm")

        def forward(self, residual, pending, ctx, binding):
            rt = self.mixer.runtime
            x = self.mixer_norm.forward(residual, pending, ctx)
            # the mixer's output is not for the stream yet: no projection may add itself into it
            sink, ctx.residual_sink = ctx.residual_sink, None
            mixed = self.mixer.forward(x, ctx, binding)
            ctx.residual_sink = sink
            mixed = rt.ops.resolve(mixed, torch.empty(residual.shape, dtype=torch.float32, device=residual.device))
            tamed = self.mixer_post_norm.forward(mixed.float().clone(), None, ctx)
            x = self.feed_forward_norm.forward(residual, tamed, ctx)
            return self.feed_forward.forward(x, ctx)

    register_part("block", "toy_sandwich", Sandwich, replace=True)

    @dataclass(frozen=True)
    class SandwichConfig:
        hidden_size: int
        intermediate_size: int
        vocab_size: int
        heads: int

        @classmethod
        def from_dict(cls, raw):
            return cls(raw["hidden_size"], raw["intermediate_size"], raw["vocab_size"], raw["heads"])

        def to_dict(self):
            return dict(architectures=["ToySandwichForCausalLM"], model_type="toy_sandwich", hidden_size=self.hidden_size,
                        intermediate_size=self.intermediate_size, vocab_size=self.vocab_size, heads=self.heads)

    def spec(config):
        head_dim = config.hidden_size // config.heads
        norm = dict(hidden_size=config.hidden_size, eps=1e-5)
        position = PartSpec("rope_neox", dict(head_dim=head_dim, rotary_dim=head_dim // 2, theta=1e4, max_positions=512,
                                              pairing="interleaved", position_scale=2.0, attention_factor=1.3))
        attention = PartSpec("attention", dict(hidden_size=config.hidden_size, num_heads=config.heads, num_kv_heads=config.heads,
                                               head_dim=head_dim, qkv_bias=True, position=position), prefix="self_attn.")
        dense = PartSpec("swiglu", dict(hidden_size=config.hidden_size, intermediate_size=config.intermediate_size), prefix="mlp.")
        layers = tuple(
            LayerSpec(prefix=f"model.layers.{index}.", block=PartSpec("toy_sandwich"), parts=dict(
                mixer=attention, feed_forward=dense,
                mixer_norm=PartSpec("rmsnorm", norm, prefix="input_layernorm."),
                mixer_post_norm=PartSpec("rmsnorm", norm, prefix="post_mixer_layernorm."),
                feed_forward_norm=PartSpec("rmsnorm", norm, prefix="post_attention_layernorm.")))
            for index in range(2))
        return ModelSpec(
            architecture="ToySandwichForCausalLM", vocab_size=config.vocab_size, hidden_size=config.hidden_size,
            embedding_tensor="model.embed_tokens.weight", layers=layers, schedule=(ScheduleEntry(0), ScheduleEntry(1)),
            final_norm=PartSpec("rmsnorm", norm), final_norm_prefix="model.norm.", head_tensor="model.embed_tokens.weight",
            max_positions=512, embedding_scale=float(config.hidden_size) ** 0.5, logit_scale=0.5, logit_softcap=2.0,
        )

    register_architecture("ToySandwichForCausalLM", "toy_sandwich", SandwichConfig.from_dict, spec, replace=True)
    return SandwichConfig(hidden_size=128, intermediate_size=176, vocab_size=411, heads=2)


def toy_sandwich_plain_forward(folder, tokens):
    _, w = plain_model.read_model_folder(folder)
    eps, heads, hidden = 1e-5, 2, 128
    dim, rot = hidden // heads, hidden // heads // 2
    count = len(tokens)
    positions = torch.arange(count, dtype=torch.float32) / 2.0
    inv_freq = 1.0 / (1e4 ** (torch.arange(0, rot, 2, dtype=torch.float32) / rot))
    angles = positions[:, None] * inv_freq[None, :]
    cos, sin = torch.cos(angles)[:, None, :], torch.sin(angles)[:, None, :]

    def rotate_pairs(x):      # x: [T, heads, dim]; pairs (2j, 2j + 1) of the first `rot` elements
        even, odd = x[..., 0:rot:2], x[..., 1:rot:2]
        out = x.clone()
        out[..., 0:rot:2] = even * cos - odd * sin
        out[..., 1:rot:2] = odd * cos + even * sin
        return out

    h = plain_model.embedding(w["model.embed_tokens.weight"], tokens) * hidden ** 0.5
    for index in range(2):
        prefix = f"model.layers.{index}."
        x = plain_model.rms_norm(h, w[prefix + "input_layernorm.weight"], eps)
        q, k, v = (plain_model.linear(x, w[prefix + f"self_attn.{n}_proj.weight"], w[prefix + f"self_attn.{n}_proj.bias"])
                   .view(count, heads, dim) for n in "qkv")
        mixed = plain_model.attention(rotate_pairs(q), rotate_pairs(k), v, 1.3 / math.sqrt(dim))
        mixed = plain_model.linear(mixed.reshape(count, hidden), w[prefix + "self_attn.o_proj.weight"])
        h = h + plain_model.rms_norm(mixed, w[prefix + "post_mixer_layernorm.weight"], eps)
        x = plain_model.rms_norm(h, w[prefix + "post_attention_layernorm.weight"], eps)
        h = h + plain_model.swiglu(x, w[prefix + "mlp.gate_proj.weight"], w[prefix + "mlp.up_proj.weight"],
                                   w[prefix + "mlp.down_proj.weight"])
    logits = plain_model.rms_norm(h, w["model.norm.weight"], eps) @ w["model.embed_tokens.weight"].t()
    return 2.0 * torch.tanh(logits * 0.5 / 2.0)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_block_with_a_post_norm_interleaved_rotary_and_scaled_ends(dtype, tmp_path):
    from cloud_inference_from_scratch_b200.engine.core import build_core
    from cloud_inference_from_scratch_b200.weights import write_random_model

    config = register_toy_sandwich()
    folder = write_random_model(tmp_path / "plain", config.to_dict(), 6)
    folder = sharpen(folder, tmp_path / "sharp", score_std=3.0 if dtype == "float32" else 1.5)
    core = build_core(folder, dtype=dtype, page_size=16, num_pages=24, max_requests=4, max_model_len=256)
    assert core.architecture == "ToySandwichForCausalLM"
    assert set(core.model.layers[0].parts) == {"mixer", "feed_forward", "mixer_norm", "mixer_post_norm", "feed_forward_norm"}
    assert "model.layers.1.post_mixer_layernorm.weight" in core.model.tensor_table()
    requests = {f"s{i}": random_tokens(411, n, 60 + i) for i, n in enumerate((45, 7, 80, 22))}
    for steps in (trace_whole(requests), trace_portions(requests), trace_mixed(requests, seed=9)):
        got = replay(core, steps)
        for rid, tokens in requests.items():
            ref = toy_sandwich_plain_forward(folder, tokens).numpy()
            mine = np.stack([got[rid][p] for p in range(len(tokens))])
            assert record("toy sandwich", dtype, relative_error(mine, ref)) <= tolerance(dtype, "toy sandwich"), (rid, relative_error(mine, ref))
