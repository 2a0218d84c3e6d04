"""Configuration, registry, loader errors and the random-weights writer (no GPU)."""

import json

import pytest
import safetensors.torch
import torch

from tiny_configs import SEED, TINY

from cloud_inference_from_scratch_b200.config import (
    ConfigError,
    Qwen2Config,
    build_config,
    register_architecture,
    registered_architectures,
    resolve_config,
    resolve_model,
    with_overrides,
)
from cloud_inference_from_scratch_b200.models import DecoderModel
from cloud_inference_from_scratch_b200.weights import (
    RandomSource,
    SafetensorsSource,
    WeightsError,
    check_tensors,
    write_random_model,
)


def test_config_reads_every_size_from_keys():
    config = Qwen2Config.from_dict(TINY["B"])
    assert (config.hidden_size, config.num_hidden_layers) == (128, 3)
    assert (config.num_attention_heads, config.num_key_value_heads, config.head_dim) == (2, 1, 64)
    assert config.rope_theta == 1e6 and config.rms_norm_eps == 1e-5
    assert config.tie_word_embeddings is False and config.attention_bias is True
    explicit = Qwen2Config.from_dict(TINY["C"])
    assert explicit.head_dim == 32 and explicit.attention_bias is False


def test_config_defaults_follow_the_reference():
    raw = dict(TINY["A"])
    del raw["rope_theta"], raw["attention_bias"], raw["architectures"]
    config = Qwen2Config.from_dict(raw)
    assert config.rope_theta == 10000.0 and config.attention_bias is True
    assert resolve_config(raw)[0].name == "Qwen2ForCausalLM"  # found through model_type


@pytest.mark.parametrize(
    "change, word",
    [
        (dict(hidden_size=None), "hidden_size"),
        (dict(model_type="llama"), "model_type"),
        (dict(hidden_act="gelu"), "hidden_act"),
        (dict(rope_scaling={"type": "yarn"}), "rope_scaling"),
        (dict(num_key_value_heads=3), "num_key_value_heads"),
        (dict(hidden_size=66), "head_dim"),
        (dict(rms_norm_eps="x"), "rms_norm_eps"),
        (dict(use_sliding_window=True, sliding_window=8, max_window_layers=1), "window"),
        (dict(vocab_size=0), "vocab_size"),
    ],
)
def test_config_errors_name_the_key(change, word):
    raw = dict(TINY["A"])
    for key, value in change.items():
        if value is None:
            raw.pop(key)
        else:
            raw[key] = value
    with pytest.raises(ConfigError, match=word):
        Qwen2Config.from_dict(raw)


def test_registry_unknown_and_custom_architecture():
    with pytest.raises(ConfigError, match="NopeForCausalLM"):
        resolve_config(dict(TINY["A"], architectures=["NopeForCausalLM"]))
    assert "Qwen2ForCausalLM" in registered_architectures()
    with pytest.raises(ValueError):
        register_architecture("Qwen2ForCausalLM", "qwen2", Qwen2Config.from_dict, lambda c: None)


def test_engine_config_names_and_overrides():
    config = build_config("ragged", block_size=8, max_batched_tokens=16, prefill_chunk_size=8)
    assert config.max_active_sequences == 16 and config.max_queue_size == 64
    assert with_overrides(config, dtype="float32").dtype == "float32"
    with pytest.raises(ValueError, match="unknown config overrides"):
        build_config("ragged", nonsense=1)
    with pytest.raises(ValueError, match="dtype"):
        build_config("ragged", dtype="float16")
    with pytest.raises(ValueError, match="mode"):
        build_config("naive")


def test_name_table_matches_reference_names():
    _, _, spec = resolve_config(TINY["B"])
    table = DecoderModel(spec).tensor_table()
    assert table["model.layers.2.self_attn.k_proj.weight"].shape == (64, 128)
    assert table["model.layers.0.self_attn.q_proj.bias"].shape == (128,)
    assert table["model.layers.1.mlp.down_proj.weight"].shape == (128, 320)
    assert table["lm_head.weight"].shape == (1000, 128)
    assert table["model.norm.weight"].role == "vector"
    assert len(table) == 2 + 1 + 3 * 12
    _, _, tied = resolve_config(TINY["A"])
    assert "lm_head.weight" not in DecoderModel(tied).tensor_table()
    _, _, nobias = resolve_config(TINY["C"])
    assert not any(name.endswith(".bias") for name in DecoderModel(nobias).tensor_table())


def test_random_model_folder_is_reproducible_and_typed(tmp_path):
    first = write_random_model(tmp_path / "a", TINY["A"], SEED["A"])
    second = write_random_model(tmp_path / "b", TINY["A"], SEED["A"])
    other = write_random_model(tmp_path / "c", TINY["A"], SEED["A"] + 1)
    one = safetensors.torch.load_file(str(first / "model.safetensors"))
    two = safetensors.torch.load_file(str(second / "model.safetensors"))
    three = safetensors.torch.load_file(str(other / "model.safetensors"))
    assert set(one) == set(two)
    for name in one:
        assert one[name].dtype == torch.bfloat16
        assert torch.equal(one[name], two[name])
    assert not torch.equal(one["model.norm.weight"], three["model.norm.weight"])
    gain = one["model.layers.0.input_layernorm.weight"].float()
    assert abs(gain.mean() - 1.0) < 0.02 and 0.005 < gain.std() < 0.04
    weight = one["model.layers.0.mlp.up_proj.weight"].float()
    assert abs(weight.mean()) < 0.002 and 0.017 < weight.std() < 0.023
    arch, config, spec = resolve_model(first)
    assert arch.name == "Qwen2ForCausalLM" and config == Qwen2Config.from_dict(TINY["A"])
    stored = json.load(open(first / "config.json"))
    assert stored["num_key_value_heads"] == 2 and stored["architectures"] == ["Qwen2ForCausalLM"]
    wide = write_random_model(tmp_path / "d", TINY["A"], SEED["A"], vector_dtype="float32")
    four = safetensors.torch.load_file(str(wide / "model.safetensors"))
    assert four["model.norm.weight"].dtype == torch.float32
    assert four["model.embed_tokens.weight"].dtype == torch.bfloat16


def test_random_tensor_does_not_depend_on_the_table(tmp_path):
    _, _, spec_a = resolve_config(TINY["A"])
    table = DecoderModel(spec_a).tensor_table()
    full = RandomSource(table, 5)
    alone = RandomSource({"model.norm.weight": table["model.norm.weight"]}, 5)
    assert torch.equal(full.get("model.norm.weight"), alone.get("model.norm.weight"))


def _rewrite(folder, edit):
    path = folder / "model.safetensors"
    tensors = safetensors.torch.load_file(str(path))
    edit(tensors)
    safetensors.torch.save_file(tensors, str(path))


def test_loader_lists_missing_unexpected_and_wrong_shapes_in_one_error(tmp_path):
    folder = write_random_model(tmp_path / "m", TINY["B"], 1)
    _, _, spec = resolve_model(folder)
    table = DecoderModel(spec).tensor_table()
    check_tensors(SafetensorsSource(folder), table, spec.optional_tensors)

    def edit(tensors):
        del tensors["model.layers.1.mlp.up_proj.weight"]
        del tensors["model.norm.weight"]
        tensors["model.layers.0.extra.weight"] = torch.zeros(3)
        tensors["model.layers.2.self_attn.v_proj.bias"] = torch.zeros(65)

    _rewrite(folder, edit)
    with pytest.raises(WeightsError) as info:
        check_tensors(SafetensorsSource(folder), table, spec.optional_tensors)
    error = info.value
    assert error.missing == ("model.layers.1.mlp.up_proj.weight", "model.norm.weight")
    assert error.unexpected == ("model.layers.0.extra.weight",)
    assert len(error.wrong_shape) == 1 and "v_proj.bias" in error.wrong_shape[0]
    text = str(error)
    assert "missing" in text and "unexpected" in text and "expected [64], found [65]" in text


def test_loader_tied_head_may_be_stored_and_duplicates_are_refused(tmp_path):
    folder = write_random_model(tmp_path / "t", TINY["A"], 1)
    _rewrite(folder, lambda t: t.__setitem__("lm_head.weight", t["model.embed_tokens.weight"].clone()))
    _, _, spec = resolve_model(folder)
    check_tensors(SafetensorsSource(folder), DecoderModel(spec).tensor_table(), spec.optional_tensors)
    safetensors.torch.save_file({"model.norm.weight": torch.ones(64)}, str(folder / "extra.safetensors"))
    with pytest.raises(WeightsError, match="more than once"):
        SafetensorsSource(folder)
    with pytest.raises(FileNotFoundError):
        SafetensorsSource(tmp_path)


def test_layer_spec_is_a_block_kind_and_a_named_map_of_parts():
    from dataclasses import replace

    from cloud_inference_from_scratch_b200.config import LayerSpec, PartSpec

    norm = PartSpec("rmsnorm", dict(hidden_size=8, eps=1e-5))
    layer = LayerSpec(prefix="l.", block=PartSpec("prenorm_residual"), mixer=PartSpec("attention"),
                      feed_forward=PartSpec("swiglu"), mixer_norm=norm, feed_forward_norm=norm)
    assert layer.mixer.family == "mixer" and layer.mixer_norm.family == "norm" and layer.feed_forward.family == "feed_forward"
    assert set(layer.parts) == {"mixer", "feed_forward", "mixer_norm", "feed_forward_norm"}
    # other slots are data too; a slot whose name does not say what it is names its family
    sandwich = LayerSpec("l.", PartSpec("toy_sandwich"), parts=dict(layer.parts, mixer_post_norm=norm,
                         second=PartSpec("swiglu", family="feed_forward")))
    assert sandwich.mixer_post_norm.family == "norm" and sandwich.second.family == "feed_forward"
    with pytest.raises(ValueError, match="family"):
        LayerSpec("l.", PartSpec("x"), gadget=PartSpec("swiglu"))
    with pytest.raises(AttributeError):
        layer.nothing
    swapped = replace(layer, mixer=PartSpec("other"))
    assert swapped.mixer.kind == "other" and swapped.feed_forward == layer.feed_forward and swapped != layer


def test_rotary_pairing_is_a_row_order_and_scales_are_constants():
    from cloud_inference_from_scratch_b200.config import PartSpec
    from cloud_inference_from_scratch_b200.parts import build_part

    def rope(**extra):
        return build_part("position", PartSpec("rope_neox", dict(head_dim=8, rotary_dim=6, theta=1e4, max_positions=64, **extra)))

    assert rope().row_order() is None and rope().attention_factor == 1.0
    assert rope(pairing="interleaved").row_order() == [0, 2, 4, 1, 3, 5, 6, 7]
    with pytest.raises(ValueError):
        rope(pairing="sideways")
    with pytest.raises(ValueError):
        rope(position_scale=0.0)
