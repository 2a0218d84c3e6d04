"""The plain implementation against the reference project's own model code (goldens), and
its own parts against each other."""

from pathlib import Path

import numpy as np
import pytest
import torch

import plain_model
from tiny_configs import TINY

GOLDEN = Path(__file__).parent / "golden"


@pytest.mark.parametrize("name", ["A", "B", "D"])
def test_plain_forward_matches_reference_golden(tiny_models, name):
    golden = np.load(GOLDEN / f"{name}.npz")
    config, weights = plain_model.read_model_folder(tiny_models[name])
    logits = plain_model.forward(config, weights, golden["prompt"].tolist())
    assert logits.shape == golden["logits"].shape
    np.testing.assert_allclose(logits.numpy(), golden["logits"], rtol=1e-5, atol=2e-6)


def test_causality_and_prefix_property(tiny_models):
    config, weights = plain_model.read_model_folder(tiny_models["A"])
    tokens = [5, 17, 3, 200, 41, 9, 77, 300]
    whole = plain_model.forward(config, weights, tokens)
    prefix = plain_model.forward(config, weights, tokens[:5])
    torch.testing.assert_close(whole[:5], prefix, rtol=1e-5, atol=1e-6)


def test_window_equals_full_when_wide_and_differs_when_narrow(tiny_models):
    config, weights = plain_model.read_model_folder(tiny_models["B"])
    tokens = list(range(3, 23))
    full = plain_model.forward(config, weights, tokens)
    wide = plain_model.forward(config, weights, tokens, window=64)
    narrow = plain_model.forward(config, weights, tokens, window=4)
    torch.testing.assert_close(full, wide)
    torch.testing.assert_close(full[:4], narrow[:4])
    assert (full[10:] - narrow[10:]).abs().max() > 1e-4


def test_rope_is_a_rotation_and_partial_passes_through():
    x = torch.randn(6, 2, 32)
    cos, sin = plain_model.rope_tables(16, list(range(6)), 10000.0)
    y = plain_model.apply_rope(x, cos, sin)
    torch.testing.assert_close(y[..., 16:], x[..., 16:])
    torch.testing.assert_close(y.norm(dim=-1), x.norm(dim=-1), rtol=1e-5, atol=1e-5)
    torch.testing.assert_close(y[0], x[0])  # position 0 is the identity


def test_schedule_shares_layers_and_caches(tiny_models):
    config, weights = plain_model.read_model_folder(tiny_models["A"])
    tokens = [1, 2, 3, 4, 5, 6]
    base = plain_model.forward(config, weights, tokens)
    same = plain_model.forward(config, weights, tokens, schedule=[(0, None), (1, None)])
    torch.testing.assert_close(base, same)
    twice = plain_model.forward(config, weights, tokens, schedule=[(0, None), (1, None), (0, None)])
    shared = plain_model.forward(config, weights, tokens, schedule=[(0, None), (1, None), (1, 1)])
    assert (twice - base).abs().max() > 1e-4
    assert (shared - twice).abs().max() > 1e-4


def test_greedy_generate_stops_on_eos(tiny_models):
    config, weights = plain_model.read_model_folder(tiny_models["A"])
    out = plain_model.greedy_generate(config, weights, [3, 9, 27], 5)
    assert len(out) == 5
    again = plain_model.greedy_generate(config, weights, [3, 9, 27], 5, eos_token_id=out[1])
    assert again == out[: out.index(out[1]) + 1]


def test_all_tiny_configs_differ():
    for key in ("hidden_size", "num_hidden_layers", "num_attention_heads", "intermediate_size",
                "vocab_size"):
        values = [TINY[name][key] for name in ("A", "B", "C")]
        assert len(set(values)) == 3, key
