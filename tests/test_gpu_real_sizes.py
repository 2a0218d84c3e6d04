"""Logits at the layer sizes the benchmark times (Qwen2.5-3B: hidden 2048, 16 q heads on 2 kv heads of
128, intermediate 11008, vocabulary 151936): two layers against the plain model on the CPU in all
four cuttings, and all 36 layers on the GPU, the bfloat16 generation path against the 32-bit path.
The reference checks its 3B model end to end (tests/remote_gpu_tests.py:99-119,
tests/remote_ragged_gpu_tests.py:73-108)."""

import numpy as np
import pytest

from helpers import (
    check_against_plain, peak_tokens, random_tokens, record, replay, requests_in, tolerance,
    trace_mixed, trace_portions, trace_tail, trace_whole,
)

pytestmark = pytest.mark.gpu

QWEN25_3B = dict(
    architectures=["Qwen2ForCausalLM"], model_type="qwen2", hidden_size=2048, num_hidden_layers=36,
    num_attention_heads=16, num_key_value_heads=2, intermediate_size=11008, vocab_size=151936,
    rope_theta=1000000.0, rms_norm_eps=1e-6, attention_bias=True, tie_word_embeddings=True,
    eos_token_id=151643, max_position_embeddings=32768, hidden_act="silu", use_sliding_window=False,
)


@pytest.fixture(scope="module")
def two_layer_folders(tmp_path_factory):
    """Two of the 36 layers at full width, written once per sharpness."""
    from cloud_inference_from_scratch_b200.engine.check import sharpening_scales
    from cloud_inference_from_scratch_b200.weights import write_random_model

    root = tmp_path_factory.mktemp("two_layers")
    config = dict(QWEN25_3B, num_hidden_layers=2)
    return {dtype: write_random_model(root / dtype, config, 5, scales=sharpening_scales(2048, score_std))
            for dtype, score_std in (("float32", 3.0), ("bfloat16", 1.5))}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_two_of_36_layers_match_the_plain_model_in_every_cutting(two_layer_folders, dtype):
    from cloud_inference_from_scratch_b200.engine.core import build_core

    folder = two_layer_folders[dtype]
    vocab = QWEN25_3B["vocab_size"]
    requests = {"long": random_tokens(vocab, 300, 1), "mid": random_tokens(vocab, 77, 2),
                "short": random_tokens(vocab, 18, 3)}
    traces = {"whole": trace_whole(requests), "tail32": trace_tail(requests, 32),
              "portions": trace_portions(requests), "mixed": trace_mixed(requests, seed=5, interrupt="mid")}
    results = {}
    for kind, steps in traces.items():
        tokens = peak_tokens(steps, 16)
        core = build_core(folder, dtype=dtype, page_size=16, num_pages=tokens // 16, max_requests=4,
                          max_model_len=512)
        results[kind] = replay(core, steps)
        check_against_plain(folder, requests_in(steps), results[kind], dtype, "3B sizes, 2 layers")
        assert core.cache.free_pages() == core.cache.total_pages()
        del core
    if dtype == "float32":
        for kind in ("tail32", "portions", "mixed"):
            for rid, rows in results[kind].items():
                for position, row in rows.items():
                    assert np.array_equal(row, results["whole"][rid.split("@")[0]][position]), (kind, rid, position)


def test_all_36_layers_bfloat16_generation_against_the_32bit_path():
    """2,048-token prompts, then 64 tokens one by one at batch 1, 8 and 64 through the scheduler and
    EngineRunner (graphs, steps launched ahead), every sampled row against the 32-bit path."""
    from cloud_inference_from_scratch_b200.engine.check import check_against_32bit

    figures = check_against_32bit(QWEN25_3B, seed=0, batches=(1, 8, 64), prompt_tokens=2048, decode_tokens=64,
                                  score_std=1.5)
    print("3B check:", figures)
    record("3B sizes, 36 layers", "bfloat16", figures["max_rel_err_bf16"])
    assert figures["positions"] == (1 + 8 + 64) * 64
    assert figures["cuda_graph_replays"] > 0 and figures["steps_ahead_adopted"] > 0
    assert figures["max_rel_err_bf16"] <= tolerance("bfloat16", "3B sizes, 36 layers"), figures
    # rounding may swap two tokens that the 32-bit path holds nearly equal, nothing else
    assert figures["top1_beyond_rounding"] == 0 and figures["top1_agree"] >= 0.9, figures
