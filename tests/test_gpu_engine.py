"""Generation through the public entry points: generate(), InferenceEngine, the cie command line;
greedy against the plain implementation, temperature sampling, EOS, pages running out."""

import json
import os
import subprocess
import sys
from pathlib import Path

import pytest
import torch

import plain_model
from helpers import check_trace_rows, random_tokens, record, tolerance
from tiny_configs import PAGE_SIZE, TINY

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


def prompts_for(name, lengths, seed=0):
    vocab = TINY[name]["vocab_size"]
    return [random_tokens(vocab, n, seed + 10 * i + n) for i, n in enumerate(lengths)]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name,lengths,steps", [("A", (5, 11, 17), 8), ("B", (1, 9, 23, 40), 6), ("D", (19, 3, 64), 5)])
def test_greedy_generation_matches_the_plain_model(tiny_models, name, lengths, steps, dtype):
    from cloud_inference_from_scratch_b200 import generate

    config, weights = plain_model.read_model_folder(tiny_models[name])
    prompts = prompts_for(name, lengths)
    results = generate(tiny_models[name], prompts, max_output_tokens=steps, dtype=dtype,
                       block_size=PAGE_SIZE[name], kv_cache_blocks=64, prefill_chunk_size=8,
                       max_batched_tokens=24, max_active_sequences=4)
    for prompt, result in zip(prompts, results):
        assert result.finish_reason == "max_output_tokens_reached" and result.input_tokens == len(prompt)
        tokens = list(prompt)
        for produced in result.token_ids:
            logits = plain_model.forward(config, weights, tokens)[-1]
            best = int(torch.argmax(logits))
            # a tie within the path's own rounding may fall either way
            assert produced == best or float(logits[best] - logits[produced]) < (1e-5 if dtype == "float32" else 2e-2)
            tokens.append(produced)
    if dtype == "float32":
        assert [r.token_ids for r in results] == [plain_model.greedy_generate(config, weights, p, steps) for p in prompts]


def _temperature_run(folder, prompts, dtype, temperature, seed, **overrides):
    """Generation at a temperature with the logits of every sampled row kept; returns the results and,
    per request, (stream number, prompt + generated tokens, prompt length, {position: logits row})."""
    from cloud_inference_from_scratch_b200 import GenerationConfig, InferenceEngine, build_config

    settings = dict(dtype=dtype, block_size=8, kv_cache_blocks=64, max_model_len=128)
    settings.update(overrides)
    with InferenceEngine(build_config("ragged", **settings), folder) as engine:
        engine.runner.trace_logits = True
        handles = [engine.submit(p, GenerationConfig(max_output_tokens=6, temperature=temperature, seed=seed))
                   for p in prompts]
        results = [h.wait() for h in handles]
        rows = {h.request_id: {} for h in handles}
        for ids, positions, logits in engine.runner.logit_trace:
            kept = logits.float().cpu().numpy()
            for row, (rid, position) in enumerate(zip(ids, positions)):
                rows[rid][position] = kept[row]
        detail = [(h.request.sequence_number, list(p) + list(r.token_ids), len(p), rows[h.request_id])
                  for h, p, r in zip(handles, prompts, results)]
    return results, detail


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_temperature_draws_do_not_depend_on_the_batch_or_the_cut(sharp_models, dtype):
    """Every drawn token is the inverse CDF of softmax(row / T) at the uniform number of its key
    (seed, stream number, output index), whatever the batch and the cut; the rows themselves match
    the plain model.  In 32-bit the tokens of all cuttings are equal as well."""
    import numpy as np

    from cloud_inference_from_scratch_b200.sampling import draw_key, uniform_from_key

    folder = sharp_models.get("B", dtype)
    config, weights = plain_model.read_model_folder(folder)
    prompts = prompts_for("B", (9, 23, 40))
    temperature, seed = 0.8, 5
    runs = {
        "alone": _temperature_run(folder, prompts[:1], dtype, temperature, seed),
        "together": _temperature_run(folder, prompts, dtype, temperature, seed),
        "chopped": _temperature_run(folder, prompts, dtype, temperature, seed, prefill_chunk_size=3, max_batched_tokens=7),
    }
    for kind, (results, detail) in runs.items():
        for stream, tokens, prompt_len, rows in detail:
            reference = plain_model.forward(config, weights, tokens).numpy()
            assert sorted(rows) == list(range(prompt_len - 1, len(tokens) - 1)), kind
            for position, row in rows.items():
                error = float(np.abs(row - reference[position]).max() / reference.std())
                assert record("B runner", dtype, error) <= tolerance(dtype, "B runner"), (kind, position, error)
                scaled = row.astype(np.float64) / temperature
                cdf = np.cumsum(np.exp(scaled - scaled.max()))
                cdf /= cdf[-1]
                u = uniform_from_key(draw_key(seed, stream, position - (prompt_len - 1)))
                drawn = tokens[position + 1]
                below = cdf[drawn - 1] if drawn else 0.0
                assert below - 1e-5 <= u <= cdf[drawn] + 1e-5, (kind, position, drawn, u, below, cdf[drawn])
    if dtype == "float32":
        assert runs["alone"][0][0].token_ids == runs["together"][0][0].token_ids == runs["chopped"][0][0].token_ids
        assert [r.token_ids for r in runs["together"][0]] == [r.token_ids for r in runs["chopped"][0]]
    greedy, _ = _temperature_run(folder, prompts, dtype, 0.0, seed)
    assert [r.token_ids for r in runs["together"][0]] != [r.token_ids for r in greedy]
    other_seed, _ = _temperature_run(folder, prompts, dtype, temperature, 6)
    assert [r.token_ids for r in other_seed] != [r.token_ids for r in runs["together"][0]]


def test_eos_stops_generation(tiny_models):
    from cloud_inference_from_scratch_b200 import generate

    prompts = prompts_for("B", (9,))
    free = generate(tiny_models["B"], prompts, max_output_tokens=6, dtype="float32", block_size=8, kv_cache_blocks=16)[0]
    stop = free.token_ids[2]
    first = free.token_ids.index(stop)
    stopped = generate(tiny_models["B"], prompts, max_output_tokens=6, eos_token_id=stop, dtype="float32",
                       block_size=8, kv_cache_blocks=16)[0]
    assert stopped.token_ids == free.token_ids[:first + 1] and stopped.finish_reason == "eos_token_reached"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_pages_running_out_preempts_and_recomputes_without_token_drift(sharp_models, tiny_models, dtype):
    from cloud_inference_from_scratch_b200 import GenerationConfig, InferenceEngine, build_config

    folder = sharp_models.get("A", dtype)
    prompts = prompts_for("A", (56, 56, 30))
    prompts[1] = list(prompts[0])            # identical prompts must give identical outputs
    def run(blocks):
        config = build_config("ragged", dtype=dtype, block_size=4, kv_cache_blocks=blocks, max_model_len=128,
                              max_batched_tokens=32, prefill_chunk_size=16, max_active_sequences=4)
        with InferenceEngine(config, folder) as engine:
            engine.runner.trace_logits = True
            handles = [engine.submit(p, GenerationConfig(max_output_tokens=12)) for p in prompts]
            results = [h.wait() for h in handles]
            snapshot = engine.snapshot_metrics()
            engine.core.cache.assert_invariants()
            assert engine.core.cache.free_pages() == engine.core.cache.total_pages()
            trace = [(ids, positions, logits.float().cpu().numpy()) for ids, positions, logits in engine.runner.logit_trace]
            requests = {h.request_id: (list(p) + list(r.token_ids), len(p), r.finish_reason)
                        for h, p, r in zip(handles, prompts, results)}
        # every row a token was sampled from, before and after the recomputation, against the plain model
        check_trace_rows(folder, requests, trace, dtype, "A runner")
        return results, snapshot
    roomy, _ = run(64)
    tight, snapshot = run(30)                # 120 tokens of cache for 142 + 36 tokens of demand
    assert snapshot["requests"]["preempted_total"] > 0 and snapshot["requests"]["recomputed_total"] > 0
    assert sum(r.preemptions for r in tight) == snapshot["requests"]["preempted_total"]
    assert all(len(r.token_ids) == 12 for r in tight)
    if dtype == "float32":
        assert [r.token_ids for r in tight] == [r.token_ids for r in roomy]
        assert tight[0].token_ids == tight[1].token_ids
    # one request that can never fit is rejected, not looped on
    config = build_config("ragged", dtype=dtype, block_size=4, kv_cache_blocks=8, max_model_len=128)
    with InferenceEngine(config, tiny_models["A"]) as engine:
        handle = engine.submit(prompts[0], GenerationConfig(max_output_tokens=4))
        with pytest.raises(RuntimeError, match="KV capacity"):
            handle.wait()
        assert engine.core.cache.free_pages() == engine.core.cache.total_pages()


def test_engine_facade_streams_and_reports(tiny_models):
    from cloud_inference_from_scratch_b200 import GenerationConfig, InferenceEngine, build_config

    config = build_config("ragged", dtype="bfloat16", block_size=8, kv_cache_blocks=64, max_model_len=128,
                          max_active_sequences=4)
    with InferenceEngine(config, tiny_models["B"]) as engine:
        prompts = prompts_for("B", (9, 23))
        first = engine.submit(prompts[0], GenerationConfig(max_output_tokens=5))
        second = engine.submit(prompts[1], GenerationConfig(max_output_tokens=9))
        streamed = [event.token_id for event in first.stream()]
        result = second.wait()
        assert len(streamed) == 5 and len(result.token_ids) == 9 and result.ttft_ms is not None
        snapshot = engine.snapshot_metrics()
        assert snapshot["requests"]["completed_total"] == 2
        assert snapshot["scheduler"]["cuda_graph_replays"] > 0 and snapshot["scheduler"]["cuda_graph_captures"] >= 1
        assert snapshot["scheduler"]["max_forward_request_count"] == 2
        assert snapshot["kv_cache"]["blocks_used"] == 0 and snapshot["gpu"]["kernel_launches"] > 0
        with pytest.raises(Exception):
            engine.submit([], GenerationConfig(max_output_tokens=1))
        with pytest.raises(ValueError, match="vocabulary"):
            engine.submit([5000], GenerationConfig(max_output_tokens=1))


def test_cie_command_line(tiny_models):
    config, weights = plain_model.read_model_folder(tiny_models["A"])
    prompt = [5, 17, 3, 200]
    env = dict(os.environ, ENGINE_MODEL=str(tiny_models["A"]))
    done = subprocess.run([sys.executable, str(ROOT / "bin" / "cie"), "generate", "5,17,3,200", "--max-output-tokens", "6",
                           "--dtype", "float32", "--block-size", "4", "--kv-cache-blocks", "32"],
                          capture_output=True, text=True, env=env, timeout=600)
    assert done.returncode == 0, done.stderr[-2000:]
    assert [int(t) for t in done.stdout.split()] == plain_model.greedy_generate(config, weights, prompt, 6)
    once = subprocess.run([sys.executable, str(ROOT / "bin" / "cie"), "generate", "5 17 3 200", "--no-stream",
                           "--max-output-tokens", "6", "--dtype", "float32", "--block-size", "4", "--kv-cache-blocks", "32"],
                          capture_output=True, text=True, env=env, timeout=600)
    assert once.stdout.split() == done.stdout.split()
    health = subprocess.run([sys.executable, str(ROOT / "bin" / "cie"), "health"], capture_output=True, text=True, timeout=600)
    assert health.returncode == 0 and json.loads(health.stdout)["readiness"]["kernels"] == "built"
    models = subprocess.run([sys.executable, str(ROOT / "bin" / "cie"), "models"], capture_output=True, text=True, env=env, timeout=600)
    assert json.loads(models.stdout)["model"]["architecture"] == "Qwen2ForCausalLM"


def test_cie_random_config_info_and_replay(tiny_models, tmp_path):
    """The added sub-commands on the device: generation from an inline random configuration, the
    one-page report, and trace replay through ``cie replay``."""
    import numpy as np

    cie = [sys.executable, str(ROOT / "bin" / "cie")]
    config = tmp_path / "config.json"
    config.write_text(json.dumps(TINY["A"]))
    common = ["--max-output-tokens", "5", "--dtype", "float32", "--block-size", "4", "--kv-cache-blocks", "32", "--no-stream"]
    first = subprocess.run([*cie, "generate", "5,17,3", "--random-config", str(config), "--weights-seed", "3", *common],
                           capture_output=True, text=True, timeout=600)
    again = subprocess.run([*cie, "generate", "5,17,3", "--random-config", json.dumps(TINY["A"]), "--weights-seed", "3", *common],
                           capture_output=True, text=True, timeout=600)
    assert first.returncode == 0, first.stderr[-2000:]
    assert len(first.stdout.split()) == 5 and first.stdout == again.stdout
    info = subprocess.run([*cie, "info", "--model", str(tiny_models["A"])], capture_output=True, text=True, timeout=600)
    report = json.loads(info.stdout)
    assert report["readiness"]["kernels"] == "built" and report["model"]["architecture"] == "Qwen2ForCausalLM"
    trace = tmp_path / "trace.jsonl"
    trace.write_text(json.dumps({"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3, 9], "want": [3]}], "end": ["a"]}) + "\n")
    done = subprocess.run([*cie, "replay", "--model", str(tiny_models["A"]), "--dtype", "float32", "--out", str(tmp_path / "out"),
                           "--max-tokens", "64", "--trace", str(trace)], capture_output=True, text=True, timeout=600)
    assert done.returncode == 0 and done.stdout.strip() == "done 0", done.stderr[-2000:]
    cfg, weights = plain_model.read_model_folder(tiny_models["A"])
    want = plain_model.forward(cfg, weights, [5, 17, 3, 9])[-1].numpy()
    got = np.fromfile(tmp_path / "out" / "0.f32", dtype="<f4")
    assert np.abs(got - want).max() <= 1e-5
