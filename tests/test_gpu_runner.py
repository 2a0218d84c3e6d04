"""The path generation really takes: scheduler -> EngineRunner -> CUDA-graph decode with the next
step launched ahead of the host.  Every sampled row's logits are compared with the plain model
run on the request's final sequence, while requests of different lengths end at different steps
(steps launched ahead are dropped), one joins in mid-decode, one stops on its EOS token and the
pool is small enough to preempt."""

import pytest

import plain_model
from helpers import check_trace_rows, random_tokens
from tiny_configs import PAGE_SIZE, TINY

pytestmark = pytest.mark.gpu


def _drive(folder, name, dtype, blocks, eos_for_first=None, **overrides):
    """Three requests from the start, a fourth after six iterations; returns per request
    (tokens, prompt length, finish reason), the logit trace, counters and the most pages in use."""
    from cloud_inference_from_scratch_b200 import GenerationConfig, InferenceEngine, build_config

    vocab = TINY[name]["vocab_size"]
    page = PAGE_SIZE[name]
    settings = dict(dtype=dtype, block_size=page, kv_cache_blocks=blocks, max_model_len=256,
                    max_batched_tokens=32, prefill_chunk_size=16, max_active_sequences=4)
    settings.update(overrides)
    config = build_config("ragged", **settings)
    plan = [(19, 12), (40, 20), (9, 7)]
    late = (25, 10)
    with InferenceEngine(config, folder) as engine:
        runner, scheduler = engine.runner, engine.scheduler
        runner.trace_logits = True
        handles = []
        for index, (length, outputs) in enumerate(plan):
            eos = eos_for_first if index == 0 else None
            handles.append(engine.submit(random_tokens(vocab, length, 300 + index),
                                         GenerationConfig(max_output_tokens=outputs, eos_token_id=eos)))
        most_pages = 0
        iteration = 0
        while scheduler.has_work:
            if iteration == 6:
                handles.append(engine.submit(random_tokens(vocab, late[0], 399),
                                             GenerationConfig(max_output_tokens=late[1])))
            scheduler.step()
            iteration += 1
            most_pages = max(most_pages, engine.core.cache.total_pages() - engine.core.cache.free_pages())
        results = [h.wait() for h in handles]
        engine.core.cache.assert_invariants()
        assert engine.core.cache.free_pages() == engine.core.cache.total_pages()
        trace = [(ids, positions, logits.float().cpu().numpy()) for ids, positions, logits in runner.logit_trace]
        counters = dict(adopted=runner.steps_ahead_adopted, dropped=runner.steps_ahead_dropped,
                        replays=runner.cuda_graph_replays, preempted=engine.snapshot_metrics()["requests"]["preempted_total"])
        requests = {h.request_id: (list(h.request.prompt_token_ids) + list(r.token_ids), r.input_tokens, r.finish_reason)
                    for h, r in zip(handles, results)}
    return requests, trace, counters, most_pages


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["B", "D"])
def test_logits_of_the_generation_path(sharp_models, name, dtype):
    folder = sharp_models.get(name, dtype)
    # roomy pool: learn the tokens (for the EOS run) and how many pages the schedule needs at most
    requests, trace, counters, most_pages = _drive(folder, name, dtype, blocks=64)
    check_trace_rows(folder, requests, trace, dtype, f"{name} runner")
    assert counters["replays"] > 0 and counters["adopted"] > 0 and counters["dropped"] > 0, counters
    assert counters["preempted"] == 0
    first = next(iter(requests))
    tokens, prompt_len, _ = requests[first]
    stop = tokens[prompt_len + 4]                       # the fifth generated token of the first request
    where = tokens[prompt_len:].index(stop)
    # an EOS hit, which the step launched ahead cannot foresee
    requests, trace, counters, most_pages = _drive(folder, name, dtype, blocks=64, eos_for_first=stop)
    check_trace_rows(folder, requests, trace, dtype, f"{name} runner")
    got, prompt_len, reason = requests[first]
    assert reason == "eos_token_reached" and len(got) == prompt_len + where + 1
    assert counters["adopted"] > 0 and counters["dropped"] > 0, counters
    # the same once more with a pool two pages short of what that schedule needs: a preemption
    requests, trace, counters, _ = _drive(folder, name, dtype, blocks=most_pages - 2, eos_for_first=stop)
    check_trace_rows(folder, requests, trace, dtype, f"{name} runner")
    assert requests[first][2] == "eos_token_reached"
    assert counters["preempted"] >= 1 and counters["adopted"] > 0, counters


def test_decode_bucket_above_the_token_budget(tiny_models):
    """A token budget that is no power of two with more decoding requests than its largest power of
    two: the padded decode batch (32 rows) is larger than the budget (24) and must still run."""
    from cloud_inference_from_scratch_b200 import generate

    config, weights = plain_model.read_model_folder(tiny_models["A"])
    prompts = [random_tokens(TINY["A"]["vocab_size"], 3 + i % 5, 500 + i) for i in range(20)]
    results = generate(tiny_models["A"], prompts, max_output_tokens=6, dtype="float32", block_size=4,
                       kv_cache_blocks=128, max_batched_tokens=24, prefill_chunk_size=8, max_active_sequences=20)
    assert [r.token_ids for r in results] == [plain_model.greedy_generate(config, weights, p, 6) for p in prompts]
    assert all(r.finish_reason == "max_output_tokens_reached" for r in results)
