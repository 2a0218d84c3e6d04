"""Self-check at real layer sizes: the bfloat16 generation path against the 32-bit path.

The serving path (scheduler, ``EngineRunner``: prompt portions, CUDA-graph decode with steps
launched ahead, tensor-core kernels) generates tokens for a few batches of random prompts and
keeps the float32 logits of every sampled row.  Then the true 32-bit path of the same model
(same seeded weights, CUDA-core products, generic attention, the step function driven directly)
runs every request's final sequence whole, in one step, and the logits are compared row by
row.  The reference checks its 3B model end to end against another implementation
(tests/remote_gpu_tests.py:99-119, logits at every position; tests/remote_ragged_gpu_tests.py:73-108,
exact tokens); with random weights there is no other implementation, so the engine's own 32-bit
path, which the tests hold to the plain model, is the yardstick.

The error of a row is max |difference| over the vocabulary divided by the standard deviation of
the 32-bit logits of that request: how large the rounding noise is against the spread of the
candidates for the next token.
"""

from __future__ import annotations

import math
from typing import Any


def sharpening_scales(hidden_size: int, score_std: float = 3.0, value_output: float = 1.5) -> dict[str, float]:
    """Factors for ``RandomSource(scales=...)`` that spread attention scores.  With N(0, 0.02)
    weights a score q.k/sqrt(D) has a standard deviation of 0.0004 * hidden: every softmax is
    close to uniform and a wrong or missing key changes almost nothing.  Scaled so, scores have
    a standard deviation of about ``score_std`` and single keys stand out."""
    qk = math.sqrt(score_std / (0.0004 * hidden_size))
    return {".q_proj.": qk, ".k_proj.": qk, ".v_proj.": value_output, ".o_proj.": value_output}


def _prompts(count: int, long_count: int, long_len: int, short_range: tuple[int, int], vocab: int,
             seed: int) -> list[list[int]]:
    import numpy as np

    rng = np.random.default_rng(seed)
    out = []
    for index in range(count):
        length = long_len if index < long_count else int(rng.integers(short_range[0], short_range[1] + 1))
        out.append(rng.integers(0, vocab, size=length).tolist())
    return out


def generate_with_logits(engine: Any, prompts: list[list[int]], max_output_tokens: int
                         ) -> list[tuple[list[int], int, dict[int, Any]]]:
    """Greedy generation through the scheduler; per prompt: (prompt + generated tokens, prompt
    length, {position of the fed token: float32 logits row on the device})."""
    from .request import GenerationConfig

    runner = engine.runner
    runner.trace_logits = True
    runner.logit_trace.clear()
    handles = [engine.submit(p, GenerationConfig(max_output_tokens=max_output_tokens, eos_token_id=None))
               for p in prompts]
    engine.run_until_idle()
    rows: dict[str, dict[int, Any]] = {h.request_id: {} for h in handles}
    for ids, positions, logits in runner.logit_trace:
        for row, (rid, position) in enumerate(zip(ids, positions)):
            if rid in rows:
                rows[rid][position] = logits[row]
    runner.logit_trace.clear()
    runner.trace_logits = False
    out = []
    for handle, prompt in zip(handles, prompts):
        result = handle.wait()
        out.append((list(prompt) + list(result.token_ids), len(prompt), rows[handle.request_id]))
    return out


def check_against_32bit(
    random_config: dict[str, Any],
    seed: int = 0,
    batches: tuple[int, ...] = (1, 8, 64),
    prompt_tokens: int = 2048,
    long_prompts: int = 8,
    short_prompts: tuple[int, int] = (128, 512),
    decode_tokens: int = 64,
    score_std: float = 3.0,
    device: str = "cuda:0",
    page_size: int = 16,
) -> dict[str, Any]:
    """Runs the comparison described in the module docstring and returns its figures:
    ``max_rel_err_bf16`` (worst row), ``mean_rel_err_bf16``, ``positions`` (rows compared),
    ``top1_agree`` (share of rows whose argmax is the same on both paths), ``top1_beyond_rounding``
    (rows whose argmax differs although the 32-bit path separates the two tokens by more than twice
    the row's own error: none, if rounding is all there is), the worst error per batch, and the
    runner's counters that show which path ran (graph replays, steps adopted ahead)."""
    import torch

    from ..config.engine_config import build_config
    from .core import build_core
    from .engine import InferenceEngine
    from .step import StepEntry

    scales = sharpening_scales(random_config["hidden_size"], score_std)
    largest = max(batches)
    prompts = _prompts(largest, min(long_prompts, largest), prompt_tokens, short_prompts,
                       random_config["vocab_size"], seed=1234)
    context = prompt_tokens + decode_tokens + page_size
    held = sum(-(-(len(p) + decode_tokens) // page_size) + 1 for p in prompts)
    config = build_config(
        "ragged", dtype="bfloat16", block_size=page_size, kv_cache_blocks=held + 8, max_model_len=context,
        max_active_sequences=largest, max_queue_size=max(64, largest), max_batched_tokens=prompt_tokens,
        prefill_chunk_size=prompt_tokens, max_output_tokens=decode_tokens, cuda_graph_decode=True,
    )
    engine = InferenceEngine(config, None, device=device, random_config=random_config, seed=seed,
                             random_scales=scales).start()
    runs: dict[int, list] = {}
    for batch in batches:
        runs[batch] = generate_with_logits(engine, prompts[:batch], decode_tokens)
    runner = engine.runner
    counters = dict(cuda_graph_replays=runner.cuda_graph_replays, steps_ahead_adopted=runner.steps_ahead_adopted,
                    steps_ahead_dropped=runner.steps_ahead_dropped)
    assert engine.core.cache.free_pages() == engine.core.cache.total_pages(), "pages were not all given back"
    engine.close()
    del engine, runner
    torch.cuda.empty_cache()

    core = build_core(None, dtype="float32", device=device, page_size=page_size,
                      num_pages=-(-context // page_size) + 2, max_requests=1, max_model_len=context,
                      random_config=random_config, seed=seed, random_device="cuda", random_scales=scales)
    reference: dict[tuple[int, ...], Any] = {}
    figures: dict[str, Any] = {}
    worst, total, rows_seen, agree, beyond = 0.0, 0.0, 0, 0, 0
    for batch, results in runs.items():
        batch_worst = 0.0
        for tokens, prompt_len, rows in results:
            fed = tuple(tokens[:-1])
            if fed not in reference:
                core.step.admit("check")
                want = tuple(range(prompt_len - 1, len(fed)))
                reference[fed] = core.step.run([StepEntry("check", list(fed), want=want)]).logits.clone()
                core.runtime.ops.check_errors()
                core.step.release("check")
            ref = reference[fed]
            spread = float(ref.std())
            for position, row in rows.items():
                ref_row = ref[position - (prompt_len - 1)]
                error = float((row - ref_row).abs().max()) / spread
                batch_worst = max(batch_worst, error)
                total += error
                rows_seen += 1
                mine, theirs = int(torch.argmax(row)), int(torch.argmax(ref_row))
                agree += int(mine == theirs)
                if mine != theirs and float(ref_row[theirs] - ref_row[mine]) > 2.0 * error * spread:
                    beyond += 1
            assert len(rows) == len(tokens) - prompt_len, "a sampled row is missing from the trace"
        figures[f"b{batch}"] = round(batch_worst, 5)
        worst = max(worst, batch_worst)
    del core, reference
    torch.cuda.empty_cache()
    return dict(max_rel_err_bf16=round(worst, 5), mean_rel_err_bf16=round(total / max(1, rows_seen), 5),
                positions=rows_seen, top1_agree=round(agree / max(1, rows_seen), 4), top1_beyond_rounding=beyond,
                per_batch=figures,
                layers=random_config["num_hidden_layers"], prompt_tokens=prompt_tokens,
                decode_tokens=decode_tokens, batches=list(batches), **counters)
