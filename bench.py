#!/usr/bin/env python3
"""Decode and prefill throughput of the engine on one B200, random weights.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--batch 8] [--impl own|reference]
                    [--config 3b|7b-mixed|14b-pressure] [--quick]

Prints ONE JSON line.  The default configuration is the Qwen2.5-3B shape: a "step" is one decode
step of a batch of requests whose prompts (2,048 random tokens each) were prefilled before;
``value`` is decoded tokens per second over exactly K steps after W warm-up steps, timed with
CUDA events on the launching stream with a synchronize on both sides.  Every step reads all
weights (6.2 GB, far larger than the 126 MB L2) and the live requests' cache, so inputs are
larger than L2 and no flush is needed.  ``e2e`` is the same metric through ``InferenceEngine``
(host token ids in, host token ids out, the step's metadata copied from pinned memory and the
sampled ids read back every step).  ``prefill`` is one 2,048-token prompt in one step.  ``points``
holds decode at batch 1 and 64 (each over at least 200 ms), the same prompt prefilled in portions
of 256 and 512 tokens, and (unless ``--quick``) the two other benchmark configurations:

* ``7b-mixed``: Qwen2.5-7B shape, 32 requests decoding at context 1,024 while 2,048-token prompts
  advance in 512-token portions; the time of a mixed step against max(bytes / HBM peak, flops /
  bf16 peak);
* ``14b-pressure``: Qwen2.5-14B shape, 64 requests with prompts of 128 to 8,192 tokens on a cache
  pool half the size of their demand: generated tokens a second, preemptions, recomputed tokens.

``check`` compares, at the full 36 layers, the logits of the bfloat16 generation path with the
32-bit path of the same weights (``engine/check.py``).  ``--config`` prints the line of one of the
other configurations alone.  The engine runs on one GPU only: for ``--gpus`` > 1 this prints one
line saying so and exits 2.
"""

from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import subprocess
import sys
import tempfile
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))


def _qwen2(hidden, layers, q_heads, kv_heads, inter, vocab, tied) -> dict:
    return dict(
        architectures=["Qwen2ForCausalLM"], model_type="qwen2", hidden_size=hidden, num_hidden_layers=layers,
        num_attention_heads=q_heads, num_key_value_heads=kv_heads, intermediate_size=inter, vocab_size=vocab,
        rope_theta=1000000.0, rms_norm_eps=1e-6, attention_bias=True, tie_word_embeddings=tied,
        eos_token_id=151643, max_position_embeddings=32768, hidden_act="silu", use_sliding_window=False,
    )


# layer sizes of the benchmark configurations; weights are random N(0, 0.02)
QWEN25_3B = _qwen2(2048, 36, 16, 2, 11008, 151936, True)
QWEN25_7B = _qwen2(3584, 28, 28, 4, 18944, 152064, False)
QWEN25_14B = _qwen2(5120, 48, 40, 8, 13824, 152064, False)
PROMPT_TOKENS = 2048
CONTEXT = 4096
PAGE = 16
MIN_TIMED_MS = 200.0          # every point is timed over at least this long
FALLBACK_PEAKS = dict(hbm_gbs=6650.0, bf16_tflops=1590.0, source="fallback")


def peaks() -> dict:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.is_file():
        try:
            raw = json.loads(path.read_text())
            return dict(hbm_gbs=float(raw["hbm_gbs"]), bf16_tflops=float(raw["bf16_tflops"]),
                        source="measured")
        except (ValueError, KeyError):
            pass
    return dict(FALLBACK_PEAKS)


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    QUERY = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self) -> None:
        self.file = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        self.process = None

    def start(self) -> None:
        try:
            self.process = subprocess.Popen(
                ["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                 "-lms", "25"], stdout=self.file, stderr=subprocess.DEVNULL)
        except OSError:
            self.process = None

    def stop(self) -> dict:
        if self.process is None:
            return dict(sm_mhz=None, sm_max_mhz=None, reasons=["nvidia-smi unavailable"])
        time.sleep(0.15)
        self.process.terminate()
        try:
            self.process.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.process.kill()
        self.file.flush()
        rows = [line.split(",") for line in Path(self.file.name).read_text().splitlines() if line.strip()]
        os.unlink(self.file.name)
        clocks, maxes, power, reasons = [], [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for row in rows:
            try:
                clocks.append(float(row[0]))
                maxes.append(float(row[1]))
                power.append(float(row[2]))
            except (ValueError, IndexError):
                continue
            for name, value in zip(names, row[3:7]):
                if value.strip().lower().startswith("active"):
                    reasons.add(name)
        return dict(
            sm_mhz=statistics.median(clocks) if clocks else None,
            sm_max_mhz=max(maxes) if maxes else None,
            power_w=statistics.median(power) if power else None,
            samples=len(clocks),
            reasons=sorted(reasons),
        )


def model_numbers(cfg: dict) -> dict:
    h, layers = cfg["hidden_size"], cfg["num_hidden_layers"]
    hq, hkv = cfg["num_attention_heads"], cfg["num_key_value_heads"]
    d = h // hq
    inter, vocab = cfg["intermediate_size"], cfg["vocab_size"]
    per_layer = (hq + 2 * hkv) * d * h + hq * d * h + 3 * inter * h
    matmul_params = layers * per_layer
    weight_bytes = 2 * (matmul_params + vocab * h) + 4 * (layers * (2 * h + (hq + 2 * hkv) * d) + h)
    kv_bytes_per_token = layers * 2 * hkv * d * 2
    return dict(matmul_params=matmul_params, head_params=vocab * h, weight_bytes=weight_bytes,
                kv_bytes_per_token=kv_bytes_per_token, head_dim=d)


def step_flops(cfg: dict, portions: list[tuple[int, int]], rows: int) -> float:
    """Floating-point operations of one step: ``portions`` is (tokens, context before them) per
    request, ``rows`` the number of logits rows."""
    numbers = model_numbers(cfg)
    hq, d, layers = cfg["num_attention_heads"], numbers["head_dim"], cfg["num_hidden_layers"]
    tokens = sum(n for n, _ in portions)
    gemm = 2.0 * numbers["matmul_params"] * tokens + 2.0 * numbers["head_params"] * rows
    keys = sum(n * before + n * (n + 1) / 2 for n, before in portions)
    return gemm + layers * 4.0 * keys * hq * d


def random_prompts(count: int, length: int, vocab: int, seed: int) -> list[list[int]]:
    import numpy as np

    rng = np.random.default_rng(seed)
    return [rng.integers(0, vocab, size=length).tolist() for _ in range(count)]


def nvtx_range(name: str):
    from cloud_inference_from_scratch_b200.engine.profiling import nvtx_range as ranged

    return ranged(name)


def make_engine(cfg: dict, batch: int, layers: int | None = None, **overrides):
    from cloud_inference_from_scratch_b200 import InferenceEngine, build_config

    cfg = dict(cfg)
    if layers:
        cfg["num_hidden_layers"] = layers
    settings = dict(
        dtype="bfloat16", block_size=PAGE, kv_cache_blocks=batch * (CONTEXT // PAGE) + 64, max_model_len=CONTEXT,
        max_active_sequences=batch, max_queue_size=max(64, batch), max_batched_tokens=PROMPT_TOKENS,
        prefill_chunk_size=PROMPT_TOKENS, max_output_tokens=CONTEXT - PROMPT_TOKENS, cuda_graph_decode=True,
    )
    settings.update(overrides)
    return InferenceEngine(build_config("ragged", **settings), None, random_config=cfg, seed=0).start(), cfg


def _timed_steps(scheduler, steps: int) -> tuple[float, float]:
    """(device milliseconds, wall seconds) of ``steps`` scheduler iterations."""
    import torch

    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    wall = time.perf_counter()
    start.record()
    for _ in range(steps):
        scheduler.step()
    stop.record()
    torch.cuda.synchronize()
    return start.elapsed_time(stop), time.perf_counter() - wall


def _until_decoding(scheduler, handles) -> None:
    """Steps until every request has its first token; a request that ended instead (a failed step)
    ends the benchmark with its reason rather than a loop that never ends."""
    while any(h.request.generated_count < 1 for h in handles):
        ended = [h.request for h in handles if h.request.is_terminal and h.request.generated_count < 1]
        if ended:
            raise RuntimeError(f"request {ended[0].request_id} ended before its first token: "
                               f"{ended[0].finish_reason} {ended[0].error_detail}")
        scheduler.step()


def time_decode(engine, cfg: dict, batch: int, steps: int, warmup: int, sample_clocks: bool) -> dict:
    """Prefills ``batch`` prompts through the public API, then times decode iterations: exactly
    ``steps`` of them, and after those as many more as make the region at least MIN_TIMED_MS long."""
    import torch

    from cloud_inference_from_scratch_b200 import GenerationConfig

    scheduler = engine.scheduler
    prompts = random_prompts(batch, PROMPT_TOKENS, cfg["vocab_size"], seed=batch)
    gen = GenerationConfig(max_output_tokens=CONTEXT - PROMPT_TOKENS, eos_token_id=None)
    handles = [engine.submit(prompt, gen) for prompt in prompts]
    _until_decoding(scheduler, handles)
    runner = engine.runner
    ops = engine.core.runtime.ops
    for _ in range(warmup):
        scheduler.step()
    torch.cuda.synchronize()
    sampler = ClockSampler() if sample_clocks else None
    if sampler:
        sampler.start()
        time.sleep(0.25)
    launches_before = ops.launches
    replays_before = runner.cuda_graph_replays
    with nvtx_range("bench.decode"):
        ms, wall = _timed_steps(scheduler, steps)
    replays = runner.cuda_graph_replays - replays_before
    per_graph = getattr(runner, "launches_per_graph", {}).get(runner._bucket(batch), 0)
    launches = (ops.launches - launches_before) + replays * per_graph
    done = 1 + warmup + steps
    room = CONTEXT - PROMPT_TOKENS - done - 2
    more = min(room, max(0, math.ceil(MIN_TIMED_MS / (ms / steps)) - steps))
    steady_ms, steady_wall, steady_steps = ms, wall, steps
    if more > 0:
        extra_ms, extra_wall = _timed_steps(scheduler, more)
        steady_ms, steady_wall, steady_steps = ms + extra_ms, wall + extra_wall, steps + more
        done += more
    clocks = sampler.stop() if sampler else None
    assert all(h.request.generated_count >= done for h in handles)
    for handle in handles:
        handle.cancel()
    return dict(ms_per_step=ms / steps, tokens_per_s=batch * steps / (ms / 1e3),
                e2e_tokens_per_s=batch * steps / wall, clocks=clocks, context=PROMPT_TOKENS + done,
                launches=launches, h2d=engine.core.step.h2d_bytes, d2h=runner.d2h_bytes,
                steady=dict(steps=steady_steps, ms_per_step=round(steady_ms / steady_steps, 4),
                            value=round(batch * steady_steps / (steady_ms / 1e3), 1),
                            e2e=round(batch * steady_steps / steady_wall, 1)))


def time_prefill(engine, cfg: dict, portion: int | None = None, repeats: int = 5) -> dict:
    """One prompt of PROMPT_TOKENS tokens through the step function: whole, or in portions of
    ``portion`` tokens (one step each).  Median of ``repeats`` runs after three warm-up runs."""
    import torch

    from cloud_inference_from_scratch_b200.engine.step import StepEntry

    core = engine.core
    prompt = random_prompts(1, PROMPT_TOKENS, cfg["vocab_size"], seed=99)[0]
    size = portion or PROMPT_TOKENS
    cuts = [(first, min(PROMPT_TOKENS, first + size)) for first in range(0, PROMPT_TOKENS, size)]
    times = []
    for index in range(repeats + 3):
        core.step.admit("prefill")
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        start.record()
        with nvtx_range("bench.prefill" if index == repeats + 2 else "bench.prefill.warm"):
            for first, last in cuts:
                want = (last - first - 1,) if last == PROMPT_TOKENS else ()
                core.step.run([StepEntry("prefill", prompt[first:last], want=want)])
        stop.record()
        torch.cuda.synchronize()
        core.step.release("prefill")
        if index >= 3:
            times.append(start.elapsed_time(stop))
    core.runtime.ops.check_errors()
    return dict(ms=statistics.median(times), steps=len(cuts))


# ---------------------------------------------------------------------------- 7B: mixed steps
def run_mixed_7b(layers: int | None = None, decoding: int = 32, decode_context: int = 1024,
                 prompt: int = 2048, portion: int = 512, prompts: int = 6) -> dict:
    """32 requests decode at a context of about 1,024 while 2,048-token prompts come in one after the
    other and advance in 512-token portions: every step then holds 32 single tokens and one portion.
    Times each mixed step (CUDA events around the scheduler iteration, device synchronised)."""
    import torch

    from cloud_inference_from_scratch_b200 import GenerationConfig

    peak = peaks()
    # the residents' own prompts come in under the same token budget, so the first of them decodes
    # for some sixty steps before the last has its prompt in: they start 64 tokens short of the
    # context they are measured at, and may go on for as long as the run lasts
    room = decoding * 2 + prompts * (prompt // portion + 2) + 64
    decode_context -= 64
    context = max(decode_context + room, prompt + 8) + PAGE
    pages = (decoding * (decode_context + room) + 2 * (prompt + 8)) // PAGE + 64
    engine, cfg = make_engine(
        QWEN25_7B, decoding + 1, layers, kv_cache_blocks=pages, max_model_len=context,
        max_batched_tokens=decoding + portion, prefill_chunk_size=portion, max_output_tokens=room,
    )
    numbers = model_numbers(cfg)
    scheduler = engine.scheduler
    residents = [engine.submit(p, GenerationConfig(max_output_tokens=room, eos_token_id=None))
                 for p in random_prompts(decoding, decode_context, cfg["vocab_size"], seed=7)]
    _until_decoding(scheduler, residents)
    times: list[float] = []
    contexts: list[int] = []
    for index, tokens in enumerate(random_prompts(prompts, prompt, cfg["vocab_size"], seed=70)):
        newcomer = engine.submit(tokens, GenerationConfig(max_output_tokens=1, eos_token_id=None))
        while not newcomer.request.is_terminal:
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            start.record()
            scheduler.step()
            stop.record()
            torch.cuda.synchronize()
            plan = engine.runner.forward_plans[-1]
            if len(plan) == decoding + 1 and index >= 2:     # the first two prompts warm up and capture
                times.append(start.elapsed_time(stop))
                contexts.append(sum(row[1] for row in plan[:decoding]) // decoding)
    engine.core.runtime.ops.check_errors()
    replays = engine.core.step.graph_replays
    for handle in residents:
        handle.cancel()
    free, total = engine.core.cache.free_pages(), engine.core.cache.total_pages()
    engine.close()
    del engine
    torch.cuda.empty_cache()
    ms = statistics.median(times)
    mean_context = statistics.mean(contexts)
    # a mixed step: 32 single tokens over their contexts, one portion over (on average) half a prompt
    portions = [(1, int(mean_context))] * decoding + [(portion, (prompt - portion) // 2)]
    flops = step_flops(cfg, portions, decoding + 0.25)
    read = numbers["weight_bytes"] + numbers["kv_bytes_per_token"] * (decoding * mean_context + prompt / 2)
    memory_ms = read / (peak["hbm_gbs"] * 1e9) * 1e3
    compute_ms = flops / (peak["bf16_tflops"] * 1e12) * 1e3
    return dict(ms_per_mixed_step=round(ms, 4), mixed_steps_timed=len(times),
                tokens_per_step=decoding + portion, tokens_per_s=round((decoding + portion) / (ms / 1e3), 1),
                memory_ms=round(memory_ms, 3), compute_ms=round(compute_ms, 3),
                frac=round(max(memory_ms, compute_ms) / ms, 4), step_bytes=int(read), step_flops=flops,
                mean_decode_context=round(mean_context, 1), layers=cfg["num_hidden_layers"],
                step_graph_replays=replays, pages_left=total - free, peaks=peak["source"])


# ---------------------------------------------------------------------------- 14B: page pressure
def run_pressure_14b(layers: int | None = None, requests: int = 64, shortest: int = 128, longest: int = 8192,
                     outputs: int = 64, pool_share: float = 0.5) -> dict:
    """64 requests with prompt lengths uniform in 128..8,192 and 64 tokens to generate each, on a
    cache pool that holds ``pool_share`` of what they need together: the scheduler preempts and
    recomputes.  Wall-clock (device synchronised) from the first submit to the last token."""
    import numpy as np
    import torch

    from cloud_inference_from_scratch_b200 import GenerationConfig

    rng = np.random.default_rng(14)
    lengths = [int(n) for n in rng.integers(shortest, longest + 1, size=requests)]
    demand = sum(-(-(n + outputs) // PAGE) for n in lengths)
    pages = max(int(demand * pool_share), -(-(longest + outputs) // PAGE) + 8)
    engine, cfg = make_engine(
        QWEN25_14B, requests, layers, kv_cache_blocks=pages, max_model_len=longest + outputs + PAGE,
        max_batched_tokens=2048, prefill_chunk_size=512, max_output_tokens=outputs, max_queue_size=requests,
    )
    numbers = model_numbers(cfg)
    prompts = [rng.integers(0, cfg["vocab_size"], size=n).tolist() for n in lengths]
    # warm-up: one short request end to end (loads kernels, captures nothing that the run reuses wrongly)
    engine.submit(prompts[0][:64], GenerationConfig(max_output_tokens=4, eos_token_id=None)).wait()
    torch.cuda.synchronize()
    started = time.perf_counter()
    handles = [engine.submit(p, GenerationConfig(max_output_tokens=outputs, eos_token_id=None)) for p in prompts]
    engine.run_until_idle()
    torch.cuda.synchronize()
    seconds = time.perf_counter() - started
    results = [h.wait() for h in handles]
    engine.core.runtime.ops.check_errors()
    counters = engine.snapshot_metrics()["requests"]
    engine.core.cache.assert_invariants()
    free, total = engine.core.cache.free_pages(), engine.core.cache.total_pages()
    iterations = counters["iterations_total"]
    engine.close()
    del engine
    torch.cuda.empty_cache()
    generated = sum(r.output_tokens for r in results)
    return dict(tokens_per_s=round(generated / seconds, 1), seconds=round(seconds, 3), generated=generated,
                prompt_tokens=sum(lengths), preempted_total=counters["preempted_total"],
                recomputed_total=counters["recomputed_total"], input_tokens_total=counters["input_tokens_total"],
                input_tokens_per_s=round(counters["input_tokens_total"] / seconds, 1), iterations=iterations,
                pool_pages=pages, demand_pages=demand, pages_left=total - free,
                pool_gb=round(pages * PAGE * numbers["kv_bytes_per_token"] / 1e9, 2),
                weights_gb=round(numbers["weight_bytes"] / 1e9, 2), layers=cfg["num_hidden_layers"],
                all_completed=all(r.output_tokens == outputs for r in results))


# ---------------------------------------------------------------------------- the lines
def size_keys(cfg: dict, layers_of_model: int, name: str) -> dict:
    numbers = model_numbers(cfg)
    return {"model": name, "layers": cfg["num_hidden_layers"], "layers_of_model": layers_of_model,
            "hidden": cfg["hidden_size"], "q_heads": cfg["num_attention_heads"],
            "kv_heads": cfg["num_key_value_heads"], "head_dim": numbers["head_dim"],
            "intermediate": cfg["intermediate_size"], "vocab": cfg["vocab_size"]}


def config_record(cfg: dict, batch: int) -> dict:
    """The flat ``config`` of the default line; the reference arm prints the same keys."""
    return {**size_keys(cfg, 36, "Qwen2.5-3B shape"), "global_batch": batch, "seq_len": CONTEXT,
            "prompt_tokens": PROMPT_TOKENS, "page_size": PAGE, "parallelism": "single GPU",
            "cuda_graph_decode": True, "l2": "inputs larger than L2 (6.2 GB of weights per step)",
            "baseline": "reference 3B c=8 on L4: 178.986 tok/s"}


def run_own(args: argparse.Namespace) -> int:
    import torch

    if not torch.cuda.is_available():
        print(json.dumps({"error": "no CUDA device; this engine has no CPU path"}))
        return 1
    peak = peaks()
    cfg = dict(QWEN25_3B)
    results = {}
    batches = (args.batch, 1, 64) if args.only == "all" else (args.batch,)
    prefill = dict(ms=float("nan"))
    portions: dict[int, dict] = {}
    for batch in batches:
        if batch in results:
            continue
        engine, used = make_engine(cfg, batch, args.layers)
        if batch == args.batch and args.only in ("all", "prefill"):
            prefill = time_prefill(engine, used)
            if args.only == "all":
                portions = {size: time_prefill(engine, used, portion=size) for size in (256, 512)}
        if args.only == "prefill":
            results[batch] = dict(ms_per_step=float("nan"), tokens_per_s=float("nan"),
                                  e2e_tokens_per_s=float("nan"), clocks=None, context=PROMPT_TOKENS,
                                  launches=0, h2d=0, d2h=0, steady=None)
        else:
            results[batch] = time_decode(engine, used, batch, args.steps, args.warmup,
                                         sample_clocks=batch == args.batch)
        engine.close()
        del engine
        torch.cuda.empty_cache()
    numbers = model_numbers(used)
    main = results[args.batch]
    step_bytes = numbers["weight_bytes"] + args.batch * main["context"] * numbers["kv_bytes_per_token"]
    achieved = step_bytes / (main["ms_per_step"] / 1e3) / 1e9
    flops = step_flops(used, [(PROMPT_TOKENS, 0)], 1)
    points: dict = {}
    for b in (1, 64):
        if b in results and b != args.batch:
            steady = results[b]["steady"]
            read = numbers["weight_bytes"] + b * results[b]["context"] * numbers["kv_bytes_per_token"]
            points[f"decode_b{b}"] = steady["value"]
            points[f"decode_b{b}_ms"] = steady["ms_per_step"]
            points[f"decode_b{b}_steps"] = steady["steps"]
            points[f"decode_b{b}_frac"] = round(read / (steady["ms_per_step"] / 1e3) / 1e9 / peak["hbm_gbs"], 4)
    for size, timed in portions.items():
        points[f"prefill_{size}"] = round(PROMPT_TOKENS / (timed["ms"] / 1e3), 1)
        points[f"prefill_{size}_ms"] = round(timed["ms"], 3)
        points[f"prefill_{size}_frac"] = round(flops / (timed["ms"] / 1e3) / (peak["bf16_tflops"] * 1e12), 4)
    check = None
    if args.only == "all" and not args.quick:
        mixed = run_mixed_7b(args.layers)
        points.update(mixed7b_ms=mixed["ms_per_mixed_step"], mixed7b_tok_s=mixed["tokens_per_s"],
                      mixed7b_frac=mixed["frac"], mixed7b_bound_ms=max(mixed["memory_ms"], mixed["compute_ms"]))
        pressure = run_pressure_14b(args.layers)
        points.update(pressure14b_tok_s=pressure["tokens_per_s"], pressure14b_preempted=pressure["preempted_total"],
                      pressure14b_recomputed=pressure["recomputed_total"], pressure14b_seconds=pressure["seconds"],
                      pressure14b_pages_left=pressure["pages_left"])
        from cloud_inference_from_scratch_b200.engine.check import check_against_32bit

        figures = check_against_32bit(used, batches=(args.batch,), prompt_tokens=PROMPT_TOKENS, decode_tokens=16,
                                      score_std=1.5)
        check = {key: figures[key] for key in ("max_rel_err_bf16", "mean_rel_err_bf16", "positions", "top1_agree",
                                               "top1_beyond_rounding", "layers", "cuda_graph_replays")}
        check["against"] = "32-bit path, same weights; error in standard deviations of the logits"
    line = {
        "metric": f"decode tok/s (Qwen2.5-3B shape, batch {args.batch}, context {PROMPT_TOKENS}+)",
        "value": round(main["tokens_per_s"], 1),
        "unit": "tokens/s",
        "n_gpus": 1,
        "steps": args.steps,
        "warmup": args.warmup,
        "ms_per_step": round(main["ms_per_step"], 4),
        "higher_is_better": True,
        "scaling": "weak",
        "vs_baseline": round(main["tokens_per_s"] / 178.986, 2),
        "dtype": "bf16",
        "data": "synthetic: random N(0,0.02) weights, uniform random token ids",
        "impl": "own",
        "config": config_record(used, args.batch),
        "e2e": {"value": round(main["e2e_tokens_per_s"], 1), "unit": "tokens/s",
                "h2d_bytes_per_step": main["h2d"], "d2h_bytes_per_step": main["d2h"]},
        "gpu_launches": main["launches"],
        "steady": main["steady"],
        "prefill": {"value": round(PROMPT_TOKENS / (prefill["ms"] / 1e3), 1), "tokens": PROMPT_TOKENS,
                    "ms": round(prefill["ms"], 3),
                    "frac": round(flops / (prefill["ms"] / 1e3) / (peak["bf16_tflops"] * 1e12), 4)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peak["hbm_gbs"],
                     "unit": "GB/s", "frac": round(achieved / peak["hbm_gbs"], 4),
                     "peaks": peak["source"]},
        "points": points,
        "check": check,
        "clocks": main["clocks"],
    }
    print(json.dumps(without_nan(line)))
    return 0


def run_other_config(args: argparse.Namespace) -> int:
    """``--config 7b-mixed`` or ``--config 14b-pressure`` alone: one line in the same form."""
    import torch

    if not torch.cuda.is_available():
        print(json.dumps({"error": "no CUDA device; this engine has no CPU path"}))
        return 1
    sampler = ClockSampler()
    sampler.start()
    if args.config == "7b-mixed":
        figures = run_mixed_7b(args.layers)
        cfg = dict(QWEN25_7B, num_hidden_layers=figures["layers"])
        line = {"metric": "ms per mixed step (Qwen2.5-7B shape, 32 decoding at context 1,024 + one 512-token portion)",
                "value": figures["ms_per_mixed_step"], "unit": "ms", "higher_is_better": False,
                "ms_per_step": figures["ms_per_mixed_step"], "steps": figures["mixed_steps_timed"],
                "config": {**size_keys(cfg, 28, "Qwen2.5-7B shape"), "global_batch": 33, "seq_len": 2048,
                           "decoding_requests": 32, "decode_context": 1024, "prompt_tokens": 2048, "portion": 512,
                           "page_size": PAGE, "parallelism": "single GPU"},
                "roofline": {"bound": "compute" if figures["compute_ms"] > figures["memory_ms"] else "hbm",
                             "memory_ms": figures["memory_ms"], "compute_ms": figures["compute_ms"],
                             "frac": figures["frac"], "peaks": figures["peaks"]},
                "detail": figures}
    else:
        figures = run_pressure_14b(args.layers)
        cfg = dict(QWEN25_14B, num_hidden_layers=figures["layers"])
        line = {"metric": "generated tok/s under page pressure (Qwen2.5-14B shape, 64 requests, prompts 128..8,192)",
                "value": figures["tokens_per_s"], "unit": "tokens/s", "higher_is_better": True,
                "ms_per_step": round(figures["seconds"] / max(1, figures["iterations"]) * 1e3, 4),
                "steps": figures["iterations"],
                "config": {**size_keys(cfg, 48, "Qwen2.5-14B shape"), "global_batch": 64, "seq_len": 8192 + 64,
                           "prompt_tokens": "uniform 128..8192", "output_tokens": 64, "page_size": PAGE,
                           "pool_pages": figures["pool_pages"], "demand_pages": figures["demand_pages"],
                           "parallelism": "single GPU"},
                "detail": figures}
    line.update({"n_gpus": 1, "warmup": args.warmup, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
                 "data": "synthetic: random N(0,0.02) weights, uniform random token ids", "impl": "own",
                 "clocks": sampler.stop()})
    print(json.dumps(without_nan(line)))
    return 0


def without_nan(value):
    """A part that was not measured (--only) is null in the record, not NaN."""
    if isinstance(value, dict):
        return {key: without_nan(item) for key, item in value.items()}
    if isinstance(value, float) and value != value:
        return None
    return value


def run_reference(args: argparse.Namespace) -> int:
    from baseline.reference_arm import run as run_reference_arm

    cfg = dict(QWEN25_3B)
    if args.layers:
        cfg["num_hidden_layers"] = args.layers
    print(json.dumps(run_reference_arm(args, QWEN25_3B, PROMPT_TOKENS, CONTEXT, config_record(cfg, args.batch))))
    return 0


def main() -> int:
    global PROMPT_TOKENS, CONTEXT
    parser = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=128)
    parser.add_argument("--warmup", type=int, default=8)
    parser.add_argument("--batch", type=int, default=8)
    parser.add_argument("--layers", type=int, default=None,
                        help="fewer layers than the model has (named in config; for quick runs)")
    parser.add_argument("--prompt-tokens", type=int, default=PROMPT_TOKENS,
                        help="prompt length of every request and of the timed prefill (the record's "
                             "default is 2048; longer ones are for profiles of long contexts, own arm only)")
    parser.add_argument("--impl", default="own", choices=("own", "reference"))
    parser.add_argument("--config", default="3b", choices=("3b", "7b-mixed", "14b-pressure"),
                        help="the benchmark configuration whose line is printed (default: the 3B line, "
                             "which also carries the other two as points)")
    parser.add_argument("--quick", action="store_true",
                        help="leave the 7B and 14B points and the logits check out of the 3B line")
    parser.add_argument("--only", default="all", choices=("all", "decode", "prefill"),
                        help="measure only the decode step at --batch, or only the prefill "
                             "(for profiling; the full line needs 'all')")
    args = parser.parse_args()
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not built")
        return 2
    if args.warmup < 3:
        args.warmup = 3
    if args.prompt_tokens != PROMPT_TOKENS:
        limit = QWEN25_3B["max_position_embeddings"]
        room = args.warmup + args.steps + 2
        if args.impl != "own" or args.prompt_tokens < 16 or args.prompt_tokens + room > limit:
            print(f"bench.py: --prompt-tokens takes 16 .. {limit - room} with these steps, own arm only")
            return 2
        PROMPT_TOKENS = args.prompt_tokens
        CONTEXT = min(limit, PROMPT_TOKENS + max(2048, room))
    if args.impl == "reference":
        return run_reference(args)
    if args.config != "3b":
        return run_other_config(args)
    return run_own(args)


if __name__ == "__main__":
    raise SystemExit(main())
