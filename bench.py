#!/usr/bin/env python3
"""Decode and prefill throughput of the engine on one B200, Qwen2.5-3B shape, random weights.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--batch 8] [--impl own|reference]

Prints ONE JSON line.  A "step" is one decode step of a batch of requests whose prompts
(2,048 random tokens each) were prefilled before; ``value`` is decoded tokens per second over
exactly K steps after W warm-up steps, timed with CUDA events on the launching stream with a
synchronize on both sides.  Every step reads all weights (6.2 GB, far larger than the 126 MB L2)
and the live requests' cache, so inputs are larger than L2 and no flush is needed.  ``e2e`` is
the same metric through ``InferenceEngine`` (host token ids in, host token ids out, the step's
metadata copied from pinned memory and the sampled ids read back every step).  ``prefill`` is
one 2,048-token prompt in one step.  ``points`` holds decode at batch 1 and 64.

The engine runs on one GPU only: for ``--gpus`` > 1 this prints one line saying so and exits 2.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

# Qwen2.5-3B layer sizes (the benchmark configuration); weights are random N(0, 0.02).
QWEN25_3B = dict(
    architectures=["Qwen2ForCausalLM"], model_type="qwen2", hidden_size=2048,
    num_hidden_layers=36, num_attention_heads=16, num_key_value_heads=2, intermediate_size=11008,
    vocab_size=151936, rope_theta=1000000.0, rms_norm_eps=1e-6, attention_bias=True,
    tie_word_embeddings=True, eos_token_id=151643, max_position_embeddings=32768,
    hidden_act="silu", use_sliding_window=False,
)
PROMPT_TOKENS = 2048
CONTEXT = 4096
PAGE = 16
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
                 "-lms", "100"], stdout=self.file, stderr=subprocess.DEVNULL)
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


def prefill_flops(cfg: dict, tokens: int, rows: int) -> float:
    numbers = model_numbers(cfg)
    hq, d, layers = cfg["num_attention_heads"], numbers["head_dim"], cfg["num_hidden_layers"]
    gemm = 2.0 * numbers["matmul_params"] * tokens + 2.0 * numbers["head_params"] * rows
    attention = layers * 4.0 * (tokens * (tokens + 1) / 2) * hq * d
    return gemm + attention


def random_prompts(count: int, length: int, vocab: int, seed: int) -> list[list[int]]:
    import numpy as np

    rng = np.random.default_rng(seed)
    return [rng.integers(0, vocab, size=length).tolist() for _ in range(count)]


def nvtx_range(name: str):
    from cloud_inference_from_scratch_b200.engine.profiling import nvtx_range as ranged

    return ranged(name)


def make_engine(cfg: dict, batch: int, layers: int | None = None):
    from cloud_inference_from_scratch_b200 import InferenceEngine, build_config

    cfg = dict(cfg)
    if layers:
        cfg["num_hidden_layers"] = layers
    pages = batch * (CONTEXT // PAGE) + 64
    config = build_config(
        "ragged", dtype="bfloat16", block_size=PAGE, kv_cache_blocks=pages, max_model_len=CONTEXT,
        max_active_sequences=batch, max_queue_size=max(64, batch), max_batched_tokens=PROMPT_TOKENS,
        prefill_chunk_size=PROMPT_TOKENS, max_output_tokens=CONTEXT - PROMPT_TOKENS,
        cuda_graph_decode=True,
    )
    return InferenceEngine(config, None, random_config=cfg, seed=0).start(), cfg


def time_decode(engine, cfg: dict, batch: int, steps: int, warmup: int, sample_clocks: bool) -> dict:
    """Prefills ``batch`` prompts through the public API, then times decode iterations."""
    import torch

    from cloud_inference_from_scratch_b200 import GenerationConfig

    scheduler = engine.scheduler
    prompts = random_prompts(batch, PROMPT_TOKENS, cfg["vocab_size"], seed=batch)
    gen = GenerationConfig(max_output_tokens=CONTEXT - PROMPT_TOKENS, eos_token_id=None)
    handles = [engine.submit(prompt, gen) for prompt in prompts]
    while any(h.request.generated_count < 1 for h in handles):
        scheduler.step()
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
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    wall = time.perf_counter()
    start.record()
    with nvtx_range("bench.decode"):
        for _ in range(steps):
            scheduler.step()
    stop.record()
    torch.cuda.synchronize()
    wall = time.perf_counter() - wall
    clocks = sampler.stop() if sampler else None
    ms = start.elapsed_time(stop)
    assert all(h.request.generated_count >= 1 + warmup + steps for h in handles)
    context_now = PROMPT_TOKENS + 1 + warmup + steps
    replays = runner.cuda_graph_replays - replays_before
    per_graph = getattr(runner, "launches_per_graph", {}).get(runner._bucket(batch), 0)
    launches = (ops.launches - launches_before) + replays * per_graph
    for handle in handles:
        handle.cancel()
    return dict(ms_per_step=ms / steps, tokens_per_s=batch * steps / (ms / 1e3),
                e2e_tokens_per_s=batch * steps / wall, clocks=clocks, context=context_now,
                launches=launches, h2d=engine.core.step.h2d_bytes, d2h=runner.d2h_bytes)


def time_prefill(engine, cfg: dict, repeats: int = 5) -> dict:
    import torch

    from cloud_inference_from_scratch_b200.engine.step import StepEntry

    core = engine.core
    prompt = random_prompts(1, PROMPT_TOKENS, cfg["vocab_size"], seed=99)[0]
    times = []
    for index in range(repeats + 3):
        core.step.admit("prefill")
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        start.record()
        with nvtx_range("bench.prefill" if index == repeats + 2 else "bench.prefill.warm"):
            core.step.run([StepEntry("prefill", prompt, want=(PROMPT_TOKENS - 1,))])
        stop.record()
        torch.cuda.synchronize()
        core.step.release("prefill")
        if index >= 3:
            times.append(start.elapsed_time(stop))
    core.runtime.ops.check_errors()
    return dict(ms=statistics.median(times))


def run_own(args: argparse.Namespace) -> int:
    import torch

    if not torch.cuda.is_available():
        print(json.dumps({"error": "no CUDA device; this engine has no CPU path"}))
        return 1
    peak = peaks()
    cfg = dict(QWEN25_3B)
    numbers = model_numbers(cfg)
    results = {}
    main = None
    batches = (args.batch, 1, 64) if args.only == "all" else (args.batch,)
    prefill = dict(ms=float("nan"))
    for batch in batches:
        if batch in results:
            continue
        engine, used = make_engine(cfg, batch, args.layers)
        numbers = model_numbers(used)
        if batch == args.batch and args.only in ("all", "prefill"):
            prefill = time_prefill(engine, used)
        if args.only == "prefill":
            results[batch] = dict(ms_per_step=float("nan"), tokens_per_s=float("nan"),
                                  e2e_tokens_per_s=float("nan"), clocks=None, context=PROMPT_TOKENS,
                                  launches=0, h2d=0, d2h=0)
        else:
            results[batch] = time_decode(engine, used, batch, args.steps, args.warmup,
                                         sample_clocks=batch == args.batch)
        engine.close()
        del engine
        torch.cuda.empty_cache()
    main = results[args.batch]
    step_bytes = numbers["weight_bytes"] + args.batch * main["context"] * numbers["kv_bytes_per_token"]
    achieved = step_bytes / (main["ms_per_step"] / 1e3) / 1e9
    flops = prefill_flops(used, PROMPT_TOKENS, 1)
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
        "config": {
            "model": "Qwen2.5-3B shape", "layers": used["num_hidden_layers"], "layers_of_model": 36,
            "hidden": used["hidden_size"], "q_heads": used["num_attention_heads"],
            "kv_heads": used["num_key_value_heads"], "head_dim": numbers["head_dim"],
            "intermediate": used["intermediate_size"], "vocab": used["vocab_size"],
            "global_batch": args.batch, "seq_len": CONTEXT, "prompt_tokens": PROMPT_TOKENS,
            "page_size": PAGE, "parallelism": "single GPU", "cuda_graph_decode": True,
            "l2": "inputs larger than L2 (6.2 GB of weights per step)",
            "baseline": "reference 3B c=8 on L4: 178.986 tok/s",
        },
        "e2e": {"value": round(main["e2e_tokens_per_s"], 1), "unit": "tokens/s",
                "h2d_bytes_per_step": main["h2d"], "d2h_bytes_per_step": main["d2h"]},
        "gpu_launches": main["launches"],
        "prefill": {"value": round(PROMPT_TOKENS / (prefill["ms"] / 1e3), 1), "tokens": PROMPT_TOKENS,
                    "ms": round(prefill["ms"], 3),
                    "frac": round(flops / (prefill["ms"] / 1e3) / (peak["bf16_tflops"] * 1e12), 4)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peak["hbm_gbs"],
                     "unit": "GB/s", "frac": round(achieved / peak["hbm_gbs"], 4),
                     "peaks": peak["source"]},
        "points": {f"decode_b{b}{suffix}": round(results[b][key], digits)
                   for b in (1, 64) if b in results
                   for suffix, key, digits in (("", "tokens_per_s", 1), ("_ms", "ms_per_step", 4))},
        "clocks": main["clocks"],
    }
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

    print(json.dumps(run_reference_arm(args, QWEN25_3B, PROMPT_TOKENS, CONTEXT)))
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
    return run_own(args)


if __name__ == "__main__":
    raise SystemExit(main())
