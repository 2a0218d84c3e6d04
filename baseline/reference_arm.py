"""The reference arm of bench.py: the unmodified reference project, installed under baseline/_ref,
driven through its own public API for the same metric and model shape.

Install (once, offline, from a writable copy of the reference's source tree):

    python -m pip install --no-index --no-build-isolation --find-links <wheel folder> \
        --target baseline/_ref <copy of the reference>

What runs is the reference's stock path: ``cloud_engine.config.build_config("ragged", pinned, ...)``,
``cloud_engine.engine.InferenceEngine(config, model_dir)``, ``await engine.start()`` (its loader, its
paged cache, its Triton attention kernel, its CUDA-graph decode), ``engine.scheduler.submit(label,
token_ids, GenerationConfig)`` and ``RequestHandle.stream()``, exactly as its own
experiments/controlled.py drives token-id workloads.  Nothing of this repository's engine is on that path.

What this file prepares is input data only: a model folder with random float16 weights whose names and
shapes come from the reference's own ``expected_tensors``, a minimal tokenizer file (the reference loads a
tokenizer at start-up although token ids are submitted directly), and the reference's pinned settings
(the values of its engine_config.json, which is not part of the installed package).  The reference pins
float16 and at most 4,096 tokens of context; both fit the benchmark configuration.

Timing: the reference has no step function to call; decode steps are counted by the tokens its streams
deliver.  After every request has produced its first token and W more (warm-up), the wall-clock time until
every request has produced K more tokens is taken, with a device synchronize on both sides.
"""

from __future__ import annotations

import asyncio
import json
import sys
import tempfile
import time
from pathlib import Path
from typing import Any

REF = Path(__file__).resolve().parent / "_ref"

# the reference's engine_config.json values (model: Qwen2.5-3B in "ragged" mode)
PINNED = {
    "model": {"id": "Qwen/Qwen2.5-0.5B", "revision": "random", "dtype": "float16", "max_model_len": 2048,
              "max_output_tokens": 256, "eos_token_id": 151643},
    "ragged_model": {"id": "Qwen/Qwen2.5-3B", "revision": "random", "dtype": "float16", "max_model_len": 4096,
                     "max_output_tokens": 256, "eos_token_id": 151643},
    "scheduler": {"max_active_sequences": 16, "max_queue_size": 64, "max_batched_tokens": 2048,
                  "prefill_chunk_size": 256, "cuda_graph_decode": True, "queue_timeout_seconds": 60,
                  "stream_queue_capacity": 32, "slow_consumer_timeout_seconds": 10},
    "kv_cache": {"block_size": 16, "bytes": 4294967296, "prefix_cache_max_blocks": 256},
}


def _write_model_folder(folder: Path, model_config: dict) -> None:
    import safetensors.torch
    import torch
    from cloud_engine.model import ModelDims  # type: ignore
    from cloud_engine.weights import expected_tensors  # type: ignore
    from tokenizers import Tokenizer, models, pre_tokenizers

    folder.mkdir(parents=True, exist_ok=True)
    (folder / "config.json").write_text(json.dumps(model_config))
    dims = ModelDims.from_hf_config(model_config)
    generator = torch.Generator(device="cuda").manual_seed(0)
    tensors = {}
    for name, shape in expected_tensors(dims).items():
        values = torch.empty(shape, dtype=torch.float32, device="cuda").normal_(0.0, 0.02, generator=generator)
        if name.endswith("norm.weight") or name.endswith("layernorm.weight"):
            values += 1.0
        tensors[name] = values.to(torch.float16).cpu()
    safetensors.torch.save_file(tensors, str(folder / "model.safetensors"))
    vocab = {"<unk>": 0, "a": 1, "b": 2}
    tokenizer = Tokenizer(models.WordLevel(vocab, unk_token="<unk>"))
    tokenizer.pre_tokenizer = pre_tokenizers.Whitespace()
    tokenizer.save(str(folder / "tokenizer.json"))
    (folder / "tokenizer_config.json").write_text(json.dumps(
        {"tokenizer_class": "PreTrainedTokenizerFast", "unk_token": "<unk>"}))


async def _decode_rate(engine: Any, batch: int, prompt_tokens: int, steps: int, warmup: int, vocab: int,
                       seed: int) -> dict:
    import numpy as np
    import torch
    from cloud_engine.engine import RequestHandle  # type: ignore
    from cloud_engine.scheduler import GenerationConfig  # type: ignore

    rng = np.random.default_rng(seed)
    total = 1 + warmup + steps
    counts = [0] * batch
    marks: dict[str, float] = {}

    def check() -> None:
        low = min(counts)
        if low >= 1 + warmup and "start" not in marks:
            torch.cuda.synchronize()
            marks["start"] = time.perf_counter()
            marks["start_tokens"] = sum(counts)
        if low >= total and "stop" not in marks:
            torch.cuda.synchronize()
            marks["stop"] = time.perf_counter()
            marks["stop_tokens"] = sum(counts)

    async def drive(index: int) -> None:
        request = await engine.scheduler.submit(
            f"bench-{batch}-{index}", rng.integers(0, vocab, prompt_tokens).tolist(),
            GenerationConfig(max_output_tokens=total, temperature=0, eos_token_id=None))
        async for _event in RequestHandle(request, engine).stream():
            counts[index] += 1
            check()

    await asyncio.gather(*(drive(index) for index in range(batch)))
    seconds = marks["stop"] - marks["start"]
    tokens = marks["stop_tokens"] - marks["start_tokens"]
    return {"tokens_per_s": tokens / seconds, "ms_per_step": seconds / steps * 1e3}


async def _prefill_rate(engine: Any, prompt_tokens: int, vocab: int) -> dict:
    import numpy as np
    import torch
    from cloud_engine.engine import RequestHandle  # type: ignore
    from cloud_engine.scheduler import GenerationConfig  # type: ignore

    rng = np.random.default_rng(99)
    times = []
    for _ in range(3):
        torch.cuda.synchronize()
        started = time.perf_counter()
        request = await engine.scheduler.submit(
            "prefill", rng.integers(0, vocab, prompt_tokens).tolist(),
            GenerationConfig(max_output_tokens=1, temperature=0, eos_token_id=None))
        async for _event in RequestHandle(request, engine).stream():
            pass
        torch.cuda.synchronize()
        times.append(time.perf_counter() - started)
    best = sorted(times)[len(times) // 2]
    return {"ms": best * 1e3, "tokens_per_s": prompt_tokens / best}


def run(args: Any, model_config: dict, prompt_tokens: int, context: int, config_record: dict | None = None) -> dict:
    if not (REF / "cloud_engine").is_dir():
        return {"impl": "reference",
                "unavailable": "baseline/_ref/cloud_engine is not installed on this machine (see baseline/reference_arm.py)"}
    try:
        import torch

        if not torch.cuda.is_available():
            return {"impl": "reference", "unavailable": "no CUDA device"}
        sys.path.insert(0, str(REF))
        from cloud_engine.config import build_config  # type: ignore
        from cloud_engine.engine import InferenceEngine  # type: ignore
    except Exception as exc:  # noqa: BLE001
        return {"impl": "reference", "unavailable": f"the reference cannot be imported: {type(exc).__name__}: {exc}"}

    config_json = dict(model_config)
    config_json.pop("use_sliding_window", None)
    if getattr(args, "layers", None):
        config_json["num_hidden_layers"] = args.layers
    results: dict[int, dict] = {}
    prefill = None
    with tempfile.TemporaryDirectory() as tmp:
        folder = Path(tmp) / "model"
        try:
            _write_model_folder(folder, config_json)
            for batch in (args.batch, 1, 64):
                if batch in results:
                    continue
                config = build_config(
                    "ragged", PINNED, max_active_sequences=max(16, batch), max_queue_size=max(64, batch),
                    kv_cache_bytes=(batch * context + 4096) * 2 * 2 * config_json["num_key_value_heads"]
                    * (config_json["hidden_size"] // config_json["num_attention_heads"]) * config_json["num_hidden_layers"],
                    prefix_cache_max_blocks=0,
                )
                engine = InferenceEngine(config, model_dir=str(folder))

                async def go(engine: Any = engine, batch: int = batch) -> tuple[dict, dict | None]:
                    await engine.start()
                    try:
                        first = None
                        if batch == args.batch:
                            first = await _prefill_rate(engine, prompt_tokens, config_json["vocab_size"])
                        rate = await _decode_rate(engine, batch, prompt_tokens, args.steps, args.warmup,
                                                  config_json["vocab_size"], seed=batch)
                        return rate, first
                    finally:
                        await engine.close()

                rate, first = asyncio.run(go())
                results[batch] = rate
                if first is not None:
                    prefill = first
                del engine
                torch.cuda.empty_cache()
        except Exception as exc:  # noqa: BLE001
            return {"impl": "reference",
                    "unavailable": f"the reference failed on this machine: {type(exc).__name__}: {str(exc)[:300]}"}
    main = results[args.batch]
    return {
        "impl": "reference",
        "metric": "decode tok/s (Qwen2.5-3B shape, batch 8, context 2048+)",
        "value": round(main["tokens_per_s"], 1),
        "unit": "tokens/s",
        "n_gpus": 1,
        "steps": args.steps,
        "warmup": args.warmup,
        "ms_per_step": round(main["ms_per_step"], 4),
        "higher_is_better": True,
        "scaling": "weak",
        "vs_baseline": round(main["tokens_per_s"] / 178.986, 2),
        "dtype": "fp16",
        "data": "synthetic: random N(0,0.02) weights, uniform random token ids",
        # the same keys and values as the own arm's line (same model shape, batch, prompt and context)
        "config": dict(config_record) if config_record else {
            "model": "Qwen2.5-3B shape", "layers": config_json["num_hidden_layers"], "layers_of_model": 36,
            "global_batch": args.batch, "seq_len": context, "prompt_tokens": prompt_tokens, "page_size": 16,
            "parallelism": "single GPU"},
        "timing": "wall clock over streamed tokens, device synchronised; prompt portions of 256 tokens (its stock setting)",
        "e2e": {"value": round(main["tokens_per_s"], 1), "unit": "tokens/s"},
        "prefill": {"value": round(prefill["tokens_per_s"], 1), "tokens": prompt_tokens, "ms": round(prefill["ms"], 3)}
        if prefill else None,
        "points": {f"decode_b{b}": round(results[b]["tokens_per_s"], 1) for b in (1, 64) if b in results},
    }
