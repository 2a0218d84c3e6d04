"""``cie``: the command line, with the reference's commands and option names.

The reference's ``cie`` is an HTTP client of a deployed server (src/cloud_engine/cli.py:53-66):
``cie [--url] [--api-key] {health | models | metrics | generate PROMPT [--model]
[--max-output-tokens 1..256, default 64] [--no-stream]}``, with ``ENGINE_MODEL`` as the default
of ``--model``.  Servers are outside this engine, so the same commands run in-process:
``--model`` (or ``ENGINE_MODEL``) is a model folder, ``PROMPT`` is a list of token ids
("5,17,3" or "5 17 3") because the tokenizer is outside this engine too, and the output is token
ids.  ``--url`` and ``--api-key`` are accepted and ignored so that existing invocations parse.

    cie generate "5,17,3" --model DIR --max-output-tokens 8
    cie generate "5 17 3" --model DIR --temperature 0.8 --seed 7 --no-stream
    cie generate "5 17 3" --random-config config.json --weights-seed 3   (random weights, no folder)
    cie models --model DIR        cie health        cie metrics --model DIR
    cie info [--model DIR]        (device, kernels, architectures, engine defaults in one report)
    cie random-model DIR --config config.json --seed 3     (writes config.json + model.safetensors)
    cie replay --model DIR --dtype float32 --out OUT --max-tokens 256 [--trace FILE]   (trace replay)
    cie bench [options of bench.py]                                    (the benchmark of the repository)
"""

from __future__ import annotations

import argparse
import json
import os
import sys
from typing import Any


def parse_token_ids(text: str) -> list[int]:
    parts = [piece for piece in text.replace(",", " ").split() if piece]
    try:
        return [int(piece) for piece in parts]
    except ValueError:
        raise SystemExit(f"cie: PROMPT must be token ids such as '5,17,3', got {text!r}") from None


def parser() -> argparse.ArgumentParser:
    cli = argparse.ArgumentParser(prog="cie", description=__doc__.split("\n\n")[0])
    cli.add_argument("--url", default=os.environ.get("ENGINE_URL"), help="ignored (no server)")
    cli.add_argument("--api-key", default=os.environ.get("ENGINE_API_KEY"), help="ignored (no server)")
    commands = cli.add_subparsers(dest="command", required=True)

    def engine_options(sub: argparse.ArgumentParser) -> None:
        sub.add_argument("--model", default=os.environ.get("ENGINE_MODEL"),
                         help="model folder (config.json + *.safetensors)")
        sub.add_argument("--random-config", default=None,
                         help="instead of --model: a config.json (path or JSON text) to draw random weights for")
        sub.add_argument("--weights-seed", type=int, default=0, help="seed of the random weights")
        sub.add_argument("--dtype", default="bfloat16", choices=("bfloat16", "float32"))
        sub.add_argument("--block-size", type=int, default=16)
        sub.add_argument("--kv-cache-blocks", type=int, default=None)
        sub.add_argument("--kv-cache-bytes", type=int, default=1 << 30)
        sub.add_argument("--max-batched-tokens", type=int, default=2048)
        sub.add_argument("--prefill-chunk-size", type=int, default=256)
        sub.add_argument("--max-active-sequences", type=int, default=16)
        sub.add_argument("--max-model-len", type=int, default=None)
        sub.add_argument("--no-cuda-graph-decode", action="store_true")

    commands.add_parser("health", help="check that the device and the kernels are usable")
    models = commands.add_parser("models", help="list registered architectures / describe a folder")
    models.add_argument("--model", default=os.environ.get("ENGINE_MODEL"))
    generate = commands.add_parser("generate", help="generate token ids")
    generate.add_argument("prompt", help="token ids, e.g. '5,17,3'")
    engine_options(generate)
    generate.add_argument("--max-output-tokens", type=int, default=64, choices=range(1, 257),
                          metavar="1..256")
    generate.add_argument("--no-stream", action="store_true")
    generate.add_argument("--temperature", type=float, default=0.0)
    generate.add_argument("--seed", type=int, default=0)
    generate.add_argument("--eos-token-id", type=int, default=None)
    metrics = commands.add_parser("metrics", help="print engine metrics as JSON")
    engine_options(metrics)
    info = commands.add_parser("info", help="device, kernels, architectures and engine defaults")
    info.add_argument("--model", default=os.environ.get("ENGINE_MODEL"))
    # their own options follow the command word and are handed on as they are
    commands.add_parser("replay", help="trace replay (the options of bin/trace_run)", add_help=False)
    commands.add_parser("bench", help="run the repository's bench.py", add_help=False)
    random_model = commands.add_parser("random-model", help="write a model folder with random weights")
    random_model.add_argument("folder")
    random_model.add_argument("--config", required=True, help="config.json to build from")
    random_model.add_argument("--seed", type=int, default=0)
    return cli


def _engine(args: argparse.Namespace, prompt_len: int = 1, max_output: int = 1) -> Any:
    from .. import InferenceEngine, build_config

    random_config = None
    if args.random_config:
        text = args.random_config
        if not text.lstrip().startswith("{"):
            with open(text, encoding="utf-8") as handle:
                text = handle.read()
        random_config = json.loads(text)
    elif not args.model:
        parser().error("--model, ENGINE_MODEL or --random-config is required")
    max_len = args.max_model_len or max(64, prompt_len + max_output)
    config = build_config(
        "ragged", dtype=args.dtype, block_size=args.block_size, kv_cache_blocks=args.kv_cache_blocks,
        kv_cache_bytes=args.kv_cache_bytes, max_batched_tokens=args.max_batched_tokens,
        prefill_chunk_size=args.prefill_chunk_size, max_active_sequences=args.max_active_sequences,
        max_model_len=max_len, max_output_tokens=max(256, max_output),
        cuda_graph_decode=not args.no_cuda_graph_decode,
    )
    if random_config is not None:
        return InferenceEngine(config, None, random_config=random_config, seed=args.weights_seed)
    return InferenceEngine(config, args.model)


def _health() -> tuple[dict[str, Any], dict[str, Any]]:
    import torch

    live = {"status": "ok"}
    ready: dict[str, Any] = {"cuda": torch.cuda.is_available()}
    if ready["cuda"]:
        from ..native.ops import Ops

        ready["device"] = torch.cuda.get_device_name(0)
        ready["capability"] = list(torch.cuda.get_device_capability(0))
        Ops("cuda:0", torch.bfloat16)
        ready["kernels"] = "built"
    ready["status"] = "ready" if ready["cuda"] else "no CUDA device"
    return live, ready


def _models(model: str | None) -> dict[str, Any]:
    from ..config.registry import registered_architectures, resolve_model

    listing: dict[str, Any] = {"architectures": list(registered_architectures())}
    if model:
        arch, config, _ = resolve_model(model)
        listing["model"] = {"folder": str(model), "architecture": arch.name, "config": config.to_dict()}
    return listing


def main(argv: list[str] | None = None) -> int:
    args, rest = parser().parse_known_args(argv)
    if rest and args.command not in ("replay", "bench"):
        parser().error("unrecognized arguments: " + " ".join(rest))
    args.rest = rest
    try:
        if args.command == "health":
            live, ready = _health()
            print(json.dumps({"liveness": live, "readiness": ready}, indent=2))
            return 0 if ready["cuda"] else 1
        if args.command == "models":
            print(json.dumps(_models(args.model), indent=2))
            return 0
        if args.command == "info":
            from dataclasses import asdict

            from .. import __version__, build_config

            live, ready = _health()
            print(json.dumps({"version": __version__, "liveness": live, "readiness": ready,
                              **_models(args.model), "engine_defaults": asdict(build_config("ragged"))}, indent=2))
            return 0
        if args.command == "replay":
            from .replay import main as replay_main

            return replay_main(args.rest)
        if args.command == "bench":
            import runpy
            from pathlib import Path

            script = Path(__file__).resolve().parents[2] / "bench.py"
            if not script.is_file():
                raise RuntimeError(f"bench.py is not beside the package ({script})")
            sys.argv = [str(script), *args.rest]
            runpy.run_path(str(script), run_name="__main__")
            return 0
        if args.command == "random-model":
            from ..weights.random_init import write_random_model

            with open(args.config, encoding="utf-8") as handle:
                config = json.load(handle)
            print(write_random_model(args.folder, config, args.seed))
            return 0
        if args.command == "metrics":
            with _engine(args) as engine:
                print(json.dumps(engine.snapshot_metrics(), indent=2, default=str))
            return 0
        # generate
        from .. import GenerationConfig

        prompt = parse_token_ids(args.prompt)
        with _engine(args, len(prompt), args.max_output_tokens) as engine:
            handle = engine.submit(
                prompt,
                GenerationConfig(max_output_tokens=args.max_output_tokens,
                                 temperature=args.temperature, eos_token_id=args.eos_token_id,
                                 seed=args.seed),
            )
            if args.no_stream:
                print(" ".join(str(t) for t in handle.wait().token_ids))
            else:
                for event in handle.stream():
                    if event.token_id is not None:
                        print(event.token_id, end=" ", flush=True)
                print()
    except (OSError, ValueError, KeyError, RuntimeError) as exc:
        print(f"cie: {type(exc).__name__}: {exc}", file=sys.stderr)
        return 1
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
