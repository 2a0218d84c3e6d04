"""Trace replay: feeds given token ids through a model step by step and writes logits.

    bin/trace_run --model DIR --dtype bfloat16|float32 --out DIR --max-tokens N [--trace FILE]

(also ``cie replay`` with the same options).  Steps come on standard input (or from ``--trace``),
one JSON object a line:

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

A request is admitted the first time its id appears and gives its pages back when a step's
``end`` names it.  For a step in which something is wanted, ``DIR/<step>.f32`` holds the logits
at the wanted places, in the order of the entries and of ``want``, as little-endian float32
[wanted, vocab].  After every step the line ``done <step>`` is printed and flushed.

Nothing is sampled, and nothing here computes: the program drives the framework's own model,
step function, cache manager and kernels (``build_core``), the ones generation uses.  The cache
pool holds ``--max-tokens`` tokens (rounded up to whole pages), so pages are used again.

The reference has no such program; the nearest pieces are ``RaggedRunner.forward_plans``
(src/cloud_engine/engine.py:210-212, 448-458) and the logit capture of
experiments/sentinel_diagnostics.py:291-315.
"""

from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

PAGE_SIZE = 16
MAX_LIVE_REQUESTS = 8


def parse_args(argv: list[str] | None = None) -> argparse.Namespace:
    parser = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    parser.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    parser.add_argument("--dtype", required=True, choices=("bfloat16", "float32"))
    parser.add_argument("--out", required=True, help="folder for <step>.f32 files")
    parser.add_argument("--max-tokens", type=int, required=True,
                        help="most tokens live requests hold at any time (sizes the cache pool)")
    parser.add_argument("--trace", default=None, help="file with the steps (default: standard input)")
    parser.add_argument("--page-size", type=int, default=PAGE_SIZE)
    parser.add_argument("--device", default="cuda:0")
    return parser.parse_args(argv)


def main(argv: list[str] | None = None) -> int:
    args = parse_args(argv)
    if args.max_tokens < 1:
        print("trace_run: --max-tokens must be positive", file=sys.stderr)
        return 2
    out_dir = Path(args.out)
    out_dir.mkdir(parents=True, exist_ok=True)

    import numpy as np

    from .. import models, parts  # noqa: F401  (registries)
    from .core import build_core
    from .step import StepEntry

    page = args.page_size
    num_pages = -(-args.max_tokens // page)
    core = build_core(
        args.model, dtype=args.dtype, device=args.device, page_size=page, num_pages=num_pages,
        max_requests=MAX_LIVE_REQUESTS, max_model_len=max(page, num_pages * page),
    )
    step_fn = core.step
    live: set[str] = set()
    steps = open(args.trace, encoding="utf-8") if args.trace else sys.stdin
    while True:
        line = steps.readline()
        if not line:
            break
        line = line.strip()
        if not line:
            continue
        record = json.loads(line)
        step = record["step"]
        entries = []
        for item in record.get("entries", []):
            request_id = str(item["id"])
            if request_id not in live:
                step_fn.admit(request_id)
                live.add(request_id)
            entries.append(StepEntry(request_id, item["tokens"], want=item.get("want", [])))
        result = step_fn.run(entries)
        if result.logits is not None and result.rows:
            logits = result.logits.float().cpu().numpy().astype("<f4", copy=False)
            np.ascontiguousarray(logits).tofile(out_dir / f"{step}.f32")
        core.runtime.ops.check_errors()
        for request_id in record.get("end", []):
            request_id = str(request_id)
            step_fn.release(request_id)
            live.discard(request_id)
        print(f"done {step}", flush=True)
    return 0
