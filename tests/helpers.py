"""Shared helpers of the GPU tests: sharpened weights, trace builders, comparisons."""

from __future__ import annotations

import random
from pathlib import Path

import numpy as np
import safetensors.torch
import torch

import plain_model

FP32_TOL = 2e-5   # max |logit difference| / max(1, max |reference logit|), 32-bit path
BF16_TOL = 2e-2   # same measure, bfloat16 path (the reference's own gate for float16 is 2e-2)


def sharpen(source: Path, target: Path, score_std: float = 3.0, vo: float = 1.5,
            qk: float | None = None) -> Path:
    """Copies a model folder with the q/k projections scaled so that attention scores have a
    standard deviation of about ``score_std`` (or by ``qk`` directly), and v/o scaled by ``vo``.

    With N(0, 0.02) weights and a normalised input, q and k elements have variance
    0.0004 * hidden, so a score (q.k / sqrt(D)) has a standard deviation of 0.0004 * hidden:
    close to zero, every softmax close to uniform, and a wrong or missing key changes almost
    nothing.  Scaled so, scores spread over several units and single keys stand out."""
    import json

    target.mkdir(parents=True, exist_ok=True)
    (target / "config.json").write_text((source / "config.json").read_text())
    hidden = json.loads((source / "config.json").read_text())["hidden_size"]
    if qk is None:
        qk = (score_std / (0.0004 * hidden)) ** 0.5
    tensors = safetensors.torch.load_file(str(source / "model.safetensors"))
    for name in list(tensors):
        if ".q_proj." in name or ".k_proj." in name:
            tensors[name] = (tensors[name].float() * qk).to(tensors[name].dtype)
        elif ".v_proj." in name or ".o_proj." in name:
            tensors[name] = (tensors[name].float() * vo).to(tensors[name].dtype)
    safetensors.torch.save_file(tensors, str(target / "model.safetensors"))
    return target


def random_tokens(vocab: int, length: int, seed: int) -> list[int]:
    generator = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (length,), generator=generator).tolist()


def relative_error(got: np.ndarray, ref: np.ndarray) -> float:
    return float(np.abs(got - ref).max() / max(1.0, float(np.abs(ref).max())))


# ---------------------------------------------------------------------------- traces
def trace_whole(requests: dict[str, list[int]]) -> list[dict]:
    return [
        {"step": i, "entries": [{"id": rid, "tokens": toks, "want": list(range(len(toks)))}],
         "end": [rid]}
        for i, (rid, toks) in enumerate(requests.items())
    ]


def trace_tail(requests: dict[str, list[int]], tail: int = 32) -> list[dict]:
    steps: list[dict] = []
    for rid, toks in requests.items():
        head = max(1, len(toks) - tail)
        steps.append({"step": len(steps),
                      "entries": [{"id": rid, "tokens": toks[:head], "want": list(range(head))}],
                      "end": []})
        for index in range(head, len(toks)):
            steps.append({"step": len(steps),
                          "entries": [{"id": rid, "tokens": [toks[index]], "want": [0]}],
                          "end": [rid] if index == len(toks) - 1 else []})
        if head == len(toks):
            steps[-1]["end"] = [rid]
    return steps


def trace_portions(requests: dict[str, list[int]], sizes=(7, 2, 13, 3, 2, 16, 5, 2, 31, 4, 2, 9)) -> list[dict]:
    steps: list[dict] = []
    for offset, (rid, toks) in enumerate(requests.items()):
        position, turn = 0, offset
        while position < len(toks):
            size = min(sizes[turn % len(sizes)], len(toks) - position)
            if len(toks) - position - size == 1:  # never leave a single token: portions are >= 2
                size += 1
            chunk = toks[position:position + size]
            position += size
            steps.append({"step": len(steps),
                          "entries": [{"id": rid, "tokens": chunk, "want": list(range(len(chunk)))}],
                          "end": [rid] if position == len(toks) else []})
            turn += 1
    return steps


def trace_mixed(requests: dict[str, list[int]], seed: int, live_limit: int = 4) -> list[dict]:
    """Up to ``live_limit`` live requests; each step takes, for a random subset of them, a portion
    of the prompt part (first two thirds) or single tokens (last third) of each; requests that
    finish end at once and the next one starts, so freed pages are taken again."""
    rng = random.Random(seed)
    pending = list(requests.items())
    live: dict[str, list] = {}
    steps: list[dict] = []
    while pending or live:
        while pending and len(live) < live_limit:
            rid, toks = pending.pop(0)
            live[rid] = [toks, 0]
        chosen = [rid for rid in live if rng.random() < 0.8] or [next(iter(live))]
        entries, ended = [], []
        for rid in chosen:
            toks, position = live[rid]
            left = len(toks) - position
            if position >= (2 * len(toks)) // 3:
                size = 1
            else:
                size = min(left, rng.choice([2, 2, 3, 5, 8, 13, 21]))
                if left - size == 1 and size > 1:
                    size += 1
            chunk = toks[position:position + size]
            live[rid][1] = position + size
            entries.append({"id": rid, "tokens": chunk, "want": list(range(len(chunk)))})
            if live[rid][1] == len(toks):
                ended.append(rid)
        for rid in ended:
            del live[rid]
        steps.append({"step": len(steps), "entries": entries, "end": ended})
    return steps


def peak_tokens(steps: list[dict], round_to: int = 64) -> int:
    """The most tokens live requests hold at any time, each rounded up to ``round_to``."""
    held: dict[str, int] = {}
    peak = 0
    for step in steps:
        for entry in step["entries"]:
            held[entry["id"]] = held.get(entry["id"], 0) + len(entry["tokens"])
        peak = max(peak, sum(-(-n // round_to) * round_to for n in held.values()))
        for rid in step["end"]:
            held.pop(rid, None)
    return peak


def replay(core, steps: list[dict]) -> dict[str, dict[int, np.ndarray]]:
    """Runs a trace through the engine's step function (what bin/trace_run does) and returns
    logits by request id and absolute position."""
    from cloud_inference_from_scratch_b200.engine.step import StepEntry

    out: dict[str, dict[int, np.ndarray]] = {}
    position: dict[str, int] = {}
    live: set[str] = set()
    for step in steps:
        entries = []
        for item in step["entries"]:
            if item["id"] not in live:
                core.step.admit(item["id"])
                live.add(item["id"])
                position.setdefault(item["id"], 0)
            entries.append(StepEntry(item["id"], item["tokens"], want=item["want"]))
        result = core.step.run(entries)
        if result.logits is not None and result.rows:
            logits = result.logits.float().cpu().numpy()
            starts = {item["id"]: position[item["id"]] for item in step["entries"]}
            for row, (rid, place) in enumerate(result.rows):
                out.setdefault(rid, {})[starts[rid] + place] = logits[row].copy()
        core.runtime.ops.check_errors()
        for item in step["entries"]:
            position[item["id"]] += len(item["tokens"])
        for rid in step["end"]:
            core.step.release(rid)
            live.discard(rid)
            position.pop(rid, None)
    core.cache.assert_invariants()
    return out


def check_against_plain(model_dir, requests, got, tolerance, schedule=None, window=0) -> float:
    config, weights = plain_model.read_model_folder(model_dir)
    worst = 0.0
    for rid, toks in requests.items():
        ref = plain_model.forward(config, weights, toks, schedule=schedule, window=window).numpy()
        assert sorted(got[rid]) == list(range(len(toks))), f"request {rid}: positions missing"
        mine = np.stack([got[rid][p] for p in range(len(toks))])
        errors = np.abs(mine - ref).max(axis=1) / max(1.0, float(np.abs(ref).max()))
        worst = max(worst, float(errors.max()))
        assert errors.max() <= tolerance, (
            f"request {rid}: first wrong position {int(np.argmax(errors > tolerance))} of {len(toks)}, "
            f"error {errors.max():.3e} > {tolerance:.1e}"
        )
    return worst
