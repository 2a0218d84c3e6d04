"""Shared helpers of the GPU tests: sharpened weights, trace builders, comparisons."""

from __future__ import annotations

import random
from pathlib import Path

import numpy as np
import safetensors.torch
import torch

import plain_model

# Error measure of every logits comparison: max |logit difference| over a row, divided by the
# standard deviation of the reference logits of that request (how far apart the candidates for the
# next token lie; 0.15 to 0.7 for the test models).  A gate is about three times the worst error
# that honest rounding was measured to give for that model and kind of run (pytest prints the worst
# errors of a session at its end); a lost page or a mis-masked key moves logits by 0.3 to several
# standard deviations on the sharpened models.
GATES = {
    "float32": {
        "A": 1.6e-5, "A long": 2e-5, "A runner": 1e-5, "B": 6e-5, "B unsharpened": 8e-6, "B far key": 2.6e-4,
        "B runner": 3e-5, "C": 1e-5, "D": 6e-5, "D runner": 5e-5, "a part alone": 5e-6, "toy models": 5e-5,
        "toy routed": 7e-6, "toy sandwich": 3e-5, "3B sizes, 2 layers": 1.7e-4,
    },
    # bfloat16: products round their inputs to 8 bits of mantissa; the error grows with the number
    # of terms, layers and decoded tokens, and the largest of a vocabulary's worth of errors is
    # 4 to 5 times their standard deviation
    "bfloat16": {
        "A": 1.3e-1, "A long": 1.3e-1, "A runner": 1.2e-1, "B": 1.5e-1, "B unsharpened": 8e-2, "B runner": 1e-1,
        "C": 8.5e-2, "D": 1.2e-1, "D runner": 1.1e-1, "a part alone": 8e-2, "toy models": 1.2e-1, "toy sandwich": 1.5e-1,
        "3B sizes, 2 layers": 2.5e-1, "3B sizes, 36 layers": 4.5e-1,
    },
}
FP32_TOL = 6e-5   # where a test has no label of its own

WORST: dict[tuple[str, str], float] = {}    # (label, dtype) -> worst error seen in this session


def tolerance(dtype: str, label: str) -> float:
    return GATES[dtype][label]


def record(label: str, dtype: str, error: float) -> float:
    WORST[label, dtype] = max(WORST.get((label, dtype), 0.0), float(error))
    return error


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
    """Largest |difference| in units of the reference's standard deviation."""
    return float(np.abs(got - ref).max() / float(ref.std()))


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


def trace_mixed(requests: dict[str, list[int]], seed: int, live_limit: int = 4,
                interrupt: str | None = None) -> list[dict]:
    """Up to ``live_limit`` live requests; each step takes, for a random subset of them, a portion
    of the prompt part (first two thirds) or single tokens (last third) of each; requests that
    finish end at once and the next one starts, so freed pages are taken again.

    ``interrupt`` names a request that is ended half-way (its pages go back) and later fed again
    from its first token under the id ``<id>@again``: a release followed by a full recompute."""
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
            elif rid == interrupt and live[rid][1] >= len(toks) // 2:
                ended.append(rid)
                pending.insert(min(1, len(pending)), (rid + "@again", toks))
        for rid in ended:
            del live[rid]
        steps.append({"step": len(steps), "entries": entries, "end": ended})
    return steps


def requests_in(steps: list[dict]) -> dict[str, list[int]]:
    """The token sequence every request id of a trace was fed, in the order of the steps."""
    fed: dict[str, list[int]] = {}
    for step in steps:
        for entry in step["entries"]:
            fed.setdefault(entry["id"], []).extend(entry["tokens"])
    return fed


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


def check_against_plain(model_dir, requests, got, dtype, label, schedule=None, window=0) -> float:
    """Every row of ``got`` against the plain model run on the whole request, under the gate of
    (``dtype``, ``label``); returns the worst error (in standard deviations of the request's
    reference logits)."""
    config, weights = plain_model.read_model_folder(model_dir)
    gate = tolerance(dtype, label)
    worst = 0.0
    known: dict[tuple, np.ndarray] = {}
    for rid, toks in requests.items():
        key = tuple(toks)
        prefix = next((ref for seen, ref in known.items() if seen[:len(key)] == key), None)
        if prefix is None:
            prefix = plain_model.forward(config, weights, toks, schedule=schedule, window=window).numpy()
            known[key] = prefix
        ref = prefix[:len(toks)]
        assert sorted(got[rid]) == list(range(len(toks))), f"request {rid}: positions missing"
        mine = np.stack([got[rid][p] for p in range(len(toks))])
        errors = np.abs(mine - ref).max(axis=1) / float(ref.std())
        worst = max(worst, float(errors.max()))
        record(label, dtype, worst)
        assert errors.max() <= gate, (
            f"request {rid}: first wrong position {int(np.argmax(errors > gate))} of {len(toks)}, "
            f"error {errors.max():.3e} > {gate:.1e}"
        )
    return worst


def check_trace_rows(folder, requests, trace, dtype, label):
    """The logit trace of an ``EngineRunner`` (``trace``: (request ids, positions, numpy rows) per
    step) against the plain model run on every request's final sequence.  ``requests``: request id
    -> (prompt + generated tokens, prompt length, finish reason).  Every sampled row must be there,
    be within the gate, and have the token the engine went on with as its (lowest) argmax."""
    config, weights = plain_model.read_model_folder(folder)
    reference = {rid: plain_model.forward(config, weights, tokens).numpy() for rid, (tokens, _, _) in requests.items()}
    seen = {rid: set() for rid in requests}
    worst = 0.0
    for ids, positions, logits in trace:
        for row, (rid, position) in enumerate(zip(ids, positions)):
            tokens, prompt_len, _ = requests[rid]
            ref = reference[rid]
            error = float(np.abs(logits[row] - ref[position]).max() / ref.std())
            worst = max(worst, error)
            assert error <= tolerance(dtype, label), (rid, position, error)
            # the token the engine went on with is the (lowest) argmax of the row it sampled from
            assert tokens[position + 1] == int(np.argmax(logits[row])), (rid, position)
            seen[rid].add(position)
    for rid, (tokens, prompt_len, _) in requests.items():
        assert seen[rid] == set(range(prompt_len - 1, len(tokens) - 1)), f"{rid}: rows missing from the trace"
    record(label, dtype, worst)
