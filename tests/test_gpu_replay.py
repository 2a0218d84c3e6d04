"""Replay of the same requests in four ways of cutting, in 32-bit and in bfloat16, against the
plain implementation: whole; most in one step and the last 32 tokens one by one; portions of
changing size down to two tokens; mixed with other requests with so few pages that they are
used again.  Also long decoding, the first tokens of a sequence, and bin/trace_run itself."""

import json
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest

import plain_model
from helpers import (
    FP32_TOL, check_against_plain, peak_tokens, random_tokens, replay, requests_in, sharpen,
    trace_mixed, trace_portions, trace_tail, trace_whole,
)
from tiny_configs import PAGE_SIZE, TINY

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent
LENGTHS = {"A": (5, 11, 17, 70, 129, 48), "B": (1, 9, 23, 40, 97, 64), "C": (33, 16, 2, 81, 50),
           "D": (19, 65, 128, 37, 3)}


def make_requests(name):
    vocab = TINY[name]["vocab_size"]
    return {f"{name}{i}": random_tokens(vocab, n, 100 * i + n) for i, n in enumerate(LENGTHS[name])}


def make_core(folder, name, dtype, tokens):
    from cloud_inference_from_scratch_b200.engine.core import build_core

    page = PAGE_SIZE[name]
    return build_core(folder, dtype=dtype, page_size=page, num_pages=-(-tokens // page),
                      max_requests=4, max_model_len=max(256, tokens))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_four_cuttings_match_the_plain_model(sharp_models, name, dtype):
    requests = make_requests(name)
    interrupted = max(requests, key=lambda rid: len(requests[rid]))
    traces = {
        "whole": trace_whole(requests),
        "tail32": trace_tail(requests, 32),
        "portions": trace_portions(requests),
        # one request is ended half-way (pages given back) and fed again from its first token
        "mixed": trace_mixed(requests, seed=7, interrupt=interrupted),
    }
    assert interrupted + "@again" in requests_in(traces["mixed"])
    results = {}
    for kind, steps in traces.items():
        # a pool just large enough for the trace, so that freed pages are taken again
        core = make_core(sharp_models.get(name, dtype), name, dtype, peak_tokens(steps, PAGE_SIZE[name]))
        total_pages = core.cache.total_pages()
        got = replay(core, steps)
        results[kind] = got
        check_against_plain(sharp_models.get(name, dtype), requests_in(steps), got, dtype, name)
        assert core.cache.free_pages() == total_pages, f"{kind}: pages were not all given back"
        assert core.cache.groups[0].allocator.allocations_total > total_pages, f"{kind}: no page reused"
    if dtype == "float32":
        # the 32-bit kernels sum in an order that does not depend on the cut: bit-equal logits,
        # also for the request that was released and computed again
        for kind in ("tail32", "portions", "mixed"):
            for rid, rows in results[kind].items():
                for position, row in rows.items():
                    assert np.array_equal(row, results["whole"][rid.split("@")[0]][position]), (kind, rid, position)
        assert len(results["mixed"][interrupted + "@again"]) == len(requests[interrupted])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_unsharpened_weights_too(tiny_models, dtype):
    requests = make_requests("B")
    core = make_core(tiny_models["B"], "B", dtype, 512)
    check_against_plain(tiny_models["B"], requests, replay(core, trace_mixed(requests, seed=3)), dtype, "B unsharpened")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_one_token_at_a_time(sharp_models, dtype):
    tokens = random_tokens(TINY["A"]["vocab_size"], 300, 5)
    requests = {"long": tokens}
    core = make_core(sharp_models.get("A", dtype), "A", dtype, 320)
    got = replay(core, trace_tail(requests, tail=296))
    check_against_plain(sharp_models.get("A", dtype), requests, got, dtype, "A long")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_first_tokens_of_a_sequence(sharp_models, name, dtype):
    vocab = TINY[name]["vocab_size"]
    requests = {"one": random_tokens(vocab, 1, 1), "two": random_tokens(vocab, 2, 2),
                "three": random_tokens(vocab, 3, 3)}
    core = make_core(sharp_models.get(name, dtype), name, dtype, 256)
    check_against_plain(sharp_models.get(name, dtype), requests, replay(core, trace_whole(requests)), dtype, name)
    single = trace_tail({"s": random_tokens(vocab, 6, 4)}, tail=5)   # every token on its own
    check_against_plain(sharp_models.get(name, dtype), {"s": random_tokens(vocab, 6, 4)}, replay(core, single), dtype, name)


def test_a_far_key_among_hundreds_is_found(tiny_models, tmp_path):
    """One early token is made a key the late queries care about: if attention lost or misplaced
    a page, the logits of the last position would change by far more than the gate.  (The
    bfloat16 kernels get the same treatment alone, with a planted key, in test_gpu_kernels.)"""
    folder = sharpen(tiny_models["B"], tmp_path / "peaky", score_std=6.0, vo=3.0)
    config, weights = plain_model.read_model_folder(folder)
    tokens = random_tokens(TINY["B"]["vocab_size"], 400, 9)
    ref = plain_model.forward(config, weights, tokens)
    altered = list(tokens)
    altered[37] = (altered[37] + 1) % TINY["B"]["vocab_size"]
    assert (plain_model.forward(config, weights, altered)[-1] - ref[-1]).abs().max() > 100 * FP32_TOL
    core = make_core(folder, "B", "float32", 448)
    got = replay(core, trace_portions({"far": tokens}, sizes=(100, 2, 57, 8)))
    check_against_plain(folder, {"far": tokens}, got, "float32", "B far key")


def test_page_running_out_is_a_host_error_that_changes_nothing(tiny_models):
    from cloud_inference_from_scratch_b200.cache import CacheCapacityFull
    from cloud_inference_from_scratch_b200.engine.step import StepEntry

    core = make_core(tiny_models["A"], "A", "float32", 16)   # 4 pages of 4 tokens
    core.step.admit("a"), core.step.admit("b")
    core.step.run([StepEntry("a", list(range(9)))])
    with pytest.raises(CacheCapacityFull):
        core.step.run([StepEntry("a", [1]), StepEntry("b", list(range(5)))])
    assert core.cache.committed_length("a") == 9 and core.cache.committed_length("b") == 0
    core.cache.assert_invariants()
    with pytest.raises(ValueError, match="position"):
        core.step.run([StepEntry("a", [1], start_pos=3)])
    with pytest.raises(ValueError, match="twice"):
        core.step.run([StepEntry("a", [1]), StepEntry("a", [2])])
    with pytest.raises(ValueError, match="vocabulary"):
        core.step.run([StepEntry("a", [512])])
    core.step.release("a"), core.step.release("b")
    assert core.cache.free_pages() == core.cache.total_pages()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run_program(sharp_models, tmp_path, dtype):
    """bin/trace_run as a user starts it: JSON lines on stdin, <step>.f32 files, 'done <step>'."""
    requests = {f"r{i}": random_tokens(TINY["B"]["vocab_size"], n, 40 + i) for i, n in enumerate((70, 33, 90, 12, 55))}
    steps = trace_mixed(requests, seed=11)
    out = tmp_path / "out"
    text = "\n".join(json.dumps(step) for step in steps) + "\n"
    done = subprocess.run(
        [sys.executable, str(ROOT / "bin" / "trace_run"), "--model", str(sharp_models.get("B", dtype)),
         "--dtype", dtype, "--out", str(out), "--max-tokens", str(peak_tokens(steps))],
        input=text, capture_output=True, text=True, timeout=600,
    )
    assert done.returncode == 0, done.stderr[-2000:]
    assert done.stdout.split("\n")[:-1] == [f"done {step['step']}" for step in steps]
    vocab = TINY["B"]["vocab_size"]
    got: dict[str, dict[int, np.ndarray]] = {}
    position = {rid: 0 for rid in requests}
    for step in steps:
        wanted = sum(len(entry["want"]) for entry in step["entries"])
        logits = np.fromfile(out / f"{step['step']}.f32", dtype="<f4").reshape(wanted, vocab)
        row = 0
        for entry in step["entries"]:
            for place in entry["want"]:
                got.setdefault(entry["id"], {})[position[entry["id"]] + place] = logits[row]
                row += 1
            position[entry["id"]] += len(entry["tokens"])
    check_against_plain(sharp_models.get("B", dtype), requests, got, dtype, "B")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["B", "D"])
def test_steps_from_captured_graphs_give_the_same_logits(sharp_models, name, dtype):
    """With graphs on, a shape of step that comes by again runs from its captured graph: the tail
    of single tokens, the repeated portions and the mixed trace all repeat shapes while contexts,
    pages and token ids change.  The logits must be those of the launches one by one, bit for bit."""
    requests = make_requests(name)
    for steps in (trace_tail(requests, 32), trace_portions(requests, sizes=(7, 7, 7, 7, 2, 2, 2, 16, 16, 16, 5)),
                  trace_mixed(requests, seed=3)):
        tokens = peak_tokens(steps, PAGE_SIZE[name])
        core = make_core(sharp_models.get(name, dtype), name, dtype, tokens)
        core.step.enable_graphs(core.max_model_len)
        graphed = replay(core, steps)
        # launch by launch with block tables of the same width (the decode kernel cuts the keys of
        # a request into as many parts as the table's width allows, and the order of a sum shows)
        one_by_one = make_core(sharp_models.get(name, dtype), name, dtype, tokens)
        one_by_one.step.fixed_table_width = core.step.fixed_table_width
        plain = replay(one_by_one, steps)
        assert core.step.graph_captures > 0 and core.step.graph_replays > 0
        assert graphed.keys() == plain.keys()
        for rid in plain:
            assert graphed[rid].keys() == plain[rid].keys()
            for position, want in plain[rid].items():
                assert np.array_equal(graphed[rid][position], want), (rid, position)
