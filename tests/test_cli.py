"""The command line's parts that need no GPU: parsing, `cie info`, `cie bench` handing its options on,
`cie random-model`."""

import json
import subprocess
import sys
from pathlib import Path

from tiny_configs import TINY

ROOT = Path(__file__).resolve().parent.parent
CIE = [sys.executable, str(ROOT / "bin" / "cie")]


def run(*args, **kwargs):
    return subprocess.run([*CIE, *args], capture_output=True, text=True, timeout=300, **kwargs)


def test_info_reports_architectures_and_defaults(tmp_path):
    done = run("info")
    assert done.returncode == 0, done.stderr
    report = json.loads(done.stdout)
    assert "Qwen2ForCausalLM" in report["architectures"]
    assert report["engine_defaults"]["block_size"] == 16 and report["engine_defaults"]["prefill_chunk_size"] == 256
    assert "cuda" in report["readiness"]


def test_bench_and_replay_take_their_own_options():
    done = run("bench", "--gpus", "2")
    assert done.returncode == 2 and "one GPU" in done.stdout
    done = run("replay", "--help")
    assert done.returncode == 0 and "--max-tokens" in done.stdout and "--trace" in done.stdout


def test_unknown_options_are_refused_and_token_ids_are_checked():
    assert run("generate", "1,2", "--bogus").returncode == 2
    done = run("generate", "five", "--model", "nowhere")
    assert done.returncode != 0 and "token ids" in done.stderr


def test_random_model_writes_a_folder(tmp_path):
    config = tmp_path / "config.json"
    config.write_text(json.dumps(TINY["A"]))
    done = run("random-model", str(tmp_path / "m"), "--config", str(config), "--seed", "3")
    assert done.returncode == 0, done.stderr
    assert (tmp_path / "m" / "config.json").is_file() and (tmp_path / "m" / "model.safetensors").is_file()
    listing = json.loads(run("models", "--model", str(tmp_path / "m")).stdout)
    assert listing["model"]["architecture"] == "Qwen2ForCausalLM"
