"""Writes tests/golden/<name>.npz: logits of the reference project's own model code on the CPU.

Run once, by hand, where the reference's sources can be imported:

    python tests/golden/make_golden.py --reference-src /path/to/cloud-inference-from-scratch/src

For each tiny configuration of tests/tiny_configs.py it writes a random-weights model folder
with this framework's writer (same seed as the tests), loads those tensors into the
reference's ``cloud_engine.model.Qwen2CausalLM`` in float32 on the CPU (its module names are
the tensor names without the ``model.`` prefix, src/cloud_engine/weights.py:117-121), runs one
whole prompt with ``AttentionBackend(cache=None)`` and stores prompt and logits.  Configuration
C gives ``head_dim`` explicitly with hidden_size != heads * head_dim, which the reference cannot
express (model.py:66-75), so it has no golden.  tests/test_plain_model.py compares
tests/plain_model.py with these files; nothing else reads them.
"""

from __future__ import annotations

import argparse
import sys
import tempfile
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent))
sys.path.insert(0, str(HERE.parent.parent))


def main() -> int:
    parser = argparse.ArgumentParser()
    parser.add_argument("--reference-src", required=True)
    args = parser.parse_args()
    sys.path.insert(0, args.reference_src)
    from cloud_engine.attention import AttentionBackend  # type: ignore
    from cloud_engine.model import ModelDims, Qwen2CausalLM  # type: ignore
    from plain_model import read_model_folder
    from tiny_configs import SEED, TINY

    from cloud_inference_from_scratch_b200.weights import write_random_model

    lengths = {"A": 17, "B": 23, "D": 19}
    for name, length in lengths.items():
        config = TINY[name]
        with tempfile.TemporaryDirectory() as folder:
            write_random_model(folder, config, SEED[name])
            stored, weights = read_model_folder(folder)
        dims = ModelDims.from_hf_config(stored)
        backend = AttentionBackend(None, dims.num_heads, dims.num_kv_heads, dims.head_dim)
        model = Qwen2CausalLM(dims, backend, dtype=torch.float32, device="cpu")
        state = {key.removeprefix("model."): value for key, value in weights.items()}
        model.load_state_dict(state, strict=True)
        generator = torch.Generator().manual_seed(1000 + SEED[name])
        prompt = torch.randint(0, config["vocab_size"], (length,), generator=generator)
        with torch.no_grad():
            logits = model(prompt, ctx=None, return_all_logits=True)
        np.savez_compressed(
            HERE / f"{name}.npz",
            prompt=prompt.numpy().astype(np.int32),
            logits=logits.numpy().astype(np.float32),
        )
        print(name, tuple(logits.shape), float(logits.abs().max()))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
