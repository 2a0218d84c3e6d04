"""Random-weights mode: writes a model folder (config.json, model.safetensors) from a
configuration and a seed.  The reference has no counterpart (its modules start from
``torch.empty``, src/cloud_engine/model.py:152,159-160); the distributions are the ones the
benchmark configurations name: weights and biases N(0, 0.02), norm gains 1 + N(0, 0.02).
"""

from __future__ import annotations

import json
from pathlib import Path
from typing import Any

from ..config.registry import resolve_config
from .source import RandomSource


def write_random_model(
    model_dir: str | Path,
    config: dict[str, Any],
    seed: int,
    std: float = 0.02,
    store_dtype: str = "bfloat16",
    vector_dtype: str | None = None,
    scales: dict[str, float] | None = None,
) -> Path:
    """``config`` is a config.json dictionary of a registered architecture."""
    import safetensors.torch

    from ..models.decoder import DecoderModel

    model_dir = Path(model_dir)
    model_dir.mkdir(parents=True, exist_ok=True)
    _, typed, spec = resolve_config(config)
    table = DecoderModel(spec).tensor_table()
    source = RandomSource(table, seed, std=std, store_dtype=store_dtype, vector_dtype=vector_dtype,
                          scales=scales)
    tensors = {name: source.get(name).contiguous() for name in source.names()}
    stored = typed.to_dict() if hasattr(typed, "to_dict") else dict(config)
    stored["torch_dtype"] = store_dtype
    with open(model_dir / "config.json", "w", encoding="utf-8") as handle:
        json.dump(stored, handle, indent=2)
    safetensors.torch.save_file(tensors, str(model_dir / "model.safetensors"))
    return model_dir
