"""Engine (scheduler and cache) configuration, with the reference's option names.

Parity: ``EngineConfig`` / ``build_config`` / ``validate_config`` / ``with_overrides`` in
src/cloud_engine/config.py:24-150 and the pinned values of engine_config.json:26-40
(16 active sequences, queue of 64, 2048 batched tokens, 256-token prefill portions,
CUDA-graph decode, 16-token blocks, 4 GiB of cache).  What is dropped: the six modes
(only the packed "ragged" engine exists here), float16, quantization, prefix reuse,
stream queues.  What is added: ``dtype`` is "bfloat16" or "float32", ``block_size`` is
free, ``kv_cache_blocks`` can fix the page count directly, and ``max_model_len`` may
go up to what the model's position range allows.
"""

from __future__ import annotations

from dataclasses import dataclass, fields, replace
from typing import Any

DTYPES = ("bfloat16", "float32")

_DEFAULTS: dict[str, Any] = dict(
    mode="ragged",
    dtype="bfloat16",
    max_model_len=4096,
    max_output_tokens=256,
    eos_token_id=None,
    max_active_sequences=16,
    max_queue_size=64,
    max_batched_tokens=2048,
    prefill_chunk_size=256,
    cuda_graph_decode=True,
    queue_timeout_seconds=60.0,
    block_size=16,
    kv_cache_bytes=4 * 1024**3,
    kv_cache_blocks=None,
)


@dataclass(frozen=True)
class EngineConfig:
    mode: str
    dtype: str
    max_model_len: int
    max_output_tokens: int
    eos_token_id: int | None
    max_active_sequences: int
    max_queue_size: int
    max_batched_tokens: int
    prefill_chunk_size: int
    cuda_graph_decode: bool
    queue_timeout_seconds: float
    block_size: int
    kv_cache_bytes: int
    kv_cache_blocks: int | None = None


def build_config(mode: str = "ragged", **overrides: Any) -> EngineConfig:
    """Defaults plus explicit overrides; an unknown override is an error (config.py:107-109)."""
    values = dict(_DEFAULTS)
    values["mode"] = mode
    unknown = set(overrides) - {f.name for f in fields(EngineConfig)}
    if unknown:
        raise ValueError(f"unknown config overrides: {sorted(unknown)}")
    values.update(overrides)
    config = EngineConfig(**values)
    validate_config(config)
    return config


def validate_config(config: EngineConfig) -> None:
    if config.mode != "ragged":
        raise ValueError(f"mode must be 'ragged' (the packed engine), got {config.mode!r}")
    if config.dtype not in DTYPES:
        raise ValueError(f"dtype must be one of {DTYPES}, got {config.dtype!r}")
    if config.max_output_tokens < 1:
        raise ValueError("max_output_tokens must be positive")
    if config.max_batched_tokens < 1 or config.prefill_chunk_size < 1:
        raise ValueError("batch token limits must be positive")
    if config.max_model_len < 1:
        raise ValueError("max_model_len must be positive")
    if config.max_active_sequences < 1:
        raise ValueError("max_active_sequences must be positive")
    if config.max_queue_size < 1:
        raise ValueError("max_queue_size must be positive")
    if config.block_size < 1:
        raise ValueError("block_size must be positive")
    if config.kv_cache_blocks is not None and config.kv_cache_blocks < 1:
        raise ValueError("kv_cache_blocks must be positive when given")
    if config.kv_cache_blocks is None and config.kv_cache_bytes < 1:
        raise ValueError("kv_cache_bytes must be positive")


def with_overrides(config: EngineConfig, **changes: Any) -> EngineConfig:
    changed = replace(config, **changes)
    validate_config(changed)
    return changed
