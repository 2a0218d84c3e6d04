"""Puts the pieces together for one model folder: description, weights, cache, step function.

This is the composition root of the engine, the counterpart of
``InferenceEngine._initialize`` (src/cloud_engine/engine.py:608-719) without modes or
backends: read config.json, resolve the architecture through the registry, check the weight
files against the name table, place tensors on the device, size the cache, build the step
function.  The trace-replay program, the scheduler's runner, the tests and the benchmark all
start here, so they drive the same model, cache and kernels.
"""

from __future__ import annotations

from dataclasses import dataclass
from pathlib import Path
from typing import Any

from ..cache.manager import CacheManager
from ..cache.pools import CachePools, plan_groups, plan_page_counts
from ..config.registry import resolve_config, resolve_model
from ..models.decoder import DecoderModel
from ..weights.loader import check_tensors, device_tensors
from ..weights.source import RandomSource, SafetensorsSource
from .runtime import Runtime
from .step import StepFunction


@dataclass
class EngineCore:
    architecture: str
    model_config: Any
    spec: Any
    model: DecoderModel
    runtime: Runtime
    cache: CacheManager
    pools: CachePools
    step: StepFunction
    page_size: int
    max_requests: int
    max_model_len: int


def build_core(
    model_dir: str | Path | None,
    *,
    dtype: str = "bfloat16",
    device: str = "cuda:0",
    page_size: int = 16,
    num_pages: int | None = None,
    kv_cache_bytes: int | None = None,
    max_requests: int = 16,
    max_model_len: int = 4096,
    max_tokens_per_step: int = 0,
    gemm: str | None = None,
    random_config: dict[str, Any] | None = None,
    seed: int = 0,
    random_device: str = "cpu",
    random_scales: dict[str, float] | None = None,
) -> EngineCore:
    """``model_dir`` is a folder with config.json and *.safetensors; or give ``random_config``
    (a config.json dictionary) and ``seed`` to draw the weights without writing a folder."""
    if model_dir is not None:
        arch, config, spec = resolve_model(model_dir)
    elif random_config is not None:
        arch, config, spec = resolve_config(random_config)
    else:
        raise ValueError("give a model folder or a random_config")
    model = DecoderModel(spec)
    table = model.tensor_table()
    if model_dir is not None:
        source: Any = SafetensorsSource(model_dir)
        check_tensors(source, table, spec.optional_tensors)
    else:
        source = RandomSource(table, seed, device=random_device, scales=random_scales)
    if max_model_len > spec.max_positions:
        raise ValueError(
            f"max_model_len {max_model_len} exceeds the model's position range {spec.max_positions}"
        )
    runtime = Runtime(device=device, dtype=dtype, max_tokens=max_tokens_per_step, gemm=gemm,
                      max_requests=max_requests)
    model.bind(device_tensors(source, table, runtime.device, runtime.dtype), runtime)

    needs = model.cache_needs()
    element_size = 4 if dtype in ("float32", "fp32") else 2
    groups, place = plan_groups(needs, element_size)
    if num_pages is None and kv_cache_bytes is None:
        raise ValueError("give num_pages or kv_cache_bytes")
    # every group's pool by what its layers can use: a windowed group needs far fewer pages
    pages_per_group = plan_page_counts(groups, page_size, max_requests, max_tokens_per_step,
                                       num_pages=num_pages, kv_cache_bytes=kv_cache_bytes)
    cache = CacheManager(groups, page_size, pages_per_group, max_requests, max_model_len)
    pools = CachePools(needs, groups, place, pages_per_group, page_size, max_requests,
                       runtime.dtype, runtime.device)
    step = StepFunction(model, runtime, cache, pools)
    return EngineCore(
        architecture=arch.name, model_config=config, spec=spec, model=model, runtime=runtime,
        cache=cache, pools=pools, step=step, page_size=page_size, max_requests=max_requests,
        max_model_len=max_model_len,
    )
