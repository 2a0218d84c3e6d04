"""The public engine: submit token ids, get tokens back.

Shape of the reference's ``InferenceEngine`` / ``RequestHandle`` / ``GenerationResult``
(src/cloud_engine/engine.py:48-57, 491-546, 549-802) without asyncio, tokenizer or HTTP:

    engine = InferenceEngine(build_config("ragged", block_size=16), model_dir)
    engine.start()
    handle = engine.submit([5, 17, 3], GenerationConfig(max_output_tokens=8))
    result = handle.wait()            # GenerationResult(token_ids=[...], finish_reason=...)
    for event in handle.stream(): ... # StreamEvent(token_id) as tokens are produced
    engine.snapshot_metrics(); engine.close()

``submit`` takes token ids (the tokenizer is outside this engine).  ``wait`` and ``stream`` drive
the scheduler loop on the caller's thread; every live request advances while one is waited for.
``runner_factory`` injects a fake runner for tests, as in the reference (engine.py:611-622).
"""

from __future__ import annotations

from collections.abc import Callable, Iterator, Sequence
from dataclasses import dataclass
from pathlib import Path
from typing import Any

from ..config.engine_config import EngineConfig, build_config
from .metrics import Metrics
from .scheduler import (
    GenerationConfig,
    PreemptionCandidate,
    Request,
    RequestState,
    Scheduler,
    SchedulingCandidate,
    StreamEvent,
    decode_first_priority,
    largest_sequence_preemption,
)


@dataclass
class GenerationResult:
    request_id: str
    token_ids: list[int]
    input_tokens: int
    output_tokens: int
    finish_reason: str
    ttft_ms: float | None
    e2e_ms: float
    preemptions: int = 0
    recomputed_tokens: int = 0


class RequestHandle:
    def __init__(self, request: Request, engine: "InferenceEngine") -> None:
        self.request = request
        self._engine = engine

    @property
    def request_id(self) -> str:
        return self.request.request_id

    @property
    def state(self) -> RequestState:
        return self.request.state

    def stream(self) -> Iterator[StreamEvent]:
        """Yields one event per produced token until the request ends."""
        request = self.request
        while True:
            while request.events:
                event = request.events.popleft()
                if event.finished:
                    return
                yield event
            if request.is_terminal:
                return
            self._engine.scheduler.step()

    def wait(self) -> GenerationResult:
        request = self.request
        scheduler = self._engine.scheduler
        while not request.is_terminal:
            scheduler.step()
        if request.state is not RequestState.COMPLETED:
            raise RuntimeError(
                f"generation {request.state.value}: {request.error_detail or request.finish_reason}"
            )
        return self._engine.result_of(request)

    def cancel(self) -> None:
        self._engine.scheduler.cancel(self.request)


class InferenceEngine:
    def __init__(
        self,
        config: EngineConfig | None = None,
        model_dir: str | Path | None = None,
        runner_factory: Callable[[EngineConfig], Any] | None = None,
        device: str | None = None,
        scheduling_priority: Callable[[SchedulingCandidate], tuple] = decode_first_priority,
        preemption_priority: Callable[[PreemptionCandidate], tuple] = largest_sequence_preemption,
        random_config: dict[str, Any] | None = None,
        seed: int = 0,
        random_scales: dict[str, float] | None = None,
    ) -> None:
        self.config = config or build_config("ragged")
        self.model_dir = Path(model_dir) if model_dir is not None else None
        self.device = device or "cuda:0"
        self._runner_factory = runner_factory
        self._random_config = random_config
        self._seed = seed
        self._random_scales = random_scales
        self.scheduling_priority = scheduling_priority
        self.preemption_priority = preemption_priority
        self.metrics = Metrics()
        self.core: Any = None
        self.runner: Any = None
        self.scheduler: Scheduler | None = None
        self.ready = False

    # ------------------------------------------------------------------ lifecycle
    def start(self) -> "InferenceEngine":
        if self.ready:
            return self
        if self._runner_factory is not None:
            self.runner = self._runner_factory(self.config)
        else:
            from .core import build_core
            from .runner import EngineRunner

            if self.model_dir is None and self._random_config is None:
                raise RuntimeError("model_dir (or random_config) required unless a runner is injected")
            config = self.config
            self.core = build_core(
                self.model_dir,
                dtype=config.dtype,
                device=self.device,
                page_size=config.block_size,
                num_pages=config.kv_cache_blocks,
                kv_cache_bytes=config.kv_cache_bytes,
                max_requests=config.max_active_sequences,
                max_model_len=config.max_model_len,
                max_tokens_per_step=config.max_batched_tokens,
                random_config=self._random_config,
                seed=self._seed,
                random_device="cuda" if self._random_config is not None else "cpu",
                random_scales=self._random_scales,
            )
            self.runner = EngineRunner(self.core, config)
        self.scheduler = Scheduler(
            self.config, self.runner, self.metrics,
            scheduling_priority=self.scheduling_priority,
            preemption_priority=self.preemption_priority,
        )
        self.ready = True
        return self

    def close(self) -> None:
        if self.scheduler is not None:
            for request in (*self.scheduler.active, *self.scheduler.waiting):
                self.scheduler.cancel(request)
        self.ready = False

    def __enter__(self) -> "InferenceEngine":
        return self.start()

    def __exit__(self, *exc: Any) -> None:
        self.close()

    # ------------------------------------------------------------------ usage
    def new_generation_config(self, max_output_tokens: int | None = None, **changes: Any) -> GenerationConfig:
        limit = self.config.max_output_tokens
        wanted = limit if max_output_tokens is None else min(max_output_tokens, limit)
        eos = changes.pop("eos_token_id", self.config.eos_token_id)
        return GenerationConfig(max_output_tokens=wanted, eos_token_id=eos, **changes)

    def submit(self, prompt_token_ids: Sequence[int], gen_config: GenerationConfig | None = None,
               label: str = "") -> RequestHandle:
        if not self.ready or self.scheduler is None:
            raise RuntimeError("engine not started")
        gen_config = gen_config or self.new_generation_config()
        prompt_token_ids = [int(t) for t in prompt_token_ids]
        if self.core is not None and prompt_token_ids:
            vocab = self.core.spec.vocab_size
            if min(prompt_token_ids) < 0 or max(prompt_token_ids) >= vocab:
                raise ValueError(f"prompt holds a token id outside the vocabulary of {vocab}")
        request = self.scheduler.submit(prompt_token_ids, gen_config, label=label)
        return RequestHandle(request, self)

    def run_until_idle(self) -> None:
        assert self.scheduler is not None
        self.scheduler.run_until_idle()

    def result_of(self, request: Request) -> GenerationResult:
        end_ns = request.finish_ns or self.metrics.now()
        return GenerationResult(
            request_id=request.request_id,
            token_ids=list(request.generated_token_ids),
            input_tokens=len(request.prompt_token_ids),
            output_tokens=request.generated_count,
            finish_reason=request.finish_reason,
            ttft_ms=(request.first_token_ns - request.arrival_ns) / 1e6 if request.first_token_ns else None,
            e2e_ms=(end_ns - request.arrival_ns) / 1e6,
            preemptions=request.preemption_count,
            recomputed_tokens=request.recomputed_tokens,
        )

    def snapshot_metrics(self) -> dict[str, Any]:
        base = self.metrics.snapshot()
        base["requests"]["waiting"] = len(self.scheduler.waiting) if self.scheduler else 0
        base["requests"]["active"] = len(self.scheduler.active) if self.scheduler else 0
        if self.core is not None:
            base["kv_cache"].update(self.core.cache.stats())
            base["kv_cache"]["pool_bytes"] = self.core.pools.bytes_held()
            base["gpu"] = dict(workspace_bytes=self.core.runtime.workspace.bytes_held(),
                               kernel_launches=self.core.runtime.ops.launches)
            import torch

            base["gpu"]["allocated_bytes"] = torch.cuda.memory_allocated()
            base["gpu"]["peak_allocated_bytes"] = torch.cuda.max_memory_allocated()
        runner = self.runner
        for name in ("forward_invocations", "max_forward_request_count", "cuda_graph_captures",
                     "cuda_graph_replays"):
            if hasattr(runner, name):
                base["scheduler"][name] = getattr(runner, name)
        plans = getattr(runner, "forward_plans", None)
        if plans is not None:
            base["scheduler"]["recent_forward_plans"] = [
                [dict(request_id=r, start_pos=s, query_length=q, sample=w) for r, s, q, w in plan]
                for plan in plans[-16:]
            ]
        return base


def generate(
    model_dir: str | Path | None,
    prompts: Sequence[Sequence[int]],
    max_output_tokens: int = 64,
    temperature: float = 0.0,
    seed: int = 0,
    eos_token_id: int | None = None,
    random_config: dict[str, Any] | None = None,
    weights_seed: int = 0,
    device: str | None = None,
    **overrides: Any,
) -> list[GenerationResult]:
    """Loads a model folder, runs every prompt (token ids) to completion, returns the results in
    the order of the prompts.  ``overrides`` are ``EngineConfig`` fields (``dtype``,
    ``block_size``, ``kv_cache_blocks``, ``max_batched_tokens``, ``prefill_chunk_size``,
    ``max_active_sequences``, ...).  A request that could not complete raises."""
    longest = max((len(p) for p in prompts), default=1)
    overrides.setdefault("max_model_len", max(longest + max_output_tokens, 64))
    overrides.setdefault("max_output_tokens", max(max_output_tokens, 1))
    overrides.setdefault("max_queue_size", max(64, len(prompts)))
    config = build_config("ragged", **overrides)
    engine = InferenceEngine(config, model_dir, device=device, random_config=random_config,
                             seed=weights_seed)
    with engine:
        handles = [
            engine.submit(
                prompt,
                GenerationConfig(max_output_tokens=max_output_tokens, temperature=temperature,
                                 eos_token_id=eos_token_id, seed=seed),
            )
            for prompt in prompts
        ]
        engine.run_until_idle()
        return [handle.wait() for handle in handles]
