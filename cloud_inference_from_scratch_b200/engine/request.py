"""The words the scheduler and its callers share: request states, refusal reasons, generation
settings, stream events, the request record itself, the columns of a step's plan and what the two
policy hooks are shown.

States, reasons, field names and the two default policies are the reference's
(src/cloud_engine/scheduler.py:29-71, 86-199) because they are the engine's public surface;
``Request`` and ``BatchPlan`` are this engine's own: a request is one growing token list (prompt
followed by what was generated) with a cursor, and a plan is four parallel columns.
"""

from __future__ import annotations

from collections import deque
from collections.abc import Sequence
from dataclasses import dataclass
from enum import Enum


class RequestState(Enum):
    WAITING = "waiting"
    PREFILL = "prefill"
    DECODING = "decoding"
    COMPLETED = "completed"
    CANCELLED = "cancelled"
    TIMED_OUT = "timed_out"
    FAILED = "failed"


TERMINAL_STATES = frozenset(
    (RequestState.COMPLETED, RequestState.CANCELLED, RequestState.TIMED_OUT, RequestState.FAILED)
)


class RejectionReason(Enum):
    QUEUE_FULL = "queue_full"
    KV_CAPACITY = "capacity_exhausted"
    CONTEXT_OVERFLOW = "context_length_exceeded"


class RejectedError(RuntimeError):
    def __init__(self, reason: RejectionReason, detail: str = "") -> None:
        super().__init__(detail or reason.value)
        self.reason = reason


@dataclass
class GenerationConfig:
    """``temperature`` 0 is greedy; otherwise tokens are drawn from softmax(logits / temperature)
    with a draw that depends only on (``seed``, the request's stream number, the output index).
    ``eos_token_id`` None means no token ends the request early."""

    max_output_tokens: int
    temperature: float = 0.0
    eos_token_id: int | None = None
    seed: int = 0

    def __post_init__(self) -> None:
        if self.max_output_tokens < 1:
            raise ValueError("max_output_tokens must be positive")
        if self.temperature < 0:
            raise ValueError("temperature must be >= 0")


@dataclass
class StreamEvent:
    token_id: int | None
    finished: bool = False
    finish_reason: str = ""


class Request:
    """One generation: ``tokens`` is the prompt followed by every generated token; the first
    ``tokens_fed`` of them are in the cache."""

    __slots__ = (
        "request_id", "config", "arrival_ns", "sequence_number", "label", "state", "tokens",
        "prompt_len", "tokens_fed", "events", "first_token_ns", "last_token_ns", "finish_ns",
        "finish_reason", "error_detail", "rejected", "preemption_count", "recomputed_tokens",
        "recompute_until",
    )

    def __init__(self, request_id: str, prompt_token_ids: Sequence[int], config: GenerationConfig,
                 arrival_ns: int, sequence_number: int = 0, label: str = "") -> None:
        self.request_id = request_id
        self.config = config
        self.arrival_ns = arrival_ns
        self.sequence_number = sequence_number
        self.label = label
        self.state = RequestState.WAITING
        self.tokens: list[int] = [int(t) for t in prompt_token_ids]
        self.prompt_len = len(self.tokens)
        self.tokens_fed = 0
        self.events: deque[StreamEvent] = deque()
        self.first_token_ns: int | None = None
        self.last_token_ns: int | None = None
        self.finish_ns: int | None = None
        self.finish_reason = ""
        self.error_detail = ""
        self.rejected = False
        self.preemption_count = 0
        self.recomputed_tokens = 0
        self.recompute_until = 0     # tokens below this position were in the cache once before

    @property
    def prompt_token_ids(self) -> list[int]:
        return self.tokens[:self.prompt_len]

    @property
    def generated_token_ids(self) -> list[int]:
        return self.tokens[self.prompt_len:]

    @property
    def generated_count(self) -> int:
        return len(self.tokens) - self.prompt_len

    @property
    def known_length(self) -> int:
        return len(self.tokens)

    @property
    def is_terminal(self) -> bool:
        return self.state in TERMINAL_STATES


class BatchItem:
    """One request's slice of tokens in a step (a view of one row of a ``BatchPlan``)."""

    __slots__ = ("request", "start_pos", "query_length", "sample")

    def __init__(self, request: Request, start_pos: int, query_length: int, sample: bool) -> None:
        self.request, self.start_pos, self.query_length, self.sample = request, start_pos, query_length, sample

    @property
    def end_pos(self) -> int:
        return self.start_pos + self.query_length

    @property
    def token_ids(self) -> list[int]:
        return self.request.tokens[self.start_pos:self.start_pos + self.query_length]

    @property
    def is_decode(self) -> bool:
        return self.query_length == 1 and self.start_pos >= self.request.prompt_len


class BatchPlan:
    """What one step runs, as columns: row i feeds ``lengths[i]`` tokens of ``requests[i]`` from
    position ``starts[i]`` and samples a token iff ``samples[i]``."""

    __slots__ = ("requests", "starts", "lengths", "samples", "token_count", "_items")

    def __init__(self, requests: list[Request], starts: list[int], lengths: list[int],
                 samples: list[bool]) -> None:
        self.requests, self.starts, self.lengths, self.samples = requests, starts, lengths, samples
        self.token_count = sum(lengths)
        self._items: tuple[BatchItem, ...] | None = None

    def __len__(self) -> int:
        return len(self.requests)

    @property
    def items(self) -> tuple[BatchItem, ...]:
        if self._items is None:
            self._items = tuple(map(BatchItem, self.requests, self.starts, self.lengths, self.samples))
        return self._items

    @property
    def request_ids(self) -> tuple[str, ...]:
        return tuple(request.request_id for request in self.requests)

    @property
    def decode_only(self) -> bool:
        """Every row is a single token whose successor is sampled."""
        return self.token_count == len(self.requests) and all(self.samples)


@dataclass(frozen=True)
class SchedulingCandidate:
    """What a custom ``scheduling_priority`` sees of a resident that has tokens to feed."""

    request_id: str
    phase: str  # "decode" or "prefill"
    remaining_tokens: int
    prompt_tokens: int
    generated_tokens: int
    arrival_ns: int


@dataclass(frozen=True)
class PreemptionCandidate:
    """What a ``preemption_priority`` sees of a resident when pages have run out."""

    request_id: str
    allocated_tokens: int
    tokens_fed: int
    generated_tokens: int
    arrival_ns: int


def decode_first_priority(candidate: SchedulingCandidate) -> tuple[int]:
    """Smallest key first: decoding requests, then prompt portions (arrival order inside each)."""
    return (0 if candidate.phase == "decode" else 1,)


def largest_sequence_preemption(candidate: PreemptionCandidate) -> tuple[int, int, int]:
    """Largest key is the victim: most pages held, then most tokens fed, then latest arrival."""
    return (candidate.allocated_tokens, candidate.tokens_fed, candidate.arrival_ns)
