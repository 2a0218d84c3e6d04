from .engine import GenerationResult, InferenceEngine, RequestHandle, generate
from .metrics import Metrics
from .scheduler import (
    BatchItem,
    BatchPlan,
    GenerationConfig,
    PreemptionCandidate,
    RejectedError,
    RejectionReason,
    Request,
    RequestState,
    Scheduler,
    SchedulingCandidate,
    StreamEvent,
    decode_first_priority,
    largest_sequence_preemption,
)

__all__ = [
    "BatchItem", "BatchPlan", "GenerationConfig", "GenerationResult", "InferenceEngine", "Metrics",
    "PreemptionCandidate", "RejectedError", "RejectionReason", "Request", "RequestHandle",
    "RequestState", "Scheduler", "SchedulingCandidate", "StreamEvent", "decode_first_priority",
    "generate", "largest_sequence_preemption",
]
