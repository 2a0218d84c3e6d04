"""Which CUDA libraries exist: the list ``build()`` compiles and the names ``Ops`` loads."""

from __future__ import annotations

GENERIC = ("elementwise.cu", "gemm_simt.cu", "attention_generic.cu", "sampling.cu")


def all_libraries() -> list[tuple[str, dict]]:
    return [(source, {}) for source in GENERIC]
