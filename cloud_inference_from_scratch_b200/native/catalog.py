"""Which CUDA libraries exist: the list ``build()`` compiles and the names ``Ops`` loads."""

from __future__ import annotations

GENERIC = ("elementwise.cu", "gemm_simt.cu", "gemm_stream.cu", "gemm_tcgen05.cu", "gemm_skinny.cu", "attention_generic.cu", "sampling.cu")


# head sizes the tensor-core attention library is built for ahead of time; any other multiple of
# 16 up to 256 is built when a model first asks for it
ATTENTION_HEAD_DIMS = (64, 128)


def all_libraries() -> list[tuple[str, dict]]:
    libraries: list[tuple[str, dict]] = [(source, {}) for source in GENERIC]
    libraries += [("attention_tensor.cu", {"HEAD_DIM": dim}) for dim in ATTENTION_HEAD_DIMS]
    libraries += [("attention_prefill_tc.cu", {"HEAD_DIM": dim}) for dim in ATTENTION_HEAD_DIMS]
    libraries += [("decode_program.cu", {"HEAD_DIM": dim}) for dim in ATTENTION_HEAD_DIMS]
    return libraries
