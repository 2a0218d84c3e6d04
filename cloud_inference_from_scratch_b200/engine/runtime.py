"""What parts need at run time: the device, the compute dtype, the kernels and a workspace.

The workspace hands out persistent activation buffers by (tag, row width, dtype): a part
asks for ``get("attention.qkv", tokens, width, dtype)`` every step and gets the first rows of
the same allocation, so addresses stay fixed from step to step (which CUDA-graph replay
needs) and layers of the same shape share their scratch.  Buffers are allocated for
``max_rows`` tokens at first use and grow only outside graph capture.  Buffers that hold one row
per request of a step (logits, the rows picked for the final norm) are bounded by the number of
requests, ``max_request_rows``, not by the token budget: at a vocabulary of 150,000 a row of
float32 logits is 600 KB.
"""

from __future__ import annotations

from typing import Any

from ..native.ops import Ops


class Workspace:
    def __init__(self, device: Any, max_rows: int = 0, max_request_rows: int = 0) -> None:
        self.device = device
        self.max_rows = int(max_rows)
        self.max_request_rows = int(max_request_rows) or self.max_rows
        self._buffers: dict[tuple[str, int, Any], Any] = {}
        self.frozen = False
        self.generation = 0   # counts buffers that were replaced by larger ones (their old address died)

    def get(self, tag: str, rows: int, width: int, dtype: Any, per_request: bool = False) -> Any:
        """The first ``rows`` rows of the buffer ``tag``; ``per_request``: the buffer holds one row
        per request of a step, not one per token."""
        import torch

        key = (tag, int(width), dtype)
        buffer = self._buffers.get(key)
        if buffer is None or buffer.shape[0] < rows:
            if self.frozen and buffer is not None:   # a new buffer harms no graph; a moved one would
                raise RuntimeError(
                    f"workspace buffer {tag!r} would have to grow to {rows} rows while a CUDA "
                    "graph that uses it is alive"
                )
            if buffer is not None:
                self.generation += 1
            capacity = max(rows, self.max_request_rows if per_request else self.max_rows, 1)
            buffer = torch.empty((capacity, int(width)), dtype=dtype, device=self.device)
            self._buffers[key] = buffer
        return buffer[:rows]

    def bytes_held(self) -> int:
        return sum(b.numel() * b.element_size() for b in self._buffers.values())


class Runtime:
    def __init__(self, device: Any = "cuda:0", dtype: str = "bfloat16", max_tokens: int = 0,
                 gemm: str | None = None, max_requests: int = 0) -> None:
        import torch

        names = {"bfloat16": torch.bfloat16, "float32": torch.float32,
                 "bf16": torch.bfloat16, "fp32": torch.float32}
        if dtype not in names:
            raise ValueError(f"dtype must be 'bfloat16' or 'float32', got {dtype!r}")
        self.device = torch.device(device)
        self.dtype = names[dtype]
        self.dtype_name = "float32" if self.dtype == torch.float32 else "bfloat16"
        if self.device.type == "cuda":
            torch.cuda.set_device(self.device)
        self.ops = Ops(self.device, self.dtype, gemm=gemm)
        # a decode-only step is padded to the next power of two of its batch, which may exceed a
        # token budget that is no power of two
        bucket = 0
        if max_tokens and max_requests:
            bucket = 1 << (min(max_requests, max_tokens) - 1).bit_length()
        self.workspace = Workspace(self.device, max(max_tokens, bucket), bucket)
