"""What parts need at run time: the device, the compute dtype, the kernels and a workspace.

The workspace hands out persistent activation buffers by (tag, row width, dtype): a part
asks for ``get("attention.qkv", tokens, width, dtype)`` every step and gets the first rows of
the same allocation, so addresses stay fixed from step to step (which CUDA-graph replay
needs) and layers of the same shape share their scratch.  Buffers are allocated for
``max_rows`` tokens at first use and grow only outside graph capture.
"""

from __future__ import annotations

from typing import Any

from ..native.ops import Ops


class Workspace:
    def __init__(self, device: Any, max_rows: int = 0) -> None:
        self.device = device
        self.max_rows = int(max_rows)
        self._buffers: dict[tuple[str, int, Any], Any] = {}
        self.frozen = False
        self.generation = 0   # counts buffers that were replaced by larger ones (their old address died)

    def get(self, tag: str, rows: int, width: int, dtype: Any) -> Any:
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
            capacity = max(rows, self.max_rows, 1)
            buffer = torch.empty((capacity, int(width)), dtype=dtype, device=self.device)
            self._buffers[key] = buffer
        return buffer[:rows]

    def bytes_held(self) -> int:
        return sum(b.numel() * b.element_size() for b in self._buffers.values())


class Runtime:
    def __init__(self, device: Any = "cuda:0", dtype: str = "bfloat16", max_tokens: int = 0,
                 gemm: str | None = None) -> None:
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
        self.workspace = Workspace(self.device, max_tokens)
