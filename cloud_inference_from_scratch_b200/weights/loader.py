"""Checks a tensor source against a model's name table and places tensors on the device.

Parity with the reference's loader (src/cloud_engine/weights.py:96-121): missing names,
unexpected names (a tied model's stored head excepted) and wrong shapes are errors.  The
reference raises on the first class it meets; here ONE ``WeightsError`` lists all three.
Dtype rule: a "matrix" tensor is held in the compute dtype (bfloat16, or float32 in a
32-bit run); a "vector" tensor (norm gain, bias) is held in float32, so one stored in
32-bit stays so and one stored in bfloat16 widens exactly; a "table" tensor is int32.
"""

from __future__ import annotations

from typing import Any

from ..parts.base import TensorSpec
from .source import WeightsError


def check_tensors(source: Any, table: dict[str, TensorSpec], optional: tuple[str, ...] = ()) -> None:
    present = set(source.names())
    missing = sorted(set(table) - present)
    unexpected = sorted(present - set(table) - set(optional))
    wrong = []
    for name in sorted(set(table) & present):
        expected = tuple(table[name].shape)
        actual = tuple(source.shape(name))
        if actual != expected:
            wrong.append(f"{name}: expected {list(expected)}, found {list(actual)}")
    if not (missing or unexpected or wrong):
        return

    def preview(items: list[str], limit: int = 12) -> str:
        shown = ", ".join(items[:limit])
        return shown + (f" (+{len(items) - limit} more)" if len(items) > limit else "")

    lines = ["model weights do not fit the configuration:"]
    if missing:
        lines.append(f"  missing tensors ({len(missing)}): {preview(missing)}")
    if unexpected:
        lines.append(f"  unexpected tensors ({len(unexpected)}): {preview(unexpected)}")
    if wrong:
        lines.append(f"  wrong shapes ({len(wrong)}): {preview(wrong)}")
    raise WeightsError("\n".join(lines), missing=missing, unexpected=unexpected, wrong_shape=wrong)


def device_tensors(source: Any, table: dict[str, TensorSpec], device: Any, compute_dtype: Any):
    """Returns ``fetch(name)``: the tensor on ``device`` in the dtype its role asks for."""
    import torch

    def fetch(name: str) -> Any:
        spec = table[name]
        tensor = source.get(name)
        if spec.role == "vector":
            dtype = torch.float32
        elif spec.role == "table":
            dtype = torch.int32
        else:
            dtype = compute_dtype
        return tensor.to(device=device, dtype=dtype).contiguous()

    return fetch
