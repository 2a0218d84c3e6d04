"""Opt-in NVTX ranges (src/cloud_engine/profiling.py:10-26): active only with ENGINE_NVTX=1."""

from __future__ import annotations

import os
from contextlib import contextmanager


@contextmanager
def nvtx_range(name: str):
    if os.environ.get("ENGINE_NVTX") != "1":
        yield
        return
    import torch

    torch.cuda.nvtx.range_push(name)
    try:
        yield
    finally:
        torch.cuda.nvtx.range_pop()
