"""Decode programs: the products and the attention of a decode step recorded as a list of phases
and run by ONE persistent kernel (csrc/decode_program.cu).

While ``Ops`` records (``Ops.begin_program``), its streaming products, the q/k/v product with the
rotary epilogue and the decode attention do not launch: they are written down here.  ``flush``
turns what was written down into phases (the C side fills them, tensor maps included), puts them
into device memory and launches the kernel; any kernel of ``Ops`` that cannot be recorded flushes
first, so the order of the work never changes.  The phases of a step depend on addresses and sizes
only, so the device copy of a list that was run before is found again by its bytes (a step
replayed from a CUDA graph never comes here at all; one captured into a graph keeps its copy for
the life of the process).
"""

from __future__ import annotations

import ctypes
import os
from collections import OrderedDict
from ctypes import c_float, c_int, c_longlong, c_void_p
from typing import Any

from .build import load_library

HEAD_DIMS = (64, 128)      # head sizes the kernel is built for
MAX_ROWS = 16              # token rows of a recorded step
MAX_SPLITS = 16            # most slices of K a product is cut into
LEAST_STAGES = 6           # the ring keeps at least this many 16 KB stages, whatever the token rows need
KEPT_TAPES = 32            # device copies kept for steps outside CUDA graphs
MIN_KEYS_PER_CTA = int(os.environ.get("CIE_PROGRAM_MIN_KEYS", "256"))


def enabled() -> bool:
    """Off unless CIE_PROGRAM=1: measured on a B200 the one-kernel step is slower than the separate
    kernels with their programmatic overlap (2.8 ms against 1.8 ms a step at batch 8): seven
    barriers in global memory a layer at 1.5 us each, and phases of a few microseconds that one CTA
    per SM runs as chains of dependent loads."""
    return os.environ.get("CIE_PROGRAM", "0") == "1"


def product_splits(tiles: int, chunks: int, ctas: int, most_chunks: int = 1 << 30) -> int:
    """Slices of K for a product of ``tiles`` 32-row weight tiles and ``chunks`` 256-column chunks on
    ``ctas`` CTAs.  A CTA works on one slice (CTA c on slice c % slices) and shares its tiles with the
    other CTAs of that slice.  One slice (every tile finished by the CTA that streams it, no finish
    phase) unless cutting K shortens the longest CTA's share by more than the finish phase and its
    barrier cost (about eight stages of streaming, and a little more with every slice it has to add
    up), or a slice may have ``most_chunks`` chunks at most (its token rows must fit shared memory)."""
    def stages(splits: int) -> int:
        return -(-tiles // (ctas // splits)) * -(-chunks // splits)

    least = max(1, -(-chunks // most_chunks))
    best, best_cost = least, float(stages(least)) + (0 if least == 1 else 8 + least / 4)
    for splits in range(max(2, least), min(chunks, MAX_SPLITS, ctas) + 1):
        cost = stages(splits) + 8 + splits / 4
        if cost < best_cost:
            best, best_cost = splits, cost
    return best


class _Library:
    def __init__(self, head_dim: int) -> None:
        from .ops import _Lib

        lib = _Lib(load_library("decode_program.cu", {"HEAD_DIM": head_dim}))
        v, i, f, ll = c_void_p, c_int, c_float, c_longlong
        self.phase_bytes = int(lib.handle.cie_program_phase_bytes())
        self.max_key_splits = int(lib.handle.cie_program_max_key_splits())
        self.gemm = lib.function("cie_program_gemm", [v, v, v, i, v, i, f, v, v, v, v, v, v, v, v, i, i, i, i, i])
        self.rope = lib.function(
            "cie_program_rope",
            [v, v, v, i, v, i, f, v, v, v, v, i, v, v, v, i, i, v, v, v, i, i, i, i, i, i, i, i, i])
        self.attention = lib.function(
            "cie_program_attention", [v, v, v, i, v, i, v, v, v, i, i, v, i, i, i, i, i, i, v, f, i])
        self.launch = lib.function("cie_program_launch", [v, i, i, v, v, v])
        self.upload = lib.function("cie_program_upload", [v, ll, v])
        self.free = lib.function("cie_program_free", [v])
        geometry = lib.function("cie_program_geometry", [i, v, v])
        ctas, slab_limit = c_int(0), c_int(0)
        geometry(LEAST_STAGES, ctypes.byref(ctas), ctypes.byref(slab_limit))
        self.ctas, self.slab_limit = ctas.value, slab_limit.value


def _ptr(tensor: Any) -> int | None:
    return None if tensor is None else tensor.data_ptr()


class DecodeProgram:
    def __init__(self, ops: Any) -> None:
        self.ops = ops
        self.recording = False
        self.calls: list[tuple] = []
        self.head_dim: int | None = None
        self._libraries: dict[int, _Library] = {}
        self._tapes: OrderedDict[bytes, list] = OrderedDict()   # bytes -> [device address, kept for a graph]
        self.counter = ops.torch.zeros(1, dtype=ops.torch.int32, device=ops.device)
        self.programs_run = 0
        self.phases_run = 0

    def library(self, head_dim: int) -> _Library:
        if head_dim not in self._libraries:
            self._libraries[head_dim] = _Library(head_dim)
        return self._libraries[head_dim]

    @property
    def pending(self) -> bool:
        return bool(self.calls)

    # ------------------------------------------------------------------ recording
    def begin(self) -> None:
        self.recording = True

    def end(self) -> None:
        self.flush()
        self.recording = False

    def gemm(self, x: Any, row_sq: Any, sq_tiles: int, eps: float, weight: Any, bias: Any, out: Any,
             residual: Any, sq: Any, scaled: Any, next_gain: Any, m: int, n: int, k: int, mode: int,
             tag: str) -> None:
        self.calls.append(("gemm", x, row_sq, sq_tiles, eps, weight, bias, out, residual, sq, scaled, next_gain,
                           m, n, k, mode, tag))

    def rope(self, x: Any, row_sq: Any, sq_tiles: int, eps: float, weight: Any, bias: Any, q_out: Any,
             positions: Any, request_of_token: Any, table: Any, num_pages: int, k_pool: Any, v_pool: Any,
             inv_freq: Any, m: int, q_heads: int, kv_heads: int, dim: int, rot: int, page_size: int,
             write_cache: bool, k: int) -> None:
        self.calls.append(("rope", x, row_sq, sq_tiles, eps, weight, bias, q_out, positions, request_of_token,
                           table, num_pages, k_pool, v_pool, inv_freq, m, q_heads, kv_heads, dim, rot, page_size,
                           write_cache, k))

    def can_attend(self, head_dim: int, page_size: int, requests: int, k_pool: Any, v_pool: Any) -> bool:
        return (self.recording and head_dim in HEAD_DIMS and requests <= MAX_ROWS and page_size >= 16
                and page_size & (page_size - 1) == 0 and (k_pool.data_ptr() | v_pool.data_ptr()) % 16 == 0)

    def attention(self, q: Any, out: Any, k_pool: Any, v_pool: Any, table: Any, num_pages: int,
                  context_lens: Any, requests: int, q_heads: int, kv_heads: int, head_dim: int, page_size: int,
                  scale: float, window: int) -> None:
        if self.head_dim is not None and self.head_dim != head_dim:
            self.flush()   # one build of the kernel per head size
        self.head_dim = head_dim
        self.calls.append(("attention", q, out, k_pool, v_pool, table, num_pages, context_lens, requests,
                           q_heads, kv_heads, page_size, scale, window))

    # ------------------------------------------------------------------ running
    def _encode(self, lib: _Library) -> tuple[bytes, int, int]:
        ops = self.ops
        size = lib.phase_bytes
        room = ctypes.create_string_buffer(2 * size)
        count = c_int(0)
        tape = bytearray()
        phases = 0
        slab = 0

        def cut(m: int, n: int, k: int) -> int:
            """Slices of K for a product, and the shared memory its token rows then need."""
            nonlocal slab
            padded = 8 if m <= 8 else 16
            chunks = -(-k // 256)
            splits = product_splits(-(-n // 32), chunks, lib.ctas, max(1, lib.slab_limit // (padded * 512)))
            slab = max(slab, padded * 512 * -(-chunks // splits))
            return splits

        for call in self.calls:
            kind = call[0]
            if kind == "gemm":
                (_, x, row_sq, sq_tiles, eps, weight, bias, out, residual, sq, scaled, next_gain, m, n, k, mode,
                 tag) = call
                splits = cut(m, n, k)
                partial = None
                if splits > 1:
                    partial = ops.scratch("program.partial." + tag, splits * m * n, reserve=MAX_SPLITS * MAX_ROWS * n)
                lib.gemm(room, ctypes.byref(count), _ptr(x), x.stride(0), _ptr(row_sq), sq_tiles, eps, _ptr(weight),
                         _ptr(bias), _ptr(out), _ptr(partial), _ptr(residual), _ptr(sq), _ptr(scaled),
                         _ptr(next_gain), m, n, k, splits, mode)
            elif kind == "rope":
                (_, x, row_sq, sq_tiles, eps, weight, bias, q_out, positions, request_of_token, table, num_pages,
                 k_pool, v_pool, inv_freq, m, q_heads, kv_heads, dim, rot, page_size, write_cache, k) = call
                n = (q_heads + 2 * kv_heads) * dim
                splits = cut(m, n, k)
                partial = None
                if splits > 1:
                    partial = ops.scratch("program.partial.qkv", splits * m * n, reserve=MAX_SPLITS * MAX_ROWS * n)
                lib.rope(room, ctypes.byref(count), _ptr(x), x.stride(0), _ptr(row_sq), sq_tiles, eps, _ptr(weight),
                         _ptr(bias), _ptr(partial), _ptr(q_out), q_out.stride(0), _ptr(positions),
                         _ptr(request_of_token), _ptr(table), table.shape[1], num_pages, _ptr(k_pool), _ptr(v_pool),
                         _ptr(inv_freq), m, q_heads, kv_heads, dim, rot, page_size, 1 if write_cache else 0, k,
                         splits)
            else:
                (_, q, out, k_pool, v_pool, table, num_pages, context_lens, requests, q_heads, kv_heads,
                 page_size, scale, window) = call
                head_dim = self.head_dim
                units = requests * kv_heads * -(-(q_heads // kv_heads) // 16)
                max_keys = table.shape[1] * page_size
                if window > 0:
                    max_keys = min(max_keys, window)
                key_splits = max(1, min(lib.max_key_splits, lib.ctas // units, max_keys // MIN_KEYS_PER_CTA))
                row = 16 * (head_dim + 4)
                most = max(lib.ctas, MAX_ROWS * kv_heads * -(-(q_heads // kv_heads) // 16))
                shares = ops.scratch(f"program.shares.{head_dim}", units * key_splits * row, reserve=most * row)
                lib.attention(room, ctypes.byref(count), _ptr(q), q.stride(0), _ptr(out), out.stride(0),
                              _ptr(k_pool), _ptr(v_pool), _ptr(table), table.shape[1], num_pages,
                              _ptr(context_lens), requests, q_heads, kv_heads, page_size, key_splits,
                              MIN_KEYS_PER_CTA, _ptr(shares), scale, window)
            tape += room.raw[: count.value * size]
            phases += count.value
        tape += bytes(size)   # the end mark: a phase of kind 0
        return bytes(tape), phases, slab

    def flush(self) -> None:
        """Runs what was recorded since the last flush (nothing, if nothing was)."""
        if not self.calls:
            return
        ops = self.ops
        lib = self.library(self.head_dim or HEAD_DIMS[-1])
        tape, phases, slab = self._encode(lib)
        self.calls = []
        self.head_dim = None
        capturing = ops.torch.cuda.is_current_stream_capturing()
        held = self._tapes.get(tape)
        if held is None:
            address = c_void_p(0)
            lib.upload(tape, len(tape), ctypes.byref(address))
            held = [address.value, capturing]
            self._tapes[tape] = held
            self._trim(lib)
        else:
            self._tapes.move_to_end(tape)
            held[1] = held[1] or capturing
        ops.launches += 1
        self.programs_run += 1
        self.phases_run += phases
        lib.launch(held[0], phases, slab, self.counter.data_ptr(), ops.error_word.data_ptr(), ops.stream)

    def _trim(self, lib: _Library) -> None:
        """Forgets the oldest device copies that no CUDA graph holds."""
        loose = [key for key, held in self._tapes.items() if not held[1]]
        if len(loose) <= KEPT_TAPES or self.ops.torch.cuda.is_current_stream_capturing():
            return
        for key in loose[: len(loose) - KEPT_TAPES]:
            lib.free(self._tapes.pop(key)[0])
