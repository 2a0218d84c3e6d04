"""Python face of the CUDA kernels: one method per kernel family, bound to a device and a dtype.

Every method launches hand-written sm_100a code from ``csrc/`` on the current CUDA stream
through a C interface (ctypes); nothing here computes on the host and there is no fallback
when a library cannot be built or the device is not a CUDA device.  Which kernel a call
reaches is decided by sizes only (for example: the tensor-core attention kernels take head
sizes that are multiples of 16 up to 256, other shapes go to the generic kernel); a size no
kernel takes raises.
"""

from __future__ import annotations

import ctypes
import os
from ctypes import c_float, c_int, c_void_p
from typing import Any

from ..lazy import Accumulated, GateUpWeight, NormedInput, Partials, ResidualSink  # noqa: F401  (re-exported)
from .build import load_library

F32, BF16 = 0, 1


class KernelError(RuntimeError):
    pass


def _ptr(tensor: Any) -> int | None:
    return None if tensor is None else tensor.data_ptr()


# More rows than this go to the tile kernels (tcgen05 or the library).  The streaming kernel
# multiplies with mma.sync, 8 tokens an instruction: built for 32 and 64 rows it was bound by that
# tensor path (the gate/up product of 64 tokens took 30 us against the library's 17) and its
# epilogues, which finish a token row per warp, by the number of rows.
STREAM_MAX_ROWS = 16
# Up to this many rows a projection adds itself into the residual stream, or rotates and stores
# q/k/v (cluster epilogues of the streaming kernel): every row count that kernel takes.
FUSED_RESIDUAL_MAX_ROWS = STREAM_MAX_ROWS


class _Lib:
    """A loaded library whose entry points return 0 or set ``cie_last_error``."""

    def __init__(self, handle: ctypes.CDLL) -> None:
        self.handle = handle
        handle.cie_last_error.restype = ctypes.c_char_p

    def function(self, name: str, argtypes: list[Any]):
        fn = getattr(self.handle, name)
        fn.argtypes = argtypes
        fn.restype = c_int
        last_error = self.handle.cie_last_error

        def call(*args: Any) -> None:
            if fn(*args) != 0:
                raise KernelError(last_error().decode(errors="replace"))

        return call


class Ops:
    def __init__(self, device: Any, dtype: Any, gemm: str | None = None) -> None:
        import torch

        self.torch = torch
        self.device = torch.device(device)
        if self.device.type != "cuda":
            raise KernelError(
                f"this engine runs on a CUDA device (sm_100a) only; got device {self.device}"
            )
        if not torch.cuda.is_available():
            raise KernelError("no CUDA device is available; there is no CPU path")
        if dtype not in (torch.float32, torch.bfloat16):
            raise KernelError(f"compute dtype must be float32 or bfloat16, got {dtype}")
        self.dtype = dtype
        self.code = F32 if dtype == torch.float32 else BF16
        self.gemm_mode = gemm or ("simt" if self.code == F32 else os.environ.get("CIE_GEMM", "cublas"))
        if self.code == F32 and self.gemm_mode != "simt":
            raise KernelError("the 32-bit path multiplies on the CUDA cores only (gemm='simt')")
        if self.gemm_mode not in ("simt", "tensor", "cublas"):
            raise KernelError(f"unknown gemm mode {self.gemm_mode!r}")
        self.error_word = torch.zeros(1, dtype=torch.int32, device=self.device)
        self.launches = 0
        self.sm_count = torch.cuda.get_device_properties(self.device).multi_processor_count

        v, i, f = c_void_p, c_int, c_float
        ew = _Lib(load_library("elementwise.cu"))
        self._embedding = ew.function("cie_embedding", [v, v, v, i, i, i, f, i, v, v])
        ll = ctypes.c_longlong
        self._shape_logits = ew.function("cie_shape_logits", [v, ll, f, f, v])
        self._add_rmsnorm = ew.function("cie_add_rmsnorm", [v, v, i, ll, v, v, v, v, i, i, f, i, v])
        self._rope_kv_write = ew.function(
            "cie_rope_kv_write",
            [v, i, ll, v, v, i, v, v, v, i, i, v, v, v, i, i, i, i, i, i, i, i, i, v, v],
        )
        self._silu_mul = ew.function("cie_silu_mul", [v, v, i, i, i, i, v])
        gs = _Lib(load_library("gemm_simt.cu"))
        self._gemm_simt = gs.function("cie_gemm_simt", [v, v, v, v, i, i, i, i, i, i, v])
        ag = _Lib(load_library("attention_generic.cu"))
        self._attention_generic = ag.function(
            "cie_attention_generic",
            [v, i, v, i, v, v, v, v, v, i, i, i, i, i, i, i, f, i, i, v, v],
        )
        self._sample = None   # sampling.cu is built when something is first sampled
        self._tensor_gemm = None
        self._fold_gemm_held = None
        # from this many rows on, projections fold the residual add / the norm / the activation
        # into the persistent tcgen05 kernel instead of running library products and separate
        # kernels (0: never)
        self.fold_rows = int(os.environ.get("CIE_FOLD_ROWS", "0"))
        # which products of 17 to 256 rows go to the weight-streaming tcgen05 kernel instead of the
        # library: "0" none, "gate_up" the gate/up product with its activation (the default: 64
        # requests decode in 3.23 instead of 3.31 ms a step, 32 in 2.80 instead of 2.88; a prompt in
        # 256-token portions takes 24.7 instead of 25.0 ms), "all" every product (for measurements)
        self.skinny_products = os.environ.get("CIE_SKINNY", "gate_up")
        if self.skinny_products == "0":
            self.skinny_products = ""
        self._skinny = None
        self._tensor_attention: dict[int, Any] = {}
        self._gemm_stream = None
        self._gemm_stream_ex = None
        self._gemm_stream_rope = None
        self.fuse_norm = False
        self._partial_buffers: dict[str, Any] = {}
        self.scratch_frozen = False
        self.scratch_generation = 0   # counts scratch buffers replaced by larger ones
        self.program = None           # recorder of decode programs (native/program.py), made on first use
        if self.code == BF16 and self.gemm_mode != "simt":
            st = _Lib(load_library("gemm_stream.cu"))
            self._gemm_stream = st.function("cie_gemm_stream", [v, v, v, v, i, i, i, i, i, i, v, v])
            self._gemm_stream_ex = st.function(
                "cie_gemm_stream_ex", [v, v, i, f, v, v, v, v, v, v, v, i, i, i, i, i, i, i, v, v])
            self._gemm_stream_rope = st.function(
                "cie_gemm_stream_rope",
                [v, v, i, f, v, v, v, i, v, v, v, i, i, v, v, v, i, i, i, i, i, i, i, i, i, v, v])
            self.fuse_norm = os.environ.get("CIE_FUSE_NORM", "1") != "0"
        if self.code == BF16 and self.gemm_mode == "tensor":
            from .tensor_gemm import TensorGemm

            self._tensor_gemm = TensorGemm(self)

    # ------------------------------------------------------------------ helpers
    @property
    def stream(self) -> int:
        return self.torch.cuda.current_stream(self.device).cuda_stream

    # ------------------------------------------------------------------ decode programs
    def begin_program(self, ctx: Any) -> bool:
        """Starts recording the streaming products and the decode attention of this step instead of
        launching them (see native/program.py), if the step is one the persistent kernel takes: a
        bfloat16 step of at most 16 tokens, each the single next token of its request.  Everything
        else that runs through ``Ops`` meanwhile flushes what was recorded first.  ``end_program``
        runs the rest."""
        from . import program

        if (self.code != BF16 or self._gemm_stream is None or not self.fuse_norm or not program.enabled()
                or ctx.num_tokens > program.MAX_ROWS or ctx.num_tokens != ctx.num_requests
                or ctx.num_single != ctx.num_requests):
            return False
        if self.program is None:
            self.program = program.DecodeProgram(self)
        self.program.begin()
        return True

    def end_program(self) -> None:
        if self.program is not None:
            self.program.end()

    def _flush(self) -> None:
        """Before a kernel that is not recorded: what was recorded so far runs first."""
        if self.program is not None and self.program.calls:
            self.program.flush()

    @property
    def recording(self) -> bool:
        return self.program is not None and self.program.recording

    def _code_of(self, tensor: Any) -> int:
        if tensor.dtype == self.torch.float32:
            return F32
        if tensor.dtype == self.torch.bfloat16:
            return BF16
        raise KernelError(f"unsupported tensor dtype {tensor.dtype}")

    def prepare_weight(self, weight: Any) -> Any:
        """A matrix [N, K] as the matrix products want it: compute dtype, contiguous."""
        return weight.to(device=self.device, dtype=self.dtype).contiguous()

    def require_attention(self, head_dim: int) -> None:
        """Builds, at model set-up, the attention kernels a head size needs."""
        if self.code == BF16:
            from . import tensor_attention

            if head_dim not in self._tensor_attention and tensor_attention.supports(head_dim):
                self._tensor_attention[head_dim] = tensor_attention.TensorAttention(self, head_dim)

    def plan_attention(self, host: Any, group: int) -> dict[str, Any]:
        """Integer work lists the attention kernels want in a step's metadata (may be empty)."""
        if self.code != BF16 or host.num_single == host.num_requests:
            return {}
        from . import tensor_attention

        return tensor_attention.plan_tiles(host.query_lens, group, skip=host.num_single)

    def check_errors(self) -> None:
        """Reads the device error word (synchronises) and raises if a kernel flagged a fault."""
        word = int(self.error_word.item())
        if word:
            self.error_word.zero_()
            faults = [name for bit, name in ((1, "a token had no valid cache page"),
                                              (2, "a token id was outside the vocabulary"),
                                              (4, "a request index was outside the batch"),
                                              (8, "a bounded wait for a tensor copy or a tensor-core "
                                                  "product ran out"))
                      if word & bit]
            if word & ~15:
                faults.append(f"unknown bits {word & ~15:#x}")
            raise KernelError("device error word set: " + "; ".join(faults))

    # ------------------------------------------------------------------ kernels
    def embedding(self, token_ids: Any, table: Any, residual: Any, scale: float = 1.0) -> None:
        """residual[t] = table[token_ids[t]] * scale, float32."""
        self._flush()
        tokens, hidden = residual.shape
        self.launches += 1
        self._embedding(_ptr(token_ids), _ptr(table), _ptr(residual), tokens, hidden,
                        table.shape[0], float(scale), self._code_of(table), _ptr(self.error_word), self.stream)

    def shape_logits(self, logits: Any, scale: float = 1.0, softcap: float = 0.0) -> None:
        """logits = softcap * tanh(logits * scale / softcap) (or logits * scale), float32, in place."""
        self._flush()
        if scale == 1.0 and softcap == 0.0:
            return
        self.launches += 1
        self._shape_logits(_ptr(logits), logits.numel(), float(scale), float(softcap), self.stream)

    def residual_sink(self, residual: Any) -> "ResidualSink":
        """The float32 stream as a target that projections may add themselves into."""
        return ResidualSink(residual)

    def add_rmsnorm(self, residual: Any, update: Any, gain: Any, eps: float, out: Any,
                    rows: Any = None) -> None:
        """``update``: None, a tensor [T, H] of the compute dtype, or ``Partials``."""
        self._flush()
        count, hidden = out.shape
        self.launches += 1
        if isinstance(update, Accumulated):
            update = None   # its kernel has added it already
        if isinstance(update, Partials) and update.splits == 0:
            update = self.resolve(update, None)
        if isinstance(update, Partials):
            self._add_rmsnorm(_ptr(residual), _ptr(update.data), update.splits,
                              update.rows * update.width, _ptr(update.bias), _ptr(gain), _ptr(out),
                              _ptr(rows), count, hidden, eps, self._code_of(out), self.stream)
        else:
            self._add_rmsnorm(_ptr(residual), _ptr(update), 0, 0, None, _ptr(gain), _ptr(out),
                              _ptr(rows), count, hidden, eps, self._code_of(out), self.stream)

    def stream_plan(self, m: int, n: int, k: int, allow_partials: bool) -> tuple[int, int] | None:
        """(weight rows per CTA, splits along K) for the streaming kernel, or None if the shape
        is not its kind (more than 16 rows, or K not a multiple of 8)."""
        if self._gemm_stream is None or m > STREAM_MAX_ROWS or k % 8 or k < 8:
            return None
        block_rows = 32
        tiles = -(-n // block_rows)
        splits = 1
        if allow_partials:
            # K is cut until the CTAs fill the slots the device has for them: an SM holds five CTAs
            # of the kernel, one is left free for the kernel that follows
            splits = max(1, min(-(-4 * self.sm_count // tiles), k // 256, 8))
        return block_rows, splits

    def scratch(self, tag: str, elements: int, reserve: int = 0) -> Any:
        """Float32 scratch memory by name.  A buffer is made for ``max(elements, reserve)`` at
        first use and may grow later, but not once ``freeze_scratch`` was called (a CUDA graph
        then holds its address)."""
        torch = self.torch
        held = self._partial_buffers.get(tag)
        if held is None or held.numel() < elements:
            if held is not None and self.scratch_frozen:
                raise KernelError(
                    f"scratch buffer {tag!r} would have to grow from {held.numel()} to {elements} "
                    "elements while a CUDA graph that uses it is alive"
                )
            if held is not None:
                self.scratch_generation += 1
            held = torch.empty(max(elements, reserve, 1), dtype=torch.float32, device=self.device)
            self._partial_buffers[tag] = held
        return held

    def freeze_scratch(self) -> None:
        self.scratch_frozen = True

    def _stream(self, x: Any, weight: Any, bias: Any, out: Any, m: int, n: int, k: int, splits: int,
                mode: int, residual: Any = None, sq: Any = None, scaled: Any = None,
                next_gain: Any = None, early_trigger: bool = False, tag: str = "linear") -> None:
        """One launch of the streaming kernel; ``x`` is a tensor or a ``NormedInput``."""
        row_sq, tiles, eps = None, 0, 0.0
        if isinstance(x, NormedInput):
            row_sq, tiles, eps, x = x.accumulated.sq, x.accumulated.tiles, x.eps, x.accumulated.scaled
        if (self.recording and mode != 2 and weight.data_ptr() % 16 == 0 and (mode != 3 or n % 32 == 0)
                and x.data_ptr() % 16 == 0 and x.stride(0) % 8 == 0):
            self.program.gemm(x, row_sq, tiles, eps, weight, bias, out, residual, sq, scaled, next_gain,
                              m, n, k, mode, tag)
            return
        self._flush()
        self.launches += 1
        self._gemm_stream_ex(_ptr(x), _ptr(row_sq), tiles, eps, _ptr(weight), _ptr(bias), _ptr(out),
                             _ptr(residual), _ptr(sq), _ptr(scaled), _ptr(next_gain), m, n, k, splits,
                             mode, 32, 1 if early_trigger else 0, _ptr(self.error_word), self.stream)

    def linear(self, x: Any, weight: Any, bias: Any, out: Any, allow_partials: bool = False,
               tag: str = "", defer_bias: bool = False, residual: Any = None) -> Any:
        """out[M, N] = x[M, K] @ weight[N, K]^T (+ bias); out is the compute dtype or float32.

        Returns ``out``; or, when ``allow_partials`` and the product was cut along K, a
        ``Partials`` that a consuming kernel adds up (then ``out`` was not written); or, when the
        caller names the ``ResidualSink`` its result is to be added to and the streaming kernel
        takes the shape, an ``Accumulated`` (the sum is in the residual stream, ``out`` was not
        written).  ``x`` may be a ``NormedInput``."""
        m, k = x.shape
        n = weight.shape[0]
        if weight.shape[1] != k or tuple(out.shape) != (m, n):
            raise KernelError(f"linear: shapes x{tuple(x.shape)} w{tuple(weight.shape)} out{tuple(out.shape)}")
        if m == 0:
            return out
        plan = self.stream_plan(m, n, k, allow_partials) if self.code == BF16 else None
        if plan is None and self.code == BF16 and self.fold_rows and m >= self.fold_rows:
            done = self._linear_folded(x, weight, bias, out, m, n, k, allow_partials, tag, residual)
            if done is not None:
                return done
        if plan is None and isinstance(x, NormedInput):
            x = x.materialize()
        if plan is not None:
            block_rows, splits = plan
            if residual is not None and self.fuse_norm and allow_partials and m <= FUSED_RESIDUAL_MAX_ROWS:
                cluster = 1
                while cluster * 2 <= splits:
                    cluster *= 2
                tiles = -(-n // 32)
                sq = self.scratch("sq." + (tag or "linear"), m * tiles, reserve=STREAM_MAX_ROWS * tiles)
                gain = residual.gain if n % 8 == 0 else None
                scaled = None
                if gain is not None:
                    scaled = self.scratch("scaled." + (tag or "linear"), (m * n + 1) // 2,
                                          reserve=STREAM_MAX_ROWS * n // 2)
                    scaled = scaled.view(self.torch.bfloat16)[: m * n].view(m, n)
                self._stream(x, weight, bias, None, m, n, k, cluster, 4, residual=residual.tensor, sq=sq,
                             scaled=scaled, next_gain=gain, early_trigger=residual.early_trigger,
                             tag=tag or "linear")
                return Accumulated(residual.tensor, sq, tiles, scaled, gain)
            if splits > 1:
                scratch = self.scratch("partials." + (tag or "linear"), splits * m * n,
                                       reserve=splits * STREAM_MAX_ROWS * n)
                self._stream(x, weight, None, scratch, m, n, k, splits, 2)
                return Partials(scratch, splits, m, n, bias)
            self._stream(x, weight, bias, out, m, n, k, 1, 1 if out.dtype == self.torch.float32 else 0,
                         tag=tag or "linear")
            return out
        self._flush()
        if self.skinny_products == "all" and self.code == BF16 and x.dtype == self.torch.bfloat16:
            skinny = self._skinny_gemm()
            if skinny.supports(x, weight, m, n, k, False, out):
                skinny.launch(x, weight, bias, out, 1 if out.dtype == self.torch.float32 else 0)
                return out
        if self._tensor_gemm is not None and self._tensor_gemm.run(x, weight, bias, out):
            return out
        if self.gemm_mode == "cublas" and self.code == BF16:
            if defer_bias and bias is not None and out.dtype == self.dtype:
                self._cublas_linear(x, weight, None, out)
                return Partials(out, 0, m, n, bias)   # the consumer adds the bias in float32
            self._cublas_linear(x, weight, bias, out)
            return out
        self.launches += 1
        self._gemm_simt(_ptr(x), _ptr(weight), _ptr(bias), _ptr(out), m, n, k, self._code_of(x),
                        self._code_of(out), 0 if self.code == F32 else 1, self.stream)
        return out

    def _skinny_gemm(self) -> Any:
        if self._skinny is None:
            from .skinny import SkinnyGemm

            self._skinny = SkinnyGemm(self)
        return self._skinny

    def _fold_gemm(self) -> Any:
        if self._tensor_gemm is not None:
            return self._tensor_gemm
        if self._fold_gemm_held is None:
            from .tensor_gemm import TensorGemm

            self._fold_gemm_held = TensorGemm(self)
        return self._fold_gemm_held

    def _linear_folded(self, x: Any, weight: Any, bias: Any, out: Any, m: int, n: int, k: int,
                       allow_partials: bool, tag: str, residual: Any) -> Any:
        """Many rows on the persistent tcgen05 kernel where that saves a whole pass over the
        activations: a projection that adds itself into the residual stream, or a product whose
        input rows are still to be divided by their root mean square.  None: not its case."""
        self._flush()
        gemm = self._fold_gemm()
        if k % 8 or weight.data_ptr() % 16:
            return None
        if isinstance(x, NormedInput):
            acc = x.accumulated
            gemm.launch_fused(acc.scaled, weight, bias, out, 1 if out.dtype == self.torch.float32 else 0,
                              row_sq=acc.sq, row_tiles=acc.tiles, eps=x.eps)
            return out
        if residual is not None and allow_partials and self.fuse_norm and x.data_ptr() % 16 == 0:
            tiles = -(-n // 32)
            sq = self.scratch("sq.rows." + (tag or "linear"), m * tiles)
            gain = residual.gain if n % 8 == 0 else None
            scaled = None
            if gain is not None:
                scaled = self.scratch("scaled.rows." + (tag or "linear"), (m * n + 1) // 2)
                scaled = scaled.view(self.torch.bfloat16)[: m * n].view(m, n)
            gemm.launch_fused(x, weight, bias, None, 4, residual=residual.tensor, sq=sq, scaled=scaled, next_gain=gain)
            return Accumulated(residual.tensor, sq, tiles, scaled, gain)
        return None

    def resolve(self, value: Any, out: Any) -> Any:
        """A plain tensor for a part that cannot consume ``Partials`` itself."""
        self._flush()
        if not isinstance(value, Partials):
            return value
        if value.splits == 0:
            if value.bias is not None:
                value.data.add_(value.bias.to(value.data.dtype))
            return value.data
        total = value.data[: value.splits * value.rows * value.width].view(value.splits, value.rows, value.width).sum(0)
        if value.bias is not None:
            total = total + value.bias
        out.copy_(total)
        return out

    def prepare_gate_up(self, gate: Any, up: Any) -> GateUpWeight:
        """Stacks gate and up; for bfloat16, interleaved in blocks of 16 rows when the channel
        count allows, so that the streaming kernel can apply SiLU(gate) * up in its epilogue."""
        torch = self.torch
        inter = gate.shape[0]
        block = inter
        if self._gemm_stream is not None and inter % 16 == 0:
            block = 16
            hidden = gate.shape[1]
            stacked = torch.stack([gate.view(inter // block, block, hidden),
                                   up.view(inter // block, block, hidden)], dim=1)
            weight = stacked.reshape(2 * inter, hidden)
        else:
            weight = torch.cat([gate, up])
        return GateUpWeight(self.prepare_weight(weight), inter, block)

    def gate_up(self, x: Any, weight: GateUpWeight, hidden_out: Any, workspace: Any) -> Any:
        """hidden_out[T, I] = SiLU(x Wg^T) * (x Wu^T)."""
        m, k = x.shape
        inter = weight.inter
        if self.code == BF16 and weight.block == 16:
            plan = self.stream_plan(m, 2 * inter, k, False)
            if plan is not None:
                self._stream(x, weight.weight, None, hidden_out, m, 2 * inter, k, 1, 3, tag="gate_up")
                return hidden_out
        if (isinstance(x, NormedInput) and self.code == BF16 and weight.block == 16 and self.fold_rows
                and m >= self.fold_rows and k % 8 == 0):
            acc = x.accumulated
            self._flush()
            self._fold_gemm().launch_fused(acc.scaled, weight.weight, None, hidden_out, 3, row_sq=acc.sq,
                                              row_tiles=acc.tiles, eps=x.eps)
            return hidden_out
        if isinstance(x, NormedInput):
            x = x.materialize()
        if self.skinny_products and self.code == BF16 and weight.block == 16 and x.dtype == self.torch.bfloat16:
            skinny = self._skinny_gemm()
            if skinny.supports(x, weight.weight, m, 2 * inter, k, True, hidden_out):
                self._flush()
                skinny.launch(x, weight.weight, None, hidden_out, 3)
                return hidden_out
        both = workspace.get("swiglu.gate_up", m, 2 * inter, self.dtype)
        self.linear(x, weight.weight, None, both)
        self.silu_mul(both, hidden_out, weight.block)
        return hidden_out

    def _cublas_linear(self, x: Any, weight: Any, bias: Any, out: Any) -> None:
        """Library matrix product (cuBLAS through torch), as the reference uses for every
        projection; kept as a yardstick for the hand-written tensor-core kernel."""
        self._flush()
        torch = self.torch
        if out.dtype == torch.float32:
            torch.mm(x, weight.t(), out_dtype=torch.float32, out=out)   # float32 straight into the caller's buffer
        else:
            torch.mm(x, weight.t(), out=out)
        if bias is not None:
            out.add_(bias.to(out.dtype))

    def rope_kv_write(self, qkv: Any, ctx: Any, kv: Any, position: Any, q_heads: int,
                      kv_heads: int, head_dim: int, write_cache: bool = True,
                      q_buffer: Any = None, paired: bool = False) -> Any:
        """Rotates q and k, writes k and v into the pages; returns the tensor that holds the
        rotated q (head h of token t at [t, h * head_dim]).  ``qkv`` is a tensor (q is rotated in
        place) or ``Partials`` (then q goes to ``q_buffer``).  ``paired``: the q and k columns of
        ``qkv`` are in the paired layout of ``pair_rotary_rows``; q then always goes to ``q_buffer``."""
        self._flush()
        rot = position.rotary_dim if position is not None else 0
        inv_freq = position.inv_freq if position is not None else None
        table = ctx.block_tables[kv.group]
        self.launches += 1
        if isinstance(qkv, Partials) and qkv.splits == 0:
            tokens = qkv.rows
            src, splits, stride, bias = qkv.data, 0, 0, qkv.bias
            target = qkv.data
        elif isinstance(qkv, Partials):
            tokens = qkv.rows
            src, splits, stride, bias = qkv.data, qkv.splits, qkv.rows * qkv.width, qkv.bias
            target = q_buffer
        else:
            tokens = qkv.shape[0]
            src, splits, stride, bias = qkv, 0, 0, None
            target = qkv
        if paired:
            if q_buffer is None:
                raise KernelError("rope_kv_write: the paired layout needs a q buffer")
            target = q_buffer
        self._rope_kv_write(_ptr(src), splits, stride, _ptr(bias), _ptr(target), target.shape[1],
                            _ptr(ctx.positions), _ptr(ctx.request_of_token), _ptr(table),
                            table.shape[1], kv.num_pages, _ptr(kv.k), _ptr(kv.v), _ptr(inv_freq),
                            tokens, q_heads, kv_heads, head_dim, rot, kv.page_size,
                            1 if write_cache else 0, 1 if paired else 0, self._code_of(target),
                            _ptr(self.error_word), self.stream)
        return target

    # ------------------------------------------------------------------ rotary epilogue of the q/k/v product
    def can_pair_rotary(self, head_dim: int, rotary_dim: int) -> bool:
        """Whether the stacked q/k/v weight of an attention layer may be kept in the paired
        layout, which lets a decode step rotate and store inside the projection's own kernel."""
        return (self._gemm_stream_rope is not None and os.environ.get("CIE_FUSE_ROPE", "1") != "0"
                and head_dim % 32 == 0 and rotary_dim % 32 == 0 and 32 <= rotary_dim <= head_dim)

    def pair_rotary_rows(self, rows: Any, heads: int, head_dim: int, rotary_dim: int) -> Any:
        """Rows [heads * head_dim, ...] of a q or k projection (weight or bias) in the paired
        layout: inside every head, blocks of 16 rotary elements followed by their 16 partners."""
        torch = self.torch
        half = rotary_dim // 2
        order = torch.empty(head_dim, dtype=torch.long)
        for d in range(head_dim):
            if d >= rotary_dim:
                column = d
            elif d < half:
                column = (d // 16) * 32 + d % 16
            else:
                column = ((d - half) // 16) * 32 + 16 + (d - half) % 16
            order[column] = d
        index = (torch.arange(heads).view(-1, 1) * head_dim + order.view(1, -1)).reshape(-1).to(rows.device)
        return rows.index_select(0, index).contiguous()

    def qkv_rope(self, x: Any, weight: Any, bias: Any, ctx: Any, kv: Any, position: Any, q_heads: int,
                 kv_heads: int, head_dim: int, write_cache: bool, q_buffer: Any) -> Any:
        """The stacked q/k/v projection (paired layout) of a few decode tokens, rotated and stored
        by the product's own kernel; returns ``q_buffer``, or None when the shape is not its kind
        (the caller then runs the product and ``rope_kv_write(..., paired=True)``)."""
        m, k = x.shape
        n = weight.shape[0]
        if (self._gemm_stream_rope is None or position is None or m > FUSED_RESIDUAL_MAX_ROWS
                or self.stream_plan(m, n, k, True) is None
                or not self.can_pair_rotary(head_dim, position.rotary_dim)):
            return None
        tiles, k_tiles = -(-n // 32), -(-k // 128)
        # K slices per block of weight rows (the size of a cluster): about two and a half CTAs an SM
        # was measured best for this small product (its successor, attention, cannot start beside it)
        splits = 8
        while splits > 1 and (2 * tiles * splits > 5 * self.sm_count or k_tiles // splits < 2):
            splits //= 2
        row_sq, row_tiles, eps = None, 0, 0.0
        if isinstance(x, NormedInput):
            row_sq, row_tiles, eps, x = x.accumulated.sq, x.accumulated.tiles, x.eps, x.accumulated.scaled
        table = ctx.block_tables[kv.group]
        if self.recording and weight.data_ptr() % 16 == 0 and x.data_ptr() % 16 == 0 and x.stride(0) % 8 == 0:
            self.program.rope(x, row_sq, row_tiles, eps, weight, bias, q_buffer, ctx.positions,
                              ctx.request_of_token, table, kv.num_pages, kv.k, kv.v, position.inv_freq, m,
                              q_heads, kv_heads, head_dim, position.rotary_dim, kv.page_size, write_cache, k)
            return q_buffer
        self._flush()
        self.launches += 1
        self._gemm_stream_rope(_ptr(x), _ptr(row_sq), row_tiles, eps, _ptr(weight), _ptr(bias),
                               _ptr(q_buffer), q_buffer.shape[1], _ptr(ctx.positions),
                               _ptr(ctx.request_of_token), _ptr(table), table.shape[1], kv.num_pages,
                               _ptr(kv.k), _ptr(kv.v), _ptr(position.inv_freq), m, q_heads, kv_heads,
                               head_dim, position.rotary_dim, kv.page_size, 1 if write_cache else 0, k,
                               splits, _ptr(self.error_word), self.stream)
        return q_buffer

    def attention(self, qkv: Any, out: Any, ctx: Any, kv: Any, q_heads: int, kv_heads: int,
                  head_dim: int, scale: float, window: int) -> None:
        fast = self._tensor_attention.get(head_dim)
        if fast is None:
            self._flush()
        if fast is not None:
            plan = ctx.extras.get(("attention", q_heads // kv_heads)) or None
            if fast.run(qkv, out, ctx, kv, q_heads, kv_heads, scale, window, plan):
                return
        self.attention_generic(qkv, out, ctx, kv, q_heads, kv_heads, head_dim, scale, window)

    def attention_generic(self, qkv: Any, out: Any, ctx: Any, kv: Any, q_heads: int,
                          kv_heads: int, head_dim: int, scale: float, window: int) -> None:
        self._flush()
        table = ctx.block_tables[kv.group]
        self.launches += 1
        self._attention_generic(_ptr(qkv), qkv.shape[1], _ptr(out), out.shape[1], _ptr(kv.k),
                                _ptr(kv.v), _ptr(ctx.positions), _ptr(ctx.request_of_token),
                                _ptr(table), table.shape[1], kv.num_pages, qkv.shape[0], q_heads,
                                kv_heads, head_dim, kv.page_size, scale, window,
                                self._code_of(qkv), _ptr(self.error_word), self.stream)

    def silu_mul(self, gate_up: Any, out: Any, block: int | None = None) -> None:
        self._flush()
        tokens, inter = out.shape
        self.launches += 1
        self._silu_mul(_ptr(gate_up), _ptr(out), tokens, inter, inter if block is None else block,
                       self._code_of(out), self.stream)

    def _load_sampling(self) -> None:
        if self._sample is None:
            v, i = c_void_p, c_int
            lib = _Lib(load_library("sampling.cu"))
            self._sample = lib.function("cie_sample", [v, i, i, v, v, v, v, v])
            self._feed_tokens = lib.function("cie_feed_tokens", [v, v, i, i, v])
            self._sample_slices = int(lib.handle.cie_sample_slices())

    def sample(self, logits: Any, temperature: Any, keys: Any, out: Any) -> None:
        """logits float32 [R, V]; temperature float32 [R] or None (greedy); keys int64 [R]."""
        self._flush()
        rows, vocab = logits.shape
        self._load_sampling()
        # the row maxima are searched by several CTAs a row first (two launches)
        scratch = self.scratch("sample.maxima", 2 * rows * self._sample_slices, reserve=2 * 1024 * self._sample_slices)
        self.launches += 2 if vocab >= 4096 else 1
        self._sample(_ptr(logits), rows, vocab, _ptr(temperature), _ptr(keys), _ptr(out), _ptr(scratch), self.stream)

    def feed_tokens(self, sampled: Any, token_ids: Any, real: int) -> None:
        """token_ids[i] = sampled[min(i, real - 1)] (int32, on the device): the token ids of a decode step
        that is launched before the step before it has been read back."""
        self._flush()
        self._load_sampling()
        self.launches += 1
        self._feed_tokens(_ptr(sampled), _ptr(token_ids), token_ids.shape[0], real, self.stream)
