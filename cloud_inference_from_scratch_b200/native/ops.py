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
from ctypes import c_float, c_int, c_void_p
from typing import Any

from .build import load_library

F32, BF16 = 0, 1


class KernelError(RuntimeError):
    pass


def _ptr(tensor: Any) -> int | None:
    return None if tensor is None else tensor.data_ptr()


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
        self.gemm_mode = gemm or ("simt" if self.code == F32 else "cublas")
        if self.code == F32 and self.gemm_mode != "simt":
            raise KernelError("the 32-bit path multiplies on the CUDA cores only (gemm='simt')")
        if self.gemm_mode not in ("simt", "tensor", "cublas"):
            raise KernelError(f"unknown gemm mode {self.gemm_mode!r}")
        self.error_word = torch.zeros(1, dtype=torch.int32, device=self.device)
        self.launches = 0

        v, i, f = c_void_p, c_int, c_float
        ew = _Lib(load_library("elementwise.cu"))
        self._embedding = ew.function("cie_embedding", [v, v, v, i, i, i, i, v, v])
        self._add_rmsnorm = ew.function("cie_add_rmsnorm", [v, v, v, v, v, i, i, f, i, v])
        self._rope_kv_write = ew.function(
            "cie_rope_kv_write", [v, v, v, v, i, i, v, v, v, i, i, i, i, i, i, i, i, v, v]
        )
        self._silu_mul = ew.function("cie_silu_mul", [v, v, i, i, i, v])
        gs = _Lib(load_library("gemm_simt.cu"))
        self._gemm_simt = gs.function("cie_gemm_simt", [v, v, v, v, i, i, i, i, i, i, v])
        ag = _Lib(load_library("attention_generic.cu"))
        self._attention_generic = ag.function(
            "cie_attention_generic",
            [v, i, v, i, v, v, v, v, v, i, i, i, i, i, i, i, f, i, i, v, v],
        )
        sm = _Lib(load_library("sampling.cu"))
        self._sample = sm.function("cie_sample", [v, i, i, v, v, v, v])
        self._tensor_gemm = None
        self._tensor_attention: dict[int, Any] = {}
        if self.code == BF16 and self.gemm_mode == "tensor":
            from .tensor_gemm import TensorGemm

            self._tensor_gemm = TensorGemm(self)

    # ------------------------------------------------------------------ helpers
    @property
    def stream(self) -> int:
        return self.torch.cuda.current_stream(self.device).cuda_stream

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
        if self.code != BF16 or bool((host.query_lens == 1).all()):
            return {}
        from . import tensor_attention

        return tensor_attention.plan_tiles(host.query_lens, group)

    def check_errors(self) -> None:
        """Reads the device error word (synchronises) and raises if a kernel flagged a fault."""
        word = int(self.error_word.item())
        if word:
            self.error_word.zero_()
            faults = [name for bit, name in ((1, "a token had no valid cache page"),
                                              (2, "a token id was outside the vocabulary"),
                                              (4, "a request index was outside the batch"))
                      if word & bit]
            raise KernelError("device error word set: " + "; ".join(faults))

    # ------------------------------------------------------------------ kernels
    def embedding(self, token_ids: Any, table: Any, residual: Any) -> None:
        tokens, hidden = residual.shape
        self.launches += 1
        self._embedding(_ptr(token_ids), _ptr(table), _ptr(residual), tokens, hidden,
                        table.shape[0], self._code_of(table), _ptr(self.error_word), self.stream)

    def add_rmsnorm(self, residual: Any, update: Any, gain: Any, eps: float, out: Any,
                    rows: Any = None) -> None:
        count, hidden = out.shape
        self.launches += 1
        self._add_rmsnorm(_ptr(residual), _ptr(update), _ptr(gain), _ptr(out), _ptr(rows), count,
                          hidden, eps, self._code_of(out), self.stream)

    def linear(self, x: Any, weight: Any, bias: Any, out: Any) -> None:
        """out[M, N] = x[M, K] @ weight[N, K]^T (+ bias); out is the compute dtype or float32."""
        m, k = x.shape
        n = weight.shape[0]
        if weight.shape[1] != k or tuple(out.shape) != (m, n):
            raise KernelError(f"linear: shapes x{tuple(x.shape)} w{tuple(weight.shape)} out{tuple(out.shape)}")
        if m == 0:
            return
        if self._tensor_gemm is not None and self._tensor_gemm.run(x, weight, bias, out):
            return
        if self.gemm_mode == "cublas" and self.code == BF16:
            self._cublas_linear(x, weight, bias, out)
            return
        self.launches += 1
        self._gemm_simt(_ptr(x), _ptr(weight), _ptr(bias), _ptr(out), m, n, k, self._code_of(x),
                        self._code_of(out), 0 if self.code == F32 else 1, self.stream)

    def _cublas_linear(self, x: Any, weight: Any, bias: Any, out: Any) -> None:
        """Library matrix product (cuBLAS through torch), as the reference uses for every
        projection; kept as a yardstick for the hand-written tensor-core kernel."""
        torch = self.torch
        if out.dtype == torch.float32:
            out.copy_(torch.mm(x, weight.t(), out_dtype=torch.float32))
        else:
            torch.mm(x, weight.t(), out=out)
        if bias is not None:
            out.add_(bias.to(out.dtype))

    def rope_kv_write(self, qkv: Any, ctx: Any, kv: Any, position: Any, q_heads: int,
                      kv_heads: int, head_dim: int, write_cache: bool = True) -> None:
        tokens = qkv.shape[0]
        rot = position.rotary_dim if position is not None else 0
        inv_freq = position.inv_freq if position is not None else None
        table = ctx.block_tables[kv.group]
        self.launches += 1
        self._rope_kv_write(_ptr(qkv), _ptr(ctx.positions), _ptr(ctx.request_of_token), _ptr(table),
                            table.shape[1], kv.num_pages, _ptr(kv.k), _ptr(kv.v), _ptr(inv_freq),
                            tokens, q_heads, kv_heads, head_dim, rot, kv.page_size,
                            1 if write_cache else 0, self._code_of(qkv), _ptr(self.error_word),
                            self.stream)

    def attention(self, qkv: Any, out: Any, ctx: Any, kv: Any, q_heads: int, kv_heads: int,
                  head_dim: int, scale: float, window: int) -> None:
        fast = self._tensor_attention.get(head_dim)
        if fast is not None:
            plan = ctx.extras.get(("attention", q_heads // kv_heads)) or None
            if fast.run(qkv, out, ctx, kv, q_heads, kv_heads, scale, window, plan):
                return
        self.attention_generic(qkv, out, ctx, kv, q_heads, kv_heads, head_dim, scale, window)

    def attention_generic(self, qkv: Any, out: Any, ctx: Any, kv: Any, q_heads: int,
                          kv_heads: int, head_dim: int, scale: float, window: int) -> None:
        table = ctx.block_tables[kv.group]
        self.launches += 1
        self._attention_generic(_ptr(qkv), qkv.shape[1], _ptr(out), out.shape[1], _ptr(kv.k),
                                _ptr(kv.v), _ptr(ctx.positions), _ptr(ctx.request_of_token),
                                _ptr(table), table.shape[1], kv.num_pages, qkv.shape[0], q_heads,
                                kv_heads, head_dim, kv.page_size, scale, window,
                                self._code_of(qkv), _ptr(self.error_word), self.stream)

    def silu_mul(self, gate_up: Any, out: Any) -> None:
        tokens, inter = out.shape
        self.launches += 1
        self._silu_mul(_ptr(gate_up), _ptr(out), tokens, inter, self._code_of(out), self.stream)

    def sample(self, logits: Any, temperature: Any, keys: Any, out: Any) -> None:
        """logits float32 [R, V]; temperature float32 [R] or None (greedy); keys int64 [R]."""
        rows, vocab = logits.shape
        self.launches += 1
        self._sample(_ptr(logits), rows, vocab, _ptr(temperature), _ptr(keys), _ptr(out), self.stream)
