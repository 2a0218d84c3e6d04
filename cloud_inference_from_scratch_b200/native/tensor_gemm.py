"""Python side of the tcgen05 matrix product (csrc/gemm_tcgen05.cu)."""

from __future__ import annotations

from ctypes import c_float, c_int, c_void_p
from typing import Any

from .build import load_library

OUT_BF16, OUT_F32, OUT_PARTIAL, OUT_SILU_MUL, OUT_RESIDUAL = 0, 1, 2, 3, 4


class TensorGemm:
    def __init__(self, ops: Any) -> None:
        from .ops import _Lib

        self.ops = ops
        lib = _Lib(load_library("gemm_tcgen05.cu"))
        v, i = c_void_p, c_int
        self._gemm = lib.function("cie_gemm_tcgen05", [v, v, v, v, i, i, i, i, i, v, v])
        self._gemm_ex = lib.function("cie_gemm_tcgen05_ex", [v, v, i, c_float, v, v, v, v, v, v, v, i, i, i, i, v, v])

    @staticmethod
    def supports(x: Any, weight: Any) -> bool:
        k = x.shape[1]
        return k % 8 == 0 and k >= 8 and x.data_ptr() % 16 == 0 and weight.data_ptr() % 16 == 0

    def launch(self, x: Any, weight: Any, bias: Any, out: Any, mode: int, splits: int = 1) -> None:
        ops = self.ops
        m, k = x.shape
        n = weight.shape[0]
        ops.launches += 1
        self._gemm(x.data_ptr(), weight.data_ptr(), None if bias is None else bias.data_ptr(),
                   out.data_ptr(), m, n, k, mode, splits, ops.error_word.data_ptr(), ops.stream)

    def launch_fused(self, x: Any, weight: Any, bias: Any, out: Any, mode: int, row_sq: Any = None,
                     row_tiles: int = 0, eps: float = 0.0, residual: Any = None, sq: Any = None,
                     scaled: Any = None, next_gain: Any = None) -> None:
        """More than 64 rows on the persistent kernel with what it can fold in: a scale per result
        row formed from sums of squares, SiLU(gate) * up, or the add into the float32 residual
        stream that leaves the sums of squares and the rows times the next norm's gain."""
        ops = self.ops
        m, k = x.shape
        n = weight.shape[0]

        def ptr(tensor: Any) -> Any:
            return None if tensor is None else tensor.data_ptr()

        ops.launches += 1
        self._gemm_ex(x.data_ptr(), ptr(row_sq), row_tiles, eps, weight.data_ptr(), ptr(bias), ptr(out),
                      ptr(residual), ptr(sq), ptr(scaled), ptr(next_gain), m, n, k, mode,
                      ops.error_word.data_ptr(), ops.stream)

    def run(self, x: Any, weight: Any, bias: Any, out: Any) -> bool:
        """out = x @ weight^T + bias for any number of rows; False if the shape is not its kind."""
        torch = self.ops.torch
        if x.dtype != torch.bfloat16 or not self.supports(x, weight):
            return False
        self.launch(x, weight, bias, out, OUT_F32 if out.dtype == torch.float32 else OUT_BF16)
        return True
