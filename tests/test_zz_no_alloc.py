"""The entry point that allocates nothing (csrc/gemm_stream_noalloc.h), called through its exported
C symbol and compared with the regular entry point, on two calls in a row.

Some users of the library cannot hand it scratch memory: code inside another runtime's execution
callback that sees only its input and output pointers, or a host that forbids cudaMalloc after
start-up.  For them ``cie_gemm_stream_noalloc`` keeps the partial sums of the split product in an
array inside the library.  The file is named so that pytest collects it last: a run that stops at
the first failure has then already run every other test.
"""

import ctypes
from ctypes import c_int, c_void_p

import pytest
import torch

pytestmark = pytest.mark.gpu


def load():
    from cloud_inference_from_scratch_b200.native.build import load_library

    lib = load_library("gemm_stream.cu")
    lib.cie_last_error.restype = ctypes.c_char_p
    v, i = c_void_p, c_int
    lib.cie_gemm_stream_noalloc.argtypes = [v, v, v, v, i, i, i, i, v]
    lib.cie_gemm_stream_noalloc.restype = c_int
    lib.cie_gemm_stream.argtypes = [v, v, v, v, i, i, i, i, i, i, v, v]
    lib.cie_gemm_stream.restype = c_int
    return lib


def regular(lib, x, w, bias, splits):
    """The existing entry point: partial sums into scratch that the caller allocated."""
    m, k = x.shape
    n = w.shape[0]
    parts = torch.empty(splits, m, n, dtype=torch.float32, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    status = lib.cie_gemm_stream(x.data_ptr(), w.data_ptr(), None, parts.data_ptr(), m, n, k, splits, 2, 32, None, stream)
    assert status == 0, lib.cie_last_error().decode()
    total = parts[0].clone()
    for s in range(1, splits):
        total += parts[s]
    return (total + bias).to(torch.bfloat16)


def test_noalloc_entry_point_matches_the_regular_one_twice():
    lib = load()
    torch.cuda.synchronize()
    stream = torch.cuda.current_stream().cuda_stream
    for call, (m, n, k, splits) in enumerate([(8, 2560, 2048, 4), (3, 2048, 11008, 8)]):
        generator = torch.Generator().manual_seed(call)
        x = torch.randn(m, k, generator=generator).to(torch.bfloat16).cuda()
        w = (torch.randn(n, k, generator=generator) * 0.05).to(torch.bfloat16).cuda()
        bias = torch.randn(n, generator=generator).cuda()
        out = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device="cuda")
        before = torch.cuda.memory_allocated()
        status = lib.cie_gemm_stream_noalloc(x.data_ptr(), w.data_ptr(), bias.data_ptr(), out.data_ptr(),
                                             m, n, k, splits, stream)
        assert status == 0, lib.cie_last_error().decode()
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == before
        want = regular(lib, x, w, bias, splits)
        torch.cuda.synchronize()
        torch.testing.assert_close(out.float(), want.float(), rtol=2e-2, atol=2e-2)
        reference = (x.float() @ w.float().t() + bias).to(torch.bfloat16)
        torch.testing.assert_close(out.float(), reference.float(), rtol=2e-2, atol=2e-2 * float(reference.abs().max()) / 4)


def test_noalloc_entry_point_refuses_what_does_not_fit():
    lib = load()
    x = torch.zeros(16, 64, dtype=torch.bfloat16, device="cuda")
    w = torch.zeros(100000, 64, dtype=torch.bfloat16, device="cuda")
    out = torch.zeros(16, 100000, dtype=torch.bfloat16, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    assert lib.cie_gemm_stream_noalloc(x.data_ptr(), w.data_ptr(), None, out.data_ptr(), 16, 100000, 64, 1, stream) == 1
    assert b"exceed the built-in scratch" in lib.cie_last_error()
    assert lib.cie_gemm_stream_noalloc(x.data_ptr(), w.data_ptr(), None, out.data_ptr(), 17, 8, 64, 1, stream) == 1
    assert b"at most 16 rows" in lib.cie_last_error()
    assert lib.cie_gemm_stream_noalloc(x.data_ptr(), w.data_ptr(), None, out.data_ptr(), 4, 8, 64, 9, stream) == 1
    assert b"splits" in lib.cie_last_error()
