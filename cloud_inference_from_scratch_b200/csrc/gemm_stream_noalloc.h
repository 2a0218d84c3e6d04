// cie_gemm_stream_noalloc: the split-K streaming matrix product for callers that cannot allocate.
//
// This entry point has no counterpart in zeeshan8281/cloud-inference-from-scratch; it exists for
// users of this library only.
//
// Who needs it.  The regular entry point, cie_gemm_stream in mode 2, writes float32 partial sums
// into scratch memory that the caller must provide, which in this framework means a torch
// allocation.  Some callers have no way to provide one: code that runs inside another runtime's
// execution callback (an inference plug-in's "enqueue", a custom operator of a host engine that
// hands out only its input and output pointers), and hosts that fixed their device memory budget
// at start-up and forbid cudaMalloc afterwards because it may synchronise the device or fail late.
// For them this variant keeps its scratch inside the library: a file-scope device array of
// CIE_NOALLOC_SCRATCH_FLOATS float32 values (4 MiB), which every GPU that loads the library holds
// from load until the process exits.
//
// What it computes.  out[M, N] (bfloat16) = x[M, K] * w[N, K]^T + bias[N] (bias may be null), with
// the product cut into `splits` slices along K exactly as cie_gemm_stream does, the slices added
// in ascending order in float32, the bias added last, and one rounding to bfloat16.
//
// Limits, checked with a clear error: M <= 16, K a multiple of 8, 1 <= splits <= 8, and
// splits * M * N <= CIE_NOALLOC_SCRATCH_FLOATS.
//
// Rules of use.
//  * The call allocates nothing: no cudaMalloc, no cudaFree, no allocating library routine.
//  * The first call on each device looks up the device address of the scratch array
//    (cudaGetSymbolAddress, with that device current) and keeps it; make that first call once
//    during set-up, outside of any stream capture.
//  * All calls share the one array, and it keeps what the last call left in it.  Nothing has to
//    start at zero: every element a call reads was written by that same call.  Two calls whose
//    kernels can overlap on the GPU (different streams, or the same stream with programmatic
//    dependent launch between them) race on the array: order them yourself.
//  * x, w and out are the caller's device pointers, 16-byte aligned; `stream` is a cudaStream_t.
//
// Returns 0, or 1 with the reason available from cie_last_error().
#pragma once

#ifdef __cplusplus
extern "C" {
#endif

#define CIE_NOALLOC_SCRATCH_FLOATS (1 << 20)

int cie_gemm_stream_noalloc(const void* x, const void* w, const float* bias, void* out, int m, int n,
                            int k, int splits, void* stream);

#ifdef __cplusplus
}
#endif
