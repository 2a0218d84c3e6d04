// Shared helpers of the sm_100a kernels: element types, conversions, reductions, error reporting.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <cstdio>
#include <cstdlib>

namespace cie {

// Element type codes passed through the C interface.
constexpr int kFloat32 = 0;
constexpr int kBFloat16 = 1;

// Bits of the device error word that kernels set instead of trapping.
constexpr int kErrBadPage = 1;      // a block-table entry needed by a token was < 0 or too large
constexpr int kErrBadToken = 2;     // a token id outside the vocabulary
constexpr int kErrBadRequest = 4;   // a request index outside the batch

template <typename T>
__device__ __forceinline__ float to_float(T v);
template <>
__device__ __forceinline__ float to_float<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_float<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T>
__device__ __forceinline__ T from_float(float v);
template <>
__device__ __forceinline__ float from_float<float>(float v) { return v; }
template <>
__device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int offset = 16; offset > 0; offset >>= 1) v += __shfl_xor_sync(0xffffffffu, v, offset);
  return v;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int offset = 16; offset > 0; offset >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, offset));
  return v;
}

// Block-wide sum for blocks of up to 1024 threads; every thread gets the result.
// The order of additions depends only on blockDim, never on the data.
__device__ __forceinline__ float block_sum(float v, float* scratch /* >= 33 floats */) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  v = warp_sum(v);
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  const int warps = (blockDim.x + 31) >> 5;
  if (warp == 0) {
    float t = lane < warps ? scratch[lane] : 0.f;
    t = warp_sum(t);
    if (lane == 0) scratch[32] = t;
  }
  __syncthreads();
  const float total = scratch[32];
  __syncthreads();
  return total;
}

// Programmatic dependent launch.  A kernel launched with the attribute may start while the
// kernel before it in the stream is still running; `pdl_wait` blocks until that kernel (and, through
// its own wait, every earlier one) has completed and its writes are visible.  Before the wait a
// kernel may only do what does not depend on earlier kernels and writes nothing they read:
// set-up and prefetching what earlier kernels do not write.  `pdl_trigger` lets the next kernel in
// the stream start its own set-up.  Kernels trigger AFTER their own wait: a kernel can then
// overlap only the ONE kernel before it (whose own predecessors have all completed).  Two kinds of
// kernel trigger first (the RMSNorm kernel and the streaming product with the residual epilogue),
// because what follows them is a product whose early part only asks for weights; the kernel after
// that one waits before it triggers, so never more than two kernels back are still running.
// The early loads (weight tiles; key/value tiles of earlier steps) stay valid under that.
// Without the launch attribute both are no-ops.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

inline bool pdl_enabled() {
  static const bool enabled = [] {
    const char* value = getenv("CIE_PDL");
    return !(value && value[0] == '0');
  }();
  return enabled;
}

// Launches `kernel` on `stream`, as a programmatic dependent of the kernel before it unless
// CIE_PDL=0 is set in the environment.
template <typename... KArgs, typename... Args>
inline cudaError_t launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                          cudaStream_t stream, Args... args) {
  cudaLaunchConfig_t config = {};
  config.gridDim = grid;
  config.blockDim = block;
  config.dynamicSmemBytes = smem;
  config.stream = stream;
  cudaLaunchAttribute attribute[1];
  attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attribute[0].val.programmaticStreamSerializationAllowed = 1;
  config.attrs = attribute;
  config.numAttrs = pdl_enabled() ? 1 : 0;
  return cudaLaunchKernelEx(&config, kernel, KArgs(args)...);
}

}  // namespace cie

// Every library keeps the text of its last failure for the Python side to raise.
#define CIE_DEFINE_LAST_ERROR()                                                       \
  static thread_local char cie_error_text[512] = "";                                  \
  extern "C" const char* cie_last_error() { return cie_error_text; }

#define CIE_FAIL(...)                                                                 \
  do {                                                                                \
    snprintf(cie_error_text, sizeof(cie_error_text), __VA_ARGS__);                    \
    return 1;                                                                         \
  } while (0)

#define CIE_LAUNCH(name, ...)                                                         \
  do {                                                                                \
    cudaError_t cie_status = cie::launch(__VA_ARGS__);                                \
    if (cie_status != cudaSuccess)                                                    \
      CIE_FAIL("%s: launch failed: %s", name, cudaGetErrorString(cie_status));        \
  } while (0)

#define CIE_CHECK_LAUNCH(name)                                                        \
  do {                                                                                \
    cudaError_t cie_status = cudaGetLastError();                                      \
    if (cie_status != cudaSuccess)                                                    \
      CIE_FAIL("%s: launch failed: %s", name, cudaGetErrorString(cie_status));        \
  } while (0)
