// C[M,N] = A[M,K] * W[N,K]^T (+ bias[N]) on the CUDA cores, float32 accumulation, any M, N, K.
//
// This is the whole-model 32-bit path's matrix product (no tensor cores, no TF32) and the
// fallback of the bfloat16 path for shapes the tensor-core kernel refuses.  Each output element
// is the sum over k in ascending order with one fused multiply-add per k, so a row's result does
// not depend on how many other rows the call has or where the row sits in it.
// The reference runs these products through cuBLAS (src/cloud_engine/model.py:100,134-136,217,227).
#include "common.cuh"

CIE_DEFINE_LAST_ERROR()

namespace cie {

constexpr int kTileM = 64, kTileN = 64, kTileK = 16;

template <typename TIn, typename TOut>
__global__ void __launch_bounds__(256)
gemm_simt_kernel(const TIn* __restrict__ a, const TIn* __restrict__ w, const float* __restrict__ bias,
                 TOut* __restrict__ c, int m_total, int n_total, int k_total) {
  __shared__ float a_tile[kTileK][kTileM + 4];
  __shared__ float w_tile[kTileK][kTileN + 4];
  pdl_wait();
  pdl_trigger();
  const int tid = threadIdx.x;
  const int m0 = blockIdx.y * kTileM, n0 = blockIdx.x * kTileN;
  const int tm = (tid / 16) * 4, tn = (tid % 16) * 4;
  float acc[4][4] = {};
  for (int k0 = 0; k0 < k_total; k0 += kTileK) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int e = tid + i * 256;      // 0..1023 over a 64 x 16 tile
      const int r = e / kTileK, kk = e % kTileK;
      const int gk = k0 + kk;
      const int gm = m0 + r, gn = n0 + r;
      a_tile[kk][r] = (gm < m_total && gk < k_total) ? to_float(a[(size_t)gm * k_total + gk]) : 0.f;
      w_tile[kk][r] = (gn < n_total && gk < k_total) ? to_float(w[(size_t)gn * k_total + gk]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < kTileK; ++kk) {
      float av[4], wv[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) av[i] = a_tile[kk][tm + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) wv[j] = w_tile[kk][tn + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], wv[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int gm = m0 + tm + i;
    if (gm >= m_total) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int gn = n0 + tn + j;
      if (gn >= n_total) continue;
      float v = acc[i][j];
      if (bias) v += bias[gn];
      c[(size_t)gm * n_total + gn] = from_float<TOut>(v);
    }
  }
}

// Few rows (decode): one warp per output column, lanes stride over k; the per-lane partial sums
// are combined by a fixed shuffle tree, so the result still does not depend on M.
// Used only when m_total <= kSmallM.
constexpr int kSmallM = 8;
template <typename TIn, typename TOut>
__global__ void __launch_bounds__(256)
gemm_small_m_kernel(const TIn* __restrict__ a, const TIn* __restrict__ w, const float* __restrict__ bias,
                    TOut* __restrict__ c, int m_total, int n_total, int k_total) {
  pdl_wait();
  pdl_trigger();
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (warp >= n_total) return;
  const TIn* wrow = w + (size_t)warp * k_total;
  float acc[kSmallM];
#pragma unroll
  for (int i = 0; i < kSmallM; ++i) acc[i] = 0.f;
  for (int k = lane; k < k_total; k += 32) {
    const float wv = to_float(wrow[k]);
#pragma unroll
    for (int i = 0; i < kSmallM; ++i)
      if (i < m_total) acc[i] = fmaf(to_float(a[(size_t)i * k_total + k]), wv, acc[i]);
  }
#pragma unroll
  for (int i = 0; i < kSmallM; ++i) {
    if (i >= m_total) break;
    float v = warp_sum(acc[i]);
    if (lane == 0) {
      if (bias) v += bias[warp];
      c[(size_t)i * n_total + warp] = from_float<TOut>(v);
    }
  }
}

}  // namespace cie

using namespace cie;

template <typename TIn, typename TOut>
static cudaError_t launch_simt(const void* a, const void* w, const float* bias, void* c, int m, int n,
                               int k, int allow_small, cudaStream_t stream) {
  if (allow_small && m <= kSmallM) {
    const int warps_per_block = 8;
    return cie::launch(gemm_small_m_kernel<TIn, TOut>, dim3((n + warps_per_block - 1) / warps_per_block),
                       dim3(256), 0, stream, (const TIn*)a, (const TIn*)w, bias, (TOut*)c, m, n, k);
  }
  dim3 grid((n + kTileN - 1) / kTileN, (m + kTileM - 1) / kTileM);
  return cie::launch(gemm_simt_kernel<TIn, TOut>, grid, dim3(256), 0, stream, (const TIn*)a,
                     (const TIn*)w, bias, (TOut*)c, m, n, k);
}

// in_dtype: element type of A and W; out_dtype: element type of C (float32 for logits).
// allow_small = 0 keeps one summation order for every M (the 32-bit check path uses that).
extern "C" int cie_gemm_simt(const void* a, const void* w, const float* bias, void* c, int m, int n,
                             int k, int in_dtype, int out_dtype, int allow_small, void* stream) {
  if (m <= 0 || n <= 0) return 0;
  if (k <= 0) CIE_FAIL("gemm_simt: K must be positive, got %d", k);
  cudaStream_t s = (cudaStream_t)stream;
  cudaError_t status;
  if (in_dtype == kFloat32 && out_dtype == kFloat32) status = launch_simt<float, float>(a, w, bias, c, m, n, k, allow_small, s);
  else if (in_dtype == kBFloat16 && out_dtype == kBFloat16) status = launch_simt<__nv_bfloat16, __nv_bfloat16>(a, w, bias, c, m, n, k, allow_small, s);
  else if (in_dtype == kBFloat16 && out_dtype == kFloat32) status = launch_simt<__nv_bfloat16, float>(a, w, bias, c, m, n, k, allow_small, s);
  else CIE_FAIL("gemm_simt: unsupported element types in=%d out=%d", in_dtype, out_dtype);
  if (status != cudaSuccess) CIE_FAIL("gemm_simt: launch failed: %s", cudaGetErrorString(status));
  return 0;
}
