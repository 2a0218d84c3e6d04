// Causal attention of a ragged batch over the paged cache, one warp per (token, query head).
// Any head size up to 256, any page size, any number of heads and groups, float32 or bfloat16
// storage; all arithmetic is float32.  This is the 32-bit path's attention and the fallback for
// head or page sizes the tensor-core kernels do not take.
//
// Formula (zeeshan8281/cloud-inference-from-scratch src/cloud_engine/kernel.py:356-405): for query
// token t at position p of its request, keys 0..p (or p-window+1..p), s = (q.k) * scale,
// running-maximum softmax, out = sum(p v) / sum(p); query head h reads kv head h / (Hq/Hkv).
// Keys are visited in blocks of 32 counted from the first visible key, so the result for a
// token depends only on its request's keys, not on the batch, the cut or the pages used.
#include "common.cuh"

#include <cfloat>

CIE_DEFINE_LAST_ERROR()

namespace cie {

constexpr int kMaxDim = 256;
constexpr int kWarps = 4;

template <typename T>
__global__ void __launch_bounds__(kWarps * 32)
attention_generic_kernel(const T* __restrict__ q, int q_stride, T* __restrict__ out, int out_stride,
                         const T* __restrict__ k_pool, const T* __restrict__ v_pool,
                         const int* __restrict__ positions, const int* __restrict__ request_of_token,
                         const int* __restrict__ table, int table_width, int num_pages, int tokens,
                         int q_heads, int kv_heads, int dim, int page_size, float scale, int window,
                         int* err) {
  __shared__ float q_s[kWarps][kMaxDim];
  __shared__ float p_s[kWarps][32];
  __shared__ long long off_s[kWarps][32];
  pdl_wait();
  pdl_trigger();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int item = blockIdx.x * kWarps + warp;
  if (item >= tokens * q_heads) return;
  const int t = item / q_heads, h = item % q_heads;
  const int kvh = h / (q_heads / kv_heads);
  const int pos = positions[t];
  const int request = request_of_token[t];
  const int* row = table + (size_t)request * table_width;
  const int length = pos + 1;
  const int first = (window > 0 && length > window) ? length - window : 0;

  const T* qv = q + (size_t)t * q_stride + (size_t)h * dim;
  for (int d = lane; d < dim; d += 32) q_s[warp][d] = to_float(qv[d]);
  __syncwarp();

  float m = -FLT_MAX, l = 0.f;
  float acc[kMaxDim / 32];
#pragma unroll
  for (int i = 0; i < kMaxDim / 32; ++i) acc[i] = 0.f;

  for (int base = first; base < length; base += 32) {
    const int key = base + lane;
    const bool valid = key < length;
    long long offset = -1;
    if (valid) {
      const int index = key / page_size;
      const int page = index < table_width ? row[index] : -1;
      if (page < 0 || page >= num_pages) {
        atomicOr(err, kErrBadPage);
      } else {
        offset = (((long long)page * kv_heads + kvh) * page_size + key % page_size) * dim;
      }
    }
    float s = -FLT_MAX;
    if (offset >= 0) {
      const T* kr = k_pool + offset;
      float dot = 0.f;
      for (int d = 0; d < dim; ++d) dot = fmaf(q_s[warp][d], to_float(kr[d]), dot);
      s = dot * scale;
    }
    const float m_new = fmaxf(m, warp_max(s));
    const float p = offset >= 0 ? expf(s - m_new) : 0.f;
    const float alpha = expf(m - m_new);
    l = l * alpha + warp_sum(p);
    m = m_new;
    p_s[warp][lane] = p;
    off_s[warp][lane] = offset;
    __syncwarp();
#pragma unroll
    for (int i = 0; i < kMaxDim / 32; ++i) acc[i] *= alpha;
    const int count = min(32, length - base);
    for (int j = 0; j < count; ++j) {
      const long long o = off_s[warp][j];
      if (o < 0) continue;
      const float pj = p_s[warp][j];
      const T* vr = v_pool + o;
#pragma unroll
      for (int i = 0; i < kMaxDim / 32; ++i) {
        const int d = lane + 32 * i;
        if (d < dim) acc[i] = fmaf(pj, to_float(vr[d]), acc[i]);
      }
    }
    __syncwarp();
  }
  T* o = out + (size_t)t * out_stride + (size_t)h * dim;
  const float inv = l > 0.f ? 1.f / l : 0.f;
#pragma unroll
  for (int i = 0; i < kMaxDim / 32; ++i) {
    const int d = lane + 32 * i;
    if (d < dim) o[d] = from_float<T>(acc[i] * inv);
  }
}

}  // namespace cie

using namespace cie;

// q: rows of q_stride elements, query head h of token t at q[t*q_stride + h*dim].
// out: [tokens, out_stride], head h at column h*dim.  Pools: [pages][kv_heads][page_size][dim].
extern "C" int cie_attention_generic(const void* q, int q_stride, void* out, int out_stride,
                                     const void* k_pool, const void* v_pool, const int* positions,
                                     const int* request_of_token, const int* table, int table_width,
                                     int num_pages, int tokens, int q_heads, int kv_heads, int dim,
                                     int page_size, float scale, int window, int dtype, int* err,
                                     void* stream) {
  if (tokens <= 0) return 0;
  if (dim > kMaxDim || dim < 1) CIE_FAIL("attention_generic: head size %d is outside 1..%d", dim, kMaxDim);
  if (kv_heads < 1 || q_heads % kv_heads) CIE_FAIL("attention_generic: %d query heads do not divide over %d kv heads", q_heads, kv_heads);
  if (page_size < 1) CIE_FAIL("attention_generic: page size %d", page_size);
  const long long items = (long long)tokens * q_heads;
  const int blocks = (int)((items + kWarps - 1) / kWarps);
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == kFloat32) {
    CIE_LAUNCH("attention_generic", attention_generic_kernel<float>, dim3(blocks), dim3(kWarps * 32), 0, s,
        (const float*)q, q_stride, (float*)out, out_stride, (const float*)k_pool, (const float*)v_pool,
        positions, request_of_token, table, table_width, num_pages, tokens, q_heads, kv_heads, dim,
        page_size, scale, window, err);
  } else if (dtype == kBFloat16) {
    CIE_LAUNCH("attention_generic", attention_generic_kernel<__nv_bfloat16>, dim3(blocks), dim3(kWarps * 32), 0, s,
        (const __nv_bfloat16*)q, q_stride, (__nv_bfloat16*)out, out_stride, (const __nv_bfloat16*)k_pool,
        (const __nv_bfloat16*)v_pool, positions, request_of_token, table, table_width, num_pages, tokens,
        q_heads, kv_heads, dim, page_size, scale, window, err);
  } else {
    CIE_FAIL("attention_generic: unknown element type code %d", dtype);
  }
  return 0;
}
