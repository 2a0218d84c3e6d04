// Sampling from float32 logits on the device: greedy (argmax, lowest index on ties) and
// temperature sampling (softmax(logits / T) in float32, inverse CDF with a counter-based draw).
//
// The reference samples greedily only: argmax over float32 logits
// (zeeshan8281/cloud-inference-from-scratch src/cloud_engine/engine.py:486-488, model.py:231-233) and
// refuses any temperature (scheduler.py:69-71).  Temperature sampling here is this framework's own:
// the uniform number of a draw is a hash of (seed, request stream, output index), so a request's
// tokens do not depend on what else is in the batch or on how its prompt was cut.
#include "common.cuh"

#include <cfloat>

CIE_DEFINE_LAST_ERROR()

namespace cie {

constexpr int kThreads = 1024;

__device__ __forceinline__ float uniform_from_key(unsigned long long x) {
  // splitmix64 finaliser; 24 high bits -> [0, 1)
  x ^= x >> 30; x *= 0xBF58476D1CE4E5B9ull;
  x ^= x >> 27; x *= 0x94D049BB133111EBull;
  x ^= x >> 31;
  return (float)(x >> 40) * (1.0f / 16777216.0f);
}

constexpr int kSlices = 16;          // CTAs that search one row's maximum
constexpr int kSliceThreads = 256;

// First pass over the logits, spread over kSlices CTAs a row (one CTA reading a whole row of a
// large vocabulary is bound by what one SM can take in): slice s of row r leaves its maximum and
// the lowest index that holds it in partial_v / partial_i [r][s].
__global__ void __launch_bounds__(kSliceThreads)
slice_max_kernel(const float* __restrict__ logits, int vocab, float* __restrict__ partial_v,
                 int* __restrict__ partial_i) {
  __shared__ float red_v[kSliceThreads / 32];
  __shared__ int red_i[kSliceThreads / 32];
  pdl_wait();
  pdl_trigger();
  const int r = blockIdx.y, s = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const float* row = logits + (size_t)r * vocab;
  const int per = (vocab + kSlices - 1) / kSlices;
  const int begin = min(s * per, vocab), end = min(begin + per, vocab);
  float best = -FLT_MAX;
  int best_i = 0x7fffffff;
  for (int i = begin + tid; i < end; i += kSliceThreads) {
    const float v = row[i];
    if (v > best || (v == best && i < best_i)) { best = v; best_i = i; }
  }
#pragma unroll
  for (int offset = 16; offset > 0; offset >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, offset);
    const int oi = __shfl_xor_sync(0xffffffffu, best_i, offset);
    if (ov > best || (ov == best && oi < best_i)) { best = ov; best_i = oi; }
  }
  if (lane == 0) { red_v[warp] = best; red_i[warp] = best_i; }
  __syncthreads();
  if (warp == 0) {
    best = lane < kSliceThreads / 32 ? red_v[lane] : -FLT_MAX;
    best_i = lane < kSliceThreads / 32 ? red_i[lane] : 0x7fffffff;
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, offset);
      const int oi = __shfl_xor_sync(0xffffffffu, best_i, offset);
      if (ov > best || (ov == best && oi < best_i)) { best = ov; best_i = oi; }
    }
    if (lane == 0) { partial_v[r * kSlices + s] = best; partial_i[r * kSlices + s] = best_i; }
  }
}

// One block per row.  temperature[r] == 0: argmax.  Else: token = first index whose inclusive
// cumulative weight exp((logit - max)/T) exceeds u * total; each thread owns one contiguous
// segment of the vocabulary, segment sums are scanned in thread order, so the result is a pure
// function of the row, the temperature and the key.
__global__ void __launch_bounds__(kThreads)
sample_kernel(const float* __restrict__ logits, int vocab, const float* __restrict__ temperature,
              const unsigned long long* __restrict__ keys, int* __restrict__ out,
              const float* __restrict__ partial_v, const int* __restrict__ partial_i) {
  __shared__ float red_v[kThreads / 32];
  __shared__ int red_i[kThreads / 32];
  __shared__ float seg_sum[kThreads];
  __shared__ float bcast[2];
  __shared__ int chosen;
  pdl_wait();
  pdl_trigger();
  const int r = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const float* row = logits + (size_t)r * vocab;

  // ---- maximum and its lowest index: from the slices' maxima if a first pass left them
  float best = -FLT_MAX;
  int best_i = 0x7fffffff;
  if (partial_v) {
    if (tid < kSlices) { best = partial_v[r * kSlices + tid]; best_i = partial_i[r * kSlices + tid]; }
  } else {
    for (int i = tid; i < vocab; i += kThreads) {
      const float v = row[i];
      if (v > best || (v == best && i < best_i)) { best = v; best_i = i; }
    }
  }
#pragma unroll
  for (int offset = 16; offset > 0; offset >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, offset);
    const int oi = __shfl_xor_sync(0xffffffffu, best_i, offset);
    if (ov > best || (ov == best && oi < best_i)) { best = ov; best_i = oi; }
  }
  if (lane == 0) { red_v[warp] = best; red_i[warp] = best_i; }
  __syncthreads();
  if (warp == 0) {
    best = lane < kThreads / 32 ? red_v[lane] : -FLT_MAX;
    best_i = lane < kThreads / 32 ? red_i[lane] : 0x7fffffff;
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, offset);
      const int oi = __shfl_xor_sync(0xffffffffu, best_i, offset);
      if (ov > best || (ov == best && oi < best_i)) { best = ov; best_i = oi; }
    }
    // a row without any comparable value (all NaN) yields token 0 rather than an index outside the vocabulary
    if (lane == 0) { bcast[0] = best; chosen = best_i == 0x7fffffff ? 0 : best_i; }
  }
  __syncthreads();
  const float temp = temperature ? temperature[r] : 0.f;
  if (!(temp > 0.f)) {
    if (tid == 0) out[r] = chosen;
    return;
  }
  const float row_max = bcast[0];
  const float inv_t = 1.f / temp;

  // ---- segment sums, in index order inside each segment
  const int seg = (vocab + kThreads - 1) / kThreads;
  const int begin = min(tid * seg, vocab), end = min(begin + seg, vocab);
  float local = 0.f;
  for (int i = begin; i < end; ++i) local += expf((row[i] - row_max) * inv_t);
  seg_sum[tid] = local;
  __syncthreads();
  if (tid == 0) {
    float total = 0.f;
    for (int i = 0; i < kThreads; ++i) total += seg_sum[i];
    const float target = uniform_from_key(keys[r]) * total;
    float before = 0.f;
    int owner = 0;
    for (int i = 0; i < kThreads; ++i) {
      owner = i;
      if (before + seg_sum[i] > target) break;
      if (i + 1 < kThreads) before += seg_sum[i];
    }
    // walk the owner's segment; if rounding left the target unreached, take the argmax
    const int b = min(owner * seg, vocab), e = min(b + seg, vocab);
    float running = before;
    int pick = -1;
    for (int i = b; i < e; ++i) {
      running += expf((row[i] - row_max) * inv_t);
      if (running > target) { pick = i; break; }
    }
    if (pick < 0) pick = chosen;
    out[r] = pick;
  }
}

// token_ids[i] = sampled[min(i, real - 1)]: the step that follows a decode step takes its token ids
// from what that step sampled, on the device; rows that only pad the batch repeat the last real one.
__global__ void feed_tokens_kernel(const int* __restrict__ sampled, int* __restrict__ token_ids, int rows, int real) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < rows) token_ids[i] = sampled[min(i, real - 1)];
}

}  // namespace cie

using namespace cie;

extern "C" int cie_sample_slices() { return kSlices; }

extern "C" int cie_feed_tokens(const int* sampled, int* token_ids, int rows, int real, void* stream) {
  if (rows <= 0) return 0;
  if (!sampled || !token_ids || real < 1 || real > rows) CIE_FAIL("feed_tokens: %d real rows of %d", real, rows);
  feed_tokens_kernel<<<(rows + 127) / 128, 128, 0, (cudaStream_t)stream>>>(sampled, token_ids, rows, real);
  CIE_CHECK_LAUNCH("feed_tokens");
  return 0;
}

// temperature may be null (all rows greedy); keys may be null only then.  scratch: room for
// rows * cie_sample_slices() floats and as many ints, or null (then one CTA a row finds the
// maximum itself, which is slow for a large vocabulary).
extern "C" int cie_sample(const float* logits, int rows, int vocab, const float* temperature,
                          const unsigned long long* keys, int* out, void* scratch, void* stream) {
  if (rows <= 0) return 0;
  if (vocab < 1) CIE_FAIL("sample: vocabulary size %d", vocab);
  if (temperature && !keys) CIE_FAIL("sample: temperature rows need draw keys");
  float* partial_v = nullptr;
  int* partial_i = nullptr;
  if (scratch && vocab >= 4096) {
    partial_v = reinterpret_cast<float*>(scratch);
    partial_i = reinterpret_cast<int*>(partial_v + (size_t)rows * kSlices);
    CIE_LAUNCH("sample", slice_max_kernel, dim3(kSlices, rows), dim3(kSliceThreads), 0, (cudaStream_t)stream,
               logits, vocab, partial_v, partial_i);
  }
  CIE_LAUNCH("sample", sample_kernel, dim3(rows), dim3(kThreads), 0, (cudaStream_t)stream, logits,
             vocab, temperature, keys, out, (const float*)partial_v, (const int*)partial_i);
  return 0;
}
