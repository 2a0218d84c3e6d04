// Memory-bound kernels of the forward pass, for float32 and bfloat16 activations:
// embedding gather into the float32 residual stream, residual-add + RMSNorm, rotary position
// encoding fused with the write of keys and values into the paged cache, SiLU * up.
// Statistics, angles and sums are float32; results are rounded once to the activation type.
//
// Reference formulas: zeeshan8281/cloud-inference-from-scratch src/cloud_engine/attention.py:52-85
// (rms_norm, rope), src/cloud_engine/cache.py:398-425 (slot = table[pos/page]*page + pos%page),
// src/cloud_engine/model.py:100 (SwiGLU), :210 (embedding).
#include "common.cuh"

CIE_DEFINE_LAST_ERROR()

namespace cie {

// ---------------------------------------------------------------- embedding
template <typename T>
__global__ void embedding_kernel(const int* __restrict__ ids, const T* __restrict__ table,
                                 float* __restrict__ residual, int hidden, int vocab, float scale, int* err) {
  pdl_wait();
  pdl_trigger();
  const int t = blockIdx.x;
  int id = ids[t];
  if (id < 0 || id >= vocab) {
    if (threadIdx.x == 0) atomicOr(err, kErrBadToken);
    id = 0;
  }
  const T* row = table + (size_t)id * hidden;
  float* out = residual + (size_t)t * hidden;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) out[i] = to_float(row[i]) * scale;
}

// ---------------------------------------------------------------- logits: scale and soft cap
// logits[i] = cap * tanh(logits[i] * scale / cap), or logits[i] * scale when cap == 0; float32, in place.
__global__ void shape_logits_kernel(float* __restrict__ logits, long long count, float scale, float cap) {
  pdl_wait();
  pdl_trigger();
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < count; i += (long long)gridDim.x * blockDim.x) {
    const float v = logits[i] * scale;
    logits[i] = cap > 0.f ? cap * tanhf(v / cap) : v;
  }
}

// ---------------------------------------------------------------- residual add + RMSNorm
// One block per output row.  rows == nullptr: row r is residual row r and residual is updated
// in place with `update`.  rows != nullptr: row r reads residual row rows[r]; residual is not
// written.  out = gain * ((x) * rsqrt(mean(x^2) + eps)), x = residual (+ update), all float32.
// `update` is either one tensor of the activation type, or (partial_splits > 0) float32 partial
// sums [splits][rows][hidden] of a matrix product cut along K, plus an optional bias; the partial
// sums are added in ascending split order.
constexpr int kMaxSplits = 8;   // partial sums a consumer adds up (the streaming product cuts K at most so often)

// Sum of up to kMaxSplits partial values; the loads are issued together, then added in split order.
__device__ __forceinline__ float sum_partials(const float* __restrict__ part, int splits, size_t stride) {
  float v[kMaxSplits];
#pragma unroll
  for (int s = 0; s < kMaxSplits; ++s) v[s] = s < splits ? part[(size_t)s * stride] : 0.f;
  float total = v[0];
#pragma unroll
  for (int s = 1; s < kMaxSplits; ++s) total += v[s];
  return total;
}

constexpr int kNormPerThread = 8;   // elements a thread keeps in registers (rows up to 8 * blockDim)

template <typename T>
__global__ void add_rmsnorm_kernel(float* __restrict__ residual, const void* __restrict__ update,
                                   int partial_splits, size_t partial_stride,
                                   const float* __restrict__ update_bias,
                                   const float* __restrict__ gain, T* __restrict__ out,
                                   const int* __restrict__ rows, int hidden, float eps) {
  __shared__ float scratch[33];
  // The one kernel that triggers BEFORE its wait: what follows a norm is a matrix product, and
  // all that product does before its own wait is to ask for weights, which no kernel writes.  It
  // may therefore start beside the kernel before this one and stream weights through its tail.
  pdl_trigger();
  pdl_wait();
  const int r = blockIdx.x;
  const int src = rows ? rows[r] : r;
  float* res = residual + (size_t)src * hidden;
  const bool has_update = update != nullptr;
  const T* upd = (has_update && partial_splits == 0) ? reinterpret_cast<const T*>(update) + (size_t)src * hidden : nullptr;
  const float* part = (has_update && partial_splits > 0) ? reinterpret_cast<const float*>(update) + (size_t)src * hidden : nullptr;
  const bool write_back = (rows == nullptr) && has_update;
  auto value = [&](int i) {
    float x = res[i];
    if (upd) x += to_float(upd[i]);
    if (part) {
      float u = sum_partials(part + i, partial_splits, partial_stride);
      if (update_bias) u += update_bias[i];
      x += u;
    }
    return x;
  };
  T* dst = out + (size_t)r * hidden;
  if (hidden <= kNormPerThread * (int)blockDim.x) {
    float x[kNormPerThread];
    float sumsq = 0.f;
#pragma unroll
    for (int j = 0; j < kNormPerThread; ++j) {
      const int i = threadIdx.x + j * blockDim.x;
      x[j] = i < hidden ? value(i) : 0.f;
      sumsq += x[j] * x[j];
    }
    const float total = block_sum(sumsq, scratch);
    const float inv = rsqrtf(total / (float)hidden + eps);
#pragma unroll
    for (int j = 0; j < kNormPerThread; ++j) {
      const int i = threadIdx.x + j * blockDim.x;
      if (i < hidden) {
        if (write_back) res[i] = x[j];
        dst[i] = from_float<T>(gain[i] * (x[j] * inv));
      }
    }
    return;
  }
  float sumsq = 0.f;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    const float x = value(i);
    if (write_back) res[i] = x;
    sumsq += x * x;
  }
  const float total = block_sum(sumsq, scratch);
  const float inv = rsqrtf(total / (float)hidden + eps);
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    const float x = write_back ? res[i] : value(i);
    dst[i] = from_float<T>(gain[i] * (x * inv));
  }
}

// The same for bfloat16 rows whose length is a multiple of 8, with a plain update or none: a thread
// owns 8 neighbouring elements (two 16-byte loads of the residual, one of the update), keeps them
// in registers across the reduction and writes them back the same way.  Up to 8192 elements a row.
__global__ void add_rmsnorm_bf16x8_kernel(float* __restrict__ residual, const __nv_bfloat16* __restrict__ update,
                                          const float* __restrict__ gain, __nv_bfloat16* __restrict__ out,
                                          const int* __restrict__ rows, int hidden, float eps) {
  __shared__ float scratch[33];
  pdl_trigger();   // see add_rmsnorm_kernel
  pdl_wait();
  const int r = blockIdx.x;
  const int src = rows ? rows[r] : r;
  const int i = threadIdx.x * 8;
  const bool active = i < hidden;
  float x[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  if (active) {
    const float4* res = reinterpret_cast<const float4*>(residual + (size_t)src * hidden + i);
    const float4 lo = res[0], hi = res[1];
    x[0] = lo.x; x[1] = lo.y; x[2] = lo.z; x[3] = lo.w; x[4] = hi.x; x[5] = hi.y; x[6] = hi.z; x[7] = hi.w;
    if (update) {
      const uint4 raw = *reinterpret_cast<const uint4*>(update + (size_t)src * hidden + i);
      const __nv_bfloat162* pairs = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 u = __bfloat1622float2(pairs[j]);
        x[2 * j] += u.x;
        x[2 * j + 1] += u.y;
      }
    }
  }
  float sumsq = 0.f;
#pragma unroll
  for (int j = 0; j < 8; ++j) sumsq += x[j] * x[j];
  const float total = block_sum(sumsq, scratch);
  const float inv = rsqrtf(total / (float)hidden + eps);
  if (!active) return;
  if (update && !rows) {
    float4* res = reinterpret_cast<float4*>(residual + (size_t)src * hidden + i);
    res[0] = make_float4(x[0], x[1], x[2], x[3]);
    res[1] = make_float4(x[4], x[5], x[6], x[7]);
  }
  const float4 g0 = *reinterpret_cast<const float4*>(gain + i), g1 = *reinterpret_cast<const float4*>(gain + i + 4);
  const float g[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
  uint4 packed;
  __nv_bfloat162* pairs = reinterpret_cast<__nv_bfloat162*>(&packed);
#pragma unroll
  for (int j = 0; j < 4; ++j)
    pairs[j] = __floats2bfloat162_rn(g[2 * j] * (x[2 * j] * inv), g[2 * j + 1] * (x[2 * j + 1] * inv));
  *reinterpret_cast<uint4*>(out + (size_t)r * hidden + i) = packed;
}

// ---------------------------------------------------------------- rotary + paged KV write
// qkv: [T, (Hq + 2 Hkv) * D], q heads first, then k heads, then v heads.  q is rotated in place.
// k is rotated and written, v is copied, to pool[page][kv_head][pos % page][D] with
// page = table[request][pos / page].  Element j < rot/2 pairs with j + rot/2 (rotate-half).
// The source row is either qkv itself (partial_splits == 0; then q_out == qkv and q is rotated
// in place; a bias not yet added may be given) or float32 partial sums [splits][T][width] of the projection plus its bias
// (partial_splits > 0; then the rotated q is written to q_out, rows of q_stride elements).
//
// paired != 0: the columns of every q and k head in the source are in the paired layout (the
// weight rows were laid out so for the rotary epilogue of the streaming product): element d < rot
// of a head stands at paired_column(d, rot), the rest (and v) where it always stands.  q_out must
// then be another buffer than the source; what is written is in the natural order.
__host__ __device__ __forceinline__ int paired_column(int d, int rot) {
  // blocks of 32 columns: 16 elements of the first half of the rotary dims, then their 16 partners
  const int half = rot / 2;
  if (d >= rot) return d;
  return d < half ? (d / 16) * 32 + d % 16 : ((d - half) / 16) * 32 + 16 + (d - half) % 16;
}

template <typename T>
__global__ void rope_kv_write_kernel(const void* __restrict__ src, int partial_splits,
                                     size_t partial_stride, const float* __restrict__ bias,
                                     T* __restrict__ q_out, int q_stride,
                                     const int* __restrict__ positions,
                                     const int* __restrict__ request_of_token,
                                     const int* __restrict__ table, int table_width, int num_pages,
                                     T* __restrict__ k_pool, T* __restrict__ v_pool,
                                     const float* __restrict__ inv_freq, int q_heads, int kv_heads,
                                     int dim, int rot, int page_size, int write_cache, int paired,
                                     int* err) {
  pdl_wait();
  pdl_trigger();
  const int t = blockIdx.x;
  const int pos = positions[t];
  const bool out_of_place = reinterpret_cast<const void*>(q_out) != src;
  const int width = (q_heads + 2 * kv_heads) * dim;
  const T* row_t = partial_splits == 0 ? reinterpret_cast<const T*>(src) + (size_t)t * width : nullptr;
  const float* row_p = partial_splits > 0 ? reinterpret_cast<const float*>(src) + (size_t)t * width : nullptr;
  auto value = [&](int i) {
    if (row_t) return bias ? to_float(row_t[i]) + bias[i] : to_float(row_t[i]);
    float v = sum_partials(row_p + i, partial_splits, partial_stride);
    if (bias) v += bias[i];
    return v;
  };
  T* q_row = q_out + (size_t)t * q_stride;
  const int half = rot / 2;

  size_t slot_base = 0;
  bool slot_ok = false;
  if (write_cache) {
    const int request = request_of_token[t];
    const int index = pos / page_size;
    int page = index < table_width ? table[(size_t)request * table_width + index] : -1;
    if (page < 0 || page >= num_pages) {
      if (threadIdx.x == 0) atomicOr(err, kErrBadPage);
    } else {
      slot_ok = true;
      slot_base = ((size_t)page * kv_heads) * page_size * dim + (size_t)(pos % page_size) * dim;
    }
  }
  const size_t head_stride = (size_t)page_size * dim;

  // rotated pairs of q and k heads: a thread owns pair j of some heads, so the sine and cosine
  // of (position, j) are computed once per thread, not once per head
  const int rot_heads = q_heads + kv_heads;
  const int lanes_per_head_set = half > 0 ? max(1, (int)blockDim.x / half) : 1;
  if (half > 0 && threadIdx.x < lanes_per_head_set * half) {
    const int j = threadIdx.x % half, first_head = threadIdx.x / half;
    float s, c;
    sincosf((float)pos * inv_freq[j], &s, &c);
    for (int h = first_head; h < rot_heads; h += lanes_per_head_set) {
      const float a = value(h * dim + (paired ? paired_column(j, rot) : j));
      const float b = value(h * dim + (paired ? paired_column(j + half, rot) : j + half));
      const T ra = from_float<T>(a * c - b * s), rb = from_float<T>(b * c + a * s);
      if (h < q_heads) {
        q_row[h * dim + j] = ra;
        q_row[h * dim + j + half] = rb;
      } else if (slot_ok) {
        T* dst = k_pool + slot_base + (size_t)(h - q_heads) * head_stride;
        dst[j] = ra;
        dst[j + half] = rb;
      }
    }
  }
  // the part of q and k beyond the rotary dims passes through
  const int tail = dim - rot;
  if (tail > 0 && (row_p || bias || out_of_place)) {
    for (int i = threadIdx.x; i < q_heads * tail; i += blockDim.x) {
      const int h = i / tail, d = rot + i % tail;
      q_row[h * dim + d] = from_float<T>(value(h * dim + d));
    }
  }
  if (!slot_ok) return;
  for (int i = threadIdx.x; i < kv_heads * tail; i += blockDim.x) {
    const int h = i / tail, d = rot + i % tail;
    k_pool[slot_base + (size_t)h * head_stride + d] = from_float<T>(value((q_heads + h) * dim + d));
  }
  for (int i = threadIdx.x; i < kv_heads * dim; i += blockDim.x) {
    const int h = i / dim, d = i % dim;
    v_pool[slot_base + (size_t)h * head_stride + d] =
        from_float<T>(value((q_heads + kv_heads + h) * dim + d));
  }
}

// The same for bfloat16 rows that are already summed (many tokens: the library product wrote them),
// with rot a multiple of 16 and head size a multiple of 8.  The work of a token is a list of
// 16-byte items: 8 neighbouring rotary pairs of a q or k head (both halves), then 8 passed-through
// columns of q, of k and of v.  A thread asks for its first item's bytes before anything else, so
// that their way from memory overlaps the position's: position -> sines and cosines (once per
// block, in shared memory) -> rotation.  q_out may be the source itself only in the natural layout
// (an item is read by the one thread that writes it, before it writes).
__global__ void rope_kv_write_bf16x8_kernel(const __nv_bfloat16* __restrict__ src, const float* __restrict__ bias,
                                            __nv_bfloat16* __restrict__ q_out, int q_stride,
                                            const int* __restrict__ positions,
                                            const int* __restrict__ request_of_token,
                                            const int* __restrict__ table, int table_width, int num_pages,
                                            __nv_bfloat16* __restrict__ k_pool, __nv_bfloat16* __restrict__ v_pool,
                                            const float* __restrict__ inv_freq, int q_heads, int kv_heads,
                                            int dim, int rot, int page_size, int write_cache, int paired,
                                            int* err) {
  extern __shared__ float trig[];  // sines of the rot / 2 pairs, then their cosines
  pdl_wait();
  pdl_trigger();
  using bf16 = __nv_bfloat16;
  const int t = blockIdx.x;
  const int width = (q_heads + 2 * kv_heads) * dim;
  const bf16* row = src + (size_t)t * width;
  bf16* q_row = q_out + (size_t)t * q_stride;
  const bool out_of_place = q_out != src;
  const int half = rot / 2;
  const int chunks = half / 8, tail_chunks = (dim - rot) / 8, value_chunks = dim / 8;
  const int rot_items = (q_heads + kv_heads) * chunks;
  const int q_tail_items = bias || out_of_place ? q_heads * tail_chunks : 0;
  const int k_tail_items = kv_heads * tail_chunks;
  const int items = rot_items + q_tail_items + k_tail_items + kv_heads * value_chunks;

  // where an item's bytes stand in the source row: column of its first (or only) piece and of
  // its partner piece (-1: none)
  auto place = [&](int i, int& col_a, int& col_b) {
    col_b = -1;
    if (i < rot_items) {
      const int h = i / chunks, c = i % chunks;
      col_a = h * dim + (paired ? paired_column(c * 8, rot) : c * 8);
      col_b = h * dim + (paired ? paired_column(c * 8 + half, rot) : c * 8 + half);
      return;
    }
    i -= rot_items;
    if (i < q_tail_items) {
      col_a = (i / tail_chunks) * dim + rot + (i % tail_chunks) * 8;
      return;
    }
    i -= q_tail_items;
    if (i < k_tail_items) {
      col_a = (q_heads + i / tail_chunks) * dim + rot + (i % tail_chunks) * 8;
      return;
    }
    i -= k_tail_items;
    col_a = (q_heads + kv_heads + i / value_chunks) * dim + (i % value_chunks) * 8;
  };
  auto fetch = [&](int i, uint4& a, uint4& b) {
    int col_a, col_b;
    place(i, col_a, col_b);
    a = *reinterpret_cast<const uint4*>(row + col_a);
    if (col_b >= 0) b = *reinterpret_cast<const uint4*>(row + col_b);
  };
  auto widen = [&](const uint4& raw, int column, float (&v)[8]) {
    const __nv_bfloat162* pairs = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 f = __bfloat1622float2(pairs[j]);
      v[2 * j] = f.x;
      v[2 * j + 1] = f.y;
    }
    if (bias) {
      const float4 lo = *reinterpret_cast<const float4*>(bias + column);
      const float4 hi = *reinterpret_cast<const float4*>(bias + column + 4);
      v[0] += lo.x, v[1] += lo.y, v[2] += lo.z, v[3] += lo.w;
      v[4] += hi.x, v[5] += hi.y, v[6] += hi.z, v[7] += hi.w;
    }
  };
  auto store8 = [&](bf16* dst, const float (&v)[8]) {
    uint4 packed;
    __nv_bfloat162* pairs = reinterpret_cast<__nv_bfloat162*>(&packed);
#pragma unroll
    for (int j = 0; j < 4; ++j) pairs[j] = __floats2bfloat162_rn(v[2 * j], v[2 * j + 1]);
    *reinterpret_cast<uint4*>(dst) = packed;
  };

  int item = threadIdx.x;
  uint4 raw_a = make_uint4(0, 0, 0, 0), raw_b = raw_a;
  if (item < items) fetch(item, raw_a, raw_b);

  const int pos = positions[t];
  long long slot_base = -1;
  if (write_cache) {
    const int request = request_of_token[t];
    const int index = pos / page_size;
    const int page = index < table_width ? table[(size_t)request * table_width + index] : -1;
    if (page < 0 || page >= num_pages) {
      if (threadIdx.x == 0) atomicOr(err, kErrBadPage);
    } else {
      slot_base = ((long long)page * kv_heads * page_size + pos % page_size) * dim;
    }
  }
  const long long head_stride = (long long)page_size * dim;
  for (int j = threadIdx.x; j < half; j += blockDim.x) sincosf((float)pos * inv_freq[j], &trig[j], &trig[half + j]);
  __syncthreads();

  while (item < items) {
    const int next = item + blockDim.x;
    uint4 next_a = raw_a, next_b = raw_b;
    if (next < items) fetch(next, next_a, next_b);
    int col_a, col_b;
    place(item, col_a, col_b);
    float a[8];
    widen(raw_a, col_a, a);
    if (item < rot_items) {
      const int h = item / chunks, c = item % chunks;
      float b[8], ra[8], rb[8];
      widen(raw_b, col_b, b);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float sn = trig[c * 8 + j], cs = trig[half + c * 8 + j];
        ra[j] = a[j] * cs - b[j] * sn;
        rb[j] = b[j] * cs + a[j] * sn;
      }
      bf16* dst = h < q_heads ? q_row + h * dim
                  : slot_base >= 0 ? k_pool + slot_base + (long long)(h - q_heads) * head_stride
                                   : nullptr;
      if (dst) {
        store8(dst + c * 8, ra);
        store8(dst + c * 8 + half, rb);
      }
    } else {
      int i = item - rot_items;
      bf16* dst = nullptr;
      if (i < q_tail_items) {
        dst = q_row + (i / tail_chunks) * dim + rot + (i % tail_chunks) * 8;
      } else if (slot_base >= 0) {
        i -= q_tail_items;
        if (i < k_tail_items) {
          dst = k_pool + slot_base + (i / tail_chunks) * head_stride + rot + (i % tail_chunks) * 8;
        } else {
          i -= k_tail_items;
          dst = v_pool + slot_base + (i / value_chunks) * head_stride + (i % value_chunks) * 8;
        }
      }
      if (dst) store8(dst, a);
    }
    item = next;
    raw_a = next_a;
    raw_b = next_b;
  }
}

// ---------------------------------------------------------------- SiLU(gate) * up
// gate_up: [T, 2 * inter] where channel c has its gate at column (c / block) * 2 * block + c % block
// and its up value `block` columns further (block == inter: all gates first, then all ups).
template <typename T>
__global__ void silu_mul_kernel(const T* __restrict__ gate_up, T* __restrict__ out, int tokens,
                                int inter, int block) {
  pdl_wait();
  pdl_trigger();
  const size_t total = (size_t)tokens * inter;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (size_t)gridDim.x * blockDim.x) {
    const size_t t = i / inter;
    const int c = (int)(i % inter);
    const size_t col = (size_t)(c / block) * 2 * block + c % block;
    const float g = to_float(gate_up[t * 2 * inter + col]);
    const float u = to_float(gate_up[t * 2 * inter + col + block]);
    out[i] = from_float<T>((g / (1.f + expf(-g))) * u);
  }
}

// bfloat16, 8 channels (16 bytes) per thread; needs inter % 8 == 0 and block % 8 == 0.
__global__ void silu_mul_bf16x8_kernel(const __nv_bfloat16* __restrict__ gate_up,
                                       __nv_bfloat16* __restrict__ out, int tokens, int inter, int block) {
  pdl_wait();
  pdl_trigger();
  const int vectors = inter / 8;
  const size_t total = (size_t)tokens * vectors;
  for (size_t v = (size_t)blockIdx.x * blockDim.x + threadIdx.x; v < total;
       v += (size_t)gridDim.x * blockDim.x) {
    const size_t t = v / vectors;
    const int c = (int)(v % vectors) * 8;
    const size_t col = (size_t)(c / block) * 2 * block + c % block;
    const uint4 graw = *reinterpret_cast<const uint4*>(gate_up + t * 2 * inter + col);
    const uint4 uraw = *reinterpret_cast<const uint4*>(gate_up + t * 2 * inter + col + block);
    const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&graw);
    const __nv_bfloat162* u2 = reinterpret_cast<const __nv_bfloat162*>(&uraw);
    uint4 packed;
    __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&packed);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 g = __bfloat1622float2(g2[j]), u = __bfloat1622float2(u2[j]);
      // the result is rounded to bfloat16: the fast exponential and division (a few ulp of
      // float32) cost a third of the instructions of the exact ones, which bound this kernel
      o2[j] = __floats2bfloat162_rn(__fdividef(g.x, 1.f + __expf(-g.x)) * u.x,
                                    __fdividef(g.y, 1.f + __expf(-g.y)) * u.y);
    }
    *reinterpret_cast<uint4*>(out + t * inter + c) = packed;
  }
}

}  // namespace cie

using namespace cie;

#define DISPATCH_DTYPE(dtype, name, ...)                                  \
  if (dtype == kFloat32) { using T = float; __VA_ARGS__ }                 \
  else if (dtype == kBFloat16) { using T = __nv_bfloat16; __VA_ARGS__ }   \
  else CIE_FAIL("%s: unknown element type code %d", name, dtype);

static int threads_for(int n) {
  int t = 32;
  while (t < n && t < 1024) t <<= 1;
  return t;
}

extern "C" int cie_embedding(const int* ids, const void* table, float* residual, int tokens,
                             int hidden, int vocab, float scale, int dtype, int* err, void* stream) {
  if (tokens <= 0) return 0;
  DISPATCH_DTYPE(dtype, "embedding", {
    CIE_LAUNCH("embedding", embedding_kernel<T>, dim3(tokens), dim3(threads_for(hidden / 4)), 0,
               (cudaStream_t)stream, ids, (const T*)table, residual, hidden, vocab, scale, err);
  })
  return 0;
}

extern "C" int cie_shape_logits(float* logits, long long count, float scale, float cap, void* stream) {
  if (count <= 0) return 0;
  if (cap < 0.f) CIE_FAIL("shape_logits: the soft cap must be >= 0, got %f", cap);
  const long long blocks = (count + 1023) / 1024;
  CIE_LAUNCH("shape_logits", shape_logits_kernel, dim3((unsigned)(blocks > 4096 ? 4096 : blocks)), dim3(256), 0,
             (cudaStream_t)stream, logits, count, scale, cap);
  return 0;
}

extern "C" int cie_add_rmsnorm(float* residual, const void* update, int partial_splits,
                               long long partial_stride, const float* update_bias,
                               const float* gain, void* out, const int* rows, int count, int hidden,
                               float eps, int dtype, void* stream) {
  if (count <= 0) return 0;
  if (partial_splits > kMaxSplits) CIE_FAIL("add_rmsnorm: at most %d partial sums, got %d", kMaxSplits, partial_splits);
  if (dtype == kBFloat16 && partial_splits == 0 && !update_bias && hidden % 8 == 0 && hidden <= 8192 &&
      ((reinterpret_cast<uintptr_t>(residual) | reinterpret_cast<uintptr_t>(update) | reinterpret_cast<uintptr_t>(gain) |
        reinterpret_cast<uintptr_t>(out)) & 15) == 0) {
    const int threads = (hidden / 8 + 31) / 32 * 32;
    CIE_LAUNCH("add_rmsnorm", add_rmsnorm_bf16x8_kernel, dim3(count), dim3(threads), 0, (cudaStream_t)stream, residual,
               (const __nv_bfloat16*)update, gain, (__nv_bfloat16*)out, rows, hidden, eps);
    return 0;
  }
  DISPATCH_DTYPE(dtype, "add_rmsnorm", {
    CIE_LAUNCH("add_rmsnorm", add_rmsnorm_kernel<T>, dim3(count), dim3(threads_for(hidden / 4)), 0,
               (cudaStream_t)stream, residual, update, partial_splits, (size_t)partial_stride,
               update_bias, gain, (T*)out, rows, hidden, eps);
  })
  return 0;
}

extern "C" int cie_rope_kv_write(const void* src, int partial_splits, long long partial_stride,
                                 const float* bias, void* q_out, int q_stride, const int* positions,
                                 const int* request_of_token, const int* table, int table_width,
                                 int num_pages, void* k_pool, void* v_pool, const float* inv_freq,
                                 int tokens, int q_heads, int kv_heads, int dim, int rot,
                                 int page_size, int write_cache, int paired, int dtype, int* err,
                                 void* stream) {
  if (tokens <= 0) return 0;
  if (rot % 2 || rot > dim || rot < 0) CIE_FAIL("rope_kv_write: rotary size %d does not fit head size %d", rot, dim);
  if (paired && (rot % 32 || q_out == src)) CIE_FAIL("rope_kv_write: the paired layout needs a rotary size that is a multiple of 32 and a q buffer of its own");
  if (partial_splits > kMaxSplits) CIE_FAIL("rope_kv_write: at most %d partial sums, got %d", kMaxSplits, partial_splits);
  if (dtype == kBFloat16 && partial_splits == 0 && tokens > 16 && rot >= 16 && rot % 16 == 0 && dim % 8 == 0 &&
      q_stride % 8 == 0 &&
      ((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(q_out) | reinterpret_cast<uintptr_t>(k_pool) |
        reinterpret_cast<uintptr_t>(v_pool) | reinterpret_cast<uintptr_t>(bias)) & 15) == 0) {
    const int items = (q_heads + kv_heads) * (rot / 16) + (q_heads + kv_heads) * ((dim - rot) / 8) + kv_heads * (dim / 8);
    const int threads = items >= 256 ? 256 : (items + 31) / 32 * 32;
    CIE_LAUNCH("rope_kv_write", rope_kv_write_bf16x8_kernel, dim3(tokens), dim3(threads), rot * sizeof(float),
               (cudaStream_t)stream, (const __nv_bfloat16*)src, bias, (__nv_bfloat16*)q_out, q_stride, positions,
               request_of_token, table, table_width, num_pages, (__nv_bfloat16*)k_pool, (__nv_bfloat16*)v_pool,
               inv_freq, q_heads, kv_heads, dim, rot, page_size, write_cache, paired, err);
    return 0;
  }
  DISPATCH_DTYPE(dtype, "rope_kv_write", {
    const int work = (q_heads + kv_heads) * (rot / 2) > kv_heads * dim ? (q_heads + kv_heads) * (rot / 2) : kv_heads * dim;
    // few tokens: spread one token over many threads; many tokens: fewer threads that each reuse
    // a pair's sine and cosine over several heads
    const int threads = tokens <= 64 ? threads_for(work) : 256;
    CIE_LAUNCH("rope_kv_write", rope_kv_write_kernel<T>, dim3(tokens), dim3(threads), 0,
               (cudaStream_t)stream, src, partial_splits, (size_t)partial_stride, bias, (T*)q_out,
               q_stride, positions, request_of_token, table, table_width, num_pages, (T*)k_pool,
               (T*)v_pool, inv_freq, q_heads, kv_heads, dim, rot, page_size, write_cache, paired, err);
  })
  return 0;
}

extern "C" int cie_silu_mul(const void* gate_up, void* out, int tokens, int inter, int block,
                            int dtype, void* stream) {
  if (tokens <= 0) return 0;
  if (block < 1 || inter % block) CIE_FAIL("silu_mul: %d channels do not divide into blocks of %d", inter, block);
  const size_t total = (size_t)tokens * inter;
  if (dtype == kBFloat16 && inter % 8 == 0 && block % 8 == 0 &&
      ((reinterpret_cast<uintptr_t>(gate_up) | reinterpret_cast<uintptr_t>(out)) & 15) == 0) {
    int vblocks = (int)((total / 8 + 255) / 256);
    if (vblocks > 148 * 16) vblocks = 148 * 16;
    CIE_LAUNCH("silu_mul", silu_mul_bf16x8_kernel, dim3(vblocks), dim3(256), 0, (cudaStream_t)stream,
               (const __nv_bfloat16*)gate_up, (__nv_bfloat16*)out, tokens, inter, block);
    return 0;
  }
  int blocks = (int)((total + 255) / 256);
  if (blocks > 148 * 16) blocks = 148 * 16;
  DISPATCH_DTYPE(dtype, "silu_mul", {
    CIE_LAUNCH("silu_mul", silu_mul_kernel<T>, dim3(blocks), dim3(256), 0, (cudaStream_t)stream,
               (const T*)gate_up, (T*)out, tokens, inter, block);
  })
  return 0;
}
