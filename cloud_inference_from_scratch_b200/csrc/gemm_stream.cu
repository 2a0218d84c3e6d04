// Weight-streaming matrix product for few rows (decode): out[M, N] = x[M, K] * W[N, K]^T, M <= 64.
//
// With at most 64 tokens a projection is bound by reading W once from HBM, so the kernel is
// built around the weight stream: a CTA owns BN weight rows and a slice of K, and pulls
// [BN x 128] weight tiles through a four-stage cp.async pipeline while tensor cores
// (mma.sync m16n8k16, bfloat16 in, float32 accumulate) multiply them with the matching slice
// of x.  Weights are the 16-row operand (the roles of the two operands are swapped), tokens are
// the 8-wide operand, so 8 tokens cost no more tensor work than 1.
// Matrices with few rows are cut along K as well (grid.y) so that every SM streams; the
// partial sums are written as float32 [splits][M][N] and added up, in a fixed order, by the
// kernel that consumes them (residual-add + RMSNorm, or rotary + cache write), which also adds
// the bias.  Epilogues: bfloat16 or float32 output with bias; float32 partials; SiLU(gate) * up
// when the weight holds gate and up rows interleaved in blocks of BN/2.
//
// The reference runs these products through cuBLAS (zeeshan8281/cloud-inference-from-scratch
// src/cloud_engine/model.py:100,134-136,217,227).
#include "common.cuh"

CIE_DEFINE_LAST_ERROR()

namespace cie {

using bf16 = __nv_bfloat16;
constexpr int BK = 128;
constexpr int WROW = BK + 8;
constexpr int STAGES = 4;
constexpr int KSTEPS = BK / 16;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void cp_async16(void* dst, const void* src, bool valid) {
  const int bytes = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(smem_u32(dst)), "l"(src), "r"(bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }
__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

constexpr int kOutBF16 = 0, kOutF32 = 1, kOutPartial = 2, kOutSiluMul = 3;

struct StreamArgs {
  const bf16* x;       // [M, K]
  const bf16* w;       // [N, K]
  const float* bias;   // [N] or null (modes 0, 1)
  void* out;           // mode 0: bf16 [M, N]; 1: float [M, N]; 2: float [splits, M, N]; 3: bf16 [M, N/2]
  int m, n, k;
  int k_per_split;     // multiple of BK
  int mode;
};

template <int MT, int BN>
__global__ void __launch_bounds__(BN * 2) gemm_stream_kernel(const StreamArgs a) {
  constexpr int THREADS = BN * 2;   // one warp per 16 weight rows
  constexpr int MP = MT * 8;        // padded token count
  extern __shared__ __align__(16) unsigned char smem_raw[];
  bf16* w_s = reinterpret_cast<bf16*>(smem_raw);            // [STAGES][BN][WROW]
  bf16* x_s = w_s + STAGES * BN * WROW;                     // [STAGES][MP][WROW]
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int n0 = blockIdx.x * BN;
  const int k_begin = blockIdx.y * a.k_per_split;
  const int k_end = min(a.k, k_begin + a.k_per_split);
  const int steps = (k_end - k_begin + BK - 1) / BK;

  // CTAs walk their K slice from different starting tiles, so that hundreds of CTAs do not ask
  // L2 for the same lines of x at the same moment
  const int rotate = steps > 0 ? (int)(blockIdx.x % (unsigned)steps) : 0;
  auto load_w = [&](int step) {
    int tile = step + rotate;
    if (tile >= steps) tile -= steps;
    const int k0 = k_begin + tile * BK;
    bf16* wd = w_s + (step % STAGES) * BN * WROW;
#pragma unroll
    for (int i = 0; i < (BN * 16) / THREADS; ++i) {   // BN rows x 16 pieces of 16 bytes
      const int e = tid + i * THREADS;
      const int r = e >> 4, c = e & 15;
      const int row = n0 + r, col = k0 + c * 8;
      const bool ok = row < a.n && col < k_end;
      cp_async16(wd + r * WROW + c * 8, ok ? a.w + (size_t)row * a.k + col : a.w, ok);
    }
  };
  auto load_x = [&](int step) {
    int tile = step + rotate;
    if (tile >= steps) tile -= steps;
    const int k0 = k_begin + tile * BK;
    bf16* xd = x_s + (step % STAGES) * MP * WROW;
    for (int e = tid; e < MP * 16; e += THREADS) {
      const int r = e >> 4, c = e & 15;
      const int col = k0 + c * 8;
      const bool ok = r < a.m && col < k_end;
      cp_async16(xd + r * WROW + c * 8, ok ? a.x + (size_t)r * a.k + col : a.x, ok);
    }
  };
  auto load_stage = [&](int step) {
    load_w(step);
    load_x(step);
  };

  // The weights do not depend on the kernel before this one: the CTA requests its first weight
  // tiles before waiting for it, so the weight stream overlaps the tail of that kernel.
  // (Asking L2 for the whole weight slice at this point was tried and made the step slower.)
#pragma unroll
  for (int s = 0; s < STAGES - 1; ++s)
    if (s < steps) load_w(s);
  pdl_wait();
  pdl_trigger();
#pragma unroll
  for (int s = 0; s < STAGES - 1; ++s) {
    if (s < steps) load_x(s);
    cp_async_commit();
  }

  float acc[MT][4];
#pragma unroll
  for (int i = 0; i < MT; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;

  for (int it = 0; it < steps; ++it) {
    cp_async_wait<STAGES - 2>();
    __syncthreads();
    if (it + STAGES - 1 < steps) load_stage(it + STAGES - 1);
    cp_async_commit();
    const bf16* wt = w_s + (it % STAGES) * BN * WROW + warp * 16 * WROW;
    const bf16* xt = x_s + (it % STAGES) * MP * WROW;
#pragma unroll
    for (int kp = 0; kp < KSTEPS / 2; ++kp) {
      uint32_t a0[4], a1[4];
      ldsm_x4(a0, wt + (lane & 15) * WROW + (2 * kp) * 16 + (lane >> 4) * 8);
      ldsm_x4(a1, wt + (lane & 15) * WROW + (2 * kp + 1) * 16 + (lane >> 4) * 8);
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) {
        uint32_t b[4];  // tokens mt*8.., k = kp*32 + {0, 8, 16, 24}
        ldsm_x4(b, xt + (mt * 8 + (lane & 7)) * WROW + kp * 32 + (lane >> 3) * 8);
        mma_bf16(acc[mt], a0, b[0], b[1]);
        mma_bf16(acc[mt], a1, b[2], b[3]);
      }
    }
  }
  cp_async_wait<0>();
  __syncthreads();

  // ---- epilogue through shared memory: out_s[token][weight row]
  float* out_s = reinterpret_cast<float*>(smem_raw);   // [MP][BN + 1]
  const int g = lane >> 2, t4 = lane & 3;
#pragma unroll
  for (int mt = 0; mt < MT; ++mt) {
    const int m0 = mt * 8 + 2 * t4, r0 = warp * 16 + g;
    out_s[m0 * (BN + 1) + r0] = acc[mt][0];
    out_s[(m0 + 1) * (BN + 1) + r0] = acc[mt][1];
    out_s[m0 * (BN + 1) + r0 + 8] = acc[mt][2];
    out_s[(m0 + 1) * (BN + 1) + r0 + 8] = acc[mt][3];
  }
  __syncthreads();
  if (a.mode == kOutSiluMul) {
    constexpr int HALF = BN / 2;
    const int c0 = blockIdx.x * HALF, channels = a.n / 2;
    bf16* out = reinterpret_cast<bf16*>(a.out);
    for (int e = tid; e < a.m * HALF; e += THREADS) {
      const int m = e / HALF, j = e % HALF;
      if (c0 + j >= channels) continue;
      const float gate = out_s[m * (BN + 1) + j], up = out_s[m * (BN + 1) + HALF + j];
      out[(size_t)m * channels + c0 + j] = __float2bfloat16_rn((gate / (1.f + expf(-gate))) * up);
    }
    return;
  }
  for (int e = tid; e < a.m * BN; e += THREADS) {
    const int m = e / BN, j = e % BN;
    const int col = n0 + j;
    if (col >= a.n) continue;
    float v = out_s[m * (BN + 1) + j];
    if (a.mode == kOutPartial) {
      reinterpret_cast<float*>(a.out)[((size_t)blockIdx.y * a.m + m) * a.n + col] = v;
    } else {
      if (a.bias) v += a.bias[col];
      if (a.mode == kOutF32) reinterpret_cast<float*>(a.out)[(size_t)m * a.n + col] = v;
      else reinterpret_cast<bf16*>(a.out)[(size_t)m * a.n + col] = __float2bfloat16_rn(v);
    }
  }
}

template <int MT, int BN>
static int launch(const StreamArgs& a, int splits, cudaStream_t stream) {
  constexpr int MP = MT * 8;
  constexpr size_t pipeline = (size_t)STAGES * (BN + MP) * WROW * sizeof(bf16);
  constexpr size_t staging = (size_t)MP * (BN + 1) * sizeof(float);
  constexpr size_t smem = pipeline > staging ? pipeline : staging;
  static bool configured = false;
  if (!configured) {
    cudaError_t status = cudaFuncSetAttribute(gemm_stream_kernel<MT, BN>,
                                              cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (status != cudaSuccess) CIE_FAIL("gemm_stream: shared memory %zu: %s", smem, cudaGetErrorString(status));
    configured = true;
  }
  dim3 grid((a.n + BN - 1) / BN, splits);
  CIE_LAUNCH("gemm_stream", gemm_stream_kernel<MT, BN>, grid, dim3(BN * 2), smem, stream, a);
  return 0;
}

}  // namespace cie

using namespace cie;

// mode: 0 bf16 out, 1 float32 out, 2 float32 partials [splits][M][N] (bias ignored),
// 3 SiLU(gate)*up with gate/up rows interleaved in blocks of block_rows/2 (splits must be 1).
// block_rows: weight rows per CTA, 32 or 64.
extern "C" int cie_gemm_stream(const void* x, const void* w, const float* bias, void* out, int m,
                               int n, int k, int splits, int mode, int block_rows, void* stream) {
  if (m <= 0 || n <= 0) return 0;
  if (m > 64) CIE_FAIL("gemm_stream: takes at most 64 rows, got %d", m);
  if (k < 8 || k % 8) CIE_FAIL("gemm_stream: K must be a multiple of 8 (16-byte rows), got %d", k);
  if (splits < 1) CIE_FAIL("gemm_stream: splits %d", splits);
  if (mode == kOutSiluMul && (splits != 1 || n % 2)) CIE_FAIL("gemm_stream: the SiLU epilogue needs one split and an even N");
  if (mode != kOutPartial && splits != 1) CIE_FAIL("gemm_stream: %d splits need the partial-sum output", splits);
  StreamArgs a;
  a.x = (const bf16*)x; a.w = (const bf16*)w; a.bias = bias; a.out = out;
  a.m = m; a.n = n; a.k = k; a.mode = mode;
  const int k_tiles = (k + BK - 1) / BK;
  a.k_per_split = ((k_tiles + splits - 1) / splits) * BK;
  cudaStream_t s = (cudaStream_t)stream;
  const int mt = m <= 8 ? 1 : m <= 16 ? 2 : m <= 32 ? 4 : 8;
  if (block_rows == 32) {
    if (mt == 1) return launch<1, 32>(a, splits, s);
    if (mt == 2) return launch<2, 32>(a, splits, s);
    if (mt == 4) return launch<4, 32>(a, splits, s);
    return launch<8, 32>(a, splits, s);
  }
  if (block_rows == 64) {
    if (mt == 1) return launch<1, 64>(a, splits, s);
    if (mt == 2) return launch<2, 64>(a, splits, s);
    if (mt == 4) return launch<4, 64>(a, splits, s);
    return launch<8, 64>(a, splits, s);
  }
  CIE_FAIL("gemm_stream: block_rows must be 32 or 64, got %d", block_rows);
}

// ------------------------------------------------------------------------------------------------
// The variant that allocates nothing (see gemm_stream_noalloc.h for who needs it and the rules).
#include "gemm_stream_noalloc.h"

namespace cie {

// Scratch for the partial sums of cie_gemm_stream_noalloc.  In host code this name is only a
// stand-in for the device symbol, never a device address: the host asks the runtime for the
// address once per device (scratch_address) and hands that to the kernels.
static __device__ __align__(256) float noalloc_scratch[CIE_NOALLOC_SCRATCH_FLOATS];

constexpr int kMaxDevices = 64;

// out[m][n] = bf16(sum over splits of partial[s][m][n] + bias[n]); the splits in ascending order.
__global__ void noalloc_reduce_kernel(const float* __restrict__ partial, const float* __restrict__ bias,
                                      bf16* __restrict__ out, int m, int n, int splits) {
  const size_t total = (size_t)m * n;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (size_t)gridDim.x * blockDim.x) {
    float v = partial[i];
    for (int s = 1; s < splits; ++s) v += partial[(size_t)s * total + i];
    if (bias) v += bias[i % n];
    out[i] = __float2bfloat16_rn(v);
  }
}

// Device address of the scratch array on the current device, looked up on first use per device.
static int scratch_address(float** address) {
  static float* known[kMaxDevices] = {};
  int device = -1;
  cudaError_t status = cudaGetDevice(&device);
  if (status != cudaSuccess) CIE_FAIL("gemm_stream_noalloc: cudaGetDevice: %s", cudaGetErrorString(status));
  if (device < 0 || device >= kMaxDevices) CIE_FAIL("gemm_stream_noalloc: device index %d is outside 0..%d", device, kMaxDevices - 1);
  if (!known[device]) {
    float* found = nullptr;
    status = cudaGetSymbolAddress(reinterpret_cast<void**>(&found), noalloc_scratch);
    if (status != cudaSuccess || !found)
      CIE_FAIL("gemm_stream_noalloc: cudaGetSymbolAddress on device %d: %s", device, cudaGetErrorString(status));
    known[device] = found;
  }
  *address = known[device];
  return 0;
}

}  // namespace cie

extern "C" int cie_gemm_stream_noalloc(const void* x, const void* w, const float* bias, void* out, int m,
                                       int n, int k, int splits, void* stream) {
  if (m <= 0 || n <= 0) return 0;
  if (m > 16) CIE_FAIL("gemm_stream_noalloc: takes at most 16 rows, got %d", m);
  if (k < 8 || k % 8) CIE_FAIL("gemm_stream_noalloc: K must be a multiple of 8, got %d", k);
  if (splits < 1 || splits > 8) CIE_FAIL("gemm_stream_noalloc: splits must be 1..8, got %d", splits);
  if ((long long)splits * m * n > (long long)CIE_NOALLOC_SCRATCH_FLOATS)
    CIE_FAIL("gemm_stream_noalloc: %d splits x %d rows x %d columns = %lld partial sums exceed the built-in scratch of %d",
             splits, m, n, (long long)splits * m * n, CIE_NOALLOC_SCRATCH_FLOATS);
  if (!x || !w || !out) CIE_FAIL("gemm_stream_noalloc: null operand");
  float* scratch = nullptr;
  if (cie::scratch_address(&scratch) != 0) return 1;
  // partial sums of the existing kernel go to the built-in scratch ...
  if (cie_gemm_stream(x, w, nullptr, scratch, m, n, k, splits, kOutPartial, 32, stream) != 0) return 1;
  // ... and are added up, with the bias, by one more kernel (launched without programmatic
  // overlap, so it starts after the product has finished)
  const size_t total = (size_t)m * n;
  int blocks = (int)((total + 255) / 256);
  if (blocks > 1024) blocks = 1024;
  noalloc_reduce_kernel<<<blocks, 256, 0, (cudaStream_t)stream>>>(scratch, bias, (bf16*)out, m, n, splits);
  CIE_CHECK_LAUNCH("gemm_stream_noalloc");
  return 0;
}
