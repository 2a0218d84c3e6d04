// out[M, N] = x[M, K] * W[N, K]^T (+ bias) on the 5th-generation tensor cores: operands come by
// TMA (cp.async.bulk.tensor, 128-byte swizzle) into a multi-stage shared-memory ring, one elected
// thread issues tcgen05.mma with the float32 accumulator in tensor memory, tcgen05.commit hands
// stages back to the TMA thread through mbarriers, and the four warps read the accumulator with
// tcgen05.ld for the epilogue.  No cluster multicast is used.
//
// Both matrices are K-major ([rows, K], K contiguous), so either can be the 128-row operand:
//  * many tokens (prefill): tokens are the 128-row operand, weight rows the N operand (BN = 128);
//  * few tokens (decode, M <= 64): the roles are swapped; 128 weight rows are the 128-row operand
//    and the tokens, padded to 16/32/64, the N operand, so a small batch does not waste a tile.
//    Here the product may also be cut along K (grid.z) into float32 partial sums that the
//    consuming kernel adds up, and gate/up rows interleaved in blocks of 16 can be finished as
//    SiLU(gate) * up in the epilogue.
//
// Every wait on an mbarrier is bounded: after about two seconds the kernel sets an error bit,
// stops issuing work, releases its tensor memory and returns.
//
// The reference runs these products through cuBLAS (zeeshan8281/cloud-inference-from-scratch
// src/cloud_engine/model.py:100,134-136,217,227).
#include "blackwell.cuh"
#include "common.cuh"

CIE_DEFINE_LAST_ERROR()

namespace cie {

using namespace bw;
using bf16 = __nv_bfloat16;

constexpr int BM = 128;              // rows of the A operand per tile (UMMA M)
constexpr int BK = 64;               // K per stage: 64 bf16 = 128 bytes = one swizzle row
constexpr int UMMA_K = 16;
constexpr int A_STAGE_BYTES = BM * BK * 2;

constexpr int kOutBF16 = 0, kOutF32 = 1, kOutPartial = 2, kOutSiluMul = 3;



__device__ __forceinline__ void tmem_load16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr));
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

struct TcArgs {
  const float* bias;   // [N] or null
  void* out;
  int m, n, k;         // tokens, weight rows, reduction size
  int ldo;             // elements between output rows (n, or n / 2 for the SiLU epilogue)
  int k_per_split;     // multiple of BK
  int mode;
  int swapped;         // 1: A operand = weight rows, B operand = tokens
  int* err;
};

template <int BN, int STAGES>
__global__ void __launch_bounds__(128) gemm_tc_kernel(const __grid_constant__ CUtensorMap map_a,
                                                       const __grid_constant__ CUtensorMap map_b,
                                                       const TcArgs a) {
  constexpr int B_STAGE_BYTES = BN * BK * 2;
  constexpr int STAGE_BYTES = A_STAGE_BYTES + B_STAGE_BYTES;
  constexpr int TMEM_COLS = BN < 32 ? 32 : BN;
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  // the dynamic shared memory window is only guaranteed 16-byte aligned: align by hand
  unsigned char* tiles = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  __shared__ __align__(8) uint64_t full_bar[STAGES];
  __shared__ __align__(8) uint64_t empty_bar[STAGES];
  __shared__ __align__(8) uint64_t acc_bar;
  __shared__ uint32_t tmem_base_s;

  pdl_wait();
  pdl_trigger();
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int a_row0 = blockIdx.x * BM;
  const int b_row0 = blockIdx.y * BN;
  const int k_begin = blockIdx.z * a.k_per_split;
  const int k_end = min(a.k, k_begin + a.k_per_split);
  const int k_tiles = (k_end - k_begin + BK - 1) / BK;

  if (tid == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    mbar_init(&acc_bar, 1);
    mbar_init_fence();
  }
  if (warp == 0) {
    __syncwarp();
    tmem_alloc<TMEM_COLS>(&tmem_base_s);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_s;

  if (warp == 0) {
    if (lane == 0) {
      // ---- TMA producer
      for (int kt = 0; kt < k_tiles; ++kt) {
        const int s = kt % STAGES;
        const uint32_t phase = (kt / STAGES) & 1;
        if (!mbar_wait(&empty_bar[s], phase ^ 1, a.err)) break;
        mbar_expect_tx(&full_bar[s], STAGE_BYTES);
        unsigned char* dst = tiles + (size_t)s * STAGE_BYTES;
        const int kc = k_begin + kt * BK;
        tma_load_2d(dst, &map_a, &full_bar[s], kc, a_row0);
        tma_load_2d(dst + A_STAGE_BYTES, &map_b, &full_bar[s], kc, b_row0);
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (lane == 0) {
      // ---- MMA issuer
      constexpr uint32_t idesc = idesc_bf16(BM, BN);
      bool alive = true;
      for (int kt = 0; kt < k_tiles && alive; ++kt) {
        const int s = kt % STAGES;
        const uint32_t phase = (kt / STAGES) & 1;
        if (!mbar_wait(&full_bar[s], phase, a.err)) { alive = false; break; }
        tc_fence_after();
        const uint32_t a_addr = smem_u32(tiles + (size_t)s * STAGE_BYTES);
        const uint64_t a_desc = smem_desc_sw128(a_addr), b_desc = smem_desc_sw128(a_addr + A_STAGE_BYTES);
#pragma unroll
        for (int kk = 0; kk < BK / UMMA_K; ++kk) {
          // advancing 16 elements (32 bytes) inside the swizzled row: +2 in 16-byte units
          umma_bf16(tmem_base, a_desc + 2 * kk, b_desc + 2 * kk, idesc, (kt > 0 || kk > 0) ? 1u : 0u);
        }
        tc_commit(&empty_bar[s]);
      }
      tc_commit(&acc_bar);
    }
    __syncwarp();
  }

  // ---- epilogue: warp w reads tensor-memory lanes 32w .. 32w+31 (rows of the A operand)
  const bool ready = k_tiles > 0 ? mbar_wait(&acc_bar, 0, a.err) : true;
  tc_fence_after();
  const int a_row = a_row0 + warp * 32 + lane;
  if (ready) {
#pragma unroll 1
    for (int c0 = 0; c0 < BN; c0 += 16) {
      uint32_t raw[16];
      if (k_tiles > 0) {
        tmem_load16(tmem_base + ((uint32_t)(warp * 32) << 16) + c0, raw);
      } else {
#pragma unroll
        for (int j = 0; j < 16; ++j) raw[j] = 0;
      }
      if (!a.swapped) {
        // lane = token row, columns = weight rows b_row0 + c0 + j
        if (a_row >= a.m) continue;
        const int col0 = b_row0 + c0;
        if (col0 >= a.n) continue;
        if (a.mode == kOutBF16) {
          bf16* dst = reinterpret_cast<bf16*>(a.out) + (size_t)a_row * a.ldo + col0;
          if (col0 + 16 <= a.n && (a.ldo % 8 == 0)) {
            uint32_t packed[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              float v0 = __uint_as_float(raw[2 * j]), v1 = __uint_as_float(raw[2 * j + 1]);
              if (a.bias) { v0 += a.bias[col0 + 2 * j]; v1 += a.bias[col0 + 2 * j + 1]; }
              __nv_bfloat162 pair = __floats2bfloat162_rn(v0, v1);
              packed[j] = *reinterpret_cast<uint32_t*>(&pair);
            }
            reinterpret_cast<uint4*>(dst)[0] = make_uint4(packed[0], packed[1], packed[2], packed[3]);
            reinterpret_cast<uint4*>(dst)[1] = make_uint4(packed[4], packed[5], packed[6], packed[7]);
          } else {
            for (int j = 0; j < 16 && col0 + j < a.n; ++j) {
              float v = __uint_as_float(raw[j]);
              if (a.bias) v += a.bias[col0 + j];
              dst[j] = __float2bfloat16_rn(v);
            }
          }
        } else {  // float32 output
          float* dst = reinterpret_cast<float*>(a.out) + (size_t)a_row * a.ldo + col0;
          for (int j = 0; j < 16 && col0 + j < a.n; ++j) {
            float v = __uint_as_float(raw[j]);
            if (a.bias) v += a.bias[col0 + j];
            dst[j] = v;
          }
        }
      } else {
        // lane = weight row a_row, columns = tokens b_row0 + c0 + j: lanes write neighbouring n
        if (a.mode == kOutSiluMul) {
          // rows come in blocks of 16 gate rows followed by their 16 up rows
          const int channel = (a_row >> 5) * 16 + (lane & 15);
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const float mine = __uint_as_float(raw[j]);
            const float other = __shfl_down_sync(0xffffffffu, mine, 16);
            const int token = b_row0 + c0 + j;
            if (lane < 16 && token < a.m && a_row < a.n && channel < a.n / 2)
              reinterpret_cast<bf16*>(a.out)[(size_t)token * a.ldo + channel] =
                  __float2bfloat16_rn((mine / (1.f + expf(-mine))) * other);
          }
          continue;
        }
        const float bias = (a.bias && a.mode != kOutPartial && a_row < a.n) ? a.bias[a_row] : 0.f;
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const int token = b_row0 + c0 + j;
          if (token >= a.m || a_row >= a.n) continue;
          const float v = __uint_as_float(raw[j]) + bias;
          if (a.mode == kOutBF16) {
            reinterpret_cast<bf16*>(a.out)[(size_t)token * a.ldo + a_row] = __float2bfloat16_rn(v);
          } else if (a.mode == kOutF32) {
            reinterpret_cast<float*>(a.out)[(size_t)token * a.ldo + a_row] = v;
          } else {
            reinterpret_cast<float*>(a.out)[((size_t)blockIdx.z * a.m + token) * a.ldo + a_row] = v;
          }
        }
      }
    }
  } else {
    // a wait ran out: give copies that may still be in flight time to land before leaving
    for (int i = 0; i < 1000; ++i) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    tmem_free<TMEM_COLS>(tmem_base);
  }
}

// ------------------------------------------------------------------------------------ host side
template <int BN, int STAGES>
static int launch(const CUtensorMap& map_a, const CUtensorMap& map_b, const TcArgs& a, dim3 grid, cudaStream_t stream) {
  constexpr size_t smem = (size_t)STAGES * (A_STAGE_BYTES + BN * BK * 2) + 1024;
  static bool configured = false;
  if (!configured) {
    cudaError_t status = cudaFuncSetAttribute(gemm_tc_kernel<BN, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (status != cudaSuccess) CIE_FAIL("gemm_tcgen05: shared memory %zu: %s", smem, cudaGetErrorString(status));
    configured = true;
  }
  CIE_LAUNCH("gemm_tcgen05", gemm_tc_kernel<BN, STAGES>, grid, dim3(128), smem, stream, map_a, map_b, a);
  return 0;
}

}  // namespace cie

using namespace cie;

// x: [M, K] bfloat16, w: [N, K] bfloat16, both with 16-byte aligned rows (K % 8 == 0).
// mode: 0 bf16 out [M, N]; 1 float32 out [M, N]; 2 float32 partials [splits][M][N] (M <= 64 only);
// 3 SiLU(gate) * up -> bf16 [M, N / 2] with gate/up rows interleaved in blocks of 16 (M <= 64 only).
extern "C" int cie_gemm_tcgen05(const void* x, const void* w, const float* bias, void* out, int m,
                                int n, int k, int mode, int splits, int* err, void* stream) {
  if (m <= 0 || n <= 0) return 0;
  if (k < 8 || k % 8) CIE_FAIL("gemm_tcgen05: K must be a multiple of 8 (16-byte rows for TMA), got %d", k);
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(w)) & 15) CIE_FAIL("gemm_tcgen05: operands must be 16-byte aligned");
  if (splits < 1) CIE_FAIL("gemm_tcgen05: splits %d", splits);
  const bool swapped = m <= 64;
  if (!swapped && (mode == kOutPartial || mode == kOutSiluMul || splits != 1))
    CIE_FAIL("gemm_tcgen05: partial sums and the SiLU epilogue exist for at most 64 rows (got %d)", m);
  if (mode != kOutPartial && splits != 1) CIE_FAIL("gemm_tcgen05: %d splits need the partial-sum output", splits);
  if (mode == kOutSiluMul && (n % 32)) CIE_FAIL("gemm_tcgen05: the SiLU epilogue needs N to be a multiple of 32");
  TcArgs a;
  a.bias = bias; a.out = out; a.m = m; a.n = n; a.k = k; a.mode = mode; a.swapped = swapped ? 1 : 0; a.err = err;
  a.ldo = mode == kOutSiluMul ? n / 2 : n;
  const int k_tiles = (k + BK - 1) / BK;
  a.k_per_split = ((k_tiles + splits - 1) / splits) * BK;
  cudaStream_t s = (cudaStream_t)stream;
  CUtensorMap map_a, map_b;
  if (swapped) {
    const int bn = m <= 16 ? 16 : m <= 32 ? 32 : 64;
    if (!tensor_map_bf16(w, n, k, BM, &map_a) || !tensor_map_bf16(x, m, k, bn, &map_b)) CIE_FAIL("gemm_tcgen05: cuTensorMapEncodeTiled failed");
    dim3 grid((n + BM - 1) / BM, 1, splits);
    if (bn == 16) return launch<16, 8>(map_a, map_b, a, grid, s);
    if (bn == 32) return launch<32, 8>(map_a, map_b, a, grid, s);
    return launch<64, 6>(map_a, map_b, a, grid, s);
  }
  if (!tensor_map_bf16(x, m, k, BM, &map_a) || !tensor_map_bf16(w, n, k, 128, &map_b)) CIE_FAIL("gemm_tcgen05: cuTensorMapEncodeTiled failed");
  dim3 grid((m + BM - 1) / BM, (n + 127) / 128, 1);
  return launch<128, 3>(map_a, map_b, a, grid, s);
}
