// out[M, N] = x[M, K] * W[N, K]^T (+ bias) on the 5th-generation tensor cores: operands come by
// TMA (cp.async.bulk.tensor, 128-byte swizzle) into a multi-stage shared-memory ring, one elected
// thread issues tcgen05.mma with the float32 accumulator in tensor memory, tcgen05.commit hands
// stages back to the TMA thread through mbarriers, and the four warps read the accumulator with
// tcgen05.ld for the epilogue.  Every CTA copies its own tiles; nothing is shared across a cluster.
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

constexpr int kOutBF16 = 0, kOutF32 = 1, kOutPartial = 2, kOutSiluMul = 3, kOutResidual = 4;



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
  // persistent kernel (more than 64 rows) only:
  // row scale: result rows are multiplied by rsqrt(sum of row_sq[m][0 .. row_tiles) / K + eps)
  const float* row_sq;
  int row_tiles;
  float eps;
  // residual epilogue (mode 4): residual[m][n] += result (+ bias); sq[m][n / 32] = sum of squares of
  // the 32 new values; with next_gain also scaled[m][n] = bfloat16(new value * next_gain[n])
  float* residual;
  float* sq;
  bf16* scaled;
  const float* next_gain;
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

// ------------------------------------------------------------------------------------ many rows
// More than 64 tokens: tokens are the 128-row operand, 256 weight rows the N operand.  CTAs are
// persistent (one per SM) and walk over the tiles, token blocks fastest, so that the CTAs running at
// one time share weight rows in L2.  Warp 0 copies (TMA), warp 1 multiplies (one thread), warps
// 2..5 finish: the accumulator is double buffered in tensor memory (2 x 256 columns), so a tile is
// written out while the next one is multiplied.
constexpr int PBN = 256;
constexpr int PSTAGES = 4;
constexpr int P_STAGE_BYTES = A_STAGE_BYTES + PBN * BK * 2;
constexpr int P_THREADS = 192;

__global__ void __launch_bounds__(P_THREADS, 1) gemm_tc_persistent_kernel(const __grid_constant__ CUtensorMap map_a,
                                                                           const __grid_constant__ CUtensorMap map_b,
                                                                           const TcArgs a) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  unsigned char* tiles = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  __shared__ __align__(8) uint64_t full_bar[PSTAGES], empty_bar[PSTAGES], acc_full[2], acc_empty[2];
  __shared__ uint32_t tmem_base_s;

  pdl_wait();
  pdl_trigger();
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int tiles_m = (a.m + BM - 1) / BM, tiles_n = (a.n + PBN - 1) / PBN;
  const int total = tiles_m * tiles_n;
  const int k_tiles = (a.k + BK - 1) / BK;

  if (tid == 0) {
    for (int s = 0; s < PSTAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(&acc_full[b], 1); mbar_init(&acc_empty[b], 128); }
    mbar_init_fence();
  }
  if (warp == 1) tmem_alloc<512>(&tmem_base_s);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_s;

  if (warp == 0) {
    if (lane == 0) {
      // ---- TMA producer
      int step = 0;
      bool alive = true;
      for (int t = blockIdx.x; t < total && alive; t += gridDim.x) {
        const int row0 = (t % tiles_m) * BM, col0 = (t / tiles_m) * PBN;
        for (int kt = 0; kt < k_tiles; ++kt, ++step) {
          const int s = step % PSTAGES;
          if (step >= PSTAGES && !mbar_wait(&empty_bar[s], ((step / PSTAGES) - 1) & 1, a.err)) { alive = false; break; }
          mbar_expect_tx(&full_bar[s], P_STAGE_BYTES);
          unsigned char* dst = tiles + (size_t)s * P_STAGE_BYTES;
          tma_load_2d(dst, &map_a, &full_bar[s], kt * BK, row0);
          tma_load_2d(dst + A_STAGE_BYTES, &map_b, &full_bar[s], kt * BK, col0);
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (lane == 0) {
      // ---- MMA issuer
      constexpr uint32_t idesc = idesc_bf16(BM, PBN);
      const uint64_t desc0 = smem_desc_sw128(smem_u32(tiles));
      int step = 0, local = 0;
      bool alive = true;
      for (int t = blockIdx.x; t < total && alive; t += gridDim.x, ++local) {
        const int buf = local & 1;
        // the epilogue warps have taken the tile before last out of this accumulator
        if (local >= 2 && !mbar_wait(&acc_empty[buf], ((local >> 1) - 1) & 1, a.err)) break;
        tc_fence_after();
        for (int kt = 0; kt < k_tiles; ++kt, ++step) {
          const int s = step % PSTAGES;
          if (!mbar_wait(&full_bar[s], (step / PSTAGES) & 1, a.err)) { alive = false; break; }
          tc_fence_after();
          const uint64_t a_desc = desc0 + (uint64_t)((s * P_STAGE_BYTES) >> 4);
          const uint64_t b_desc = a_desc + (uint64_t)(A_STAGE_BYTES >> 4);
#pragma unroll
          for (int kk = 0; kk < BK / UMMA_K; ++kk)
            umma_bf16(tmem_base + buf * PBN, a_desc + 2 * kk, b_desc + 2 * kk, idesc, (kt > 0 || kk > 0) ? 1u : 0u);
          tc_commit(&empty_bar[s]);
        }
        if (alive) tc_commit(&acc_full[buf]);
      }
    }
    __syncwarp();
  } else {
    // ---- epilogue: this warp reads tensor-memory lanes 32 * (warp % 4) ..+31 (token rows)
    const int quarter = warp & 3;
    const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
    const int sq_tiles = (a.n + 31) / 32;
    int local = 0;
    for (int t = blockIdx.x; t < total; t += gridDim.x, ++local) {
      const int buf = local & 1;
      const int row = (t % tiles_m) * BM + quarter * 32 + lane, col_tile = (t / tiles_m) * PBN;
      const bool row_ok = row < a.m;
      // the row's scale, while the tile is still being multiplied
      float scale = 1.f;
      if (a.row_sq && row_ok) {
        float parts[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        const float* src = a.row_sq + (size_t)row * a.row_tiles;
        for (int i = 0; i < a.row_tiles; i += 8) {
#pragma unroll
          for (int j = 0; j < 8; ++j) parts[j] += i + j < a.row_tiles ? src[i + j] : 0.f;
        }
        const float sum = ((parts[0] + parts[1]) + (parts[2] + parts[3])) + ((parts[4] + parts[5]) + (parts[6] + parts[7]));
        scale = rsqrtf(sum / (float)a.k + a.eps);
      }
      if (k_tiles > 0 && !mbar_wait(&acc_full[buf], (local >> 1) & 1, a.err)) break;
      tc_fence_after();
#pragma unroll 1
      for (int c = 0; c < PBN / 32; ++c) {
        const int col0 = col_tile + c * 32;
        uint32_t raw[32];
        if (k_tiles > 0) {
          tmem_ld32(tmem_base + lane_base + buf * PBN + c * 32, raw);
          tc_wait_ld();
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) raw[j] = 0;
        }
        if (c == PBN / 32 - 1) {   // the accumulator is in registers: the next tile but one may use it
          tc_fence_before();
          mbar_arrive(&acc_empty[buf]);
        }
        if (!row_ok || col0 >= a.n) continue;
        const bool whole = col0 + 32 <= a.n;
        float v[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(raw[j]) * scale;
        if (a.bias && a.mode != kOutSiluMul) {
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] += col0 + j < a.n ? a.bias[col0 + j] : 0.f;
        }
        if (a.mode == kOutBF16) {
          bf16* dst = reinterpret_cast<bf16*>(a.out) + (size_t)row * a.ldo + col0;
          if (whole && a.ldo % 8 == 0) {
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              uint32_t packed[4];
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                __nv_bfloat162 pair = __floats2bfloat162_rn(v[q * 8 + 2 * j], v[q * 8 + 2 * j + 1]);
                packed[j] = *reinterpret_cast<uint32_t*>(&pair);
              }
              reinterpret_cast<uint4*>(dst)[q] = make_uint4(packed[0], packed[1], packed[2], packed[3]);
            }
          } else {
            for (int j = 0; j < 32 && col0 + j < a.n; ++j) dst[j] = __float2bfloat16_rn(v[j]);
          }
        } else if (a.mode == kOutF32) {
          float* dst = reinterpret_cast<float*>(a.out) + (size_t)row * a.ldo + col0;
          if (whole && a.ldo % 4 == 0) {
#pragma unroll
            for (int q = 0; q < 8; ++q) reinterpret_cast<float4*>(dst)[q] = make_float4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
          } else {
            for (int j = 0; j < 32 && col0 + j < a.n; ++j) dst[j] = v[j];
          }
        } else if (a.mode == kOutSiluMul) {
          // 16 gate columns followed by their 16 up columns (N is a multiple of 32)
          bf16* dst = reinterpret_cast<bf16*>(a.out) + (size_t)row * a.ldo + col0 / 2;
          uint32_t packed[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const float g0 = v[2 * j], g1 = v[2 * j + 1];
            __nv_bfloat162 pair = __floats2bfloat162_rn(__fdividef(g0, 1.f + __expf(-g0)) * v[16 + 2 * j],
                                                        __fdividef(g1, 1.f + __expf(-g1)) * v[16 + 2 * j + 1]);
            packed[j] = *reinterpret_cast<uint32_t*>(&pair);
          }
          if (a.ldo % 8 == 0) {
            reinterpret_cast<uint4*>(dst)[0] = make_uint4(packed[0], packed[1], packed[2], packed[3]);
            reinterpret_cast<uint4*>(dst)[1] = make_uint4(packed[4], packed[5], packed[6], packed[7]);
          } else {
#pragma unroll
            for (int j = 0; j < 8; ++j) reinterpret_cast<uint32_t*>(dst)[j] = packed[j];
          }
        } else {   // kOutResidual
          float* res = a.residual + (size_t)row * a.n + col0;
          float square = 0.f;
          if (whole && a.n % 8 == 0) {
            float4 old[8];
#pragma unroll
            for (int q = 0; q < 8; ++q) old[q] = reinterpret_cast<const float4*>(res)[q];
#pragma unroll
            for (int q = 0; q < 8; ++q) {
              v[4 * q] += old[q].x; v[4 * q + 1] += old[q].y; v[4 * q + 2] += old[q].z; v[4 * q + 3] += old[q].w;
              reinterpret_cast<float4*>(res)[q] = make_float4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
            }
#pragma unroll
            for (int j = 0; j < 32; ++j) square += v[j] * v[j];
            if (a.scaled) {
              bf16* dst = a.scaled + (size_t)row * a.n + col0;
#pragma unroll
              for (int q = 0; q < 4; ++q) {
                const float4 g0 = *reinterpret_cast<const float4*>(a.next_gain + col0 + q * 8);
                const float4 g1 = *reinterpret_cast<const float4*>(a.next_gain + col0 + q * 8 + 4);
                const float g[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
                uint32_t packed[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                  __nv_bfloat162 pair = __floats2bfloat162_rn(v[q * 8 + 2 * j] * g[2 * j], v[q * 8 + 2 * j + 1] * g[2 * j + 1]);
                  packed[j] = *reinterpret_cast<uint32_t*>(&pair);
                }
                reinterpret_cast<uint4*>(dst)[q] = make_uint4(packed[0], packed[1], packed[2], packed[3]);
              }
            }
          } else {
            for (int j = 0; j < 32 && col0 + j < a.n; ++j) {
              const float updated = res[j] + v[j];
              res[j] = updated;
              square += updated * updated;
              if (a.scaled) a.scaled[(size_t)row * a.n + col0 + j] = __float2bfloat16_rn(updated * a.next_gain[col0 + j]);
            }
          }
          a.sq[(size_t)row * sq_tiles + col0 / 32] = square;
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_free<512>(tmem_base);
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

static int launch_persistent(const void* x, const void* w, const TcArgs& a, cudaStream_t stream) {
  CUtensorMap map_a, map_b;
  if (!tensor_map_bf16(x, a.m, a.k, BM, &map_a) || !tensor_map_bf16(w, a.n, a.k, PBN, &map_b))
    CIE_FAIL("gemm_tcgen05: cuTensorMapEncodeTiled failed");
  constexpr size_t smem = (size_t)PSTAGES * P_STAGE_BYTES + 1024;
  static bool configured = false;
  static int sms = 0;
  if (!configured) {
    cudaError_t status = cudaFuncSetAttribute(gemm_tc_persistent_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (status != cudaSuccess) CIE_FAIL("gemm_tcgen05: shared memory %zu: %s", smem, cudaGetErrorString(status));
    int device = 0;
    cudaGetDevice(&device);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
    if (sms < 1) sms = 1;
    configured = true;
  }
  const int total = ((a.m + BM - 1) / BM) * ((a.n + PBN - 1) / PBN);
  CIE_LAUNCH("gemm_tcgen05", gemm_tc_persistent_kernel, dim3(total < sms ? total : sms), dim3(P_THREADS), smem, stream, map_a, map_b, a);
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
  TcArgs a = {};
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
  return launch_persistent(x, w, a, s);
}

// More than 64 rows with everything the persistent kernel can fold in.
//  row_sq ([M, row_tiles] float32, or null): every result row m is multiplied by
//  rsqrt(sum of row_sq[m] / K + eps) before bias, activation or residual add.
//  mode 0 bf16 out, 1 float32 out, 3 SiLU(gate) * up (gate/up rows interleaved in blocks of 16),
//  4 residual[M, N] += result (+ bias), sq[M, ceil(N / 32)] = sums of squares of the new values per
//  32 columns and, with next_gain, scaled[M, N] = bfloat16(new value * next_gain).
extern "C" int cie_gemm_tcgen05_ex(const void* x, const float* row_sq, int row_tiles, float eps, const void* w,
                                   const float* bias, void* out, float* residual, float* sq, void* scaled,
                                   const float* next_gain, int m, int n, int k, int mode, int* err, void* stream) {
  if (m <= 0 || n <= 0) return 0;
  if (m <= 64) CIE_FAIL("gemm_tcgen05_ex: the persistent kernel is for more than 64 rows (got %d)", m);
  if (k < 8 || k % 8) CIE_FAIL("gemm_tcgen05_ex: K must be a multiple of 8, got %d", k);
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(w)) & 15) CIE_FAIL("gemm_tcgen05_ex: operands must be 16-byte aligned");
  if (mode != kOutBF16 && mode != kOutF32 && mode != kOutSiluMul && mode != kOutResidual) CIE_FAIL("gemm_tcgen05_ex: mode %d", mode);
  if (mode == kOutSiluMul && n % 32) CIE_FAIL("gemm_tcgen05_ex: the SiLU epilogue needs N to be a multiple of 32");
  if (mode == kOutResidual && (!residual || !sq)) CIE_FAIL("gemm_tcgen05_ex: the residual epilogue needs the residual and a place for the sums of squares");
  if (mode != kOutResidual && !out) CIE_FAIL("gemm_tcgen05_ex: null output");
  if ((scaled != nullptr) != (next_gain != nullptr)) CIE_FAIL("gemm_tcgen05_ex: the scaled copy needs both its buffer and the gain");
  if (row_sq && row_tiles < 1) CIE_FAIL("gemm_tcgen05_ex: %d tiles of sums of squares", row_tiles);
  TcArgs a = {};
  a.bias = bias; a.out = out; a.m = m; a.n = n; a.k = k; a.mode = mode; a.swapped = 0; a.err = err;
  a.ldo = mode == kOutSiluMul ? n / 2 : n;
  a.row_sq = row_sq; a.row_tiles = row_tiles; a.eps = eps;
  a.residual = residual; a.sq = sq; a.scaled = (bf16*)scaled; a.next_gain = next_gain;
  return launch_persistent(x, w, a, (cudaStream_t)stream);
}
