// out[M, N] = x[M, K] * W[N, K]^T (+ bias) for 17 to 256 tokens: a product that is bound by reading
// the weights once, on the 5th-generation tensor cores.
//
// The tokens are the 128-row operand of tcgen05.mma (one or two tiles of 128, rows past M read as
// zero), the weight rows the N operand, whose width is a launch parameter: every CTA takes `rows`
// weight rows (a multiple of 16 up to 256), so that the weight matrix is dealt out evenly over the
// SMs whatever its height, which tiles of 128 rows cannot do (22,016 rows are 172 tiles for 148
// SMs).  Products with few weight rows and a long K are also cut along K: the `k_parts` CTAs of a
// thread-block cluster take one K range each of the same weight rows, leave their float32 sums in
// their own shared memory and, after a cluster barrier, each adds up and finishes some token rows,
// reading the others' sums through distributed shared memory.  Nothing goes through global memory
// twice and no second kernel adds anything up.
//
// Warp 0 copies (TMA, 128-byte swizzle) into a ring of stages of [tokens 128 x 64][weights rows x
// 64]; it asks for the weights of the first stages BEFORE `griddepcontrol.wait`, since weights do
// not depend on the kernel before this one (tensor memory is allocated after the wait).  Warp 1
// multiplies (one thread; accumulators in tensor memory), tcgen05.commit hands stages back.  Warps 2..5 read the accumulators with tcgen05.ld and
// finish: bias, bfloat16 or float32 rows, or SiLU(gate) * up for gate/up rows interleaved in
// blocks of 16.
//
// Every wait on an mbarrier is bounded: after about two seconds the kernel sets an error bit,
// stops issuing work, releases its tensor memory and returns; cluster barriers are reached by
// every thread on every path.
//
// The reference runs these products through cuBLAS (zeeshan8281/cloud-inference-from-scratch
// src/cloud_engine/model.py:100,134-136,217,227).
#include "blackwell.cuh"
#include "common.cuh"

CIE_DEFINE_LAST_ERROR()

namespace cie {

using namespace bw;
using bf16 = __nv_bfloat16;

constexpr int BM = 128;              // token rows of a tile (UMMA M)
constexpr int BK = 64;               // K per stage: 64 bf16 = 128 bytes = one swizzle row
constexpr int UMMA_K = 16;
constexpr int X_TILE_BYTES = BM * BK * 2;
constexpr int THREADS = 192;
constexpr int MAX_STAGES = 12;
constexpr int SMEM_LIMIT = 232448;   // most dynamic shared memory of a CTA on sm_100

constexpr int kOutBF16 = 0, kOutF32 = 1, kOutSiluMul = 3;

struct SkinnyArgs {
  const float* bias;   // [N] or null
  void* out;
  int m, n, k;         // tokens, weight rows, reduction size
  int ldo;             // elements between output rows (n, or n / 2 for the SiLU epilogue)
  int rows;            // weight rows a CTA takes: a multiple of 16 (32 with the SiLU epilogue), 16 .. 256
  int k_parts;         // CTAs of a cluster that share the K range of the same weight rows: 1, 2, 4, 8
  int stages;          // depth of the ring
  int x_rows;          // token rows a copy brings (the rest of a 128-row tile is never looked at): 16 .. 128
  int mode;
  int* err;
};

__device__ __forceinline__ void tmem_alloc_cols(uint32_t* slot, uint32_t cols) {   // whole warp; cols a power of two >= 32
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(slot)), "r"(cols));
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
}
__device__ __forceinline__ void tmem_free_cols(uint32_t base, uint32_t cols) {     // whole warp
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(base), "r"(cols));
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr));
}
__device__ __forceinline__ void cluster_arrive() { asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_wait() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }
// the shared::cluster address, in CTA `rank` of the cluster, of what lies at shared::cta address `local` here
__device__ __forceinline__ uint32_t peer_address(uint32_t local, int rank) {
  uint32_t remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local), "r"(rank));
  return remote;
}
__device__ __forceinline__ float4 peer_load4(uint32_t address) {
  float4 v;
  asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(address) : "memory");
  return v;
}

__device__ __forceinline__ float silu(float g) { return __fdividef(g, 1.f + __expf(-g)); }

__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  __nv_bfloat162 pair = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&pair);
}

// One token row's 16 (SiLU: 32 -> 16) finished values, starting at weight row `col`, go to global memory.
// v: 32 values (only the first 16 are used unless the mode is SiLU).
__device__ __forceinline__ void store_chunk(const SkinnyArgs& a, int row, int col, float* v, int width) {
  if (a.mode == kOutSiluMul) {
    // 16 gate rows followed by their 16 up rows (N and `rows` are multiples of 32)
    bf16* dst = reinterpret_cast<bf16*>(a.out) + (size_t)row * a.ldo + col / 2;
    uint32_t packed[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) packed[j] = pack2(silu(v[2 * j]) * v[16 + 2 * j], silu(v[2 * j + 1]) * v[16 + 2 * j + 1]);
    if (a.ldo % 8 == 0) {
      reinterpret_cast<uint4*>(dst)[0] = make_uint4(packed[0], packed[1], packed[2], packed[3]);
      reinterpret_cast<uint4*>(dst)[1] = make_uint4(packed[4], packed[5], packed[6], packed[7]);
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) reinterpret_cast<uint32_t*>(dst)[j] = packed[j];
    }
    return;
  }
#pragma unroll 1
  for (int half = 0; half < width; half += 16) {
    const int c = col + half;
    if (c >= a.n) return;
    float* w = v + half;
    if (a.bias) {
#pragma unroll
      for (int j = 0; j < 16; ++j) w[j] += c + j < a.n ? a.bias[c + j] : 0.f;
    }
    const bool whole = c + 16 <= a.n;
    if (a.mode == kOutBF16) {
      bf16* dst = reinterpret_cast<bf16*>(a.out) + (size_t)row * a.ldo + c;
      if (whole && a.ldo % 8 == 0) {
        reinterpret_cast<uint4*>(dst)[0] = make_uint4(pack2(w[0], w[1]), pack2(w[2], w[3]), pack2(w[4], w[5]), pack2(w[6], w[7]));
        reinterpret_cast<uint4*>(dst)[1] = make_uint4(pack2(w[8], w[9]), pack2(w[10], w[11]), pack2(w[12], w[13]), pack2(w[14], w[15]));
      } else {
        for (int j = 0; j < 16 && c + j < a.n; ++j) dst[j] = __float2bfloat16_rn(w[j]);
      }
    } else {
      float* dst = reinterpret_cast<float*>(a.out) + (size_t)row * a.ldo + c;
      if (whole && a.ldo % 4 == 0) {
#pragma unroll
        for (int q = 0; q < 4; ++q) reinterpret_cast<float4*>(dst)[q] = make_float4(w[4 * q], w[4 * q + 1], w[4 * q + 2], w[4 * q + 3]);
      } else {
        for (int j = 0; j < 16 && c + j < a.n; ++j) dst[j] = w[j];
      }
    }
  }
}

template <int MT>
__global__ void __launch_bounds__(THREADS, 1) gemm_skinny_kernel(const __grid_constant__ CUtensorMap map_x,
                                                                  const __grid_constant__ CUtensorMap map_w,
                                                                  const SkinnyArgs a) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  // the dynamic shared memory window is only guaranteed 16-byte aligned: align by hand (the same
  // offset in every CTA of a cluster, since they run the same kernel with the same static data)
  unsigned char* tiles = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  __shared__ __align__(8) uint64_t full_bar[MAX_STAGES];
  __shared__ __align__(8) uint64_t empty_bar[MAX_STAGES];
  __shared__ __align__(8) uint64_t acc_bar;
  __shared__ uint32_t tmem_base_s;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int rank = blockIdx.x;                       // which K range (the cluster lies along x)
  const int w_row0 = blockIdx.y * a.rows;
  const int stages = a.stages;
  const int stage_bytes = MT * X_TILE_BYTES + a.rows * BK * 2;
  // what the copies of a stage bring: token rows past x_rows of the tile stay as they were, and the
  // accumulator rows they feed are never read
  const int stage_tx = MT * a.x_rows * BK * 2 + a.rows * BK * 2;
  const int k_tiles = (a.k + BK - 1) / BK;
  const int share = k_tiles / a.k_parts, extra = k_tiles % a.k_parts;
  const int kt0 = rank * share + min(rank, extra);
  const int count = share + (rank < extra ? 1 : 0);
  const int acc_stride = (a.rows + 31) & ~31;        // columns of tensor memory between the accumulators
  uint32_t tmem_cols = 32;
  while ((int)tmem_cols < MT * acc_stride) tmem_cols <<= 1;

  if (tid == 0) {
    for (int s = 0; s < stages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    mbar_init(&acc_bar, 1);
    mbar_init_fence();
  }
  __syncthreads();
  // Tensor memory is asked for after `griddepcontrol.wait` only: a CTA of an earlier kernel that is
  // still to allocate its own on this SM must never find it taken by a CTA that waits for that
  // kernel.  Warps 1..5 (the product and the epilogue) meet once it is there.
  uint32_t tmem_base = 0;
  if (warp >= 1) {
    pdl_wait();
    pdl_trigger();
    if (warp == 1) tmem_alloc_cols(&tmem_base_s, tmem_cols);
    tc_fence_before();
    asm volatile("bar.sync 1, %0;" ::"n"(THREADS - 32) : "memory");
    tc_fence_after();
    tmem_base = tmem_base_s;
  }

  if (warp == 0) {
    if (lane == 0) {
      // ---- TMA producer: the weights of the first stages do not wait for the kernel before
      const int early = min(stages, count);
      for (int kt = 0; kt < early; ++kt) {
        mbar_expect_tx(&full_bar[kt], stage_tx);
        tma_load_2d(tiles + (size_t)kt * stage_bytes + MT * X_TILE_BYTES, &map_w, &full_bar[kt], (kt0 + kt) * BK, w_row0);
      }
      pdl_wait();
      pdl_trigger();
      for (int kt = 0; kt < early; ++kt) {
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
          tma_load_2d(tiles + (size_t)kt * stage_bytes + mt * X_TILE_BYTES, &map_x, &full_bar[kt], (kt0 + kt) * BK, mt * BM);
      }
      for (int kt = early; kt < count; ++kt) {
        const int s = kt % stages;
        if (!mbar_wait(&empty_bar[s], ((kt / stages) - 1) & 1, a.err)) break;
        mbar_expect_tx(&full_bar[s], stage_tx);
        unsigned char* dst = tiles + (size_t)s * stage_bytes;
        tma_load_2d(dst + MT * X_TILE_BYTES, &map_w, &full_bar[s], (kt0 + kt) * BK, w_row0);
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) tma_load_2d(dst + mt * X_TILE_BYTES, &map_x, &full_bar[s], (kt0 + kt) * BK, mt * BM);
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (lane == 0) {
      // ---- MMA issuer
      const uint32_t idesc = idesc_bf16(BM, a.rows);
      for (int kt = 0; kt < count; ++kt) {
        const int s = kt % stages;
        if (!mbar_wait(&full_bar[s], (kt / stages) & 1, a.err)) break;
        tc_fence_after();
        const uint32_t x_addr = smem_u32(tiles + (size_t)s * stage_bytes);
        const uint64_t w_desc = smem_desc_sw128(x_addr + MT * X_TILE_BYTES);
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
          const uint64_t x_desc = smem_desc_sw128(x_addr + mt * X_TILE_BYTES);
#pragma unroll
          for (int kk = 0; kk < BK / UMMA_K; ++kk) {
            // advancing 16 elements (32 bytes) inside the swizzled row: +2 in 16-byte units
            umma_bf16(tmem_base + mt * acc_stride, x_desc + 2 * kk, w_desc + 2 * kk, idesc, (kt > 0 || kk > 0) ? 1u : 0u);
          }
        }
        tc_commit(&empty_bar[s]);
      }
      tc_commit(&acc_bar);   // arrives when every product issued so far has finished (at once if there was none)
    }
    __syncwarp();
  }

  // ---- epilogue: warps 2..5; a warp reads the tensor-memory lanes of its quarter (token rows)
  const int pitch = a.rows + 4;   // floats between token rows of the sums a cluster exchanges
  float* sums = reinterpret_cast<float*>(tiles);
  bool ready = true;
  if (warp >= 2) {
    ready = mbar_wait(&acc_bar, 0, a.err);
    tc_fence_after();
    const int quarter = warp & 3;
    if (ready) {
#pragma unroll 1
      for (int mt = 0; mt < MT; ++mt) {
        const int row = mt * BM + quarter * 32 + lane;
#pragma unroll 1
        for (int c0 = 0; c0 < a.rows; c0 += 32) {
          const int width = min(32, a.rows - c0);   // 32 or 16
          uint32_t raw[32];
          if (count > 0) {
            const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + mt * acc_stride + c0;
            tmem_ld16(taddr, raw);
            if (width > 16) tmem_ld16(taddr + 16, raw + 16);
            tc_wait_ld();
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) raw[j] = 0;
          }
          if (row >= a.m) continue;
          float v[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(raw[j]);
          if (a.k_parts == 1) {
            if (w_row0 + c0 < a.n) store_chunk(a, row, w_row0 + c0, v, width);
          } else {
            float4* dst = reinterpret_cast<float4*>(sums + (size_t)row * pitch + c0);
#pragma unroll
            for (int q = 0; q < 8; ++q)
              if (q * 4 < width) dst[q] = make_float4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
          }
        }
      }
    }
  }
  if (a.k_parts > 1) {
    // every CTA of the cluster has left its sums (or has given up: then the result is void and the
    // error word says so); token row r is finished by the CTA of rank r % k_parts
    cluster_arrive();
    cluster_wait();
    if (warp >= 2 && ready) {
      const int t = (warp - 2) * 32 + lane;
      const int live = min(a.m, MT * BM);
      const int mine = live > rank ? (live - rank + a.k_parts - 1) / a.k_parts : 0;
      const int per_row = a.mode == kOutSiluMul ? a.rows / 32 : a.rows / 16;   // chunks of a token row
      const int lanes_per_chunk = 4;                                           // four threads share a chunk
      const int items = mine * per_row * lanes_per_chunk;
      const uint32_t base = smem_u32(sums);
      for (int i = t; i < items; i += 4 * 32) {
        const int part = i % lanes_per_chunk;
        const int chunk = (i / lanes_per_chunk) % per_row;
        const int row = rank + (i / (lanes_per_chunk * per_row)) * a.k_parts;
        if (a.mode == kOutSiluMul) {
          // this thread: four channels of a block of 16: gates at 32 * chunk + 4 * part, ups 16 further
          const int col = chunk * 32 + part * 4;
          float4 gate = make_float4(0.f, 0.f, 0.f, 0.f), up = gate;
          const uint32_t local = base + (uint32_t)(((size_t)row * pitch + col) * sizeof(float));
          for (int p = 0; p < a.k_parts; ++p) {
            const uint32_t peer = peer_address(local, p);
            const float4 g = peer_load4(peer), u = peer_load4(peer + 16 * sizeof(float));
            gate.x += g.x; gate.y += g.y; gate.z += g.z; gate.w += g.w;
            up.x += u.x; up.y += u.y; up.z += u.z; up.w += u.w;
          }
          const int channel = (w_row0 + chunk * 32) / 2 + part * 4;
          if (w_row0 + chunk * 32 < a.n) {
            bf16* dst = reinterpret_cast<bf16*>(a.out) + (size_t)row * a.ldo + channel;
            const uint32_t lo = pack2(silu(gate.x) * up.x, silu(gate.y) * up.y), hi = pack2(silu(gate.z) * up.z, silu(gate.w) * up.w);
            if (a.ldo % 4 == 0) {
              *reinterpret_cast<uint2*>(dst) = make_uint2(lo, hi);
            } else {
              reinterpret_cast<uint32_t*>(dst)[0] = lo;
              reinterpret_cast<uint32_t*>(dst)[1] = hi;
            }
          }
        } else {
          const int col = chunk * 16 + part * 4;
          float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
          const uint32_t local = base + (uint32_t)(((size_t)row * pitch + col) * sizeof(float));
          for (int p = 0; p < a.k_parts; ++p) {
            const float4 s = peer_load4(peer_address(local, p));
            sum.x += s.x; sum.y += s.y; sum.z += s.z; sum.w += s.w;
          }
          const int c = w_row0 + col;
          float w[4] = {sum.x, sum.y, sum.z, sum.w};
          if (a.bias) {
#pragma unroll
            for (int j = 0; j < 4; ++j) w[j] += c + j < a.n ? a.bias[c + j] : 0.f;
          }
          if (c < a.n) {
            const bool whole = c + 4 <= a.n;
            if (a.mode == kOutBF16) {
              bf16* dst = reinterpret_cast<bf16*>(a.out) + (size_t)row * a.ldo + c;
              if (whole && a.ldo % 4 == 0) {
                *reinterpret_cast<uint2*>(dst) = make_uint2(pack2(w[0], w[1]), pack2(w[2], w[3]));
              } else {
                for (int j = 0; j < 4 && c + j < a.n; ++j) dst[j] = __float2bfloat16_rn(w[j]);
              }
            } else {
              float* dst = reinterpret_cast<float*>(a.out) + (size_t)row * a.ldo + c;
              if (whole && a.ldo % 4 == 0) {
                *reinterpret_cast<float4*>(dst) = make_float4(w[0], w[1], w[2], w[3]);
              } else {
                for (int j = 0; j < 4 && c + j < a.n; ++j) dst[j] = w[j];
              }
            }
          }
        }
      }
    }
    // nobody leaves while a peer may still read its sums
    cluster_arrive();
    cluster_wait();
  }
  if (!ready) {
    // a wait ran out: give copies that may still be in flight time to land before leaving
    for (int i = 0; i < 1000; ++i) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_free_cols(tmem_base, tmem_cols);
}

static size_t skinny_smem(int tiles_m, int rows, int stages) {
  return (size_t)stages * (tiles_m * X_TILE_BYTES + rows * BK * 2) + 1024;
}

template <int MT>
static cudaError_t configure(size_t smem) {
  static size_t configured = 0;
  if (smem <= configured) return cudaSuccess;
  cudaError_t status = cudaFuncSetAttribute(gemm_skinny_kernel<MT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (status == cudaSuccess) configured = smem;
  return status;
}

template <int MT>
static int launch_skinny(const CUtensorMap& map_x, const CUtensorMap& map_w, const SkinnyArgs& a, int row_parts, cudaStream_t stream) {
  const size_t smem = skinny_smem(MT, a.rows, a.stages);
  cudaError_t status = configure<MT>(smem);
  if (status != cudaSuccess) CIE_FAIL("gemm_skinny: shared memory %zu: %s", smem, cudaGetErrorString(status));
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3(a.k_parts, row_parts, 1);
  config.blockDim = dim3(THREADS);
  config.dynamicSmemBytes = smem;
  config.stream = stream;
  cudaLaunchAttribute attributes[2];
  int count = 0;
  if (a.k_parts > 1) {
    attributes[count].id = cudaLaunchAttributeClusterDimension;
    attributes[count].val.clusterDim.x = a.k_parts;
    attributes[count].val.clusterDim.y = 1;
    attributes[count].val.clusterDim.z = 1;
    ++count;
  }
  if (pdl_enabled()) {
    attributes[count].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attributes[count].val.programmaticStreamSerializationAllowed = 1;
    ++count;
  }
  config.attrs = attributes;
  config.numAttrs = count;
  status = cudaLaunchKernelEx(&config, gemm_skinny_kernel<MT>, map_x, map_w, a);
  if (status != cudaSuccess) CIE_FAIL("gemm_skinny: launch failed: %s", cudaGetErrorString(status));
  return 0;
}

template <int MT>
static int clusters_at_once(int rows, int k_parts, int stages) {
  const size_t smem = skinny_smem(MT, rows, stages);
  if (configure<MT>(smem) != cudaSuccess) {
    cudaGetLastError();
    return -1;
  }
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3(k_parts, 1, 1);
  config.blockDim = dim3(THREADS);
  config.dynamicSmemBytes = smem;
  cudaLaunchAttribute attribute;
  attribute.id = cudaLaunchAttributeClusterDimension;
  attribute.val.clusterDim.x = k_parts;
  attribute.val.clusterDim.y = 1;
  attribute.val.clusterDim.z = 1;
  config.attrs = &attribute;
  config.numAttrs = 1;
  int clusters = 0;
  if (cudaOccupancyMaxActiveClusters(&clusters, gemm_skinny_kernel<MT>, &config) != cudaSuccess) {
    cudaGetLastError();
    return -1;
  }
  return clusters;
}

}  // namespace cie

using namespace cie;

// Most bytes of dynamic shared memory a launch may ask for, and what a launch with these sizes asks for.
extern "C" int cie_gemm_skinny_smem_limit() { return SMEM_LIMIT; }
extern "C" long long cie_gemm_skinny_smem(int m, int rows, int stages) { return (long long)skinny_smem(m > BM ? 2 : 1, rows, stages); }

// How many clusters of `k_parts` CTAs with these sizes the device runs at one time (-1: the query failed).
extern "C" int cie_gemm_skinny_clusters(int m, int rows, int k_parts, int stages) {
  if (rows < 16 || rows > 256 || rows % 16 || stages < 2 || stages > MAX_STAGES) return 0;
  if (k_parts != 1 && k_parts != 2 && k_parts != 4 && k_parts != 8) return 0;
  if (skinny_smem(m > BM ? 2 : 1, rows, stages) > (size_t)SMEM_LIMIT) return 0;
  return m > BM ? clusters_at_once<2>(rows, k_parts, stages) : clusters_at_once<1>(rows, k_parts, stages);
}

// x: [M, K] bfloat16, w: [N, K] bfloat16, both with 16-byte aligned rows (K % 8 == 0); 1 <= M <= 256.
// mode: 0 bf16 out [M, N]; 1 float32 out [M, N]; 3 SiLU(gate) * up -> bf16 [M, N / 2] with gate/up
// rows interleaved in blocks of 16.  rows: weight rows a CTA takes (a multiple of 16, of 32 for
// mode 3, at most 256); k_parts: 1, 2, 4 or 8 CTAs of a cluster share the K range (each needs at
// least one block of 64); stages: depth of the ring, 2 .. 12, within the shared memory of an SM,
// and, with k_parts > 1, large enough to hold the float32 sums of the CTA's tile afterwards.
extern "C" int cie_gemm_skinny(const void* x, const void* w, const float* bias, void* out, int m, int n, int k,
                               int mode, int rows, int k_parts, int stages, int* err, void* stream) {
  if (m <= 0 || n <= 0) return 0;
  if (m > 2 * BM) CIE_FAIL("gemm_skinny: at most %d rows, got %d", 2 * BM, m);
  if (k < 8 || k % 8) CIE_FAIL("gemm_skinny: K must be a multiple of 8 (16-byte rows for TMA), got %d", k);
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(w)) & 15) CIE_FAIL("gemm_skinny: operands must be 16-byte aligned");
  if (mode != kOutBF16 && mode != kOutF32 && mode != kOutSiluMul) CIE_FAIL("gemm_skinny: mode %d", mode);
  if (mode == kOutSiluMul && (n % 32 || rows % 32 || bias)) CIE_FAIL("gemm_skinny: the SiLU epilogue needs N and the rows of a CTA to be multiples of 32 and no bias");
  if (rows < 16 || rows > 256 || rows % 16) CIE_FAIL("gemm_skinny: a CTA takes 16 .. 256 weight rows in steps of 16, got %d", rows);
  if (k_parts != 1 && k_parts != 2 && k_parts != 4 && k_parts != 8) CIE_FAIL("gemm_skinny: 1, 2, 4 or 8 K ranges, got %d", k_parts);
  const int k_tiles = (k + BK - 1) / BK;
  if (k_parts > k_tiles) CIE_FAIL("gemm_skinny: %d K ranges of a K of %d", k_parts, k);
  if (stages < 2 || stages > MAX_STAGES) CIE_FAIL("gemm_skinny: 2 .. %d stages, got %d", MAX_STAGES, stages);
  const int tiles_m = m > BM ? 2 : 1;
  const size_t smem = skinny_smem(tiles_m, rows, stages);
  if (smem > (size_t)SMEM_LIMIT) CIE_FAIL("gemm_skinny: %d stages of %d weight rows need %zu bytes of shared memory", stages, rows, smem);
  if (k_parts > 1 && (size_t)tiles_m * BM * (rows + 4) * sizeof(float) > smem - 1024)
    CIE_FAIL("gemm_skinny: the ring (%zu bytes) cannot hold the sums of %d x %d", smem - 1024, tiles_m * BM, rows);
  const int row_parts = (n + rows - 1) / rows;
  if (row_parts > 65535) CIE_FAIL("gemm_skinny: %d parts of weight rows", row_parts);
  SkinnyArgs a = {};
  a.bias = bias; a.out = out; a.m = m; a.n = n; a.k = k; a.mode = mode; a.err = err;
  a.ldo = mode == kOutSiluMul ? n / 2 : n;
  a.rows = rows; a.k_parts = k_parts; a.stages = stages;
  a.x_rows = tiles_m == 1 ? (m + 15) / 16 * 16 : BM;
  CUtensorMap map_x, map_w;
  if (!tensor_map_bf16(x, m, k, a.x_rows, &map_x) || !tensor_map_bf16(w, n, k, rows, &map_w)) CIE_FAIL("gemm_skinny: cuTensorMapEncodeTiled failed");
  cudaStream_t s = (cudaStream_t)stream;
  return tiles_m == 2 ? launch_skinny<2>(map_x, map_w, a, row_parts, s) : launch_skinny<1>(map_x, map_w, a, row_parts, s);
}
