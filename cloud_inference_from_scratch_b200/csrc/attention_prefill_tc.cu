// Ragged causal attention of prompt portions over the paged cache on the 5th-generation tensor
// cores (tcgen05), bfloat16, head size 64 or 128 (-DHEAD_DIM), pages of a multiple of 16 tokens.
//
// One CTA takes 128 query rows of ONE request and ONE kv head; a row is a (token, query head of the
// group) pair, so the heads of a group share every key and value.  Keys go by in tiles of 128:
//
//   TMA warp      key/value pages -> shared memory, boxes of 16 keys x 64 columns with 128-byte
//                 swizzle, two stages, one mbarrier per stage.
//   MMA thread    S = Q K^T (128 x 128, float32, in tensor memory, double buffered), then
//                 O += P V (128 x HEAD_DIM, in tensor memory).  V is the N operand with N
//                 contiguous, exactly as it lies in the cache; nothing is transposed.
//   4 softmax     thread r owns row r: reads S from tensor memory, keeps the running maximum and
//   warps         sum in float32, writes P as bfloat16 into shared memory in the swizzled layout
//                 the tensor core reads, and rescales O in tensor memory when the maximum of some
//                 row of its warp grew by more than 2^8 (the result does not depend on when).
//
// S of tile j+1 is computed while the softmax of tile j runs; O += P V of tile j runs while the
// maximum of tile j+1 is searched.  Every wait is bounded (about two seconds, then an error bit).
//
// Formula: zeeshan8281/cloud-inference-from-scratch src/cloud_engine/kernel.py:324-405 (one
// program per query token and head on CUDA cores there).
#include "blackwell.cuh"
#include "common.cuh"

#include <cfloat>

#ifndef HEAD_DIM
#define HEAD_DIM 128
#endif

CIE_DEFINE_LAST_ERROR()

namespace cie {

using namespace bw;
using bf16 = __nv_bfloat16;
constexpr int D = HEAD_DIM;
static_assert(D == 64 || D == 128, "this kernel is built for head sizes 64 and 128");

constexpr int BM = 128;                 // query rows per CTA (tensor-memory lanes)
constexpr int BN = 128;                 // keys per tile
constexpr int HALVES = D / 64;          // 64-column sub-tiles of a row of Q, K or V
constexpr int SUB_BYTES = 128 * 128;    // one sub-tile: 128 rows of 128 bytes
constexpr int TILE_BYTES = HALVES * SUB_BYTES;
constexpr int P_BYTES = 2 * SUB_BYTES;  // 128 rows x 128 keys
constexpr int STAGES = 2;
constexpr int SMEM_BYTES = TILE_BYTES * (1 + 2 * STAGES) + P_BYTES + 1024;
constexpr int THREADS = 192;            // 4 softmax warps, 1 TMA warp, 1 MMA warp
constexpr int TMEM_COLS = 512;          // S0 | S1 | O
constexpr uint32_t COL_S = 0, COL_O = 2 * BN;
constexpr float kGrow = 8.f;            // rescale when a maximum moved by more than this (log2 units)

struct Args {
  const bf16* q;
  int q_stride;
  bf16* out;
  int out_stride;
  const int* table;        // [requests][table_width]
  int table_width;
  int num_pages;
  int kv_heads;
  int page_size;
  const int* tile_request;
  const int* tile_q0;
  int num_tiles;
  const int* context_lens;
  const int* query_lens;
  const int* query_start;
  int group, hpt, tpt, head_chunks;
  float scale_log2;
  int* err;
};

__global__ void __launch_bounds__(THREADS, 1) prefill_tc_kernel(const __grid_constant__ CUtensorMap k_map,
                                                                 const __grid_constant__ CUtensorMap v_map,
                                                                 const Args a) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  unsigned char* q_s = smem;
  unsigned char* k_s = q_s + TILE_BYTES;             // [STAGES][TILE_BYTES]
  unsigned char* v_s = k_s + STAGES * TILE_BYTES;    // [STAGES][TILE_BYTES]
  unsigned char* p_s = v_s + STAGES * TILE_BYTES;
  __shared__ __align__(8) uint64_t kv_full[STAGES], kv_empty[STAGES], s_full[2], p_full, pv_done;
  __shared__ uint32_t tmem_slot;

  pdl_wait();
  pdl_trigger();
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int tile = blockIdx.x;   // the list puts the tiles with the most keys first
  const int kvh = blockIdx.y / a.head_chunks, h0 = (blockIdx.y % a.head_chunks) * a.hpt;
  const int request = a.tile_request[tile], q0 = a.tile_q0[tile];
  const int context = a.context_lens[request], q_len = a.query_lens[request];
  const int first_token = a.query_start[request] + q0;
  const int ntok = min(a.tpt, q_len - q0);
  const int* table_row = a.table + (size_t)request * a.table_width;
  const int pos_lo = context + q0;
  const int valid_hi = context + q0 + ntok;          // keys [0, valid_hi) are visible to some row
  const int tiles = (valid_hi + BN - 1) / BN;

  if (tid == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(&kv_full[s], 1); mbar_init(&kv_empty[s], 1); }
    mbar_init(&s_full[0], 1); mbar_init(&s_full[1], 1);
    mbar_init(&p_full, 128);
    mbar_init(&pv_done, 1);
    mbar_init_fence();
  }
  if (warp == 5) tmem_alloc<TMEM_COLS>(&tmem_slot);

  // ---- Q tile, swizzled by hand: row r is token r / hpt, head h0 + r % hpt of the group.
  // Value stages start as zeros: rows that no copy fills must not hold NaN or Inf bits.
  for (int idx = tid; idx < BM * (D / 8); idx += THREADS) {
    const int r = idx / (D / 8), c = idx % (D / 8);
    const int tok = r / a.hpt, hh = h0 + r % a.hpt;
    uint4 value = make_uint4(0u, 0u, 0u, 0u);
    if (tok < ntok && hh < a.group)
      value = *reinterpret_cast<const uint4*>(a.q + (size_t)(first_token + tok) * a.q_stride +
                                              (size_t)(kvh * a.group + hh) * D + c * 8);
    *reinterpret_cast<uint4*>(q_s + (c >> 3) * SUB_BYTES + r * 128 + (((c & 7) ^ (r & 7)) << 4)) = value;
  }
  for (int idx = tid; idx < STAGES * TILE_BYTES / 16; idx += THREADS)
    reinterpret_cast<uint4*>(v_s)[idx] = make_uint4(0u, 0u, 0u, 0u);
  fence_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_slot;

  if (warp == 4) {
    // ---- TMA producer: lane b fetches the b-th block of 16 keys of a tile
    for (int j = 0; j < tiles; ++j) {
      const int s = j % STAGES;
      if (j >= STAGES && !mbar_wait(&kv_empty[s], ((j / STAGES) - 1) & 1, a.err)) break;
      const int k0 = j * BN;
      const int blocks = min(BN / 16, (valid_hi - k0 + 15) / 16);
      if (lane == 0) mbar_expect_tx(&kv_full[s], (uint32_t)blocks * 2u * 16u * D * 2u);
      __syncwarp();
      if (lane < blocks) {
        const int key = k0 + lane * 16;
        const int index = key / a.page_size;
        int page = index < a.table_width ? table_row[index] : -1;
        if (page < 0 || page >= a.num_pages) {
          atomicOr(a.err, kErrBadPage);
          page = 0;                     // the copy must still happen: the barrier counts its bytes
        }
        const int row = (page * a.kv_heads + kvh) * a.page_size + key % a.page_size;
#pragma unroll
        for (int h = 0; h < HALVES; ++h) {
          tma_load_2d(k_s + s * TILE_BYTES + h * SUB_BYTES + lane * 2048, &k_map, &kv_full[s], h * 64, row);
          tma_load_2d(v_s + s * TILE_BYTES + h * SUB_BYTES + lane * 2048, &v_map, &kv_full[s], h * 64, row);
        }
      }
      __syncwarp();
    }
  } else if (warp == 5) {
    if (lane == 0) {
      // ---- MMA issuer
      constexpr uint32_t idesc_qk = idesc_bf16(BM, BN);
      constexpr uint32_t idesc_pv = idesc_bf16(BM, D, true);
      const uint32_t q_addr = smem_u32(q_s), p_addr = smem_u32(p_s);
      auto issue_qk = [&](int j) -> bool {
        const int s = j % STAGES;
        if (!mbar_wait(&kv_full[s], (j / STAGES) & 1, a.err)) return false;
        tc_fence_after();
        const uint32_t k_addr = smem_u32(k_s + s * TILE_BYTES);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t off = (kk >> 2) * SUB_BYTES + (kk & 3) * 32;
          umma_bf16(tmem + COL_S + (j & 1) * BN, smem_desc_sw128(q_addr + off), smem_desc_sw128(k_addr + off),
                    idesc_qk, kk > 0 ? 1u : 0u);
        }
        tc_commit(&s_full[j & 1]);
        return true;
      };
      bool alive = issue_qk(0);
      for (int j = 0; j < tiles && alive; ++j) {
        if (j + 1 < tiles) alive = issue_qk(j + 1);
        if (!alive || !mbar_wait(&p_full, j & 1, a.err)) { alive = false; break; }
        tc_fence_after();
        const uint32_t v_addr = smem_u32(v_s + (j % STAGES) * TILE_BYTES);
#pragma unroll
        for (int kk = 0; kk < BN / 16; ++kk) {
          // P: 16 keys further inside the swizzled row; V: 16 key rows further down
          const uint64_t p_desc = smem_desc_sw128(p_addr + (kk >> 2) * SUB_BYTES + (kk & 3) * 32);
          const uint64_t v_desc = smem_desc_sw128(v_addr + kk * 2048, SUB_BYTES);
          umma_bf16(tmem + COL_O, p_desc, v_desc, idesc_pv, (j > 0 || kk > 0) ? 1u : 0u);
        }
        tc_commit(&kv_empty[j % STAGES]);
        tc_commit(&pv_done);
      }
    }
    __syncwarp();
  } else {
    // ---- softmax: thread r owns row r = tensor-memory lane r
    const int r = tid;
    const int tok = r / a.hpt, hh = h0 + r % a.hpt;
    const bool row_used = tok < ntok && hh < a.group;
    const int pos = row_used ? context + q0 + tok : -1;
    const uint32_t lane_base = (uint32_t)(warp * 32) << 16;
    float m_used = -INFINITY, l = 0.f;
    bool alive = true;
    for (int j = 0; j < tiles && alive; ++j) {
      if (!mbar_wait(&s_full[j & 1], (j >> 1) & 1, a.err)) { alive = false; break; }
      tc_fence_after();
      const int k0 = j * BN;
      const int rel = pos - k0;                       // columns 0..rel of this tile are visible
      const bool masked = k0 + BN - 1 > pos_lo;       // the same for the whole CTA
      const uint32_t s_addr = tmem + lane_base + COL_S + (j & 1) * BN;
      float mx = -INFINITY;
#pragma unroll
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t raw[32];
        tmem_ld32(s_addr + c * 32, raw);
        tc_wait_ld();
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const float s = __uint_as_float(raw[i]);
          mx = fmaxf(mx, (masked && c * 32 + i > rel) ? -INFINITY : s);
        }
      }
      mx *= a.scale_log2;
      const bool grow = mx > m_used + kGrow;          // false while the row has seen no key
      if (j > 0 && !mbar_wait(&pv_done, (j - 1) & 1, a.err)) { alive = false; break; }
      if (__any_sync(0xffffffffu, grow)) {
        float alpha = 1.f;
        if (grow) {
          alpha = exp2f(m_used - mx);                 // 0 at the row's first keys
          m_used = mx;
          l *= alpha;
        }
        if (j > 0) {
          tc_fence_after();
#pragma unroll
          for (int c = 0; c < D / 32; ++c) {
            uint32_t raw[32];
            tmem_ld32(tmem + lane_base + COL_O + c * 32, raw);
            tc_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; ++i) raw[i] = __float_as_uint(__uint_as_float(raw[i]) * alpha);
            tmem_st32(tmem + lane_base + COL_O + c * 32, raw);
          }
          tc_wait_st();
        }
      }
      const float m_eff = m_used == -INFINITY ? 0.f : m_used;
#pragma unroll
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t raw[32];
        tmem_ld32(s_addr + c * 32, raw);
        tc_wait_ld();
        uint32_t packed[16];
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          float p0 = exp2f(fmaf(__uint_as_float(raw[i]), a.scale_log2, -m_eff));
          float p1 = exp2f(fmaf(__uint_as_float(raw[i + 1]), a.scale_log2, -m_eff));
          if (masked) {
            if (c * 32 + i > rel) p0 = 0.f;
            if (c * 32 + i + 1 > rel) p1 = 0.f;
          }
          l += p0 + p1;
          __nv_bfloat162 pair = __floats2bfloat162_rn(p0, p1);
          packed[i >> 1] = *reinterpret_cast<uint32_t*>(&pair);
        }
        // columns 32c .. 32c+31 are the 16-byte pieces 4c .. 4c+3 of the row
#pragma unroll
        for (int piece = 0; piece < 4; ++piece) {
          const int chunk = c * 4 + piece;
          *reinterpret_cast<uint4*>(p_s + (chunk >> 3) * SUB_BYTES + r * 128 + (((chunk & 7) ^ (r & 7)) << 4)) =
              make_uint4(packed[piece * 4], packed[piece * 4 + 1], packed[piece * 4 + 2], packed[piece * 4 + 3]);
        }
      }
      fence_async_smem();
      tc_fence_before();
      mbar_arrive(&p_full);
    }
    // ---- write out
    if (alive && tiles > 0 && mbar_wait(&pv_done, (tiles - 1) & 1, a.err)) {
      tc_fence_after();
      const float inv = l > 0.f ? 1.f / l : 0.f;
      bf16* dst = a.out + (size_t)(first_token + tok) * a.out_stride + (size_t)(kvh * a.group + hh) * D;
#pragma unroll
      for (int c = 0; c < D / 32; ++c) {
        uint32_t raw[32];
        tmem_ld32(tmem + lane_base + COL_O + c * 32, raw);
        tc_wait_ld();
        if (row_used) {
#pragma unroll
          for (int piece = 0; piece < 4; ++piece) {
            uint32_t packed[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              __nv_bfloat162 pair = __floats2bfloat162_rn(__uint_as_float(raw[piece * 8 + 2 * i]) * inv,
                                                          __uint_as_float(raw[piece * 8 + 2 * i + 1]) * inv);
              packed[i] = *reinterpret_cast<uint32_t*>(&pair);
            }
            *reinterpret_cast<uint4*>(dst + c * 32 + piece * 8) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 5) tmem_free<TMEM_COLS>(tmem);
}

}  // namespace cie

using namespace cie;

extern "C" int cie_attention_prefill_tc_head_dim() { return D; }

// Same arguments as the mma.sync prefill kernel's entry point, without a window: the caller keeps
// windowed layers, other head sizes and pages that are no multiple of 16 tokens on that kernel.
extern "C" int cie_attention_prefill_tc(const void* q, int q_stride, void* out, int out_stride,
                                        const void* k_pool, const void* v_pool, const int* table,
                                        int table_width, int num_pages, const int* tile_request,
                                        const int* tile_q0, int num_tiles, const int* context_lens,
                                        const int* query_lens, const int* query_start, int q_heads,
                                        int kv_heads, int page_size, int hpt, float scale, int* err,
                                        void* stream) {
  if (num_tiles <= 0) return 0;
  if (kv_heads < 1 || q_heads % kv_heads) CIE_FAIL("attention_prefill_tc: %d query heads over %d kv heads", q_heads, kv_heads);
  const int group = q_heads / kv_heads;
  if (hpt < 1 || hpt > BM || hpt > group) CIE_FAIL("attention_prefill_tc: %d heads per tile with a group of %d", hpt, group);
  if (page_size < 16 || page_size % 16) CIE_FAIL("attention_prefill_tc: pages of %d tokens (a multiple of 16 is needed)", page_size);
  if (q_stride % 8 || out_stride % 8) CIE_FAIL("attention_prefill_tc: row strides must keep 16-byte alignment");
  if ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(k_pool) |
       reinterpret_cast<uintptr_t>(v_pool)) & 15)
    CIE_FAIL("attention_prefill_tc: buffers must be 16-byte aligned");
  Args a;
  a.q = (const bf16*)q; a.q_stride = q_stride; a.out = (bf16*)out; a.out_stride = out_stride;
  a.table = table; a.table_width = table_width; a.num_pages = num_pages; a.kv_heads = kv_heads; a.page_size = page_size;
  a.tile_request = tile_request; a.tile_q0 = tile_q0; a.num_tiles = num_tiles; a.context_lens = context_lens;
  a.query_lens = query_lens; a.query_start = query_start;
  a.group = group; a.hpt = hpt; a.tpt = BM / hpt; a.head_chunks = (group + hpt - 1) / hpt;
  a.scale_log2 = scale * 1.4426950408889634f; a.err = err;
  CUtensorMap k_map, v_map;
  const long long rows = (long long)num_pages * kv_heads * page_size;
  // the pools as matrices [pages * kv_heads * page_size, D], read in boxes of 16 rows
  if (!tensor_map_bf16(k_pool, rows, D, 16, &k_map) || !tensor_map_bf16(v_pool, rows, D, 16, &v_map))
    CIE_FAIL("attention_prefill_tc: cuTensorMapEncodeTiled failed");
  static bool configured = false;
  if (!configured) {
    cudaError_t status = cudaFuncSetAttribute(prefill_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    if (status != cudaSuccess) CIE_FAIL("attention_prefill_tc: shared memory %d: %s", SMEM_BYTES, cudaGetErrorString(status));
    configured = true;
  }
  dim3 grid(num_tiles, kv_heads * a.head_chunks);
  CIE_LAUNCH("attention_prefill_tc", prefill_tc_kernel, grid, dim3(THREADS), (size_t)SMEM_BYTES, (cudaStream_t)stream, k_map, v_map, a);
  return 0;
}
