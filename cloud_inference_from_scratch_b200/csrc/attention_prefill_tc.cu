// Ragged causal attention of prompt portions over the paged cache on the 5th-generation tensor
// cores (tcgen05), bfloat16, head size 64 or 128 (-DHEAD_DIM), pages of a multiple of 16 tokens.
//
// One CTA takes 128 query rows of ONE request and ONE kv head; a row is a (token, query head of the
// group) pair, so the heads of a group share every key and value.  Keys go by in tiles of 128:
//
//   TMA warps     key/value pages -> shared memory: one copy per tile where the tile's pages follow
//                 each other in the pool (a 5-dimensional box over consecutive pages of one kv
//                 head), else one copy per 16 keys (a 4-dimensional box
//                 that leaves every 8 keys as two swizzled 8 x 64 pieces side by side: few, large
//                 copies, because the TMA unit's rate of copies bounds this kernel); two stages of keys and two of values, each with its own mbarriers, so
//                 the keys of tile j+2 are on their way while the values of tile j are still in use.
//   MMA threads   one issues S = Q K^T (128 x 128, float32, in tensor memory, double buffered),
//                 another O += P V (128 x HEAD_DIM, in tensor memory).  V is the N operand with N
//                 contiguous, exactly as it lies in the cache; nothing is transposed.
//   4 softmax     thread r owns row r: reads S from tensor memory, keeps the running maximum and
//   warps         sum in float32, writes P as bfloat16 into shared memory (two buffers) in the
//                 swizzled layout the tensor core reads, and rescales O in tensor memory when the
//                 maximum of some row of its warp grew by more than 2^8 (the result does not
//                 depend on when).
//
// A launch with few query tiles (a prompt portion over a long context) may cut the keys of a query
// tile into ranges, one CTA each (grid.z): such a CTA leaves its unnormalised output, maximum and
// sum in global memory, and whichever CTA of the tile draws the last ticket adds the shares up.
// Nobody waits for anybody.
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
#ifndef TC_BN
#define TC_BN 128
#endif
#ifndef TC_STAGES
#define TC_STAGES 2
#endif
constexpr int BN = TC_BN;               // keys per tile: 64 or 128
static_assert(BN == 64 || BN == 128, "key tiles of 64 or 128");
constexpr int HALVES = D / 64;          // 64-column sub-tiles of a row of Q, K or V
constexpr int SUB_BYTES = 128 * 128;    // a sub-tile of Q or P: 128 rows of 128 bytes (64 columns)
constexpr int Q_BYTES = HALVES * SUB_BYTES;
constexpr int GROUP_BYTES = HALVES * 1024;          // 8 keys of K or V: 8 x 64 left columns, then the right ones
constexpr int BLOCK_BYTES = 2 * GROUP_BYTES;        // 16 keys: what one TMA copy brings
constexpr int TILE_BYTES = (BN / 16) * BLOCK_BYTES; // one stage of keys (or of values)
constexpr int P_BYTES = (BN / 64) * SUB_BYTES;      // 128 rows x BN keys
constexpr int STAGES = TC_STAGES;
constexpr int SMEM_BYTES = Q_BYTES + TILE_BYTES * 2 * STAGES + 2 * P_BYTES + 1024;   // P is double buffered
static_assert(SMEM_BYTES <= 227 * 1024, "shared memory");
#ifndef TC_KEY_PRODUCERS
#define TC_KEY_PRODUCERS 1
#endif
#ifndef TC_VALUE_PRODUCERS
#define TC_VALUE_PRODUCERS 1
#endif
// TMA warps per ring: the copies of a tile are issued by several threads at once (one warp issuing
// all of them was measured slower).  No more than 8 warps in all: the softmax threads keep a row
// of S in registers and need the 255 a thread of a 256-thread CTA may have.
constexpr int KEY_PRODUCERS = TC_KEY_PRODUCERS, VALUE_PRODUCERS = TC_VALUE_PRODUCERS;
constexpr int MMA_WARP = 4;            // issues S = Q K^T (and owns the tensor-memory allocation)
constexpr int PV_WARP = 5 + KEY_PRODUCERS + VALUE_PRODUCERS;   // issues O += P V
constexpr int THREADS = (PV_WARP + 1) * 32;   // 4 softmax warps, two MMA warps, the TMA warps
static_assert(THREADS <= 256, "at most 8 warps");
constexpr int TMEM_COLS = 512;          // S0 | S1 | O
constexpr uint32_t COL_S = 0, COL_O = 2 * BN;
constexpr int TABLE_SLOTS = 256;       // block-table entries kept in shared memory (more are read from global memory)
constexpr float kGrow = 8.f;            // rescale when a maximum moved by more than this (log2 units)

// 2^x by the special-function unit alone (results below 2^-126 become 0; -inf gives 0).
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

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
  // one copy per tile when the pages of a tile follow each other in the pool (0: never):
  int run_pages;           // pages a tile spans (1 if a page holds several tiles)
  // key ranges: up to `splits` CTAs (grid.z) share the keys of a query tile, each with at least
  // `min_tiles` key tiles; shares: [query tile][kv head, head chunk][split][D + 2][128] float32;
  // tickets: one int per (query tile, kv head, head chunk), zero between launches
  int splits, min_tiles;
  float* shares;
  int* tickets;
};
constexpr int SHARE_FLOATS = (D + 2) * BM;
constexpr int MAX_RANGES = 4;          // most key ranges of a query tile (the CTA that adds them up holds 32 columns of each)

__global__ void __launch_bounds__(THREADS, 1) prefill_tc_kernel(const __grid_constant__ CUtensorMap k_map,
                                                                 const __grid_constant__ CUtensorMap v_map,
                                                                 const __grid_constant__ CUtensorMap k_run_map,
                                                                 const __grid_constant__ CUtensorMap v_run_map,
                                                                 const Args a) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  unsigned char* q_s = smem;
  unsigned char* k_s = q_s + Q_BYTES;                // [STAGES][TILE_BYTES]
  unsigned char* v_s = k_s + STAGES * TILE_BYTES;    // [STAGES][TILE_BYTES]
  unsigned char* p_s = v_s + STAGES * TILE_BYTES;
  __shared__ __align__(8) uint64_t k_full[STAGES], k_empty[STAGES], v_full[STAGES], v_empty[STAGES], s_full[2], s_free[2], p_full, pv_done[2];
  __shared__ uint32_t tmem_slot;
  __shared__ int pages_s[TABLE_SLOTS];   // the block-table entries this CTA's keys need
  __shared__ int last_s;                 // key ranges: did this CTA draw the tile's last ticket?

  // Before `griddepcontrol.wait`: only what the kernel before this one does not write.  Lengths and
  // block tables come with the step's metadata, and keys and values below a request's context
  // were written by earlier steps (the kernel before writes this step's tokens only).
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
  const int all_tiles = (valid_hi + BN - 1) / BN;
  // how many of the launched key ranges this query tile uses (the launch is sized for the longest
  // context the tables hold); the CTAs of the others leave before they set anything up
  // (adding shares up costs about as much as walking six key tiles: not below three ranges' worth of keys)
  const int used = a.splits > 1 && all_tiles >= 3 * a.min_tiles ? min(a.splits, all_tiles / a.min_tiles) : 1;
  const int split = blockIdx.z;
  if (split >= used) return;
  const int tile_begin = split * (all_tiles / used) + min(split, all_tiles % used);
  const int tiles = all_tiles / used + (split < all_tiles % used ? 1 : 0);
  // CTAs that share keys walk them from different starting tiles (the running-maximum softmax does
  // not care about the order), so that they do not all ask L2 for the same lines at the same time
  const int first_tile = tiles > 0 ? (int)((blockIdx.x * 5u + blockIdx.y * 3u) % (unsigned)tiles) : 0;
  auto tile_of = [&](int j) { const int t = j + first_tile; return tile_begin + (t >= tiles ? t - tiles : t); };

  if (tid == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&k_full[s], 1); mbar_init(&k_empty[s], 1);
      mbar_init(&v_full[s], 1); mbar_init(&v_empty[s], 1);
    }
    mbar_init(&s_full[0], 1); mbar_init(&s_full[1], 1);
    mbar_init(&s_free[0], 128); mbar_init(&s_free[1], 128);
    mbar_init(&p_full, 128);
    mbar_init(&pv_done[0], 1); mbar_init(&pv_done[1], 1);
    mbar_init_fence();
  }
  // Value stages start as zeros: rows that no copy fills must not hold NaN or Inf bits.
  for (int idx = tid; idx < STAGES * TILE_BYTES / 16; idx += THREADS)
    reinterpret_cast<uint4*>(v_s)[idx] = make_uint4(0u, 0u, 0u, 0u);
  {
    const int needed = min((valid_hi + a.page_size - 1) / a.page_size, min(a.table_width, TABLE_SLOTS));
    for (int idx = tid; idx < needed; idx += THREADS) pages_s[idx] = table_row[idx];
  }
  fence_async_smem();
  __syncthreads();
  uint32_t tmem = 0;
  const bool producer = warp > MMA_WARP && warp < PV_WARP;
  if (!producer) {
  // ---- everybody but the TMA warps (which go ahead with the keys and values of earlier steps):
  // the Q tile, swizzled by hand: row r is token r / hpt, head h0 + r % hpt of the group.
  // Tensor memory is asked for after the wait only: a CTA of an earlier kernel that is still to
  // allocate its own on this SM must never find it taken by a CTA that waits for that kernel.
  pdl_wait();
  pdl_trigger();
  if (warp == MMA_WARP) tmem_alloc<TMEM_COLS>(&tmem_slot);
  constexpr int STAGERS = THREADS - (PV_WARP - MMA_WARP - 1) * 32;
  const int stager = warp <= MMA_WARP ? tid : tid - (PV_WARP - MMA_WARP - 1) * 32;
  for (int idx = stager; idx < BM * (D / 8); idx += STAGERS) {
    const int r = idx / (D / 8), c = idx % (D / 8);
    const int tok = r / a.hpt, hh = h0 + r % a.hpt;
    uint4 value = make_uint4(0u, 0u, 0u, 0u);
    if (tok < ntok && hh < a.group)
      value = *reinterpret_cast<const uint4*>(a.q + (size_t)(first_token + tok) * a.q_stride +
                                              (size_t)(kvh * a.group + hh) * D + c * 8);
    *reinterpret_cast<uint4*>(q_s + (c >> 3) * SUB_BYTES + r * 128 + (((c & 7) ^ (r & 7)) << 4)) = value;
  }
  fence_async_smem();
  tc_fence_before();
  asm volatile("bar.sync 2, %0;" ::"n"(STAGERS) : "memory");   // the Q tile is whole before a product reads it
  tc_fence_after();
  tmem = tmem_slot;
  }

  if (producer) {
    // ---- TMA producers: some warps for the keys, some for the values; a lane fetches one
    // block of 16 keys of a tile.  Keys and values have rings of their own: a key stage is free again
    // as soon as S of its tile is computed, long before the values of that tile have been used.
    const bool for_keys = warp - MMA_WARP - 1 < KEY_PRODUCERS;
    const int sharers = for_keys ? KEY_PRODUCERS : VALUE_PRODUCERS;
    const int part = for_keys ? warp - MMA_WARP - 1 : warp - MMA_WARP - 1 - KEY_PRODUCERS;   // which share of a tile's blocks
    const int per_warp = (BN / 16 + sharers - 1) / sharers;
    const int block = part * per_warp + lane;                    // this lane's block, if lane < per_warp
    auto block_row = [&](int j) -> int {
      const int key = tile_of(j) * BN + block * 16;
      const int index = key / a.page_size;
      int page = index >= a.table_width ? -1 : index < TABLE_SLOTS ? pages_s[index] : table_row[index];
      if (page < 0 || page >= a.num_pages) {
        atomicOr(a.err, kErrBadPage);
        page = 0;                     // the copy must still happen: the barrier counts its bytes
      }
      return (page * a.kv_heads + kvh) * a.page_size + key % a.page_size;
    };
    auto blocks_of = [&](int j) { return min(BN / 16, (valid_hi - tile_of(j) * BN + 15) / 16); };
    auto page_at = [&](int key) -> int {
      const int index = key / a.page_size;
      return index >= a.table_width ? -1 : index < TABLE_SLOTS ? pages_s[index] : table_row[index];
    };
    auto load = [&](int j, unsigned char* ring, const CUtensorMap* map, const CUtensorMap* run_map, uint64_t* full,
                    uint64_t* empty) -> bool {
      const int s = j % STAGES;
      const int blocks = blocks_of(j);
      const int k0 = tile_of(j) * BN;
      // Do the pages of this tile follow each other in the pool?  Then one copy brings the tile.
      bool run = a.run_pages > 0;
      int first_page = 0;
      if (run) {
        const int page = lane < blocks ? page_at(k0 + lane * 16) : 0;
        first_page = __shfl_sync(0xffffffffu, page, 0);
        const bool follows = lane >= blocks || page == first_page + (lane * 16) / a.page_size;
        run = __all_sync(0xffffffffu, follows) && first_page >= 0 && first_page < a.num_pages;
      }
      const bool mine = !run && lane < per_warp && block < blocks;
      const int row = mine ? block_row(j) : 0;
      if (j >= STAGES && !mbar_wait(&empty[s], ((j / STAGES) - 1) & 1, a.err)) return false;
      if (run) {
        if (part == 0 && lane == 0) {
          // the whole box counts, also where it reaches past the keys in use or past the pool's end
          mbar_expect_tx(&full[s], TILE_BYTES);
          const int group = kvh * (a.page_size / 8) + (k0 % a.page_size) / 8;
          if constexpr (HALVES == 2) tma_load_5d(ring + s * TILE_BYTES, run_map, &full[s], 0, 0, 0, group, first_page);
          else tma_load_4d(ring + s * TILE_BYTES, run_map, &full[s], 0, 0, group, first_page);
        }
        __syncwarp();
        return true;
      }
      // the first warp of the ring announces the bytes of the whole tile (a copy of another warp
      // may complete before that: the phase still waits for this arrival)
      if (part == 0 && lane == 0) mbar_expect_tx(&full[s], (uint32_t)blocks * 16u * D * 2u);
      __syncwarp();
      if (mine) {   // one copy per block of 16 keys (they lie in one page)
        if constexpr (HALVES == 2) tma_load_4d(ring + s * TILE_BYTES + block * BLOCK_BYTES, map, &full[s], 0, 0, 0, row / 8);
        else tma_load_3d(ring + s * TILE_BYTES + block * BLOCK_BYTES, map, &full[s], 0, 0, row / 8);
      }
      __syncwarp();
      return true;
    };
    bool alive = true, waited = false;
    for (int j = 0; j < tiles && alive; ++j) {
      if (!waited && tile_of(j) * BN + BN > context) {   // a tile with keys of this step: the kernel before writes them
        pdl_wait();
        waited = true;
      }
      alive = for_keys ? load(j, k_s, &k_map, &k_run_map, k_full, k_empty) : load(j, v_s, &v_map, &v_run_map, v_full, v_empty);
    }
    if (!waited) pdl_wait();
  } else if (warp == MMA_WARP) {
    if (lane == 0) {
      // ---- S = Q K^T, issued as far ahead as the two S buffers allow; the other products are
      // issued by a thread of their own, so that neither waits behind the other's operands
      constexpr uint32_t idesc_qk = idesc_bf16(BM, BN);
      // descriptors differ only in their address field (bits 0..13, in units of 16 bytes): one is
      // built per operand and the others follow by adding to it
      const uint64_t q_desc = smem_desc_sw128(smem_u32(q_s));
      // keys: rows are keys, groups of 8 keys GROUP_BYTES apart, the right 64 columns 1 KB further
      const uint64_t k_desc0 = smem_desc_sw128(smem_u32(k_s), 16, GROUP_BYTES);
      for (int j = 0; j < tiles; ++j) {
        const int s = j % STAGES;
        // the softmax threads have taken S of tile j-2 out of this buffer
        if (j > 1 && !mbar_wait(&s_free[j & 1], ((j >> 1) - 1) & 1, a.err)) break;
        if (!mbar_wait(&k_full[s], (j / STAGES) & 1, a.err)) break;
        tc_fence_after();
        const uint64_t k_desc = k_desc0 + (uint64_t)((s * TILE_BYTES) >> 4);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          constexpr int unit = 16;
          const uint32_t q_off = ((kk >> 2) * SUB_BYTES + (kk & 3) * 32) / unit, k_off = ((kk >> 2) * 1024 + (kk & 3) * 32) / unit;
          umma_bf16(tmem + COL_S + (j & 1) * BN, q_desc + q_off, k_desc + k_off, idesc_qk, kk > 0 ? 1u : 0u);
        }
        tc_commit(&s_full[j & 1]);
        tc_commit(&k_empty[s]);
      }
    }
    __syncwarp();
  } else if (warp == PV_WARP) {
    if (lane == 0) {
      // ---- O += P V
      constexpr uint32_t idesc_pv = idesc_bf16(BM, D, true);
      const uint64_t p_desc0 = smem_desc_sw128(smem_u32(p_s));
      // values: the N-contiguous operand, 64-column blocks 1 KB apart, groups of 8 keys GROUP_BYTES apart
      const uint64_t v_desc0 = smem_desc_sw128(smem_u32(v_s), 1024, GROUP_BYTES);
      for (int j = 0; j < tiles; ++j) {
        if (!mbar_wait(&p_full, j & 1, a.err)) break;
        if (!mbar_wait(&v_full[j % STAGES], (j / STAGES) & 1, a.err)) break;
        tc_fence_after();
        const uint64_t p_desc = p_desc0 + (uint64_t)(((j & 1) * P_BYTES) >> 4);
        const uint64_t v_desc = v_desc0 + (uint64_t)(((j % STAGES) * TILE_BYTES) >> 4);
#pragma unroll
        for (int kk = 0; kk < BN / 16; ++kk) {
          // P: 16 keys further inside the swizzled row; V: 16 key rows further down
          umma_bf16(tmem + COL_O, p_desc + (uint32_t)(((kk >> 2) * SUB_BYTES + (kk & 3) * 32) >> 4),
                    v_desc + (uint32_t)((kk * BLOCK_BYTES) >> 4), idesc_pv, (j > 0 || kk > 0) ? 1u : 0u);
        }
        tc_commit(&v_empty[j % STAGES]);
        tc_commit(&pv_done[j & 1]);
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
      const int k0 = tile_of(j) * BN;
      const int rel = pos - k0;                       // columns 0..rel of this tile are visible
      const bool masked = k0 + BN - 1 > pos_lo;       // the same for the whole CTA
      const uint32_t s_addr = tmem + lane_base + COL_S + (j & 1) * BN;
      // the whole row of S comes into registers once; maxima and sums run as four independent
      // chains (a thread has no other warp on its scheduler to hide a dependent chain behind)
      uint32_t sraw[BN / 32][32];
#pragma unroll
      for (int c = 0; c < BN / 32; ++c) tmem_ld32(s_addr + c * 32, sraw[c]);
      tc_wait_ld();
      tc_fence_before();
      mbar_arrive(&s_free[j & 1]);   // the buffer may take S of tile j+2
      float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
      if (masked) {   // a tile on the diagonal: compare every column with the row's position
#pragma unroll
        for (int c = 0; c < BN / 32; ++c) {
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            if (c * 32 + i > rel) sraw[c][i] = 0xff800000u;   // -inf: stays out of maximum and sum
            mx4[i & 3] = fmaxf(mx4[i & 3], __uint_as_float(sraw[c][i]));
          }
        }
      } else {
#pragma unroll
        for (int c = 0; c < BN / 32; ++c) {
#pragma unroll
          for (int i = 0; i < 32; ++i) mx4[i & 3] = fmaxf(mx4[i & 3], __uint_as_float(sraw[c][i]));
        }
      }
      float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
      mx *= a.scale_log2;
      const bool grow = mx > m_used + kGrow;          // false while the row has seen no key
      // this tile's P buffer was last read by O += P V of tile j-2
      if (j > 1 && !mbar_wait(&pv_done[j & 1], ((j >> 1) - 1) & 1, a.err)) { alive = false; break; }
      if (__any_sync(0xffffffffu, grow)) {
        float alpha = 1.f;
        if (grow) {
          alpha = exp2f(m_used - mx);                 // 0 at the row's first keys
          m_used = mx;
          l *= alpha;
        }
        if (j > 0) {
          // O must be complete up to tile j-1 before it is rescaled
          if (!mbar_wait(&pv_done[(j - 1) & 1], ((j - 1) >> 1) & 1, a.err)) { alive = false; break; }
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
      float l4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t packed[16];
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          // masked columns hold -inf since the first pass: 2^(-inf) is 0
          const float p0 = fast_exp2(fmaf(__uint_as_float(sraw[c][i]), a.scale_log2, -m_eff));
          const float p1 = fast_exp2(fmaf(__uint_as_float(sraw[c][i + 1]), a.scale_log2, -m_eff));
          l4[(i >> 1) & 3] += p0 + p1;
          __nv_bfloat162 pair = __floats2bfloat162_rn(p0, p1);
          packed[i >> 1] = *reinterpret_cast<uint32_t*>(&pair);
        }
        // columns 32c .. 32c+31 are the 16-byte pieces 4c .. 4c+3 of the row
#pragma unroll
        for (int piece = 0; piece < 4; ++piece) {
          const int chunk = c * 4 + piece;
          *reinterpret_cast<uint4*>(p_s + (j & 1) * P_BYTES + (chunk >> 3) * SUB_BYTES + r * 128 + (((chunk & 7) ^ (r & 7)) << 4)) =
              make_uint4(packed[piece * 4], packed[piece * 4 + 1], packed[piece * 4 + 2], packed[piece * 4 + 3]);
        }
      }
      l += (l4[0] + l4[1]) + (l4[2] + l4[3]);
      fence_async_smem();
      tc_fence_before();
      mbar_arrive(&p_full);
    }
    bf16* dst = a.out + (size_t)(first_token + tok) * a.out_stride + (size_t)(kvh * a.group + hh) * D;
    if (used > 1) {
      // ---- one key range of several: leave the share, draw a ticket, and add all shares up if it
      // was the last one.  A share is stored column by column, so that the 128 threads write and
      // read neighbouring words.
      const int unit = blockIdx.x * gridDim.y + blockIdx.y;
      float* unit_shares = a.shares + (size_t)unit * a.splits * SHARE_FLOATS;
      float* share = unit_shares + (size_t)split * SHARE_FLOATS;
      const bool finished = alive && tiles > 0 && mbar_wait(&pv_done[(tiles - 1) & 1], ((tiles - 1) >> 1) & 1, a.err);
      if (finished) {
        tc_fence_after();
#pragma unroll
        for (int c = 0; c < D / 32; ++c) {
          uint32_t raw[32];
          tmem_ld32(tmem + lane_base + COL_O + c * 32, raw);
          tc_wait_ld();
#pragma unroll
          for (int i = 0; i < 32; ++i) __stcg(share + (c * 32 + i) * BM + r, __uint_as_float(raw[i]));
        }
        __stcg(share + D * BM + r, m_used);
        __stcg(share + (D + 1) * BM + r, l);
      }
      __threadfence();
      asm volatile("bar.sync 1, 128;" ::: "memory");   // the four softmax warps
      if (tid == 0) {
        const int drawn = atomicAdd(a.tickets + unit, 1);
        last_s = drawn == used - 1 ? 1 : 0;
        if (drawn == used - 1) a.tickets[unit] = 0;     // ready for the next launch
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (last_s && finished) {
        __threadfence();
        float m_all = -INFINITY;
        for (int s = 0; s < used; ++s) m_all = fmaxf(m_all, __ldcg(unit_shares + (size_t)s * SHARE_FLOATS + D * BM + r));
        float weight[MAX_RANGES];
        float sum = 0.f;
#pragma unroll
        for (int s = 0; s < MAX_RANGES; ++s) {
          weight[s] = 0.f;
          if (s < used) {
            const float m_s = __ldcg(unit_shares + (size_t)s * SHARE_FLOATS + D * BM + r);
            weight[s] = m_s == -INFINITY ? 0.f : exp2f(m_s - m_all);
            sum += weight[s] * __ldcg(unit_shares + (size_t)s * SHARE_FLOATS + (D + 1) * BM + r);
          }
        }
        const float inv = sum > 0.f ? 1.f / sum : 0.f;
        if (row_used) {
          // 32 columns at a time, every load of them asked for before the first addition
#pragma unroll 1
          for (int c0 = 0; c0 < D; c0 += 32) {
            float acc32[32];
#pragma unroll
            for (int i = 0; i < 32; ++i) acc32[i] = 0.f;
            float part[MAX_RANGES][32];
#pragma unroll
            for (int s = 0; s < MAX_RANGES; ++s) {
              if (s < used) {
#pragma unroll
                for (int i = 0; i < 32; ++i) part[s][i] = __ldcg(unit_shares + (size_t)s * SHARE_FLOATS + (c0 + i) * BM + r);
              }
            }
#pragma unroll
            for (int s = 0; s < MAX_RANGES; ++s) {
              if (s < used) {
#pragma unroll
                for (int i = 0; i < 32; ++i) acc32[i] += weight[s] * part[s][i];
              }
            }
#pragma unroll
            for (int c = c0; c < c0 + 32; c += 8) {
            const float* acc = acc32 + (c - c0);
            uint32_t packed[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              __nv_bfloat162 pair = __floats2bfloat162_rn(acc[2 * i] * inv, acc[2 * i + 1] * inv);
              packed[i] = *reinterpret_cast<uint32_t*>(&pair);
            }
            *reinterpret_cast<uint4*>(dst + c) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
            }
          }
        }
      }
    } else
    // ---- write out
    if (alive && tiles > 0 && mbar_wait(&pv_done[(tiles - 1) & 1], ((tiles - 1) >> 1) & 1, a.err)) {
      tc_fence_after();
      const float inv = l > 0.f ? 1.f / l : 0.f;
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
  if (warp == MMA_WARP) tmem_free<TMEM_COLS>(tmem);
}

}  // namespace cie

using namespace cie;

extern "C" int cie_attention_prefill_tc_head_dim() { return D; }
extern "C" int cie_attention_prefill_tc_key_tile() { return BN; }
extern "C" int cie_attention_prefill_tc_max_ranges() { return MAX_RANGES; }

// Same arguments as the mma.sync prefill kernel's entry point, without a window: the caller keeps
// windowed layers, other head sizes and pages that are no multiple of 16 tokens on that kernel.
// splits: key ranges launched per query tile (1 .. 4); a tile uses as many as leave each min_tiles
// key tiles.  shares: float32 [num_tiles * kv_heads * head chunks][splits][head size + 2][128];
// tickets: one int per (query tile, kv head, head chunk), zero before the first launch.
extern "C" int cie_attention_prefill_tc(const void* q, int q_stride, void* out, int out_stride,
                                        const void* k_pool, const void* v_pool, const int* table,
                                        int table_width, int num_pages, const int* tile_request,
                                        const int* tile_q0, int num_tiles, const int* context_lens,
                                        const int* query_lens, const int* query_start, int q_heads,
                                        int kv_heads, int page_size, int hpt, float scale, int splits,
                                        int min_tiles, float* shares, int* tickets, int* err, void* stream) {
  if (num_tiles <= 0) return 0;
  if (splits < 1 || splits > MAX_RANGES) CIE_FAIL("attention_prefill_tc: 1 to %d key ranges, got %d", MAX_RANGES, splits);
  if (splits > 1 && (min_tiles < 1 || !shares || !tickets)) CIE_FAIL("attention_prefill_tc: key ranges need scratch memory and a least number of key tiles each");
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
  a.splits = splits; a.min_tiles = min_tiles; a.shares = shares; a.tickets = tickets;
  CUtensorMap k_map, v_map;
  const long long rows = (long long)num_pages * kv_heads * page_size;
  // the pools as matrices [pages * kv_heads * page_size, D], read in blocks of 16 whole rows
  if (!tensor_map_bf16_row_blocks(k_pool, rows, D, 16, &k_map) || !tensor_map_bf16_row_blocks(v_pool, rows, D, 16, &v_map))
    CIE_FAIL("attention_prefill_tc: cuTensorMapEncodeTiled failed");
  // copies of whole tiles, for tiles whose pages follow each other in the pool
  CUtensorMap k_run = k_map, v_run = v_map;
  a.run_pages = 0;
  {
    int run_pages = 0, groups = 0;
    if (page_size <= BN && BN % page_size == 0) { run_pages = BN / page_size; groups = page_size / 8; }
    else if (page_size > BN && page_size % BN == 0) { run_pages = 1; groups = BN / 8; }
    static const bool allowed = [] {
      const char* value = getenv("CIE_TC_RUNS");
      return !(value && value[0] == '0');
    }();
    if (allowed && run_pages > 0 && tensor_map_bf16_page_runs(k_pool, num_pages, kv_heads, page_size, D, groups, run_pages, &k_run) &&
        tensor_map_bf16_page_runs(v_pool, num_pages, kv_heads, page_size, D, groups, run_pages, &v_run))
      a.run_pages = run_pages;
  }
  static bool configured = false;
  if (!configured) {
    cudaError_t status = cudaFuncSetAttribute(prefill_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    if (status != cudaSuccess) CIE_FAIL("attention_prefill_tc: shared memory %d: %s", SMEM_BYTES, cudaGetErrorString(status));
    configured = true;
  }
  dim3 grid(num_tiles, kv_heads * a.head_chunks, splits);
  CIE_LAUNCH("attention_prefill_tc", prefill_tc_kernel, grid, dim3(THREADS), (size_t)SMEM_BYTES, (cudaStream_t)stream, k_map, v_map, k_run, v_run, a);
  return 0;
}
