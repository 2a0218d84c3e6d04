// Tensor-core attention over the paged cache for bfloat16, one head size per build (-DHEAD_DIM).
//
//  * prefill_kernel: ragged causal attention of prompt portions (cached prefix + the portion
//    itself) on mma.sync, for what the tcgen05 kernel (attention_prefill_tc.cu) does not take:
//    head sizes other than 64 and 128, windows, pages that are no multiple of 16 tokens.  One CTA
//    takes a tile of 128 query rows of ONE request and ONE kv head; a row is a (token, query head
//    of the group) pair, so the heads of a group share every K/V load.  K/V tiles of 64 keys are
//    gathered row by row from the pages with bulk asynchronous copies (any page size), double
//    buffered; QK^T and PV run on mma.sync m16n8k16 with float32 accumulators and a float32
//    running-maximum softmax.
//  * decode_kernel: one query token per request.  The keys of a request are split over the CTAs
//    of a thread-block cluster and, inside a CTA, over 12 warps that each stream 16-key tiles
//    through private stages (TMA tensor copies where pages, head size and window allow, else
//    cp.async); partial (max, sum, output) triples are merged in shared memory, then across the
//    cluster through distributed shared memory.
//
// Formula: zeeshan8281/cloud-inference-from-scratch src/cloud_engine/kernel.py:324-405 (one
// program per query token and head, CUDA-core reductions, page size fixed at 16, head size
// 64 or 128).  Here head sizes are the multiples of 16 up to 256, any page size and grouping.
#include "attention_tiles.cuh"
#include "blackwell.cuh"
#include "common.cuh"

#include <cooperative_groups.h>
#include <cuda.h>

#include <cfloat>

#ifndef HEAD_DIM
#define HEAD_DIM 128
#endif

CIE_DEFINE_LAST_ERROR()

namespace cie {

namespace cg = cooperative_groups;
// (fragment loads, tile addressing, score / accumulate / softmax steps: attention_tiles.cuh)
// ------------------------------------------------------------------------------------ prefill
constexpr int BM = 128, BN = 64, PREFILL_WARPS = 8;

struct PrefillArgs {
  const bf16* q;
  int q_stride;
  bf16* out;
  int out_stride;
  Pools pools;
  const int* tile_request;
  const int* tile_q0;
  const int* context_lens;
  const int* query_lens;
  const int* query_start;
  int group;         // query heads per kv head
  int hpt;           // heads of the group per tile (rows of one token)
  int tpt;           // tokens per tile
  int head_chunks;   // ceil(group / hpt)
  float scale_log2;
  int window;
  int* err;
};

// One 64-key tile: thread t < 64 copies key row t of K, thread 64 + t row t of V, each with one bulk
// asynchronous copy of a whole row (a row never crosses a page, so any page size works).  Rows
// outside [valid_lo, valid_hi) are not copied.  Thread 0 arms the stage's mbarrier.
__device__ __forceinline__ void load_kv_tile(const PrefillArgs& a, const int* row, int kvh, int k0,
                                             int valid_lo, int valid_hi, bf16* k_dst, bf16* v_dst,
                                             uint64_t* bar, int tid) {
  const int lo = max(k0, valid_lo), hi = min(k0 + BN, valid_hi);
  const int rows = max(0, hi - lo);
  if (tid == 0) mbar_expect_tx(bar, (uint32_t)rows * 2u * ROW_BYTES);
  if (tid >= 2 * BN) return;
  const int r = tid & (BN - 1);
  const int key = k0 + r;
  if (key < lo || key >= hi) return;
  long long off = kv_offset(a.pools, row, key, kvh, a.err);
  if (off < 0) off = (long long)kvh * a.pools.page_size * D;   // page 0: the copy must still happen
  if (tid < BN) bulk_copy(k_dst + r * ROW, a.pools.k + off, ROW_BYTES, bar);
  else bulk_copy(v_dst + r * ROW, a.pools.v + off, ROW_BYTES, bar);
}

__global__ void __launch_bounds__(PREFILL_WARPS * 32) prefill_kernel(const PrefillArgs a) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  bf16* q_s = reinterpret_cast<bf16*>(smem_raw);  // [BM][ROW]
  bf16* k_s = q_s + BM * ROW;                     // [2][BN][ROW]
  bf16* v_s = k_s + 2 * BN * ROW;                 // [2][BN][ROW]
  pdl_wait();
  pdl_trigger();
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int tile = blockIdx.x;
  const int kvh = blockIdx.y / a.head_chunks, h0 = (blockIdx.y % a.head_chunks) * a.hpt;
  const int request = a.tile_request[tile], q0 = a.tile_q0[tile];
  const int context = a.context_lens[request], q_len = a.query_lens[request];
  const int first_token = a.query_start[request] + q0;
  const int ntok = min(a.tpt, q_len - q0);
  const int* table_row = a.pools.table + (size_t)request * a.pools.table_width;

  // ---- Q tile: row r is token r / hpt, head h0 + r % hpt of the group
  for (int idx = tid; idx < BM * CHUNKS; idx += PREFILL_WARPS * 32) {
    const int r = idx / CHUNKS, c = idx % CHUNKS;
    const int tok = r / a.hpt, hh = h0 + r % a.hpt;
    const bool ok = tok < ntok && hh < a.group;
    const bf16* src = ok ? a.q + (size_t)(first_token + tok) * a.q_stride + (size_t)(kvh * a.group + hh) * D + c * 8 : a.q;
    cp_async16(q_s + r * ROW + c * 8, src, ok);
  }
  cp_async_commit();

  const int pos_lo = context + q0, pos_hi = context + q0 + ntok - 1;
  const int valid_lo = a.window > 0 ? max(0, pos_lo - a.window + 1) : 0;
  const int valid_hi = pos_hi + 1;
  const int k_begin = (valid_lo / BN) * BN;
  const int tiles = (valid_hi - k_begin + BN - 1) / BN;

  __shared__ __align__(8) uint64_t bars[2];
  if (tid < 2) mbar_init(&bars[tid], 1);
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  __syncthreads();
  load_kv_tile(a, table_row, kvh, k_begin, valid_lo, valid_hi, k_s, v_s, &bars[0], tid);

  uint32_t q_frag[KSTEPS][4];
  float o[NTILES_D][4];
#pragma unroll
  for (int i = 0; i < NTILES_D; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};

  // positions of the two rows this thread holds (-1: row not in use)
  const int g = lane >> 2, t4 = lane & 3;
  int row_pos[2];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int r = warp * 16 + g + h * 8;
    const int tok = r / a.hpt, hh = h0 + r % a.hpt;
    row_pos[h] = (tok < ntok && hh < a.group) ? context + q0 + tok : -1;
  }

  bool alive = true;
  for (int it = 0; it < tiles && alive; ++it) {
    const int stage = it & 1;
    if (it + 1 < tiles)
      load_kv_tile(a, table_row, kvh, k_begin + (it + 1) * BN, valid_lo, valid_hi,
                   k_s + (stage ^ 1) * BN * ROW, v_s + (stage ^ 1) * BN * ROW, &bars[stage ^ 1], tid);
    if (it == 0) cp_async_wait<0>();   // the queries
    alive = mbar_wait(&bars[stage], (it >> 1) & 1, a.err);
    const int k0 = k_begin + it * BN;
    {
      // rows of this tile that were not copied: their V must not hold NaN or Inf bits
      const int lo = max(k0, valid_lo), hi = min(k0 + BN, valid_hi);
      if (hi - lo < BN) {
        bf16* v_tile = v_s + stage * BN * ROW;
        for (int e = tid; e < BN * (D / 2); e += PREFILL_WARPS * 32) {
          const int r = e / (D / 2), c = e % (D / 2);
          if (k0 + r < lo || k0 + r >= hi) reinterpret_cast<uint32_t*>(v_tile + r * ROW)[c] = 0u;
        }
        // these ordinary stores must be ordered before later bulk copies into the same stage
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      }
    }
    __syncthreads();
    if (it == 0) {
#pragma unroll
      for (int kk = 0; kk < KSTEPS; ++kk)
        ldsm_x4(q_frag[kk], q_s + (warp * 16 + (lane & 15)) * ROW + kk * 16 + (lane >> 4) * 8);
    }
    // a warp whose rows all lie before this tile's first key has nothing to add
    const int warp_pos_hi = context + q0 + min(ntok - 1, (warp * 16 + 15) / a.hpt);
    if (k0 <= warp_pos_hi) {
      float s[BN / 8][4];
      scores<BN / 16>(q_frag, k_s + stage * BN * ROW, s, lane);
#pragma unroll
      for (int i = 0; i < BN / 8; ++i) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int key = k0 + i * 8 + 2 * t4 + (e & 1);
          const int pos = row_pos[e >> 1];
          const bool ok = key <= pos && (a.window <= 0 || key > pos - a.window);
          s[i][e] = ok ? s[i][e] * a.scale_log2 : -INFINITY;
        }
      }
      softmax_update<BN / 8>(s, m, l, o);
      accumulate<BN / 16>(s, v_s + stage * BN * ROW, o, lane);
    }
    __syncthreads();
  }

  // ---- write out
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    if (row_pos[h] < 0) continue;
    const float total = quad_sum(l[h]);
    const float inv = total > 0.f ? 1.f / total : 0.f;
    const int r = warp * 16 + g + h * 8;
    const int tok = r / a.hpt, hh = h0 + r % a.hpt;
    bf16* dst = a.out + (size_t)(first_token + tok) * a.out_stride + (size_t)(kvh * a.group + hh) * D;
#pragma unroll
    for (int i = 0; i < NTILES_D; ++i) {
      const uint32_t packed = pack_bf16(o[i][2 * h] * inv, o[i][2 * h + 1] * inv);
      *reinterpret_cast<uint32_t*>(dst + i * 8 + 2 * t4) = packed;
    }
  }
}

// ------------------------------------------------------------------------------------ decode
#ifndef DECODE_WARPS_N
#define DECODE_WARPS_N 12
#endif
constexpr int DECODE_WARPS = DECODE_WARPS_N;
constexpr int DN = 16;   // keys per warp and iteration

struct DecodeArgs {
  const bf16* q;          // row b of q_stride elements: the request's single query token
  int q_stride;
  bf16* out;
  int out_stride;
  Pools pools;
  const int* context_lens;  // keys before the query token; it attends to context + 1 keys
  int group;
  int head_chunks;          // ceil(group / 16)
  int page_shift;           // log2(page_size), or -1 if it is not a power of two
  int splits;               // CTAs per cluster: 1, 2, 4 or 8
  int chunks;               // clusters that may share a request's keys (1 .. DECODE_MAX_CHUNKS)
  int chunk_keys;           // a request uses only as many of them as leave every CTA this many keys
  float* partials;          // chunks > 1: [unit][chunk][16][D + 2] shares of the clusters
  int* counters;            // chunks > 1: [unit] CTAs that have delivered; zero between launches
  float scale_log2;
  int window;
  int q_heads;
  int* err;
};

constexpr int DECODE_MAX_CHUNKS = 16;
constexpr int DECODE_PAGE_SLOTS = 1024;   // block-table entries of a CTA's key range kept in shared memory

// Stages per warp: all but one are in flight while one is multiplied.
//  cp.async variant: padded rows (ROW elements), two stages (one for head sizes over 128).
//  TMA variant: unpadded swizzled tiles, two stages.
constexpr int DECODE_STAGES_LSU = D <= 128 ? 2 : 1;
#ifndef DECODE_STAGES_TMA_N
#define DECODE_STAGES_TMA_N (HEAD_DIM <= 128 ? 2 : 1)
#endif
constexpr int DECODE_STAGES_TMA = DECODE_STAGES_TMA_N;
constexpr int DECODE_STAGE_LSU = 2 * DN * ROW;   // K and V of one stage, elements
constexpr int DECODE_STAGE_TMA = 2 * DN * D;
constexpr size_t DECODE_Q_BYTES = ((size_t)16 * ROW * sizeof(bf16) + 1023) / 1024 * 1024;
constexpr size_t DECODE_MERGE_BYTES = (size_t)DECODE_WARPS * 16 * (D + 2) * sizeof(float);
constexpr size_t DECODE_PART_BYTES = (size_t)16 * (D + 2) * sizeof(float);
template <bool kTma>
constexpr size_t decode_work_bytes() {
  const size_t kv = (size_t)DECODE_WARPS * (kTma ? DECODE_STAGES_TMA * DECODE_STAGE_TMA : DECODE_STAGES_LSU * DECODE_STAGE_LSU) * sizeof(bf16);
  const size_t need = kv > DECODE_MERGE_BYTES ? kv : DECODE_MERGE_BYTES;
  return (need + 1023) / 1024 * 1024;
}
template <bool kTma>
constexpr size_t decode_smem() { return 1024 + DECODE_Q_BYTES + decode_work_bytes<kTma>() + DECODE_PART_BYTES; }

// One 16-key tile of K and V for one warp with 16-byte cp.async, two lanes per key row.  The page
// of a key comes from the CTA's copy of its block-table range (or from global memory if the range
// did not fit).  Rows past `valid_hi` are filled with zeros.
__device__ __forceinline__ void load_kv_tile_warp(const DecodeArgs& a, const int* row, const int* pages_s,
                                                  int first_index, int cached, int kvh, int k0,
                                                  int valid_hi, bf16* k_dst, bf16* v_dst, int lane) {
  const int half = lane & 1;
  const int r = lane >> 1;
  const int key = k0 + r;
  long long off = -1;
  if (key < valid_hi) {
    int index, within;
    if (a.page_shift >= 0) { index = key >> a.page_shift; within = key & (a.pools.page_size - 1); }
    else { index = key / a.pools.page_size; within = key - index * a.pools.page_size; }
    int page;
    if (index - first_index < cached) page = pages_s[index - first_index];
    else page = index < a.pools.table_width ? row[index] : -1;
    if (page < 0 || page >= a.pools.num_pages) atomicOr(a.err, kErrBadPage);
    else off = (((long long)page * a.pools.kv_heads + kvh) * a.pools.page_size + within) * D;
  }
  // one source pointer and one destination address per row; the pieces are constant offsets
  const int bytes = off >= 0 ? 16 : 0;
  const bf16* ks = a.pools.k + (off >= 0 ? off : 0) + half * 8;
  const bf16* vs = a.pools.v + (off >= 0 ? off : 0) + half * 8;
  const uint32_t kd = smem_u32(k_dst + r * ROW + half * 8), vd = smem_u32(v_dst + r * ROW + half * 8);
#pragma unroll
  for (int c = 0; c < CHUNKS / 2; ++c) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(kd + c * 32), "l"(ks + c * 16), "r"(bytes));
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(vd + c * 32), "l"(vs + c * 16), "r"(bytes));
  }
}


// Several clusters per request: the CTA that delivered last adds up the clusters' shares
// ([chunk][16][D + 2] floats: unnormalised output, maximum, sum) and writes the output rows.
// Kept out of line so that it costs the kernel's main loop no registers.
__device__ __noinline__ void merge_chunks(const float* unit_partials, int chunks, bf16* out_rows, int rows,
                                          int tid) {
  // out_rows: the first of this unit's head rows in the output; rows: how many of the 16 exist
  for (int idx = tid; idx < 16 * D; idx += DECODE_WARPS * 32) {
    const int r = idx / D, d = idx % D;
    if (r >= rows) continue;
    float ms[DECODE_MAX_CHUNKS], ls[DECODE_MAX_CHUNKS], os[DECODE_MAX_CHUNKS];
#pragma unroll
    for (int c = 0; c < DECODE_MAX_CHUNKS; ++c) {
      if (c < chunks) {
        const float* share = unit_partials + (size_t)(c * 16 + r) * (D + 2);
        ms[c] = __ldcg(share + D);
        ls[c] = __ldcg(share + D + 1);
        os[c] = __ldcg(share + d);
      } else {
        ms[c] = -INFINITY; ls[c] = 0.f; os[c] = 0.f;
      }
    }
    float m_all = -INFINITY;
#pragma unroll
    for (int c = 0; c < DECODE_MAX_CHUNKS; ++c) m_all = fmaxf(m_all, ms[c]);
    float sum = 0.f, acc = 0.f;
#pragma unroll
    for (int c = 0; c < DECODE_MAX_CHUNKS; ++c) {
      const float f = (ms[c] == -INFINITY) ? 0.f : exp2f(ms[c] - m_all);
      sum += ls[c] * f;
      acc += os[c] * f;
    }
    out_rows[(size_t)r * D + d] = __float2bfloat16_rn(sum > 0.f ? acc / sum : 0.f);
  }
}

// kTma == false: keys and values come through the load/store unit (cp.async), any page size and
// window.  kTma == true: each 16-key tile is fetched by one lane with D/64 tensor copies per
// matrix (boxes of 16 rows x 64 columns, 128-byte swizzle) that complete on the stage's mbarrier;
// it needs pages of a multiple of 16 tokens, a head size that is a multiple of 64 and no window,
// so that a tile never straddles two pages.
template <bool kTma>
__global__ void __launch_bounds__(DECODE_WARPS * 32)
decode_kernel(const __grid_constant__ CUtensorMap k_map, const __grid_constant__ CUtensorMap v_map,
              const DecodeArgs a) {
  constexpr int STAGES = kTma ? DECODE_STAGES_TMA : DECODE_STAGES_LSU;
  constexpr int STAGE = kTma ? DECODE_STAGE_TMA : DECODE_STAGE_LSU;
  extern __shared__ __align__(16) unsigned char smem_unaligned[];
  unsigned char* smem_raw = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_unaligned) + 1023) & ~(uintptr_t)1023);
  bf16* q_s = reinterpret_cast<bf16*>(smem_raw);                          // [16][ROW]
  bf16* kv_s = reinterpret_cast<bf16*>(smem_raw + DECODE_Q_BYTES);        // per warp: STAGES of K,V
  float* merge_s = reinterpret_cast<float*>(smem_raw + DECODE_Q_BYTES);   // aliased after the loop
  float* part_s = reinterpret_cast<float*>(smem_raw + DECODE_Q_BYTES + decode_work_bytes<kTma>());
  __shared__ int pages_s[DECODE_PAGE_SLOTS];
  __shared__ __align__(8) uint64_t bars[DECODE_WARPS][kTma ? DECODE_STAGES_TMA : 1];
  // The TMA variant waits for the kernel before it only after it has asked for its first key
  // tiles: block tables and context lengths come with the step's metadata, and older keys and
  // values are not touched by the kernel before this one (it writes the newest token only), so
  // only a tile that holds the newest key has to wait.  This rests on every kernel triggering its
  // dependents AFTER its own wait: then at most the one kernel before this one is still running.
  if constexpr (!kTma) {
    pdl_wait();
    pdl_trigger();
  }
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int split = blockIdx.x;
  const int kvh = blockIdx.y / a.head_chunks, h0 = (blockIdx.y % a.head_chunks) * 16;
  const int request = blockIdx.z;
  const int* table_row = a.pools.table + (size_t)request * a.pools.table_width;
  const int length = a.context_lens[request] + 1;
  const int first = (a.window > 0 && length > a.window) ? length - a.window : 0;
  // how many of the launched clusters this request needs: the launch is sized for the longest
  // context the tables can hold, the request may be far shorter; the others leave at once
  int chunks = a.chunks;
  if (chunks > 1) chunks = max(1, min(chunks, (length - first) / (a.splits * a.chunk_keys)));
  if ((int)blockIdx.x / a.splits >= chunks) return;
  const int ranges = a.splits * chunks;   // blockIdx.x counts key ranges; a cluster holds neighbours
  const int per_split = (((length - first + ranges - 1) / ranges) + DN - 1) / DN * DN;
  const int begin = first + split * per_split;
  const int end = min(length, begin + per_split);

  if constexpr (kTma) {
    if (tid < DECODE_WARPS * STAGES) mbar_init(&bars[tid / STAGES][tid % STAGES], 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  // this CTA's stretch of the block table goes to shared memory once, so that no tile load has
  // to wait for a table entry from global memory first
  const int first_index = begin / a.pools.page_size;
  int cached = begin < end ? (end - 1) / a.pools.page_size - first_index + 1 : 0;
  if (cached > DECODE_PAGE_SLOTS) cached = DECODE_PAGE_SLOTS;
  for (int i = tid; i < cached; i += DECODE_WARPS * 32)
    pages_s[i] = first_index + i < a.pools.table_width ? table_row[first_index + i] : -1;
  __syncthreads();

  bf16* mine = kv_s + warp * STAGES * STAGE;
  const int tiles = begin < end ? (end - begin + DN - 1) / DN : 0;
  // warp w takes tiles w, w + DECODE_WARPS, ...
  auto issue = [&](int tile, int slot) {
    bf16* dst = mine + slot * STAGE;
    if constexpr (kTma) {
      if (tile < tiles && lane == 0) {
        const int key = begin + tile * DN;   // a multiple of 16: the tile lies inside one page
        const int index = key >> a.page_shift, within = key & (a.pools.page_size - 1);
        int page;
        if (index - first_index < cached) page = pages_s[index - first_index];
        else page = index < a.pools.table_width ? table_row[index] : -1;
        if (page < 0 || page >= a.pools.num_pages) {
          atomicOr(a.err, kErrBadPage);
          page = 0;   // the copies must still happen, or the barrier would never complete
        }
        const int row0 = (page * a.pools.kv_heads + kvh) * a.pools.page_size + within;
        uint64_t* bar = &bars[warp][slot];
        mbar_expect_tx(bar, (uint32_t)(2 * DN * D * sizeof(bf16)));
        if constexpr (kBlockCopies) {
          if constexpr (D == 128) {
            bw::tma_load_4d(dst, &k_map, bar, 0, 0, 0, row0 / 8);
            bw::tma_load_4d(dst + DN * D, &v_map, bar, 0, 0, 0, row0 / 8);
          } else {
            bw::tma_load_3d(dst, &k_map, bar, 0, 0, row0 / 8);
            bw::tma_load_3d(dst + DN * D, &v_map, bar, 0, 0, row0 / 8);
          }
        } else {
#pragma unroll
          for (int sub = 0; sub < D / 64; ++sub) {
            tma_load_2d(dst + sub * 1024, &k_map, bar, sub * 64, row0);
            tma_load_2d(dst + DN * D + sub * 1024, &v_map, bar, sub * 64, row0);
          }
        }
      }
    } else {
      if (tile < tiles)
        load_kv_tile_warp(a, table_row, pages_s, first_index, cached, kvh, begin + tile * DN, end, dst,
                          dst + DN * ROW, lane);
      cp_async_commit();
    }
  };
  // tiles that can be asked for before the kernels before this one have finished: all but the
  // one that holds the newest key (position length - 1)
  int early = 0;   // how many of the first STAGES - 1 tiles of this warp were issued early
  if constexpr (kTma) {
#pragma unroll
    for (int p = 0; p < STAGES - 1; ++p) {
      const int tile = warp + p * DECODE_WARPS;
      if (tile < tiles && begin + (tile + 1) * DN <= length - 1) {
        issue(tile, p);
        early |= 1 << p;
      }
    }
    pdl_wait();
    pdl_trigger();
  }
  for (int idx = tid; idx < 16 * CHUNKS; idx += DECODE_WARPS * 32) {
    const int r = idx / CHUNKS, c = idx % CHUNKS;
    const bool ok = h0 + r < a.group;
    const bf16* src = ok ? a.q + (size_t)request * a.q_stride + (size_t)(kvh * a.group + h0 + r) * D + c * 8 : a.q;
    cp_async16(q_s + r * ROW + c * 8, src, ok);
  }
  cp_async_commit();
#pragma unroll
  for (int p = 0; p < STAGES - 1; ++p)
    if (!(early & (1 << p))) issue(warp + p * DECODE_WARPS, p);
  if constexpr (kTma) cp_async_wait<0>();
  else cp_async_wait<STAGES - 1>();   // the queries (first group) have landed
  __syncthreads();
  uint32_t q_frag[KSTEPS][4];
#pragma unroll
  for (int kk = 0; kk < KSTEPS; ++kk)
    ldsm_x4(q_frag[kk], q_s + (lane & 15) * ROW + kk * 16 + (lane >> 4) * 8);

  float o[NTILES_D][4];
#pragma unroll
  for (int i = 0; i < NTILES_D; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
  const int t4 = lane & 3;

  int stage = 0;
  uint32_t phases = 0;   // TMA variant: bit s is the parity to wait for on stage s
  bool alive = true;
  for (int it = warp; it < tiles && alive; it += DECODE_WARPS) {
    issue(it + (STAGES - 1) * DECODE_WARPS, (stage + STAGES - 1) % STAGES);
    if constexpr (kTma) {
      alive = mbar_wait(&bars[warp][stage], (phases >> stage) & 1u, a.err);
      phases ^= 1u << stage;
    } else {
      cp_async_wait<STAGES - 1>();
      __syncwarp();
    }
    const bf16* k_tile = mine + stage * STAGE;
    const bf16* v_tile = k_tile + (kTma ? DN * D : DN * ROW);
    const int k0 = begin + it * DN;
    float s[DN / 8][4];
    scores<DN / 16, kTma>(q_frag, k_tile, s, lane);
    if (k0 + DN <= end) {
#pragma unroll
      for (int i = 0; i < DN / 8; ++i)
#pragma unroll
        for (int e = 0; e < 4; ++e) s[i][e] *= a.scale_log2;
    } else {
#pragma unroll
      for (int i = 0; i < DN / 8; ++i)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int key = k0 + i * 8 + 2 * t4 + (e & 1);
          s[i][e] = key < end ? s[i][e] * a.scale_log2 : -INFINITY;
        }
    }
    if (a.group - h0 <= 8) softmax_update<DN / 8, 1>(s, m, l, o);
    else softmax_update<DN / 8, 2>(s, m, l, o);
    accumulate<DN / 16, kTma>(s, v_tile, o, lane);
    __syncwarp();
    stage = (stage + 1) % STAGES;
  }
  if constexpr (!kTma) cp_async_wait<0>();
  __syncthreads();   // every warp is done with its K/V buffers: reuse them for the merge

  // ---- merge the warps: per warp [16][D + 2] floats (o, then max, then sum)
  const int g = lane >> 2;
  float* my_merge = merge_s + warp * 16 * (D + 2);
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int r = g + h * 8;
    const float total = quad_sum(l[h]);
#pragma unroll
    for (int i = 0; i < NTILES_D; ++i) {
      my_merge[r * (D + 2) + i * 8 + 2 * t4] = o[i][2 * h];
      my_merge[r * (D + 2) + i * 8 + 2 * t4 + 1] = o[i][2 * h + 1];
    }
    if (t4 == 0) {
      my_merge[r * (D + 2) + D] = m[h];
      my_merge[r * (D + 2) + D + 1] = total;
    }
  }
  __syncthreads();
  // this CTA's share: part_s[16][D + 2] = (unnormalised output, running maximum, sum)
  for (int idx = tid; idx < 16 * (D + 1); idx += DECODE_WARPS * 32) {
    const int r = idx / (D + 1), d = idx % (D + 1);
    float m_all = -INFINITY;
#pragma unroll
    for (int w = 0; w < DECODE_WARPS; ++w) m_all = fmaxf(m_all, merge_s[(w * 16 + r) * (D + 2) + D]);
    float acc = 0.f;
#pragma unroll
    for (int w = 0; w < DECODE_WARPS; ++w) {
      const float mw = merge_s[(w * 16 + r) * (D + 2) + D];
      const float f = (mw == -INFINITY) ? 0.f : exp2f(mw - m_all);
      // column D of a warp's block holds its maximum; column D + 1 its sum
      acc += merge_s[(w * 16 + r) * (D + 2) + (d < D ? d : D + 1)] * f;
    }
    if (d < D) {
      part_s[r * (D + 2) + d] = acc;
    } else {
      part_s[r * (D + 2) + D] = m_all;
      part_s[r * (D + 2) + D + 1] = acc;
    }
  }
  if (a.splits == 1 && chunks == 1) {
    __syncthreads();
    for (int idx = tid; idx < 16 * D; idx += DECODE_WARPS * 32) {
      const int r = idx / D, d = idx % D;
      if (h0 + r >= a.group) continue;
      const float sum = part_s[r * (D + 2) + D + 1];
      a.out[(size_t)request * a.out_stride + (size_t)(kvh * a.group + h0 + r) * D + d] =
          __float2bfloat16_rn(sum > 0.f ? part_s[r * (D + 2) + d] / sum : 0.f);
    }
    return;
  }
  // ---- the CTAs of a cluster hold the splits of one (request, kv head, head chunk): after a
  // cluster barrier each CTA merges some of the 16 head rows, reading its peers' shares through
  // distributed shared memory.  No scratch in global memory, no second kernel.
  // With several clusters per request (long contexts at small batches) a cluster's merged rows
  // go to global memory instead, unnormalised, and whichever CTA of the request delivers last
  // (a ticket from an atomic counter: nobody waits for anybody) merges the clusters.
  cg::cluster_group cluster = cg::this_cluster();
  cluster.sync();
  const int rank = (int)cluster.block_rank();
  const bool chunked = chunks > 1;
  const int unit = request * gridDim.y + blockIdx.y;
  float* unit_partials = chunked ? a.partials + (size_t)unit * a.chunks * 16 * (D + 2) : nullptr;
  float* my_partials = chunked ? unit_partials + (size_t)(blockIdx.x / a.splits) * 16 * (D + 2) : nullptr;
  for (int idx = tid; idx < 16 * D; idx += DECODE_WARPS * 32) {
    const int r = idx / D, d = idx % D;
    if (r % a.splits != rank || h0 + r >= a.group) continue;
    float ms[8], ls[8], os[8];
#pragma unroll
    for (int c = 0; c < 8; ++c) {
      if (c < a.splits) {
        const float* peer = cluster.map_shared_rank(part_s, c);
        ms[c] = peer[r * (D + 2) + D];
        ls[c] = peer[r * (D + 2) + D + 1];
        os[c] = peer[r * (D + 2) + d];
      } else {
        ms[c] = -INFINITY; ls[c] = 0.f; os[c] = 0.f;
      }
    }
    float m_all = -INFINITY;
#pragma unroll
    for (int c = 0; c < 8; ++c) m_all = fmaxf(m_all, ms[c]);
    float sum = 0.f, acc = 0.f;
#pragma unroll
    for (int c = 0; c < 8; ++c) {
      const float f = (ms[c] == -INFINITY) ? 0.f : exp2f(ms[c] - m_all);
      sum += ls[c] * f;
      acc += os[c] * f;
    }
    if (!chunked) {
      a.out[(size_t)request * a.out_stride + (size_t)(kvh * a.group + h0 + r) * D + d] =
          __float2bfloat16_rn(sum > 0.f ? acc / sum : 0.f);
    } else {
      my_partials[r * (D + 2) + d] = acc;
      if (d == 0) {
        my_partials[r * (D + 2) + D] = m_all;
        my_partials[r * (D + 2) + D + 1] = sum;
      }
    }
  }
  cluster.sync();   // nobody leaves while a peer may still read its share
  if (!chunked) return;
  __shared__ int last_s;
  __threadfence();   // this thread's shares are visible before the ticket is drawn
  __syncthreads();
  if (tid == 0) last_s = atomicAdd(&a.counters[unit], 1) == a.splits * chunks - 1;
  __syncthreads();
  if (!last_s) return;
  __threadfence();
  merge_chunks(unit_partials, chunks, a.out + (size_t)request * a.out_stride + (size_t)(kvh * a.group + h0) * D,
               a.group - h0, tid);
  if (tid == 0) a.counters[unit] = 0;   // ready for the next launch
}

// ------------------------------------------------------------------------------------ decode, split over CTAs
// The decode kernel for pools that TMA can read (pages of a power of two >= 16 tokens, head size a
// multiple of 64).  A request's keys are cut into `splits` ranges, one CTA each:
// a CTA is 4 warps and a ring of SPLIT_STAGES stages of 64 keys (K and V of a stage arrive by
// one mbarrier; 16 KB of keys and 16 KB of values at head size 128), so two or three CTAs fit an
// SM and every SM has work at small batches.  Warp w multiplies the w-th 16 keys of a stage.  A
// The CTAs of a unit (request, kv head, 16 heads) that lie in one thread-block cluster divide the
// head rows among themselves and send each other their shares of them (unnormalised output,
// maximum, sum) with asynchronous stores into the owner's shared memory that complete on a barrier
// there; every CTA adds up the rows it owns and writes them out.  A unit that spans several
// clusters (or a launch without clusters) leaves the shares in global memory instead and draws a
// ticket: whoever draws the last ticket of the unit adds the shares up.  Nobody waits for a CTA that
// may not be running.
//
// Before `griddepcontrol.wait` a CTA already asks for the stages that do not hold the newest key:
// block tables and context lengths come with the step's metadata and older keys and values are
// not touched by the kernel before this one (it writes the newest token only).
constexpr int SPLIT_WARPS = 4;
constexpr int SPLIT_TILE = SPLIT_WARPS * DN;          // keys per stage
constexpr int SPLIT_MAX_STAGES = 8;                   // one lane of the first warp per 16-key block in flight
constexpr int SPLIT_MAX = 64;                         // most CTAs that share a request's keys
constexpr int SPLIT_BLOCK = DN * D;                   // elements of one 16-key block of K (or V)
constexpr int SPLIT_STAGE = 2 * SPLIT_TILE * D;       // elements of a stage: 4 K blocks, then 4 V blocks
constexpr int SPLIT_SHARE_ROW = D + 4;                // floats of a share's row: D outputs, maximum, sum, padding
constexpr int SPLIT_SHARE = 16 * SPLIT_SHARE_ROW;     // floats of a CTA's share
constexpr int SPLIT_PAGE_SLOTS = 512;                 // the first block-table entries of a request, kept in shared memory
constexpr size_t SPLIT_STAGE_BYTES = (size_t)SPLIT_STAGE * sizeof(bf16);
constexpr size_t SPLIT_MERGE_BYTES = ((size_t)SPLIT_WARPS * 16 * D + 16 * (D + 4)) * sizeof(float);   // the warps' blocks, then the CTA's own rows
constexpr int SPLIT_MIN_STAGES = (int)((SPLIT_MERGE_BYTES + SPLIT_STAGE_BYTES - 1) / SPLIT_STAGE_BYTES);   // the merge buffers reuse the ring
static_assert(SPLIT_MAX_STAGES * SPLIT_WARPS <= 32, "one lane of the first warp per 16-key block in flight");
// A CTA that shares a unit of `rows` head rows with p - 1 others in its cluster owns at most
// ceil(rows / p) of them and receives p - 1 shares of each; p is anything up to the cluster size
// (the last cluster of a unit may be partly used).
constexpr int split_inbox_rows(int rows, int cluster) {
  int most = 0;
  for (int p = 2; p <= cluster; ++p) {
    const int need = (p - 1) * ((rows + p - 1) / p);
    if (need > most) most = need;
  }
  return most;
}
// dynamic shared memory: alignment slack, the queries, the ring, and (with clusters) the inbox
constexpr size_t split_smem(int stages, int cluster, int rows) {
  return 1024 + DECODE_Q_BYTES + (size_t)stages * SPLIT_STAGE_BYTES +
         (size_t)split_inbox_rows(rows, cluster) * SPLIT_SHARE_ROW * sizeof(float);
}

__device__ __forceinline__ uint32_t cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// the shared::cluster address, in CTA `rank` of the cluster, of what lies at `p` in this CTA
__device__ __forceinline__ uint32_t map_to_rank(const void* p, uint32_t rank) {
  uint32_t remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(smem_u32(p)), "r"(rank));
  return remote;
}
__device__ __forceinline__ void cluster_arrive() { asm volatile("barrier.cluster.arrive.release;" ::: "memory"); }
__device__ __forceinline__ void cluster_wait() { asm volatile("barrier.cluster.wait.acquire;" ::: "memory"); }
// asynchronous stores into another CTA's shared memory; the bytes count on the barrier `bar` there
__device__ __forceinline__ void push_f4(uint32_t remote, float4 v, uint32_t bar) {
  asm volatile("st.async.shared::cluster.mbarrier::complete_tx::bytes.v4.f32 [%0], {%1, %2, %3, %4}, [%5];"
               ::"r"(remote), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w), "r"(bar) : "memory");
}
__device__ __forceinline__ void push_f2(uint32_t remote, float a, float b, uint32_t bar) {
  asm volatile("st.async.shared::cluster.mbarrier::complete_tx::bytes.v2.f32 [%0], {%1, %2}, [%3];"
               ::"r"(remote), "f"(a), "f"(b), "r"(bar) : "memory");
}

struct SplitArgs {
  const bf16* q;            // row b of q_stride elements: the request's single query token
  int q_stride;
  bf16* out;
  int out_stride;
  Pools pools;
  const int* context_lens;  // keys before the query token; it attends to context + 1 keys
  int group;
  int head_chunks;          // ceil(group / 16)
  int page_shift;           // log2(page_size)
  int splits;               // CTAs launched per unit (1 .. SPLIT_MAX)
  int min_keys;             // a request uses only as many of them as leave every CTA this many keys
  int stages;               // stages of the ring (SPLIT_MIN_STAGES .. SPLIT_MAX_STAGES)
  int cluster;              // CTAs of a thread-block cluster along the splits (1: no clusters)
  float* shares;            // [unit][split / cluster][16][D + 4]
  int* tickets;             // [unit]; zero between launches
  float scale_log2;
  int window;
  int* err;
};

// The CTA that drew a unit's last ticket adds up the unit's shares: every thread takes four columns
// of one head row, asks for the maxima, sums and outputs of eight shares at one time and merges
// them with a running maximum (in the order of the shares, so the result does not depend on who
// came last).
__device__ __noinline__ void merge_shares(const float* unit_shares, int count, bf16* out_rows, int rows, int tid) {
  for (int idx = tid; idx < rows * (D / 4); idx += SPLIT_WARPS * 32) {
    const int r = idx / (D / 4), c4 = idx % (D / 4);
    const float* row = unit_shares + r * SPLIT_SHARE_ROW;
    float m_run = -INFINITY, sum = 0.f;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int c0 = 0; c0 < count; c0 += 8) {
      float ms[8], ls[8];
      float4 part[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const bool live = c0 + j < count;
        const float* share = row + (size_t)(live ? c0 + j : c0) * SPLIT_SHARE;
        ms[j] = live ? __ldcg(share + D) : -INFINITY;
        ls[j] = live ? __ldcg(share + D + 1) : 0.f;
        part[j] = __ldcg(reinterpret_cast<const float4*>(share + c4 * 4));
      }
      float m_new = m_run;
#pragma unroll
      for (int j = 0; j < 8; ++j) m_new = fmaxf(m_new, ms[j]);
      const float keep = (m_run == -INFINITY) ? 0.f : exp2f(m_run - m_new);
      sum *= keep; acc.x *= keep; acc.y *= keep; acc.z *= keep; acc.w *= keep;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float f = (ms[j] == -INFINITY) ? 0.f : exp2f(ms[j] - m_new);
        sum += ls[j] * f;
        acc.x += part[j].x * f; acc.y += part[j].y * f; acc.z += part[j].z * f; acc.w += part[j].w * f;
      }
      m_run = m_new;
    }
    const float inv = sum > 0.f ? 1.f / sum : 0.f;
    uint2 packed;
    packed.x = pack_bf16(acc.x * inv, acc.y * inv);
    packed.y = pack_bf16(acc.z * inv, acc.w * inv);
    *reinterpret_cast<uint2*>(out_rows + (size_t)r * D + c4 * 4) = packed;
  }
}

#ifdef SPLIT_TRACE
// Debug builds only (-DSPLIT_TRACE): every CTA leaves the global timer at eight points of its life.
__device__ long long* g_split_trace = nullptr;
__device__ __forceinline__ void split_mark(int point) {
  if (threadIdx.x == 0 && g_split_trace) {
    long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    const int cta = (blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x;
    g_split_trace[cta * 8 + point] = t;
  }
}
#define SPLIT_MARK(point) split_mark(point)
#else
#define SPLIT_MARK(point)
#endif

template <bool kCluster>
__global__ void __launch_bounds__(SPLIT_WARPS * 32)
decode_split_kernel(const __grid_constant__ CUtensorMap k_map, const __grid_constant__ CUtensorMap v_map,
                    const SplitArgs a) {
  extern __shared__ __align__(16) unsigned char smem_unaligned[];
  unsigned char* smem_raw = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_unaligned) + 1023) & ~(uintptr_t)1023);
  bf16* q_s = reinterpret_cast<bf16*>(smem_raw);                          // [16][ROW]
  bf16* ring = reinterpret_cast<bf16*>(smem_raw + DECODE_Q_BYTES);        // a.stages stages
  float* merge_s = reinterpret_cast<float*>(smem_raw + DECODE_Q_BYTES);   // reused after the loop: [warp][16][D]
  __shared__ __align__(8) uint64_t full[SPLIT_MAX_STAGES];
  __shared__ int pages_s[SPLIT_PAGE_SLOTS];
  __shared__ float warp_max_s[SPLIT_WARPS][16], warp_sum_s[SPLIT_WARPS][16];
  __shared__ int last_s;
  __shared__ __align__(8) uint64_t inbox_bar;   // cluster variant: counts the bytes of the peers' shares
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if constexpr (kCluster) {
    // every CTA of the cluster sets its inbox up and says so, whether it has keys or not; a CTA
    // that hands its share over first makes sure that everybody has said so
    if (tid == 0) {
      mbar_init(&inbox_bar, 1);
      asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    cluster_arrive();
  }
  SPLIT_MARK(0);
  // the split is the slowest index of the grid: the CTAs a short request does not use come last
  const int split = blockIdx.z;
  const int kvh = blockIdx.x / a.head_chunks, h0 = (blockIdx.x % a.head_chunks) * 16;
  const int request = blockIdx.y;
  const int stages = a.stages;
  const int* table_row = a.pools.table + (size_t)request * a.pools.table_width;
  // the request's block-table row goes to shared memory once, asked for together with its length,
  // so that no copy has to wait for a table entry from global memory first
  const int cached = min(a.pools.table_width, SPLIT_PAGE_SLOTS);
  for (int i = tid; i < cached; i += SPLIT_WARPS * 32) pages_s[i] = table_row[i];
  const int length = a.context_lens[request] + 1;
  const int first = (a.window > 0 && length > a.window) ? length - a.window : 0;
  const int first_block = first / DN;                      // 16-key blocks are the unit of a copy
  const int blocks = (length + DN - 1) / DN - first_block;
  // how many of the launched CTAs this request uses: the launch is sized for the longest context
  // the tables can hold, the request may be far shorter; the others leave at once
  const int used = max(1, min(a.splits, (length - first) / a.min_keys));
  if (split >= used) return;
  // the CTAs of this unit that lie in this CTA's cluster, and the clusters the unit uses
  const int rank = kCluster ? (int)cluster_rank() : 0;
  const int cluster_index = split / a.cluster;
  const int peers = min(a.cluster, used - cluster_index * a.cluster);   // working CTAs of this cluster
  const int clusters_used = (used + a.cluster - 1) / a.cluster;
  const int live_rows = min(16, a.group - h0);
  // head row r of the unit is finished by the CTA of rank r % peers; this CTA owns rows rank,
  // rank + peers, ... and keeps them at local index r / peers
  const int rows_owned = rank < live_rows ? (live_rows - rank + peers - 1) / peers : 0;
  const int rows_per_owner = (live_rows + peers - 1) / peers;
  float* inbox = reinterpret_cast<float*>(smem_raw + DECODE_Q_BYTES + (size_t)a.stages * SPLIT_STAGE_BYTES);
  if constexpr (kCluster) {
    if (peers > 1 && rows_owned > 0 && tid == 0)
      mbar_expect_tx(&inbox_bar, (uint32_t)((peers - 1) * rows_owned * (D + 2) * sizeof(float)));
  }
  const int per_split = (blocks + used - 1) / used;        // in blocks
  const int begin = (first_block + split * per_split) * DN;
  const int end = min(length, begin + per_split * DN);
  const int tiles = begin < end ? (end - begin + SPLIT_TILE - 1) / SPLIT_TILE : 0;

  if (tid < stages) mbar_init(&full[tid], 1);
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  __syncthreads();

  // The first warp feeds the ring: tiles [tile0, tile0 + count) go to stages slot0, slot0 + 1, ...;
  // lane 4 t + b copies the b-th 16 keys (and values) of the t-th of them.
  auto issue = [&](int tile0, int count, int slot0) {
    const int t = lane >> 2, b = lane & 3;
    const int tile = tile0 + t;
    const int k0 = begin + tile * SPLIT_TILE;
    const bool active = t < count && tile < tiles;
    const int in_tile = active ? min(SPLIT_WARPS, (end - k0 + DN - 1) / DN) : 0;   // 16-key blocks of the tile
    int slot = slot0 + t;
    if (slot >= stages) slot -= stages;
    uint64_t* bar = &full[slot];
    if (active && b == 0) mbar_expect_tx(bar, (uint32_t)(in_tile * 2 * SPLIT_BLOCK * sizeof(bf16)));
    __syncwarp();
    if (b < in_tile) {
      const int key = k0 + b * DN;
      const int index = key >> a.page_shift, within = key & (a.pools.page_size - 1);
      int page;
      if (index < cached) page = pages_s[index];
      else page = index < a.pools.table_width ? table_row[index] : -1;
      if (page < 0 || page >= a.pools.num_pages) {
        atomicOr(a.err, kErrBadPage);
        page = 0;   // the copies must still happen, or the barrier would never complete
      }
      const int row0 = (page * a.pools.kv_heads + kvh) * a.pools.page_size + within;
      bf16* k_dst = ring + slot * SPLIT_STAGE + b * SPLIT_BLOCK;
      bf16* v_dst = k_dst + SPLIT_WARPS * SPLIT_BLOCK;
      if constexpr (kBlockCopies) {
        if constexpr (D == 128) {
          bw::tma_load_4d(k_dst, &k_map, bar, 0, 0, 0, row0 / 8);
          bw::tma_load_4d(v_dst, &v_map, bar, 0, 0, 0, row0 / 8);
        } else {
          bw::tma_load_3d(k_dst, &k_map, bar, 0, 0, row0 / 8);
          bw::tma_load_3d(v_dst, &v_map, bar, 0, 0, row0 / 8);
        }
      } else {
#pragma unroll
        for (int sub = 0; sub < D / 64; ++sub) {
          tma_load_2d(k_dst + sub * 1024, &k_map, bar, sub * 64, row0);
          tma_load_2d(v_dst + sub * 1024, &v_map, bar, sub * 64, row0);
        }
      }
    }
  };
  // stages that can be asked for before the kernels before this one have finished: those that do
  // not hold the newest key (position length - 1)
  int early = 0;
  while (early < stages && early < tiles && begin + (early + 1) * SPLIT_TILE <= length - 1) ++early;
  SPLIT_MARK(1);
  if (warp == 0 && early) issue(0, early, 0);
  pdl_wait();
  pdl_trigger();
  SPLIT_MARK(2);
  for (int idx = tid; idx < 16 * CHUNKS; idx += SPLIT_WARPS * 32) {
    const int r = idx / CHUNKS, c = idx % CHUNKS;
    const bool ok = h0 + r < a.group;
    const bf16* src = ok ? a.q + (size_t)request * a.q_stride + (size_t)(kvh * a.group + h0 + r) * D + c * 8 : a.q;
    cp_async16(q_s + r * ROW + c * 8, src, ok);
  }
  cp_async_commit();
  if (warp == 0 && early < stages && early < tiles) issue(early, stages - early, early);
  cp_async_wait<0>();
  __syncthreads();
  uint32_t q_frag[KSTEPS][4];
#pragma unroll
  for (int kk = 0; kk < KSTEPS; ++kk)
    ldsm_x4(q_frag[kk], q_s + (lane & 15) * ROW + kk * 16 + (lane >> 4) * 8);

  float o[NTILES_D][4];
#pragma unroll
  for (int i = 0; i < NTILES_D; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
  const int t4 = lane & 3;

  // A copy that did not arrive in time has set the error bit.  Before the CTA gives up the shared
  // memory that copies still in flight target, every one of them gets one more bounded wait: the
  // tiles from `it` on that were asked for, each on its stage and parity.
  auto drain = [&](int it, int stage, uint32_t phases) {
    for (int j = 0; j < stages && it + j < tiles; ++j) {
      int slot = stage + j;
      if (slot >= stages) slot -= stages;
      mbar_wait(&full[slot], (phases >> slot) & 1u, a.err);
    }
  };
  int stage = 0, failed_at = -1, failed_stage = 0;
  uint32_t phases = 0;   // bit s: the parity to wait for on stage s
  for (int it = 0; it < tiles; ++it) {
    const uint32_t parity = (phases >> stage) & 1u;
    const bool landed = mbar_wait(&full[stage], parity, a.err);
    if (it == 0) SPLIT_MARK(3);
    const int k0 = begin + it * SPLIT_TILE + warp * DN;      // this warp's 16 keys of the stage
    if (landed && k0 < end) {
      const bf16* k_tile = ring + stage * SPLIT_STAGE + warp * SPLIT_BLOCK;
      const bf16* v_tile = k_tile + SPLIT_WARPS * SPLIT_BLOCK;
      float s[DN / 8][4];
      scores<DN / 16, true>(q_frag, k_tile, s, lane);
      if (k0 >= first && k0 + DN <= end) {
#pragma unroll
        for (int i = 0; i < DN / 8; ++i)
#pragma unroll
          for (int e = 0; e < 4; ++e) s[i][e] *= a.scale_log2;
      } else {
#pragma unroll
        for (int i = 0; i < DN / 8; ++i)
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int key = k0 + i * 8 + 2 * t4 + (e & 1);
            s[i][e] = (key >= first && key < end) ? s[i][e] * a.scale_log2 : -INFINITY;
          }
      }
      if (a.group - h0 <= 8) softmax_update<DN / 8, 1>(s, m, l, o);
      else softmax_update<DN / 8, 2>(s, m, l, o);
      accumulate<DN / 16, true>(s, v_tile, o, lane);
    }
    if (it + stages < tiles) {
      // everybody is done with the stage (and agrees on whether its copies arrived) before it is refilled
      if (!__syncthreads_and(landed)) {
        if (tid == 0) drain(it, stage, phases);
        return;
      }
      if (warp == 0) issue(it + stages, 1, stage);
    } else if (!landed) {
      // nothing is refilled any more, so no barrier lies ahead in the loop: leave it, and find out
      // together below
      failed_at = it;
      failed_stage = stage;
      break;
    }
    phases ^= 1u << stage;
    if (++stage == stages) stage = 0;
  }
  SPLIT_MARK(4);

  // ---- merge the warps.  Each warp puts its row maxima and sums down; then everybody knows the
  // CTA's maxima, scales its own outputs to them in registers and puts them down too ([warp][16][D],
  // the ring is free by then); the sums over the warps are formed while the share is written.
  const int g = lane >> 2;
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const float total = quad_sum(l[h]);
    if (t4 == 0) {
      warp_max_s[warp][g + h * 8] = m[h];
      warp_sum_s[warp][g + h * 8] = total;
    }
  }
  // (this barrier lies behind every warp's last use of the ring, which the merge buffers reuse)
  if (!__syncthreads_and(failed_at < 0)) {
    if (tid == 0 && failed_at >= 0) drain(failed_at, failed_stage, phases);
    return;
  }
  float scale_mine[2];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int r = g + h * 8;
    float m_all = -INFINITY;
#pragma unroll
    for (int w = 0; w < SPLIT_WARPS; ++w) m_all = fmaxf(m_all, warp_max_s[w][r]);
    scale_mine[h] = (m[h] == -INFINITY) ? 0.f : exp2f(m[h] - m_all);
  }
  float* my_merge = merge_s + warp * 16 * D;
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int r = g + h * 8;
#pragma unroll
    for (int i = 0; i < NTILES_D; ++i)
      *reinterpret_cast<float2*>(my_merge + r * D + i * 8 + 2 * t4) =
          make_float2(o[i][2 * h] * scale_mine[h], o[i][2 * h + 1] * scale_mine[h]);
  }
  __syncthreads();
  const int unit = request * gridDim.x + blockIdx.x;
  const int shares_per_unit = a.splits / a.cluster;
  float* unit_shares = a.shares + (size_t)unit * shares_per_unit * SPLIT_SHARE;
  float* cluster_share = unit_shares + (size_t)cluster_index * SPLIT_SHARE;
  bf16* out_rows = a.out + (size_t)request * a.out_stride + (size_t)(kvh * a.group + h0) * D;
  const bool exchange = kCluster && peers > 1;
  // the rows this CTA owns, from itself: [rows_per_owner][SPLIT_SHARE_ROW] behind the warps' blocks
  float* own_s = merge_s + SPLIT_WARPS * 16 * D;
  if (exchange) cluster_wait();   // every CTA of the cluster has set its inbox up (they said so when they started)

  // this CTA's share: every thread takes four columns of one head row and adds the warps up
  for (int idx = tid; idx < live_rows * (D / 4); idx += SPLIT_WARPS * 32) {
    const int r = idx / (D / 4), c4 = idx % (D / 4);
    float4 acc = *reinterpret_cast<const float4*>(merge_s + r * D + c4 * 4);
#pragma unroll
    for (int w = 1; w < SPLIT_WARPS; ++w) {
      const float4 part = *reinterpret_cast<const float4*>(merge_s + (w * 16 + r) * D + c4 * 4);
      acc.x += part.x; acc.y += part.y; acc.z += part.z; acc.w += part.w;
    }
    float m_all = -INFINITY;
#pragma unroll
    for (int w = 0; w < SPLIT_WARPS; ++w) m_all = fmaxf(m_all, warp_max_s[w][r]);
    float sum = 0.f;
#pragma unroll
    for (int w = 0; w < SPLIT_WARPS; ++w) {
      const float mw = warp_max_s[w][r];
      sum += warp_sum_s[w][r] * ((mw == -INFINITY) ? 0.f : exp2f(mw - m_all));
    }
    if (exchange) {
      const int owner = r % peers, local = r / peers;
      if (owner == rank) {
        float* mine = own_s + local * SPLIT_SHARE_ROW;
        *reinterpret_cast<float4*>(mine + c4 * 4) = acc;
        if (c4 == 0) { mine[D] = m_all; mine[D + 1] = sum; }
      } else {
        // the owner keeps the shares of its peers in the order of their ranks, itself left out
        const int slot = rank < owner ? rank : rank - 1;
        const float* theirs = inbox + (size_t)(slot * rows_per_owner + local) * SPLIT_SHARE_ROW;
        const uint32_t bar = map_to_rank(&inbox_bar, owner);
        push_f4(map_to_rank(theirs + c4 * 4, owner), acc, bar);
        if (c4 == 0) push_f2(map_to_rank(theirs + D, owner), m_all, sum, bar);
      }
    } else if (clusters_used == 1) {   // the request is this CTA's alone: the output itself
      const float inv = sum > 0.f ? 1.f / sum : 0.f;
      uint2 packed;
      packed.x = pack_bf16(acc.x * inv, acc.y * inv);
      packed.y = pack_bf16(acc.z * inv, acc.w * inv);
      *reinterpret_cast<uint2*>(out_rows + (size_t)r * D + c4 * 4) = packed;
    } else {
      __stcg(reinterpret_cast<float4*>(cluster_share + r * SPLIT_SHARE_ROW + c4 * 4), acc);
      if (c4 == 0) {
        __stcg(cluster_share + r * SPLIT_SHARE_ROW + D, m_all);
        __stcg(cluster_share + r * SPLIT_SHARE_ROW + D + 1, sum);
      }
    }
  }
  if (!exchange && clusters_used == 1) return;
  if (exchange) {
    if (rows_owned == 0) return;          // more CTAs than head rows: nothing to finish here
    __syncthreads();                      // this CTA's own rows are in own_s
    if (!mbar_wait(&inbox_bar, 0, a.err)) return;   // and its peers' shares of them in the inbox
    // the rows this CTA owns: its own share and its peers', in the order of their ranks
    for (int idx = tid; idx < rows_owned * (D / 4); idx += SPLIT_WARPS * 32) {
      const int local = idx / (D / 4), c4 = idx % (D / 4);
      const int r = local * peers + rank;
      float m_all = -INFINITY, sum = 0.f;
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int peer = 0; peer < peers; ++peer) {
        const float* share = peer == rank ? own_s + local * SPLIT_SHARE_ROW
                                          : inbox + (size_t)((peer < rank ? peer : peer - 1) * rows_per_owner + local) * SPLIT_SHARE_ROW;
        const float m_theirs = share[D], sum_theirs = share[D + 1];
        const float4 part = *reinterpret_cast<const float4*>(share + c4 * 4);
        const float m_new = fmaxf(m_all, m_theirs);
        const float keep = (m_all == -INFINITY) ? 0.f : exp2f(m_all - m_new);
        const float take = (m_theirs == -INFINITY) ? 0.f : exp2f(m_theirs - m_new);
        sum = sum * keep + sum_theirs * take;
        acc.x = acc.x * keep + part.x * take; acc.y = acc.y * keep + part.y * take;
        acc.z = acc.z * keep + part.z * take; acc.w = acc.w * keep + part.w * take;
        m_all = m_new;
      }
      if (clusters_used == 1) {
        const float inv = sum > 0.f ? 1.f / sum : 0.f;
        uint2 packed;
        packed.x = pack_bf16(acc.x * inv, acc.y * inv);
        packed.y = pack_bf16(acc.z * inv, acc.w * inv);
        *reinterpret_cast<uint2*>(out_rows + (size_t)r * D + c4 * 4) = packed;
      } else {
        __stcg(reinterpret_cast<float4*>(cluster_share + r * SPLIT_SHARE_ROW + c4 * 4), acc);
        if (c4 == 0) {
          __stcg(cluster_share + r * SPLIT_SHARE_ROW + D, m_all);
          __stcg(cluster_share + r * SPLIT_SHARE_ROW + D + 1, sum);
        }
      }
    }
    if (clusters_used == 1) return;
  }
  // ---- several clusters share the unit: every CTA that wrote rows of its cluster's share draws a
  // ticket; whoever draws the last one adds the clusters' shares up
  int writers = 0;
  for (int c = 0; c < clusters_used; ++c) {
    const int in_cluster = min(a.cluster, used - c * a.cluster);
    writers += kCluster && in_cluster > 1 ? min(in_cluster, live_rows) : 1;
  }
  SPLIT_MARK(5);
  __threadfence();   // this thread's part of the share is visible before the ticket is drawn
  __syncthreads();
  if (tid == 0) last_s = atomicAdd(&a.tickets[unit], 1) == writers - 1;
  __syncthreads();
  SPLIT_MARK(6);
  if (!last_s) return;
  __threadfence();
  merge_shares(unit_shares, clusters_used, out_rows, live_rows, tid);
  if (tid == 0) a.tickets[unit] = 0;   // ready for the next launch
  SPLIT_MARK(7);
}

// ------------------------------------------------------------------------------------ tensor maps
}  // namespace cie

using namespace cie;

static const float kLog2e = 1.4426950408889634f;

extern "C" int cie_attention_head_dim() { return D; }

extern "C" int cie_attention_prefill(const void* q, int q_stride, void* out, int out_stride,
                                     const void* k_pool, const void* v_pool, const int* table,
                                     int table_width, int num_pages, const int* tile_request,
                                     const int* tile_q0, int num_tiles, const int* context_lens,
                                     const int* query_lens, const int* query_start, int q_heads,
                                     int kv_heads, int page_size, int hpt, float scale, int window,
                                     int* err, void* stream) {
  if (num_tiles <= 0) return 0;
  if (kv_heads < 1 || q_heads % kv_heads) CIE_FAIL("attention_prefill: %d query heads over %d kv heads", q_heads, kv_heads);
  const int group = q_heads / kv_heads;
  if (hpt < 1 || hpt > BM || hpt > group) CIE_FAIL("attention_prefill: %d heads per tile with a group of %d", hpt, group);
  if (q_stride % 8 || out_stride % 2) CIE_FAIL("attention_prefill: row strides must keep 16-byte alignment");
  PrefillArgs a;
  a.q = (const bf16*)q; a.q_stride = q_stride; a.out = (bf16*)out; a.out_stride = out_stride;
  a.pools = Pools{(const bf16*)k_pool, (const bf16*)v_pool, table, table_width, num_pages, kv_heads, page_size};
  a.tile_request = tile_request; a.tile_q0 = tile_q0; a.context_lens = context_lens;
  a.query_lens = query_lens; a.query_start = query_start;
  a.group = group; a.hpt = hpt; a.tpt = BM / hpt; a.head_chunks = (group + hpt - 1) / hpt;
  a.scale_log2 = scale * kLog2e; a.window = window; a.err = err;
  const size_t smem = (size_t)(BM + 4 * BN) * ROW * sizeof(bf16);
  static bool configured = false;
  if (!configured) {
    cudaError_t status = cudaFuncSetAttribute(prefill_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (status != cudaSuccess) CIE_FAIL("attention_prefill: shared memory %zu: %s", smem, cudaGetErrorString(status));
    configured = true;
  }
  dim3 grid(num_tiles, kv_heads * a.head_chunks);
  CIE_LAUNCH("attention_prefill", prefill_kernel, grid, dim3(PREFILL_WARPS * 32), smem, (cudaStream_t)stream, a);
  return 0;
}

// splits: CTAs that share the keys of one request (a thread-block cluster): 1, 2, 4 or 8.
// chunks: clusters launched per request (1 .. 16); a request uses as many of them as leave each
// of its CTAs `chunk_keys` keys.  More than one needs `partials`, float32
// [requests * kv_heads * ceil(group / 16)][chunks][16][head size + 2], and `counters`, one int per
// (request, kv head, 16 heads) that is zero before the first launch (the kernel leaves it zero).
// use_tma: 1 lets the kernel fetch keys and values with tensor copies where the shapes allow it
// (pages of a multiple of 16 tokens, head size a multiple of 64, no window); 0 keeps cp.async.
template <bool kTma>
static int launch_decode(const CUtensorMap& k_map, const CUtensorMap& v_map, const DecodeArgs& a,
                         int requests, cudaStream_t stream) {
  constexpr size_t smem = decode_smem<kTma>();
  static bool configured = false;
  if (!configured) {
    cudaError_t status = cudaFuncSetAttribute(decode_kernel<kTma>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (status != cudaSuccess) CIE_FAIL("attention_decode: shared memory %zu: %s", smem, cudaGetErrorString(status));
    configured = true;
  }
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3(a.splits * a.chunks, a.pools.kv_heads * a.head_chunks, requests);
  config.blockDim = dim3(DECODE_WARPS * 32);
  config.dynamicSmemBytes = smem;
  config.stream = stream;
  cudaLaunchAttribute attributes[2];
  int count = 0;
  attributes[count].id = cudaLaunchAttributeClusterDimension;
  attributes[count].val.clusterDim.x = a.splits;
  attributes[count].val.clusterDim.y = 1;
  attributes[count].val.clusterDim.z = 1;
  ++count;
  if (pdl_enabled()) {
    attributes[count].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attributes[count].val.programmaticStreamSerializationAllowed = 1;
    ++count;
  }
  config.attrs = attributes;
  config.numAttrs = count;
  cudaError_t status = cudaLaunchKernelEx(&config, decode_kernel<kTma>, k_map, v_map, a);
  if (status != cudaSuccess) CIE_FAIL("attention_decode: launch failed: %s", cudaGetErrorString(status));
  return 0;
}

// How many clusters of `splits` CTAs of the decode kernel the device runs at one time (a cluster
// stays inside one GPC and a CTA takes most of an SM's shared memory); -1 if the query fails.
template <bool kTma>
static int decode_clusters_at_once(int splits) {
  constexpr size_t smem = decode_smem<kTma>();
  if (cudaFuncSetAttribute(decode_kernel<kTma>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) return -1;
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3(splits, 1, 1);
  config.blockDim = dim3(DECODE_WARPS * 32);
  config.dynamicSmemBytes = smem;
  cudaLaunchAttribute attribute;
  attribute.id = cudaLaunchAttributeClusterDimension;
  attribute.val.clusterDim.x = splits;
  attribute.val.clusterDim.y = 1;
  attribute.val.clusterDim.z = 1;
  config.attrs = &attribute;
  config.numAttrs = 1;
  int clusters = 0;
  if (cudaOccupancyMaxActiveClusters(&clusters, decode_kernel<kTma>, &config) != cudaSuccess) {
    cudaGetLastError();
    return -1;
  }
  return clusters;
}

extern "C" int cie_attention_decode_clusters(int splits, int use_tma) {
  if (splits != 1 && splits != 2 && splits != 4 && splits != 8) return -1;
  return use_tma && D % 64 == 0 ? decode_clusters_at_once<true>(splits) : decode_clusters_at_once<false>(splits);
}

extern "C" int cie_attention_decode(const void* q, int q_stride, void* out, int out_stride,
                                    const void* k_pool, const void* v_pool, const int* table,
                                    int table_width, int num_pages, const int* context_lens,
                                    int requests, int q_heads, int kv_heads, int page_size,
                                    int splits, int chunks, int chunk_keys, float* partials, int* counters, float scale,
                                    int window, int use_tma, int* err, void* stream) {
  if (requests <= 0) return 0;
  if (kv_heads < 1 || q_heads % kv_heads) CIE_FAIL("attention_decode: %d query heads over %d kv heads", q_heads, kv_heads);
  if (splits != 1 && splits != 2 && splits != 4 && splits != 8) CIE_FAIL("attention_decode: splits must be 1, 2, 4 or 8, got %d", splits);
  if (q_stride % 8) CIE_FAIL("attention_decode: row stride must keep 16-byte alignment");
  if (chunks < 1 || chunks > DECODE_MAX_CHUNKS) CIE_FAIL("attention_decode: 1 to %d clusters per request, got %d", DECODE_MAX_CHUNKS, chunks);
  if (chunks > 1 && (!partials || !counters || chunk_keys < 1)) CIE_FAIL("attention_decode: several clusters per request need scratch memory and a least number of keys per CTA");
  DecodeArgs a;
  a.q = (const bf16*)q; a.q_stride = q_stride; a.out = (bf16*)out; a.out_stride = out_stride;
  a.pools = Pools{(const bf16*)k_pool, (const bf16*)v_pool, table, table_width, num_pages, kv_heads, page_size};
  a.context_lens = context_lens; a.group = q_heads / kv_heads; a.head_chunks = (a.group + 15) / 16;
  a.splits = splits; a.chunks = chunks; a.chunk_keys = chunk_keys; a.partials = partials; a.counters = counters; a.scale_log2 = scale * kLog2e; a.window = window; a.q_heads = q_heads; a.err = err;
  a.page_shift = -1;
  for (int shift = 0; shift < 31; ++shift)
    if ((1 << shift) == page_size) a.page_shift = shift;
  CUtensorMap k_map = {}, v_map = {};
  const bool tma = use_tma && D % 64 == 0 && window <= 0 && a.page_shift >= 4 &&
                   ((reinterpret_cast<uintptr_t>(k_pool) | reinterpret_cast<uintptr_t>(v_pool)) & 15) == 0;
  if (tma) {
    const long long rows = (long long)num_pages * kv_heads * page_size;
    const bool mapped = kBlockCopies
        ? bw::tensor_map_bf16_row_blocks(k_pool, rows, D, 16, &k_map) && bw::tensor_map_bf16_row_blocks(v_pool, rows, D, 16, &v_map)
        : bw::tensor_map_bf16(k_pool, rows, D, 16, &k_map) && bw::tensor_map_bf16(v_pool, rows, D, 16, &v_map);
    if (!mapped)
      CIE_FAIL("attention_decode: cuTensorMapEncodeTiled failed");
    return launch_decode<true>(k_map, v_map, a, requests, (cudaStream_t)stream);
  }
  return launch_decode<false>(k_map, v_map, a, requests, (cudaStream_t)stream);
}

// How many CTAs of the split decode kernel with a ring of `stages` stages, clusters of `cluster`
// CTAs and `rows` head rows a unit fit one SM (its shared memory decides); 0 if the head size is not its kind or the sizes are
// out of range, -1 on failure.
template <bool kCluster>
static int split_ctas_per_sm(int stages, int cluster, int rows) {
  const size_t smem = split_smem(stages, cluster, rows);
  if (cudaFuncSetAttribute(decode_split_kernel<kCluster>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  int ctas = 0;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&ctas, decode_split_kernel<kCluster>, SPLIT_WARPS * 32, smem) != cudaSuccess) {
    cudaGetLastError();
    return -1;
  }
  return ctas;
}

// rows: head rows of a unit (query heads per kv head, at most 16)
extern "C" int cie_attention_decode_split_ctas_per_sm(int stages, int cluster, int rows) {
  if (D % 64 || stages < SPLIT_MIN_STAGES || stages > SPLIT_MAX_STAGES || cluster < 1 || cluster > 16 || rows < 1 || rows > 16) return 0;
  return cluster > 1 ? split_ctas_per_sm<true>(stages, cluster, rows) : split_ctas_per_sm<false>(stages, 1, rows);
}

// How many clusters of `cluster` CTAs of the split decode kernel the device runs at one time with a
// ring of `stages` stages and `rows` head rows a unit (a cluster stays inside one GPC); -1 if the
// query fails, 0 if the sizes are not the kernel's.
extern "C" int cie_attention_decode_split_clusters(int stages, int cluster, int rows) {
  if (D % 64 || stages < SPLIT_MIN_STAGES || stages > SPLIT_MAX_STAGES || rows < 1 || rows > 16) return 0;
  if (cluster != 2 && cluster != 4 && cluster != 8 && cluster != 16) return 0;
  const size_t smem = split_smem(stages, cluster, rows);
  if (cudaFuncSetAttribute(decode_split_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess ||
      (cluster > 8 && cudaFuncSetAttribute(decode_split_kernel<true>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1) != cudaSuccess)) {
    cudaGetLastError();
    return -1;
  }
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3(1, 1, cluster);
  config.blockDim = dim3(SPLIT_WARPS * 32);
  config.dynamicSmemBytes = smem;
  cudaLaunchAttribute attribute;
  attribute.id = cudaLaunchAttributeClusterDimension;
  attribute.val.clusterDim.x = 1;
  attribute.val.clusterDim.y = 1;
  attribute.val.clusterDim.z = cluster;
  config.attrs = &attribute;
  config.numAttrs = 1;
  int clusters = 0;
  if (cudaOccupancyMaxActiveClusters(&clusters, decode_split_kernel<true>, &config) != cudaSuccess) {
    cudaGetLastError();
    return -1;
  }
  return clusters;
}

extern "C" int cie_attention_decode_split_max() { return SPLIT_MAX; }
extern "C" int cie_attention_decode_split_tile() { return SPLIT_TILE; }

#ifdef SPLIT_TRACE
extern "C" int cie_attention_decode_split_trace(void* buffer) {
  return cudaMemcpyToSymbol(g_split_trace, &buffer, sizeof(buffer)) == cudaSuccess ? 0 : 1;
}
#endif

// The split decode kernel.  splits: CTAs launched per (request, kv head, 16 heads) unit, 1 ..
// cie_attention_decode_split_max(); a request uses as many of them as leave each `min_keys` keys.
// cluster: 1, 2, 4, 8 or 16 neighbouring splits of a unit form a thread-block cluster and hand their
// shares to its first CTA through shared memory (splits must be a multiple of it).
// shares: float32 [requests * kv_heads * ceil(group / 16)][splits][16][head size + 4]; tickets: one
// int per unit, zero before the first launch (the kernel leaves them zero).  Needs pages of a power
// of two >= 16 tokens, a head size that is a multiple of 64 and 16-byte-aligned pools (the caller
// checks and takes the other decode kernel where that does not hold).
extern "C" int cie_attention_decode_split(const void* q, int q_stride, void* out, int out_stride,
                                          const void* k_pool, const void* v_pool, const int* table,
                                          int table_width, int num_pages, const int* context_lens,
                                          int requests, int q_heads, int kv_heads, int page_size,
                                          int splits, int min_keys, int stages, int cluster, float* shares,
                                          int* tickets, float scale, int window, int* err, void* stream) {
  if (requests <= 0) return 0;
  if (kv_heads < 1 || q_heads % kv_heads) CIE_FAIL("attention_decode_split: %d query heads over %d kv heads", q_heads, kv_heads);
  if (splits < 1 || splits > SPLIT_MAX) CIE_FAIL("attention_decode_split: 1 to %d CTAs per request, got %d", SPLIT_MAX, splits);
  if (q_stride % 8) CIE_FAIL("attention_decode_split: row stride must keep 16-byte alignment");
  if (min_keys < 1) CIE_FAIL("attention_decode_split: min_keys must be positive");
  if (stages < SPLIT_MIN_STAGES || stages > SPLIT_MAX_STAGES)
    CIE_FAIL("attention_decode_split: %d to %d stages, got %d", SPLIT_MIN_STAGES, SPLIT_MAX_STAGES, stages);
  if (cluster != 1 && cluster != 2 && cluster != 4 && cluster != 8 && cluster != 16)
    CIE_FAIL("attention_decode_split: clusters of 1, 2, 4, 8 or 16 CTAs, got %d", cluster);
  if (splits % cluster) CIE_FAIL("attention_decode_split: %d CTAs per request are no multiple of the cluster size %d", splits, cluster);
  if (splits > cluster && (!shares || !tickets)) CIE_FAIL("attention_decode_split: several clusters per request need scratch memory");
  int page_shift = -1;
  for (int shift = 0; shift < 31; ++shift)
    if ((1 << shift) == page_size) page_shift = shift;
  if (D % 64 || page_shift < 4 ||
      ((reinterpret_cast<uintptr_t>(k_pool) | reinterpret_cast<uintptr_t>(v_pool)) & 15) != 0)
    CIE_FAIL("attention_decode_split: needs head size %% 64 == 0 (got %d), pages of a power of two >= 16 "
             "(got %d) and 16-byte-aligned pools", D, page_size);
  SplitArgs a;
  a.q = (const bf16*)q; a.q_stride = q_stride; a.out = (bf16*)out; a.out_stride = out_stride;
  a.pools = Pools{(const bf16*)k_pool, (const bf16*)v_pool, table, table_width, num_pages, kv_heads, page_size};
  a.context_lens = context_lens; a.group = q_heads / kv_heads; a.head_chunks = (a.group + 15) / 16;
  a.page_shift = page_shift; a.splits = splits; a.min_keys = min_keys; a.stages = stages; a.cluster = cluster;
  a.shares = shares; a.tickets = tickets;
  a.scale_log2 = scale * kLog2e; a.window = window; a.err = err;
  CUtensorMap k_map = {}, v_map = {};
  const long long rows = (long long)num_pages * kv_heads * page_size;
  const bool mapped = kBlockCopies
      ? bw::tensor_map_bf16_row_blocks(k_pool, rows, D, 16, &k_map) && bw::tensor_map_bf16_row_blocks(v_pool, rows, D, 16, &v_map)
      : bw::tensor_map_bf16(k_pool, rows, D, 16, &k_map) && bw::tensor_map_bf16(v_pool, rows, D, 16, &v_map);
  if (!mapped) CIE_FAIL("attention_decode_split: cuTensorMapEncodeTiled failed");
  const size_t smem = split_smem(stages, cluster, a.group < 16 ? a.group : 16);
  static size_t configured[2] = {0, 0};
  const int variant = cluster > 1 ? 1 : 0;
  if (smem > configured[variant]) {
    cudaError_t status = variant
        ? cudaFuncSetAttribute(decode_split_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)
        : cudaFuncSetAttribute(decode_split_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (status != cudaSuccess) CIE_FAIL("attention_decode_split: shared memory %zu: %s", smem, cudaGetErrorString(status));
    configured[variant] = smem;
  }
  if (cluster > 8) {
    // clusters of more than 8 CTAs need the kernel's consent
    static bool allowed = false;
    if (!allowed) {
      cudaError_t status = cudaFuncSetAttribute(decode_split_kernel<true>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
      if (status != cudaSuccess) CIE_FAIL("attention_decode_split: clusters of %d: %s", cluster, cudaGetErrorString(status));
      allowed = true;
    }
  }
  if (requests > 65535) CIE_FAIL("attention_decode_split: at most 65535 requests a launch, got %d", requests);
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3(kv_heads * a.head_chunks, requests, splits);
  config.blockDim = dim3(SPLIT_WARPS * 32);
  config.dynamicSmemBytes = smem;
  config.stream = (cudaStream_t)stream;
  cudaLaunchAttribute attributes[2];
  int count = 0;
  if (cluster > 1) {
    attributes[count].id = cudaLaunchAttributeClusterDimension;
    attributes[count].val.clusterDim.x = 1;
    attributes[count].val.clusterDim.y = 1;
    attributes[count].val.clusterDim.z = cluster;
    ++count;
  }
  if (pdl_enabled()) {
    attributes[count].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attributes[count].val.programmaticStreamSerializationAllowed = 1;
    ++count;
  }
  config.attrs = attributes;
  config.numAttrs = count;
  cudaError_t status = cluster > 1 ? cudaLaunchKernelEx(&config, decode_split_kernel<true>, k_map, v_map, a)
                                   : cudaLaunchKernelEx(&config, decode_split_kernel<false>, k_map, v_map, a);
  if (status != cudaSuccess) CIE_FAIL("attention_decode_split: launch failed: %s", cudaGetErrorString(status));
  return 0;
}
