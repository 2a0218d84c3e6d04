// A decode step's matrix products and attention as ONE persistent kernel that runs a list of phases.
//
// A decode step of a few tokens is bound by reading every weight once, and between two of its
// kernels the memory system drains and fills again: a launch, a ramp, a tail, five times a layer.
// Here the host writes the step down as a list of phases (a "program": q/k/v product with rotary
// epilogue, attention over the pages, output projection into the residual stream, gate/up product
// with SiLU, down projection, layer after layer) and one kernel with one CTA per SM walks the list.
// Between phases the CTAs meet at a barrier in global memory; the weight stream does not stop
// there:
//
//  * warp 0 of a CTA is the producer.  It walks the CTA's share of every phase in order and pulls
//    what the phase reads from HBM (weight tiles, key and value tiles) through one ring of 16 KB
//    stages with TMA copies that complete on the stage's mbarrier.  Weights and the keys and
//    values of earlier steps do not depend on anything the step computes, so the producer runs
//    ahead across phase boundaries, as far as the ring has room: while the consumers wait at a
//    barrier or for their input rows, the next phases' bytes are already arriving.  Only a stage
//    that holds a key written by this step (the newest token's) waits for the phase that writes it.
//  * warps 1..4 are the consumers.  For a product they take one 64-column box of a stage each
//    ([32 weight rows x 256 columns] per stage), with the token rows as the 8-wide operand of
//    mma.sync m16n8k16 read straight from global memory (L2) into registers one stage ahead; at
//    the end of a tile they add their four slices up in shared memory and run the epilogue
//    (rotary + cache write, residual add + sums of squares + pre-scaled rows, SiLU * up, plain).
//    A product with few weight rows and a long K is cut along K over the CTAs; its partial sums
//    go to global memory and a short "finish" phase adds them up in a fixed order and runs the
//    epilogue.  For attention a CTA takes a range of one request's keys (64-key tiles, the warps
//    16 keys each), leaves an unnormalised share, and a short "merge" phase joins the shares.
//
// Everything a phase reads that another CTA wrote earlier in the same kernel is read past L1
// (ld.global.cg, cp.async.cg, TMA); the barrier between phases is a release/acquire counter.
// Every wait is bounded: one that runs out sets the time-out bit of the error word, after which the
// CTA stops waiting and runs to its end (its results are void), so the kernel always returns.
//
// The reference runs a decode step as separate library and Triton kernels per projection
// (zeeshan8281/cloud-inference-from-scratch src/cloud_engine/model.py:86-100,132-137,212-227;
// kernel.py:324-405); the formulas are the same, the arrangement is this engine's.
#include "attention_tiles.cuh"
#include "blackwell.cuh"
#include "common.cuh"

#include <cuda.h>

CIE_DEFINE_LAST_ERROR()

namespace cie {

#ifndef PG_GROUPS
#define PG_GROUPS 2
#endif
constexpr int PG_BOXES = 4;                       // warps that share a stage: one 64-column box (or 16 keys) each
constexpr int PG_CONSUMERS = PG_BOXES * PG_GROUPS;   // groups of four warps take the stages in turn
constexpr int PG_THREADS = 32 * (1 + PG_CONSUMERS);
constexpr int PG_STAGE_BYTES = 16384;
constexpr int PG_MAX_STAGES = 12;
constexpr int PG_KC = 256;          // K columns of a stage: four boxes of 64
constexpr int PG_BN = 32;           // weight rows of a tile
constexpr int PG_TILE_KEYS = 64;    // keys of an attention tile: four blocks of 16
constexpr int PG_BLOCK_BYTES = 16 * D * 2;                  // one 16-key block of K (or V)
constexpr int PG_KEY_STAGES = (2 * PG_TILE_KEYS * D * 2) / PG_STAGE_BYTES;   // stages of a tile: K and V
constexpr int PG_RED_ROW = PG_BN + 1;
constexpr int PG_RED_BYTES = (PG_CONSUMERS * 16 * PG_RED_ROW * 4 + 1023) / 1024 * 1024;   // [warp][16 tokens][33]
constexpr int PG_MERGE_BYTES = PG_BOXES * 16 * D * 4;                          // [warp of a group][16 heads][D]
// Shared memory behind the ring: the sums' buffer of the products, then a region that holds the token
// rows of a product (the "slab": [64-column group][8 or 16 rows][128 bytes], sized by the launch) or,
// in an attention phase, the merge buffer.
constexpr int region_bytes(int slab_bytes) {
  return ((slab_bytes > PG_MERGE_BYTES ? slab_bytes : PG_MERGE_BYTES) + 1023) / 1024 * 1024;
}
constexpr int PG_Q_BYTES = 16 * ROW * 2;
constexpr int PG_SHARE_ROW = D + 4;                          // floats of a share's row: outputs, maximum, sum, padding
constexpr int PG_MAX_KEY_SPLITS = 64;
static_assert(D == 64 || D == 128, "the decode program is built for head sizes 64 and 128");
static_assert(PG_KEY_STAGES == 1 || PG_KEY_STAGES == 2, "a key tile is one or two stages");
static_assert(16 % PG_CONSUMERS == 0 || PG_CONSUMERS > 16, "the merge phase gives a unit's 16 head rows to whole groups of warps");

enum : int { kEnd = 0, kGemm = 1, kFinish = 2, kAttention = 3, kMerge = 4 };
constexpr int kOutBF16 = 0, kOutF32 = 1, kOutSiluMul = 3, kOutResidual = 4, kOutRope = 5;

// One phase of the program.  The host fills it (cie_program_* below); the kernel reads it from
// global memory.  Fields a kind does not use are zero.
struct alignas(128) Phase {
  CUtensorMap map0;   // product: the weight [N, K] in boxes of [32 rows x 64 columns]; attention: the key pool
  CUtensorMap map1;   // attention: the value pool
  int kind;
  int m;              // token rows of a product; requests of an attention phase
  // ---- product and its finish
  int n, k;
  int row_tiles;      // ceil(N / 32)
  int chunks;         // ceil(K / 256)
  int splits;         // slices of K, each a unit of its own; > 1: partial sums, a finish phase follows
  int mode;           // epilogue (kOut...)
  const bf16* x;      // [m, x_stride]
  int x_stride;
  const float* row_sq;   // [m, sq_tiles] sums of squares of the rows x was made from, or null
  int sq_tiles;
  float eps;
  const float* bias;
  void* out;          // kOutBF16 / kOutF32: [m, n]; kOutSiluMul: bf16 [m, n / 2]
  float* partial;     // [splits][m][n]
  float* residual;    // kOutResidual: [m, n] float32, added into
  float* sq;          // kOutResidual: [m, row_tiles] sums of squares of the new rows per 32 columns
  bf16* scaled;       // kOutResidual, optional: bf16(new row * next_gain)
  const float* next_gain;
  bf16* q_out;        // kOutRope: rotated q [m, q_stride]; attention: the queries
  int q_stride;
  const int* positions;
  const int* request_of_token;
  const int* table;   // [requests][table_width]
  int table_width, num_pages;
  bf16* k_pool;       // [pages][kv_heads][page_size][dim]
  bf16* v_pool;
  const float* inv_freq;
  int q_heads, kv_heads, dim, rot, page_size, write_cache;
  // ---- attention and its merge
  bf16* attn_out;     // [requests, out_stride]
  int out_stride;
  const int* context_lens;   // keys before the query token
  int group, head_chunks, page_shift;
  int key_splits;     // CTAs a unit (request, kv head, 16 heads) may use
  int min_keys;       // a request uses only as many of them as leave each this many keys
  int window;
  float scale_log2;
  float* shares;      // [unit][key_splits][16][D + 4]
};

struct ProgramShared {
  uint64_t full[PG_MAX_STAGES];
  uint64_t empty[PG_MAX_STAGES];
  float rstd[16];
  float warp_max[PG_CONSUMERS][16];
  float warp_sum[PG_CONSUMERS][16];
  volatile int epoch;   // barriers between phases that this CTA has passed
  volatile int dead;    // a wait ran out somewhere in this CTA
};

// Diagnostics: with a buffer set (cie_program_set_trace) the first consumer thread of every CTA leaves
// the global timer when it begins a phase (0), at two points inside it (2, 3: a product's token rows are
// in shared memory; its last stage is multiplied) and when it has done its share of it (1).
__device__ long long* g_program_trace = nullptr;
__device__ int g_program_trace_phases = 0;
__device__ __forceinline__ void trace_mark(int phase, int which, int ctid) {
  if (ctid == 0 && g_program_trace && phase < g_program_trace_phases) {
    long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    g_program_trace[((size_t)phase * gridDim.x + blockIdx.x) * 4 + which] = t;
  }
}

#ifdef PROGRAM_PROBE
// Debug builds only (-DPROGRAM_PROBE): the first consumer warp of one CTA leaves the clock around
// every stage it multiplies (before the wait, after it, after the stage is given back).
__device__ long long* g_program_probe = nullptr;
__device__ int g_program_probe_cta = 0;
__device__ int g_program_probe_slots = 0;
__device__ int g_program_probe_used = 0;
#define PROBE_DECLARE() long long probe_t[8] = {0, 0, 0, 0, 0, 0, 0, 0}
#define PROBE_AT(i) probe_t[i] = clock64()
#define PROBE_STORE()                                                                             \
  if (g_program_probe && (int)blockIdx.x == g_program_probe_cta && c.cw == 0 && lane == 0 &&      \
      g_program_probe_used < g_program_probe_slots) {                                             \
    const int at = g_program_probe_used++;                                                        \
    for (int i = 0; i < 8; ++i) g_program_probe[at * 8 + i] = probe_t[i];                         \
  }
#else
#define PROBE_DECLARE()
#define PROBE_AT(i)
#define PROBE_STORE()
#endif

constexpr long long kWaitCycles = 4000000000ll;    // about two seconds
constexpr long long kDrainCycles = 200000000ll;    // about a tenth of a second, per stage, at the very end

__device__ __forceinline__ bool wait_bar(uint64_t* bar, uint32_t parity, long long cycles, int* err) {
  if (bw::mbar_try_wait(bar, parity)) return true;
  const long long start = clock64();
  while (!bw::mbar_try_wait(bar, parity)) {
    if (clock64() - start > cycles) {
      atomicOr(err, bw::kErrTimeout);
      return false;
    }
  }
  return true;
}

__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, %0;" ::"n"(PG_CONSUMERS * 32) : "memory"); }
// the four warps of one group (barriers 2, 3, ...)
__device__ __forceinline__ void group_sync(int group) { asm volatile("bar.sync %0, %1;" ::"r"(group + 2), "n"(PG_BOXES * 32) : "memory"); }
__device__ __forceinline__ void fence_proxy_async_all() { asm volatile("fence.proxy.async;" ::: "memory"); }
__device__ __forceinline__ unsigned load_acquire(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// ---- which part of a phase a CTA takes (the producer and the consumers must agree on every line)
//
// A product of row_tiles tiles of 32 weight rows, its K cut into `splits` slices of whole 256-column
// chunks.  CTA c works on ONE slice, c % splits, for the whole phase (so the token columns it needs
// fit shared memory and are fetched once), together with the other CTAs of that slice: it is number
// c / splits among them and takes the tiles rank, rank + peers, rank + 2 peers, ...  Inside a tile the
// chunks are walked from a chunk that differs between the CTAs of a slice, so that they do not all
// ask for the same lines at the same moment.
struct ProductShare {
  int first_chunk, count;   // the slice's chunks
  int rotate;               // the chunk (relative) a tile's walk begins with
  int rank, peers;          // tiles rank, rank + peers, ... < row_tiles
  int tiles;                // how many that is
  __device__ __forceinline__ int chunk(int i) const {   // the i-th stage of a tile
    int c = i + rotate;
    if (c >= count) c -= count;
    return first_chunk + c;
  }
};
__device__ __forceinline__ ProductShare product_share(const Phase& p) {
  ProductShare s;
  const int slice = (int)(blockIdx.x % (unsigned)p.splits);
  s.rank = (int)(blockIdx.x / (unsigned)p.splits);
  s.peers = ((int)gridDim.x - slice + p.splits - 1) / p.splits;
  s.first_chunk = (slice * p.chunks) / p.splits;            // splits * chunks stays far below 2^31
  s.count = ((slice + 1) * p.chunks) / p.splits - s.first_chunk;
  s.rotate = s.count > 0 ? s.rank % s.count : 0;
  s.tiles = s.rank < p.row_tiles ? (p.row_tiles - s.rank + s.peers - 1) / s.peers : 0;
  if (s.count <= 0) s.tiles = 0;
  return s;
}
// How the stages of a CTA's tiles reach the two groups of consumer warps.
//  * Several tiles: they go to the groups in turn, whole (the CTA's tile number j to group j % 2), and
//    the producer fills stages of the two groups' tiles alternately for as long as both have some
//    left, so that both groups stream at the same time and each finishes its own tiles.
//  * One tile: the two groups share it, stage i going to group i % 2, and add their sums up at its end.
// Either way the ring's stages go to group 0 and group 1 in turn while both have stages left (group
// 0 first), and to the one that has some left after that.
static_assert(PG_GROUPS == 2, "the stages of a product are dealt to two groups of consumer warps");

struct KeyUnit {
  int unit, split, request, kvh, h0;
  int length, first, begin, end, tiles, used;
};
__device__ __forceinline__ KeyUnit key_unit(const Phase& p, int u) {
  KeyUnit k;
  const int base = p.m * p.kv_heads * p.head_chunks;
  k.unit = u % base;           // the split is the slowest index: the CTAs a short request leaves unused are spread
  k.split = u / base;
  k.request = k.unit / (p.kv_heads * p.head_chunks);
  const int rest = k.unit % (p.kv_heads * p.head_chunks);
  k.kvh = rest / p.head_chunks;
  k.h0 = (rest % p.head_chunks) * 16;
  k.length = p.context_lens[k.request] + 1;
  k.first = (p.window > 0 && k.length > p.window) ? k.length - p.window : 0;
  const int first_block = k.first / 16;
  const int blocks = (k.length + 15) / 16 - first_block;
  k.used = max(1, min(p.key_splits, (k.length - k.first) / p.min_keys));
  const int per_split = (blocks + k.used - 1) / k.used;
  k.begin = (first_block + k.split * per_split) * 16;
  k.end = min(k.length, k.begin + per_split * 16);
  k.tiles = (k.split < k.used && k.begin < k.end) ? (k.end - k.begin + PG_TILE_KEYS - 1) / PG_TILE_KEYS : 0;
  return k;
}

// ------------------------------------------------------------------------------------------ producer
struct Ring {
  unsigned char* base;
  ProgramShared* sh;
  int stages;
  int slot;
  uint32_t parity;   // producer: parity to wait for on empty[slot]; consumer: on full[slot]
  __device__ __forceinline__ void advance() {
    if (++slot == stages) {
      slot = 0;
      parity ^= 1u;
    }
  }
  __device__ __forceinline__ void skip(int count) {   // stages that somebody else takes
    slot += count;
    while (slot >= stages) {
      slot -= stages;
      parity ^= 1u;
    }
  }
};

__device__ void run_producer(const Phase* __restrict__ tape, Ring ring, int* err, int lane) {
  ProgramShared& sh = *ring.sh;
  bool alive = true;
  long long issued = 0;   // stages filled so far
  // waits until the stage at ring.slot is free; false once a wait has run out
  auto acquire = [&]() -> bool {
    int ok = 1;
    if (lane == 0) ok = wait_bar(&sh.empty[ring.slot], ring.parity, kWaitCycles, err) ? 1 : 0;
    ok = __shfl_sync(0xffffffffu, ok, 0);
    return ok != 0;
  };
  for (int pi = 0; alive; ++pi) {
    const Phase& p = tape[pi];
    const int kind = p.kind;
    if (kind == kEnd) break;
    if (kind == kGemm) {
      auto issue = [&](int tile, int chunk) -> bool {
        if (!acquire()) return false;
        uint64_t* bar = &sh.full[ring.slot];
        if (lane == 0) bw::mbar_expect_tx(bar, PG_STAGE_BYTES);
        __syncwarp();
        if (lane < 4)
          bw::tma_load_2d(ring.base + (size_t)ring.slot * PG_STAGE_BYTES + lane * 4096, &p.map0, bar,
                          chunk * PG_KC + lane * 64, tile * PG_BN);
        ring.advance();
        ++issued;
        return true;
      };
      const ProductShare share = product_share(p);
      if (share.tiles == 1) {
        for (int i = 0; i < share.count && alive; ++i) alive = issue(share.rank, share.chunk(i));
      } else if (share.tiles > 1) {
        // two streams of tiles: rank, rank + 2 peers, ... and rank + peers, rank + 3 peers, ...
        int tile0 = share.rank, tile1 = share.rank + share.peers, i0 = 0, i1 = 0, turn = 0;
        bool live0 = true, live1 = tile1 < p.row_tiles;
        while ((live0 || live1) && alive) {
          if (live0 && (turn == 0 || !live1)) {
            alive = issue(tile0, share.chunk(i0));
            if (++i0 == share.count) {
              i0 = 0;
              tile0 += 2 * share.peers;
              live0 = tile0 < p.row_tiles;
            }
            turn = 1;
          } else {
            alive = issue(tile1, share.chunk(i1));
            if (++i1 == share.count) {
              i1 = 0;
              tile1 += 2 * share.peers;
              live1 = tile1 < p.row_tiles;
            }
            turn = 0;
          }
        }
      }
    } else if (kind == kAttention) {
      const int units = p.m * p.kv_heads * p.head_chunks * p.key_splits;
      for (int u = blockIdx.x; u < units && alive; u += gridDim.x) {
        const KeyUnit k = key_unit(p, u);
        for (int tile = 0; tile < k.tiles && alive; ++tile) {
          const int k0 = k.begin + tile * PG_TILE_KEYS;
          const int in_tile = min(4, (k.end - k0 + 15) / 16);   // 16-key blocks of the tile
          if (k0 + PG_TILE_KEYS > k.length - 1 && k.end == k.length) {
            // the tile holds the newest key, which the q/k/v phase of this step writes: wait until this
            // CTA has passed the barrier in front of this phase
            if (lane == 0) {
              const long long start = clock64();
              while (sh.epoch < pi && !sh.dead) {
                if (clock64() - start > kWaitCycles) {
                  atomicOr(err, bw::kErrTimeout);
                  sh.dead = 1;
                }
              }
            }
            __syncwarp();
            if (sh.dead) { alive = false; break; }
            fence_proxy_async_all();
          }
          int page = 0, within = 0;
          if (lane < in_tile) {
            const int key = k0 + lane * 16;
            const int index = key >> p.page_shift;
            within = key & (p.page_size - 1);
            page = index < p.table_width ? __ldg(p.table + (size_t)k.request * p.table_width + index) : -1;
            if (page < 0 || page >= p.num_pages) {
              atomicOr(err, kErrBadPage);
              page = 0;   // the copy must still happen, or the barrier would never complete
            }
          }
          const int row0 = (page * p.kv_heads + k.kvh) * p.page_size + within;
          if constexpr (PG_KEY_STAGES == 2) {
#pragma unroll
            for (int which = 0; which < 2; ++which) {
              if (!acquire()) { alive = false; break; }
              uint64_t* bar = &sh.full[ring.slot];
              if (lane == 0) bw::mbar_expect_tx(bar, (uint32_t)(in_tile * PG_BLOCK_BYTES));
              __syncwarp();
              if (lane < in_tile)
                bw::tma_load_4d(ring.base + (size_t)ring.slot * PG_STAGE_BYTES + lane * PG_BLOCK_BYTES,
                                which == 0 ? &p.map0 : &p.map1, bar, 0, 0, 0, row0 / 8);
              ring.advance();
              ++issued;
            }
          } else {
            if (!acquire()) { alive = false; break; }
            uint64_t* bar = &sh.full[ring.slot];
            if (lane == 0) bw::mbar_expect_tx(bar, (uint32_t)(in_tile * 2 * PG_BLOCK_BYTES));
            __syncwarp();
            if (lane < in_tile) {
              unsigned char* dst = ring.base + (size_t)ring.slot * PG_STAGE_BYTES + lane * PG_BLOCK_BYTES;
              bw::tma_load_3d(dst, &p.map0, bar, 0, 0, row0 / 8);
              bw::tma_load_3d(dst + 4 * PG_BLOCK_BYTES, &p.map1, bar, 0, 0, row0 / 8);
            }
            ring.advance();
            ++issued;
          }
        }
      }
    }
  }
  // Before the CTA gives its shared memory up, every copy it asked for has landed: the last
  // `stages` fills each get one more (short) bounded wait.  Normally they completed long ago.
  if (lane == 0) {
    const long long pending = issued < ring.stages ? issued : ring.stages;
    for (long long back = 1; back <= pending; ++back) {
      const long long fill = issued - back;
      wait_bar(&sh.full[(int)(fill % ring.stages)], (uint32_t)((fill / ring.stages) & 1), kDrainCycles, err);
    }
  }
}

// ------------------------------------------------------------------------------------------ consumers
struct Consumer {
  Ring ring;
  float* scratch;
  unsigned char* slab;   // the token rows of a product (behind the sums' buffer); attention's merge buffer
  bf16* q_s;
  int* err;
  int phase_index;      // (for the trace)
  int cw, lane, ctid;   // consumer warp 0 .. PG_CONSUMERS - 1, lane, thread among the consumers
  int group, box;       // cw / 4: which stages it takes; cw % 4: which part of a stage
  bool alive;
  // waits for the stage at ring.slot to be full
  __device__ __forceinline__ void wait_full() {
    if (alive) {   // the same in every lane of the warp
      const bool landed = wait_bar(&ring.sh->full[ring.slot], ring.parity, kWaitCycles, err);
      if (!__all_sync(0xffffffffu, landed)) {
        alive = false;
        ring.sh->dead = 1;
      }
    }
  }
  __device__ __forceinline__ void release(int slot) {
    __syncwarp();
    if (lane == 0) bw::mbar_arrive(&ring.sh->empty[slot]);
  }
  __device__ __forceinline__ void sync() {
    consumer_sync();
    if (ring.sh->dead) alive = false;
  }
};

__device__ __forceinline__ float load_cg(const float* p) { return __ldcg(p); }
__device__ __forceinline__ void ldsm_x4_at(uint32_t (&r)[4], uint32_t shared_address) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(shared_address));
}

// The epilogue of one finished value: row m (token), column `col` = tile * 32 + lane of the product.
// The whole warp calls this for one token row.
__device__ __forceinline__ void finish_value(const Phase& p, int m, int tile, int lane, float v, int* err) {
  const int col = tile * PG_BN + lane;
  if (p.mode == kOutBF16 || p.mode == kOutF32) {
    if (col < p.n) {
      if (p.bias) v += p.bias[col];
      if (p.mode == kOutF32) reinterpret_cast<float*>(p.out)[(size_t)m * p.n + col] = v;
      else reinterpret_cast<bf16*>(p.out)[(size_t)m * p.n + col] = __float2bfloat16_rn(v);
    }
    return;
  }
  if (p.mode == kOutSiluMul) {
    // gate and up rows interleaved in blocks of 16: lanes 0..15 hold gate, 16..31 the matching up
    const float up = __shfl_sync(0xffffffffu, v, (lane & 15) + 16);
    const int channels = p.n / 2, channel = tile * 16 + lane;
    if (lane < 16 && channel < channels)
      reinterpret_cast<bf16*>(p.out)[(size_t)m * channels + channel] = __float2bfloat16_rn((v / (1.f + expf(-v))) * up);
    return;
  }
  if (p.mode == kOutResidual) {
    float square = 0.f;
    if (col < p.n) {
      const float bias = p.bias ? p.bias[col] : 0.f;
      const float updated = load_cg(p.residual + (size_t)m * p.n + col) + (v + bias);
      p.residual[(size_t)m * p.n + col] = updated;
      if (p.scaled) p.scaled[(size_t)m * p.n + col] = __float2bfloat16_rn(updated * p.next_gain[col]);
      square = updated * updated;
    }
    square = warp_sum(square);
    if (lane == 0) p.sq[(size_t)m * p.row_tiles + tile] = square;
    return;
  }
  // kOutRope: the stacked q/k/v projection, q and k rows in the paired layout (inside every head,
  // blocks of 16 rotary elements followed by their 16 partners); the 32 columns lie in one head
  const int n0 = tile * PG_BN;
  const int q_width = p.q_heads * p.dim, kv_width = p.kv_heads * p.dim;
  const int region = n0 < q_width ? 0 : n0 < q_width + kv_width ? 1 : 2;   // q, k, v
  const int local = n0 - (region == 0 ? 0 : region == 1 ? q_width : q_width + kv_width);
  const int head = local / p.dim, p0 = local % p.dim;
  const int half = p.rot / 2;
  const bool rotary = region < 2 && p0 < p.rot;
  const int pair = (p0 >> 5) * 16 + (lane & 15);
  const int d_out = rotary ? (lane < 16 ? pair : half + pair) : p0 + lane;
  if (p.bias) v += p.bias[n0 + lane];
  const int pos = p.positions[m];
  float result = v;
  if (rotary) {
    float sn, cs;
    sincosf((float)pos * p.inv_freq[pair], &sn, &cs);
    const float other = __shfl_xor_sync(0xffffffffu, v, 16);
    result = lane < 16 ? v * cs - other * sn : v * cs + other * sn;
  }
  const bf16 rounded = __float2bfloat16_rn(result);
  if (region == 0) {
    p.q_out[(size_t)m * p.q_stride + head * p.dim + d_out] = rounded;
  } else if (p.write_cache) {
    const int index = pos / p.page_size;
    const int page = index < p.table_width ? p.table[(size_t)p.request_of_token[m] * p.table_width + index] : -1;
    if (page < 0 || page >= p.num_pages) {
      if (lane == 0) atomicOr(err, kErrBadPage);
    } else {
      bf16* pool = region == 1 ? p.k_pool : p.v_pool;
      pool[(((long long)page * p.kv_heads + head) * p.page_size + pos % p.page_size) * p.dim + d_out] = rounded;
      // the attention phase reads the pages with TMA copies
      fence_proxy_async_all();
    }
  }
}

// The slices of a finished tile are in red[warp][token][weight row] (`slices` of them: a group's four,
// or all consumers' when the groups shared the unit).  The warps taking part (number `part` of
// `parts`) add them up for the token rows part, part + parts, ... and run the epilogue (or leave the
// partial sums of a K slice).
__device__ __noinline__ void tile_epilogue(const Phase& p, const Consumer& c, const float* red, int slices, int part,
                                           int parts, int tile, int split) {
  const int lane = c.lane;
  for (int m = part; m < p.m; m += parts) {
    float v = 0.f;
    for (int w = 0; w < slices; ++w) v += red[(w * 16 + m) * PG_RED_ROW + lane];
    if (p.row_sq) v *= c.ring.sh->rstd[m];
    if (p.splits > 1) {
      const int col = tile * PG_BN + lane;
      if (col < p.n) __stcg(p.partial + ((size_t)split * p.m + m) * p.n + col, v);
    } else {
      finish_value(p, m, tile, lane, v, c.err);
    }
  }
}

template <int MT>
__device__ __noinline__ void gemm_phase(const Phase& p, Consumer& shared_state) {
  Consumer c = shared_state;   // in registers while the phase runs
  constexpr int MP = MT * 8;
  constexpr int XG = MP * 128;   // bytes of one 64-column group of the slab: MP rows of 128 bytes
  ProgramShared& sh = *c.ring.sh;
  const int lane = c.lane, box_index = c.box, group = c.group;
  const int g = lane >> 2, t4 = lane & 3;
  const ProductShare share = product_share(p);
  // ---- the token rows of this CTA's slice of K go to shared memory once, for the whole phase: the
  // slab, [64-column group][MP rows][128 bytes], the 16-byte piece c of row r at position c ^ (r & 7)
  // as in the weight boxes (rows beyond the step's and columns beyond K are zeros)
  {
    const int k_begin = share.first_chunk * PG_KC, k_total = p.k, rows = p.m, x_stride = p.x_stride;
    const bf16* x = p.x;
    const int pieces = share.tiles > 0 ? share.count * (PG_KC / 8) * MP : 0;
    for (int index = c.ctid; index < pieces; index += PG_CONSUMERS * 32) {
      const int piece = index & 7, row = (index >> 3) % MP, group64 = (index >> 3) / MP;
      const int k0 = k_begin + group64 * 64 + piece * 8;
      const bool ok = row < rows && k0 < k_total;
      cp_async16(c.slab + group64 * XG + row * 128 + ((piece ^ (row & 7)) << 4),
                 ok ? x + (size_t)row * x_stride + k0 : x, ok);
    }
    cp_async_commit();
  }
  if (p.row_sq) {
    // rstd of the token rows from the sums of squares that an earlier phase left per 32 columns
    for (int m = c.cw; m < MP; m += PG_CONSUMERS) {
      float sum = 0.f;
      if (m < p.m)
        for (int t = lane; t < p.sq_tiles; t += 32) sum += load_cg(p.row_sq + (size_t)m * p.sq_tiles + t);
      sum = warp_sum(sum);
      if (lane == 0) sh.rstd[m] = m < p.m ? rsqrtf(sum / (float)p.k + p.eps) : 0.f;
    }
  }
  // ---- this group's stages.  One tile: every second stage of it.  Several: every stage of every
  // second tile.  The ring's stages go to the groups in turn while both have some left.
  const bool shared = share.tiles == 1;
  const int own_tiles = shared ? 1 : (share.tiles + 1 - group) / 2;
  const int own_total = shared ? (share.count + 1 - group) / 2 : own_tiles * share.count;
  const int other_total = shared ? share.count - own_total : (share.tiles - own_tiles) * share.count;
  const int both = own_total < other_total ? own_total : other_total;
  // per-lane offsets that do not change with the stage
  int a_offset[4][2];   // of the A fragments inside this warp's box
#pragma unroll
  for (int i16 = 0; i16 < 4; ++i16)
#pragma unroll
    for (int rt = 0; rt < 2; ++rt) {
      const int row = rt * 16 + (lane & 15), piece = 2 * i16 + (lane >> 4);
      a_offset[i16][rt] = box_index * 4096 + row * 128 + ((piece ^ (row & 7)) << 4);
    }
  int b_offset[2][MT];  // of the B fragments inside a chunk of the slab (this warp's 64-column group)
#pragma unroll
  for (int pair = 0; pair < 2; ++pair)
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
      b_offset[pair][mt] = box_index * XG + (mt * 8 + (lane & 7)) * 128 + (((4 * pair + (lane >> 3)) ^ (lane & 7)) << 4);
  // two accumulator sets a row tile (even and odd k-steps) halve the chains of dependent
  // tensor-core instructions; they are added when the tile is complete
  float acc[2][2][MT][4];
#pragma unroll
  for (int e = 0; e < 2; ++e)
#pragma unroll
    for (int rt = 0; rt < 2; ++rt)
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) acc[e][rt][mt][0] = acc[e][rt][mt][1] = acc[e][rt][mt][2] = acc[e][rt][mt][3] = 0.f;
  // sums of a tile: a group's own four slices, or all eight when the groups share the tile
  float* red = shared ? c.scratch : c.scratch + group * (PG_BOXES * 16 * PG_RED_ROW);
  const int slice = shared ? c.cw : box_index;
  auto put_sums = [&]() {
#pragma unroll
    for (int rt = 0; rt < 2; ++rt)
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) {
        const int m0 = mt * 8 + 2 * t4, r0 = rt * 16 + g;
        float* mine = red + (slice * 16 + m0) * PG_RED_ROW + r0;
        mine[0] = acc[0][rt][mt][0] + acc[1][rt][mt][0];
        mine[PG_RED_ROW] = acc[0][rt][mt][1] + acc[1][rt][mt][1];
        mine[8] = acc[0][rt][mt][2] + acc[1][rt][mt][2];
        mine[PG_RED_ROW + 8] = acc[0][rt][mt][3] + acc[1][rt][mt][3];
#pragma unroll
        for (int e = 0; e < 2; ++e)
          acc[e][rt][mt][0] = acc[e][rt][mt][1] = acc[e][rt][mt][2] = acc[e][rt][mt][3] = 0.f;
      }
  };
  cp_async_wait<0>();
  c.sync();   // the slab and rstd are there for everybody
  trace_mark(c.phase_index, 2, c.ctid);
  int tile = share.rank + (shared ? 0 : group * share.peers);
  int in_tile = shared ? group : 0;          // stage of the tile that comes next for this group
  const int in_tile_step = shared ? 2 : 1;
  for (int done = 0; done < own_total; ++done) {
    PROBE_DECLARE();
    PROBE_AT(0);
    if (group == 1 && done < both) c.ring.advance();   // the other group's stage lies in front of this one
    PROBE_AT(1);
    int relative = in_tile + share.rotate;             // the chunk of this stage, counted from the slice's first
    if (relative >= share.count) relative -= share.count;
    PROBE_AT(2);
    c.wait_full();
    PROBE_AT(3);
    PROBE_AT(4);
#ifndef PROGRAM_SKIP_MATH   // (debug builds may leave the products out to see what the rest costs)
    const uint32_t box = smem_u32(c.ring.base) + c.ring.slot * PG_STAGE_BYTES;
    const uint32_t xb = smem_u32(c.slab) + relative * (4 * XG);
    // every fragment of the stage is asked for before the first product needs one
    uint32_t bfrag[2][MT][4], afrag[4][2][4];
#pragma unroll
    for (int pair = 0; pair < 2; ++pair)
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) ldsm_x4_at(bfrag[pair][mt], xb + b_offset[pair][mt]);
#pragma unroll
    for (int i16 = 0; i16 < 4; ++i16)
#pragma unroll
      for (int rt = 0; rt < 2; ++rt) ldsm_x4_at(afrag[i16][rt], box + a_offset[i16][rt]);
#pragma unroll
    for (int i16 = 0; i16 < 4; ++i16)
#pragma unroll
      for (int rt = 0; rt < 2; ++rt)
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
          mma_bf16(acc[i16 & 1][rt][mt], afrag[i16][rt], bfrag[i16 >> 1][mt][2 * (i16 & 1)], bfrag[i16 >> 1][mt][2 * (i16 & 1) + 1]);
#endif
    PROBE_AT(5);
    c.release(c.ring.slot);
    c.ring.advance();
    if (group == 0 && done < both) c.ring.advance();   // the other group's stage lies behind this one
    PROBE_AT(6);
    PROBE_STORE();
    in_tile += in_tile_step;
    if (!shared && in_tile == share.count) {
      // ---- the group's tile is complete: its four slices meet in shared memory
      group_sync(group);   // the group's tile before has been read
      put_sums();
      group_sync(group);
      tile_epilogue(p, c, red, PG_BOXES, box_index, PG_BOXES, tile, (int)(blockIdx.x % (unsigned)p.splits));
      in_tile = 0;
      tile += 2 * share.peers;
    }
  }
  trace_mark(c.phase_index, 3, c.ctid);
  // what is left of the phase's stages in this CTA belongs to the other group
  c.ring.skip(other_total - both);
  if (shared) {
    // ---- the tile the groups shared: all eight slices meet (a group without a stage brings zeros)
    put_sums();
    c.sync();
    tile_epilogue(p, c, red, PG_CONSUMERS, c.cw, PG_CONSUMERS, tile, (int)(blockIdx.x % (unsigned)p.splits));
  }
  if (sh.dead) c.alive = false;
  shared_state = c;
}

// The rstd scale of a product that was cut along K is applied to its partial sums (gemm_phase);
// this phase adds the slices up in ascending order and runs the epilogue.
__device__ __noinline__ void finish_phase(const Phase& p, Consumer& c) {
  const int lane = c.lane;
  for (int tile = blockIdx.x; tile < p.row_tiles; tile += gridDim.x) {
    const int col = tile * PG_BN + lane;
    for (int m = c.cw; m < p.m; m += PG_CONSUMERS) {
      float v = 0.f;
      if (col < p.n) {
        const float* src = p.partial + (size_t)m * p.n + col;
        const size_t stride = (size_t)p.m * p.n;
        int s = 0;
        for (; s + 4 <= p.splits; s += 4) {
          const float a0 = load_cg(src + (size_t)s * stride), a1 = load_cg(src + (size_t)(s + 1) * stride);
          const float a2 = load_cg(src + (size_t)(s + 2) * stride), a3 = load_cg(src + (size_t)(s + 3) * stride);
          v += a0; v += a1; v += a2; v += a3;
        }
        for (; s < p.splits; ++s) v += load_cg(src + (size_t)s * stride);
      }
      finish_value(p, m, tile, lane, v, c.err);
    }
  }
}

__device__ __noinline__ void attention_phase(const Phase& p, Consumer& shared_state) {
  Consumer c = shared_state;   // in registers while the phase runs
  ProgramShared& sh = *c.ring.sh;
  const int lane = c.lane, cw = c.cw, box_index = c.box;
  const int g = lane >> 2, t4 = lane & 3;
  float* merge_s = reinterpret_cast<float*>(c.slab);   // [warp of a group][16][D]
  const int units = p.m * p.kv_heads * p.head_chunks * p.key_splits;
  for (int u = blockIdx.x; u < units; u += gridDim.x) {
    const KeyUnit k = key_unit(p, u);
    if (k.tiles == 0) continue;
    const int live_rows = min(16, p.group - k.h0);
    c.sync();   // the unit before is done with the queries and the merge buffer
    for (int idx = c.ctid; idx < 16 * CHUNKS; idx += PG_CONSUMERS * 32) {
      const int r = idx / CHUNKS, piece = idx % CHUNKS;
      const bool ok = k.h0 + r < p.group;
      const bf16* src = ok ? p.q_out + (size_t)k.request * p.q_stride + (size_t)(k.kvh * p.group + k.h0 + r) * D + piece * 8
                           : p.q_out;
      cp_async16(c.q_s + r * ROW + piece * 8, src, ok);
    }
    cp_async_commit();
    cp_async_wait<0>();
    c.sync();
    uint32_t q_frag[KSTEPS][4];
#pragma unroll
    for (int kk = 0; kk < KSTEPS; ++kk)
      ldsm_x4(q_frag[kk], c.q_s + (lane & 15) * ROW + kk * 16 + (lane >> 4) * 8);
    float o[NTILES_D][4];
#pragma unroll
    for (int i = 0; i < NTILES_D; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    float mx[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
    for (int tile = 0; tile < k.tiles; ++tile) {
      if (tile % PG_GROUPS != c.group) {   // another group's tile
#pragma unroll
        for (int i = 0; i < PG_KEY_STAGES; ++i) c.ring.advance();
        continue;
      }
      const int k0 = k.begin + tile * PG_TILE_KEYS + box_index * 16;   // this warp's 16 keys of the tile
      const bool mine = k0 < k.end;
      c.wait_full();
      const int k_slot = c.ring.slot;
      const bf16* k_tile = reinterpret_cast<const bf16*>(c.ring.base + (size_t)k_slot * PG_STAGE_BYTES + box_index * PG_BLOCK_BYTES);
      float s[2][4];
      if (mine && c.alive) {
        scores<1, true>(q_frag, k_tile, s, lane);
        if (k0 >= k.first && k0 + 16 <= k.end) {
#pragma unroll
          for (int i = 0; i < 2; ++i)
#pragma unroll
            for (int e = 0; e < 4; ++e) s[i][e] *= p.scale_log2;
        } else {
#pragma unroll
          for (int i = 0; i < 2; ++i)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const int key = k0 + i * 8 + 2 * t4 + (e & 1);
              s[i][e] = (key >= k.first && key < k.end) ? s[i][e] * p.scale_log2 : -INFINITY;
            }
        }
        if (live_rows <= 8) softmax_update<2, 1>(s, mx, l, o);
        else softmax_update<2, 2>(s, mx, l, o);
      }
      const bf16* v_tile;
      if constexpr (PG_KEY_STAGES == 2) {
        c.release(k_slot);
        c.ring.advance();
        c.wait_full();
        v_tile = reinterpret_cast<const bf16*>(c.ring.base + (size_t)c.ring.slot * PG_STAGE_BYTES + box_index * PG_BLOCK_BYTES);
      } else {
        v_tile = k_tile + 4 * PG_BLOCK_BYTES / 2;
      }
      if (mine && c.alive) accumulate<1, true>(s, v_tile, o, lane);
      c.release(c.ring.slot);
      c.ring.advance();
    }
    // ---- the warps of the CTA: maxima and sums first, then the outputs scaled to the CTA's maxima.
    // The warps of the other groups hand their outputs to the first group's warp with the same part
    // of a tile (the same thread holds the same elements), which adds them to its own; then the
    // first group's four slices meet in the merge buffer.
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const float total = quad_sum(l[h]);
      if (t4 == 0) {
        sh.warp_max[cw][g + h * 8] = mx[h];
        sh.warp_sum[cw][g + h * 8] = total;
      }
    }
    c.sync();
    float* my_merge = merge_s + box_index * 16 * D;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int r = g + h * 8;
      float m_all = -INFINITY;
#pragma unroll
      for (int w = 0; w < PG_CONSUMERS; ++w) m_all = fmaxf(m_all, sh.warp_max[w][r]);
      const float scale_mine = (mx[h] == -INFINITY) ? 0.f : exp2f(mx[h] - m_all);
#pragma unroll
      for (int i = 0; i < NTILES_D; ++i) {
        o[i][2 * h] *= scale_mine;
        o[i][2 * h + 1] *= scale_mine;
      }
    }
#pragma unroll
    for (int other = 1; other < PG_GROUPS; ++other) {
      if (c.group == other) {
#pragma unroll
        for (int h = 0; h < 2; ++h)
#pragma unroll
          for (int i = 0; i < NTILES_D; ++i)
            *reinterpret_cast<float2*>(my_merge + (g + h * 8) * D + i * 8 + 2 * t4) = make_float2(o[i][2 * h], o[i][2 * h + 1]);
      }
      c.sync();
      if (c.group == 0) {
#pragma unroll
        for (int h = 0; h < 2; ++h)
#pragma unroll
          for (int i = 0; i < NTILES_D; ++i) {
            const float2 theirs = *reinterpret_cast<const float2*>(my_merge + (g + h * 8) * D + i * 8 + 2 * t4);
            o[i][2 * h] += theirs.x;
            o[i][2 * h + 1] += theirs.y;
          }
      }
      c.sync();
    }
    if (c.group == 0) {
#pragma unroll
      for (int h = 0; h < 2; ++h)
#pragma unroll
        for (int i = 0; i < NTILES_D; ++i)
          *reinterpret_cast<float2*>(my_merge + (g + h * 8) * D + i * 8 + 2 * t4) = make_float2(o[i][2 * h], o[i][2 * h + 1]);
    }
    c.sync();
    bf16* out_rows = p.attn_out + (size_t)k.request * p.out_stride + (size_t)(k.kvh * p.group + k.h0) * D;
    float* share = p.shares + ((size_t)k.unit * p.key_splits + k.split) * 16 * PG_SHARE_ROW;
    for (int idx = c.ctid; idx < live_rows * (D / 4); idx += PG_CONSUMERS * 32) {
      const int r = idx / (D / 4), c4 = idx % (D / 4);
      float4 acc = *reinterpret_cast<const float4*>(merge_s + r * D + c4 * 4);
#pragma unroll
      for (int w = 1; w < PG_BOXES; ++w) {
        const float4 part = *reinterpret_cast<const float4*>(merge_s + (w * 16 + r) * D + c4 * 4);
        acc.x += part.x; acc.y += part.y; acc.z += part.z; acc.w += part.w;
      }
      float m_all = -INFINITY;
#pragma unroll
      for (int w = 0; w < PG_CONSUMERS; ++w) m_all = fmaxf(m_all, sh.warp_max[w][r]);
      float sum = 0.f;
#pragma unroll
      for (int w = 0; w < PG_CONSUMERS; ++w) {
        const float mw = sh.warp_max[w][r];
        sum += sh.warp_sum[w][r] * ((mw == -INFINITY) ? 0.f : exp2f(mw - m_all));
      }
      if (k.used == 1) {   // the request's keys are this CTA's alone: the output itself
        const float inv = sum > 0.f ? 1.f / sum : 0.f;
        uint2 packed;
        packed.x = pack_bf16(acc.x * inv, acc.y * inv);
        packed.y = pack_bf16(acc.z * inv, acc.w * inv);
        *reinterpret_cast<uint2*>(out_rows + (size_t)r * D + c4 * 4) = packed;
      } else {
        __stcg(reinterpret_cast<float4*>(share + r * PG_SHARE_ROW + c4 * 4), acc);
        if (c4 == 0) {
          __stcg(share + r * PG_SHARE_ROW + D, m_all);
          __stcg(share + r * PG_SHARE_ROW + D + 1, sum);
        }
      }
    }
  }
  shared_state = c;
}

// Joins the shares of the CTAs that divided a request's keys: a warp takes one head row and merges
// the shares in the order of the key ranges, eight at a time, with a running maximum.
__device__ __noinline__ void merge_phase(const Phase& p, Consumer& c) {
  const int lane = c.lane;
  const int base = p.m * p.kv_heads * p.head_chunks;
  constexpr int PARTS = 16 / PG_CONSUMERS;   // a unit's 16 head rows: one a warp
  for (int u = blockIdx.x; u < base * PARTS; u += gridDim.x) {
    const KeyUnit k = key_unit(p, u / PARTS);   // split 0 of the unit: lengths and the count of shares
    const int r = (u % PARTS) * PG_CONSUMERS + c.cw;
    const int live_rows = min(16, p.group - k.h0);
    if (k.used == 1 || r >= live_rows || lane >= D / 4) continue;
    const float* row = p.shares + ((size_t)k.unit * p.key_splits * 16 + r) * PG_SHARE_ROW;
    float m_run = -INFINITY, sum = 0.f;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int c0 = 0; c0 < k.used; c0 += 8) {
      float ms[8], ls[8];
      float4 part[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const bool live = c0 + j < k.used;
        const float* share = row + (size_t)(live ? c0 + j : c0) * 16 * PG_SHARE_ROW;
        ms[j] = live ? __ldcg(share + D) : -INFINITY;
        ls[j] = live ? __ldcg(share + D + 1) : 0.f;
        part[j] = __ldcg(reinterpret_cast<const float4*>(share + lane * 4));
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
    bf16* out_row = p.attn_out + (size_t)k.request * p.out_stride + (size_t)(k.kvh * p.group + k.h0 + r) * D;
    *reinterpret_cast<uint2*>(out_row + lane * 4) = packed;
  }
}

// All CTAs meet: what they wrote before is visible to all of them after.  `passed` barriers lie
// behind; the counter only grows (the host zeroes it before the launch).
__device__ void grid_barrier(Consumer& c, unsigned* counter, int passed) {
  ProgramShared& sh = *c.ring.sh;
  consumer_sync();
  if (c.ctid == 0) {
    // a release at GPU scope: what the CTA's threads wrote before the barrier above is visible to
    // whoever sees the count
    asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(counter) : "memory");
    const unsigned target = (unsigned)(passed + 1) * gridDim.x;
    if (!sh.dead) {
      const long long start = clock64();
      while (load_acquire(counter) < target) {
        if (clock64() - start > kWaitCycles) {
          atomicOr(c.err, bw::kErrTimeout);
          sh.dead = 1;
          break;
        }
      }
    }
    sh.epoch = passed + 1;
  }
  c.sync();
}

__device__ void run_consumers(const Phase* __restrict__ tape, Consumer c, unsigned* counter) {
  for (int pi = 0;; ++pi) {
    const Phase& p = tape[pi];
    const int kind = p.kind;
    if (kind == kEnd) break;
    trace_mark(pi, 0, c.ctid);
    c.phase_index = pi;
    if (kind == kGemm) {
      if (p.m <= 8) gemm_phase<1>(p, c);
      else gemm_phase<2>(p, c);
    } else if (kind == kFinish) {
      finish_phase(p, c);
    } else if (kind == kAttention) {
      attention_phase(p, c);
    } else if (kind == kMerge) {
      merge_phase(p, c);
    }
    trace_mark(pi, 1, c.ctid);
    if (tape[pi + 1].kind == kEnd) break;   // what the last phase wrote is visible when the kernel ends
    grid_barrier(c, counter, pi);
  }
}

__global__ void __launch_bounds__(PG_THREADS, 1)
decode_program_kernel(const Phase* __restrict__ tape, unsigned* counter, int* err, int stages, int slab_bytes) {
  extern __shared__ __align__(16) unsigned char smem_unaligned[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_unaligned) + 1023) & ~(uintptr_t)1023);
  __shared__ ProgramShared sh;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (tid == 0) {
    for (int s = 0; s < stages; ++s) {
      bw::mbar_init(&sh.full[s], 1);
      bw::mbar_init(&sh.empty[s], PG_BOXES);
    }
    sh.epoch = 0;
    sh.dead = 0;
    bw::mbar_init_fence();
  }
  __syncthreads();
  Ring ring;
  ring.base = smem;
  ring.sh = &sh;
  ring.stages = stages;
  ring.slot = 0;
  if (warp == 0) {
    ring.parity = 1;   // a fresh barrier counts as "the phase before has completed": every stage starts free
    run_producer(tape, ring, err, lane);
  } else {
    ring.parity = 0;
    Consumer c;
    c.ring = ring;
    c.scratch = reinterpret_cast<float*>(smem + (size_t)stages * PG_STAGE_BYTES);
    c.slab = smem + (size_t)stages * PG_STAGE_BYTES + PG_RED_BYTES;
    c.q_s = reinterpret_cast<bf16*>(smem + (size_t)stages * PG_STAGE_BYTES + PG_RED_BYTES + region_bytes(slab_bytes));
    c.group = (warp - 1) / PG_BOXES;
    c.box = (warp - 1) % PG_BOXES;
    c.err = err;
    c.cw = warp - 1;
    c.lane = lane;
    c.ctid = tid - 32;
    c.alive = true;
    run_consumers(tape, c, counter);
  }
}

// ------------------------------------------------------------------------------------------ host
struct LaunchPlan {
  int device = -1;
  int sms = 0;
  long long room = 0;        // dynamic shared memory a CTA may have
  size_t configured = 0;     // what the kernel has been allowed so far
  bool cooperative = true;
};

static int launch_plan(LaunchPlan** out) {
  static LaunchPlan plans[64];
  int device = -1;
  cudaError_t status = cudaGetDevice(&device);
  if (status != cudaSuccess) CIE_FAIL("decode_program: cudaGetDevice: %s", cudaGetErrorString(status));
  if (device < 0 || device >= 64) CIE_FAIL("decode_program: device index %d", device);
  LaunchPlan& plan = plans[device];
  if (plan.device != device) {
    int sms = 0, optin = 0;
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
    cudaDeviceGetAttribute(&optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, device);
    cudaFuncAttributes attributes;
    status = cudaFuncGetAttributes(&attributes, decode_program_kernel);
    if (status != cudaSuccess) CIE_FAIL("decode_program: cudaFuncGetAttributes: %s", cudaGetErrorString(status));
    plan.room = (long long)optin - (long long)attributes.sharedSizeBytes;
    const char* plain = getenv("CIE_PROGRAM_COOPERATIVE");
    plan.cooperative = !(plain && plain[0] == '0');
    plan.sms = sms;
    plan.device = device;
  }
  *out = &plan;
  return 0;
}

// Stages of the ring and bytes of dynamic shared memory for a slab of `slab_bytes`.
static int ring_for(const LaunchPlan& plan, int slab_bytes, int* stages, size_t* smem) {
  const long long fixed = 1024 + PG_RED_BYTES + region_bytes(slab_bytes) + PG_Q_BYTES;
  long long count = (plan.room - fixed) / PG_STAGE_BYTES;
  if (count > PG_MAX_STAGES) count = PG_MAX_STAGES;
  const char* forced = getenv("CIE_PROGRAM_STAGES");
  if (forced && atoi(forced) >= 3 && atoi(forced) < count) count = atoi(forced);
  if (count < 3) CIE_FAIL("decode_program: a slab of %d bytes leaves room for %lld stages only", slab_bytes, count);
  *stages = (int)count;
  *smem = (size_t)(fixed + count * PG_STAGE_BYTES);
  return 0;
}

static int page_shift_of(int page_size) {
  for (int shift = 0; shift < 31; ++shift)
    if ((1 << shift) == page_size) return shift;
  return -1;
}

}  // namespace cie

using namespace cie;

extern "C" int cie_program_head_dim() { return D; }

#ifdef PROGRAM_PROBE
extern "C" int cie_program_set_probe(void* buffer, int slots, int cta) {
  const int zero = 0;
  if (cudaMemcpyToSymbol(g_program_probe, &buffer, sizeof(buffer)) != cudaSuccess ||
      cudaMemcpyToSymbol(g_program_probe_slots, &slots, sizeof(slots)) != cudaSuccess ||
      cudaMemcpyToSymbol(g_program_probe_cta, &cta, sizeof(cta)) != cudaSuccess ||
      cudaMemcpyToSymbol(g_program_probe_used, &zero, sizeof(zero)) != cudaSuccess)
    CIE_FAIL("decode_program: cudaMemcpyToSymbol failed");
  return 0;
}
#endif

// Diagnostics: `buffer` (device memory, 4 * phases * CTAs 64-bit words, zeroed, or null to stop)
// receives the global timer at the points of trace_mark for the first `phases` phases.
extern "C" int cie_program_set_trace(void* buffer, int phases) {
  if (cudaMemcpyToSymbol(g_program_trace, &buffer, sizeof(buffer)) != cudaSuccess ||
      cudaMemcpyToSymbol(g_program_trace_phases, &phases, sizeof(phases)) != cudaSuccess)
    CIE_FAIL("decode_program: cudaMemcpyToSymbol failed");
  return 0;
}
extern "C" int cie_program_phase_bytes() { return (int)sizeof(Phase); }
extern "C" int cie_program_max_key_splits() { return PG_MAX_KEY_SPLITS; }

// CTAs of a launch (one per SM), and the largest slab of token rows (bytes) that still leaves the
// ring `least_stages` stages, on the current device.
extern "C" int cie_program_geometry(int least_stages, int* ctas, int* slab_limit) {
  LaunchPlan* plan = nullptr;
  if (launch_plan(&plan) != 0) return 1;
  *ctas = plan->sms;
  const long long left = plan->room - 1024 - PG_RED_BYTES - PG_Q_BYTES - (long long)least_stages * PG_STAGE_BYTES;
  *slab_limit = left < 0 ? 0 : (int)(left / 1024 * 1024);
  return 0;
}

// Writes the phases of one matrix product out[m, n] = x[m, k] * w[n, k]^T into `phases` (room for
// two) and their number into `count`: the product, and with splits > 1 the finish phase that adds
// the K slices up (partial: float32 [splits][m][n]).  x: bfloat16 rows of x_stride elements; with
// row_sq every result row is multiplied by rsqrt(sum of row_sq[m][0 .. sq_tiles) / k + eps).
// mode: 0 bfloat16 out, 1 float32 out (both + bias), 3 SiLU(gate) * up with gate and up rows
// interleaved in blocks of 16 (n even; out is [m, n / 2]), 4 residual[m, n] += product (+ bias),
// sq[m, ceil(n / 32)] = sums of squares of the new rows per 32 columns and, with next_gain,
// scaled = bfloat16(new row * next_gain).  (The rotary epilogue has its own entry point.)
static int fill_gemm(Phase* phases, int* count, Phase& p, const void* w, int splits, float* partial) {
  if (p.m <= 0 || p.m > 16) CIE_FAIL("decode_program: a product takes 1 to 16 rows, got %d", p.m);
  if (p.n <= 0 || p.k < 8 || p.k % 8) CIE_FAIL("decode_program: product [%d x %d]: K must be a multiple of 8", p.n, p.k);
  if (!p.x || !w || (reinterpret_cast<uintptr_t>(w) & 15) || (reinterpret_cast<uintptr_t>(p.x) & 15) || p.x_stride % 8)
    CIE_FAIL("decode_program: operands must be present and their rows 16-byte aligned");
  p.row_tiles = (p.n + PG_BN - 1) / PG_BN;
  p.chunks = (p.k + PG_KC - 1) / PG_KC;
  if (splits < 1 || splits > p.chunks) CIE_FAIL("decode_program: %d slices of %d chunks of K", splits, p.chunks);
  {
    LaunchPlan* plan = nullptr;
    if (launch_plan(&plan) != 0) return 1;
    if (splits > plan->sms) CIE_FAIL("decode_program: %d slices of K on %d CTAs", splits, plan->sms);
  }
  if (splits > 1 && !partial) CIE_FAIL("decode_program: slices of K need memory for their partial sums");
  if (p.row_sq && p.sq_tiles < 1) CIE_FAIL("decode_program: %d tiles of sums of squares", p.sq_tiles);
  p.splits = splits;
  p.partial = partial;
  if (!bw::tensor_map_bf16(w, p.n, p.k, PG_BN, &p.map0)) CIE_FAIL("decode_program: cuTensorMapEncodeTiled failed for a weight");
  p.kind = kGemm;
  phases[0] = p;
  *count = 1;
  if (splits > 1) {
    p.kind = kFinish;
    phases[1] = p;
    *count = 2;
  }
  return 0;
}

extern "C" int cie_program_gemm(void* phases, int* count, const void* x, int x_stride, const float* row_sq,
                                int sq_tiles, float eps, const void* w, const float* bias, void* out,
                                float* partial, float* residual, float* sq, void* scaled, const float* next_gain,
                                int m, int n, int k, int splits, int mode) {
  if (mode != kOutBF16 && mode != kOutF32 && mode != kOutSiluMul && mode != kOutResidual)
    CIE_FAIL("decode_program: product mode %d", mode);
  if (mode == kOutSiluMul && n % 32) CIE_FAIL("decode_program: the SiLU epilogue needs N a multiple of 32, got %d", n);
  if (mode == kOutResidual && (!residual || !sq)) CIE_FAIL("decode_program: the residual epilogue needs the stream and a place for the sums of squares");
  if ((scaled != nullptr) != (next_gain != nullptr)) CIE_FAIL("decode_program: the scaled copy needs both its buffer and the gain");
  if ((mode == kOutBF16 || mode == kOutF32 || mode == kOutSiluMul) && !out) CIE_FAIL("decode_program: no output");
  Phase p = {};
  p.m = m; p.n = n; p.k = k; p.mode = mode;
  p.x = (const bf16*)x; p.x_stride = x_stride; p.row_sq = row_sq; p.sq_tiles = sq_tiles; p.eps = eps;
  p.bias = bias; p.out = out; p.residual = residual; p.sq = sq; p.scaled = (bf16*)scaled; p.next_gain = next_gain;
  return fill_gemm(static_cast<Phase*>(phases), count, p, w, splits, partial);
}

// The stacked q/k/v projection with the rotary epilogue: q rotated to q_out [m, q_stride], k
// (rotated) and v into the token's slot of the cache pages unless write_cache is 0.  The weight
// and bias rows of q and k heads are in the paired layout; head and rotary size multiples of 32.
extern "C" int cie_program_rope(void* phases, int* count, const void* x, int x_stride, const float* row_sq,
                                int sq_tiles, float eps, const void* w, const float* bias, float* partial,
                                void* q_out, int q_stride, const int* positions, const int* request_of_token,
                                const int* table, int table_width, int num_pages, void* k_pool, void* v_pool,
                                const float* inv_freq, int m, int q_heads, int kv_heads, int dim, int rot,
                                int page_size, int write_cache, int k, int splits) {
  if (!q_out || !positions || !inv_freq) CIE_FAIL("decode_program: the rotary epilogue needs q_out, positions and frequencies");
  if (dim < 32 || dim % 32 || rot < 32 || rot % 32 || rot > dim)
    CIE_FAIL("decode_program: head size %d and rotary size %d must be multiples of 32", dim, rot);
  if (q_heads < 1 || kv_heads < 1) CIE_FAIL("decode_program: %d query and %d kv heads", q_heads, kv_heads);
  if (write_cache && (!request_of_token || !table || !k_pool || !v_pool || page_size < 1))
    CIE_FAIL("decode_program: the cache write needs the block table and the pools");
  Phase p = {};
  p.m = m; p.n = (q_heads + 2 * kv_heads) * dim; p.k = k; p.mode = kOutRope;
  p.x = (const bf16*)x; p.x_stride = x_stride; p.row_sq = row_sq; p.sq_tiles = sq_tiles; p.eps = eps;
  p.bias = bias;
  p.q_out = (bf16*)q_out; p.q_stride = q_stride; p.positions = positions; p.request_of_token = request_of_token;
  p.table = table; p.table_width = table_width; p.num_pages = num_pages;
  p.k_pool = (bf16*)k_pool; p.v_pool = (bf16*)v_pool; p.inv_freq = inv_freq;
  p.q_heads = q_heads; p.kv_heads = kv_heads; p.dim = dim; p.rot = rot; p.page_size = page_size;
  p.write_cache = write_cache;
  return fill_gemm(static_cast<Phase*>(phases), count, p, w, splits, partial);
}

// One query token for each of `requests` requests (token row = request index) over the paged
// cache.  key_splits: CTAs a unit (request, kv head, 16 heads) may use, 1 .. cie_program_max_key_splits();
// a request uses as many as leave each min_keys keys.  shares: float32 [requests * kv_heads *
// ceil(group / 16)][key_splits][16][head size + 4].  Writes the attention phase and, with
// key_splits > 1, the merge phase.  Needs pages of a power of two >= 16 tokens and 16-byte-aligned pools.
extern "C" int cie_program_attention(void* phases, int* count, const void* q, int q_stride, void* out, int out_stride,
                                     const void* k_pool, const void* v_pool, const int* table, int table_width,
                                     int num_pages, const int* context_lens, int requests, int q_heads,
                                     int kv_heads, int page_size, int key_splits, int min_keys, float* shares,
                                     float scale, int window) {
  if (requests <= 0 || requests > 16) CIE_FAIL("decode_program: attention takes 1 to 16 requests, got %d", requests);
  if (kv_heads < 1 || q_heads % kv_heads) CIE_FAIL("decode_program: %d query heads over %d kv heads", q_heads, kv_heads);
  if (key_splits < 1 || key_splits > PG_MAX_KEY_SPLITS) CIE_FAIL("decode_program: 1 to %d CTAs per request, got %d", PG_MAX_KEY_SPLITS, key_splits);
  if (q_stride % 8 || out_stride % 4) CIE_FAIL("decode_program: row strides must keep the alignment of the rows");
  if (min_keys < 1) CIE_FAIL("decode_program: min_keys must be positive");
  if (key_splits > 1 && !shares) CIE_FAIL("decode_program: several CTAs per request need memory for their shares");
  const int shift = page_shift_of(page_size);
  if (shift < 4 || ((reinterpret_cast<uintptr_t>(k_pool) | reinterpret_cast<uintptr_t>(v_pool)) & 15) != 0)
    CIE_FAIL("decode_program: needs pages of a power of two >= 16 (got %d) and 16-byte-aligned pools", page_size);
  Phase p = {};
  p.kind = kAttention;
  p.m = requests;
  p.q_out = (bf16*)q; p.q_stride = q_stride; p.attn_out = (bf16*)out; p.out_stride = out_stride;
  p.k_pool = (bf16*)k_pool; p.v_pool = (bf16*)v_pool; p.table = table; p.table_width = table_width;
  p.num_pages = num_pages; p.context_lens = context_lens; p.q_heads = q_heads; p.kv_heads = kv_heads;
  p.page_size = page_size; p.page_shift = shift; p.group = q_heads / kv_heads; p.head_chunks = (p.group + 15) / 16;
  p.key_splits = key_splits; p.min_keys = min_keys; p.shares = shares; p.window = window;
  p.scale_log2 = scale * 1.4426950408889634f;
  const long long rows = (long long)num_pages * kv_heads * page_size;
  if (!bw::tensor_map_bf16_row_blocks(k_pool, rows, D, 16, &p.map0) || !bw::tensor_map_bf16_row_blocks(v_pool, rows, D, 16, &p.map1))
    CIE_FAIL("decode_program: cuTensorMapEncodeTiled failed for the cache pools");
  Phase* list = static_cast<Phase*>(phases);
  list[0] = p;
  *count = 1;
  if (key_splits > 1) {
    p.kind = kMerge;
    list[1] = p;
    *count = 2;
  }
  return 0;
}

// Device memory holding a copy of `bytes` bytes at `host` (a program's phases and its end mark).
// May be called while the calling thread captures a CUDA graph on some stream: the allocation and
// the copy are not part of the capture (they run at once, on a stream of their own).
extern "C" int cie_program_upload(const void* host, long long bytes, void** device) {
  if (!host || bytes <= 0 || !device) CIE_FAIL("decode_program: nothing to upload");
  cudaStreamCaptureMode mode = cudaStreamCaptureModeRelaxed;
  cudaError_t status = cudaThreadExchangeStreamCaptureMode(&mode);
  if (status != cudaSuccess) CIE_FAIL("decode_program: cudaThreadExchangeStreamCaptureMode: %s", cudaGetErrorString(status));
  void* memory = nullptr;
  cudaStream_t side = nullptr;
  status = cudaMalloc(&memory, (size_t)bytes);
  if (status == cudaSuccess) status = cudaStreamCreateWithFlags(&side, cudaStreamNonBlocking);
  if (status == cudaSuccess) status = cudaMemcpyAsync(memory, host, (size_t)bytes, cudaMemcpyHostToDevice, side);
  if (status == cudaSuccess) status = cudaStreamSynchronize(side);
  if (side) cudaStreamDestroy(side);
  cudaThreadExchangeStreamCaptureMode(&mode);
  if (status != cudaSuccess) {
    if (memory) cudaFree(memory);
    CIE_FAIL("decode_program: uploading %lld bytes: %s", bytes, cudaGetErrorString(status));
  }
  *device = memory;
  return 0;
}

// Gives back what cie_program_upload returned (waits for the device first: not during a capture).
extern "C" int cie_program_free(void* device) {
  if (device && cudaFree(device) != cudaSuccess) CIE_FAIL("decode_program: cudaFree failed");
  return 0;
}

// Runs a program: `tape` is device memory holding `phases` phases followed by one zeroed phase
// (the end mark); `slab_bytes` the most shared memory any of its products needs for its token rows
// (8 or 16 rows x the columns of the longest K slice x 2 bytes; the ring gets what is left);
// `counter` one 32-bit word of device memory for the barriers (zeroed here, on the
// stream).  One CTA per SM, launched cooperatively so that all of them are resident at one time.
extern "C" int cie_program_launch(const void* tape, int phases, int slab_bytes, void* counter, int* err, void* stream) {
  if (phases <= 0) return 0;
  if (!tape || !counter || !err) CIE_FAIL("decode_program: null argument");
  if (slab_bytes < 0) CIE_FAIL("decode_program: slab of %d bytes", slab_bytes);
  if (reinterpret_cast<uintptr_t>(tape) & 127) CIE_FAIL("decode_program: the phases must be 128-byte aligned");
  LaunchPlan* plan = nullptr;
  if (launch_plan(&plan) != 0) return 1;
  cudaError_t status = cudaMemsetAsync(counter, 0, sizeof(unsigned), (cudaStream_t)stream);
  if (status != cudaSuccess) CIE_FAIL("decode_program: cudaMemsetAsync: %s", cudaGetErrorString(status));
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3(plan->sms);
  config.blockDim = dim3(PG_THREADS);
  int stages = 0;
  size_t smem = 0;
  if (ring_for(*plan, slab_bytes, &stages, &smem) != 0) return 1;
  if (smem > plan->configured) {
    status = cudaFuncSetAttribute(decode_program_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (status != cudaSuccess) CIE_FAIL("decode_program: shared memory %zu: %s", smem, cudaGetErrorString(status));
    plan->configured = smem;
  }
  config.dynamicSmemBytes = smem;
  config.stream = (cudaStream_t)stream;
  cudaLaunchAttribute attributes[1];
  attributes[0].id = cudaLaunchAttributeCooperative;
  attributes[0].val.cooperative = 1;
  config.attrs = attributes;
  config.numAttrs = plan->cooperative ? 1 : 0;
  status = cudaLaunchKernelEx(&config, decode_program_kernel, static_cast<const Phase*>(tape),
                              static_cast<unsigned*>(counter), err, stages, slab_bytes);
  if (status != cudaSuccess) CIE_FAIL("decode_program: launch failed: %s", cudaGetErrorString(status));
  return 0;
}
