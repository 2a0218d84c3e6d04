// Weight-streaming matrix product for few rows (decode): out[M, N] = x[M, K] * W[N, K]^T, M <= 16.
//
// With so few tokens a projection is bound by reading W once from HBM, so the kernel is
// built around the weight stream: a CTA owns BN weight rows and a slice of K, and pulls
// [BN x 128] weight tiles through a four-stage pipeline (two TMA tensor copies per tile with
// 128-byte swizzle, completing on the stage's mbarrier; cp.async for a weight whose address or
// row length TMA cannot take) while tensor cores
// (mma.sync m16n8k16, bfloat16 in, float32 accumulate) multiply them with the matching slice
// of x.  Weights are the 16-row operand (the roles of the two operands are swapped), tokens are
// the 8-wide operand, so 8 tokens cost no more tensor work than 1.
// Matrices with few rows are cut along K as well (grid.y) so that every SM streams; the
// partial sums are written as float32 [splits][M][N] and added up, in a fixed order, by the
// kernel that consumes them (residual-add + RMSNorm, or rotary + cache write), which also adds
// the bias.  Epilogues: bfloat16 or float32 output with bias; float32 partials; SiLU(gate) * up
// when the weight holds gate and up rows interleaved in blocks of BN/2; and the residual
// epilogue: the CTAs that share weight rows form a thread-block cluster, add their K slices up
// through distributed shared memory in a fixed order, add the sum into the float32 residual
// stream and leave the sum of squares of each new row slice for the product that normalises next.
//
// The rotary epilogue works the same way for the stacked q/k/v projection of a decode step: the
// cluster adds its K slices, then rotates q and k (weight rows of a head are laid out so that the
// two elements of a rotary pair are 16 lanes apart in one CTA), writes q for the attention kernel
// and k and v straight into their cache pages.
//
// With the gain of the norm that follows, the residual epilogue also writes bfloat16(new row * gain): the
// un-normalised input of the next product, which multiplies its own result rows by
// rstd = rsqrt(mean square + eps), formed from those sums of squares, in its epilogue.  One
// rounding to bfloat16 either way, and no RMSNorm kernel in between.
//
// The reference runs these products through cuBLAS (zeeshan8281/cloud-inference-from-scratch
// src/cloud_engine/model.py:100,134-136,217,227).
#include "blackwell.cuh"
#include "common.cuh"

#include <cooperative_groups.h>

CIE_DEFINE_LAST_ERROR()

namespace cie {

namespace cg = cooperative_groups;
using bf16 = __nv_bfloat16;
constexpr int BK = 128;
constexpr int WROW = BK + 8;
// Pipeline depth: four stages for up to 8 tokens; three for 9..16, whose larger x tiles would
// otherwise cost an SM one resident CTA (and a wide product a second wave).
template <int MT>
constexpr int stages_for() { return MT == 1 ? 4 : 3; }
// A CTA's tile is divided among more warps than its 16-row halves: the small products of a step are
// chains of dependent instructions of a few warps an SM, so the work of ONE warp, not the weight
// stream, sets their time (measured on a B200 at 13 cycles an instruction and 7 % of the issue slots
// in use).  A warp takes 16 weight rows, one 8-token tile and every second pair of k-steps of a
// tile: four warps a CTA up to 8 tokens, eight for 9 to 16; the shares of K meet in shared memory
// before the epilogue, whose rows are then divided among all warps too.  (Four shares of K at up to
// 8 tokens were slower again: 1.82 ms a step against 1.77.)
template <int MT>
constexpr int token_split_for() { return MT; }
#ifndef STREAM_K_SPLIT_1
#define STREAM_K_SPLIT_1 2
#endif
#ifndef STREAM_K_SPLIT_2
#define STREAM_K_SPLIT_2 2
#endif
template <int MT>
constexpr int k_split_for() { return MT == 1 ? STREAM_K_SPLIT_1 : STREAM_K_SPLIT_2; }
constexpr int KSTEPS = BK / 16;

using bw::smem_u32;
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

// ---- exchange inside a cluster without meeting: asynchronous stores into a peer's shared memory
// that count on a barrier there
__device__ __forceinline__ uint32_t map_to_rank(const void* p, uint32_t rank) {
  uint32_t remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(smem_u32(p)), "r"(rank));
  return remote;
}
__device__ __forceinline__ void cluster_arrive() { asm volatile("barrier.cluster.arrive.release;" ::: "memory"); }
__device__ __forceinline__ void cluster_wait() { asm volatile("barrier.cluster.wait.acquire;" ::: "memory"); }
__device__ __forceinline__ void push_f32(uint32_t remote, float v, uint32_t bar) {
  asm volatile("st.async.shared::cluster.mbarrier::complete_tx::bytes.f32 [%0], %1, [%2];"
               ::"r"(remote), "f"(v), "r"(bar) : "memory");
}

[[maybe_unused]] constexpr int kOutBF16 = 0;
constexpr int kOutF32 = 1, kOutPartial = 2, kOutSiluMul = 3, kOutResidual = 4, kOutRope = 5;

struct StreamArgs {
  const bf16* x;       // [M, K]
  const bf16* w;       // [N, K]
  const float* bias;   // [N] or null (modes 0, 1)
  void* out;           // mode 0: bf16 [M, N]; 1: float [M, N]; 2: float [splits, M, N]; 3: bf16 [M, N/2]
  int m, n, k;
  int k_per_split;     // multiple of BK
  int mode;
  int early_trigger;   // mode 4: let the next kernel start before this one has waited for its predecessor
  int push;            // modes 4, 5: the K slices reach the CTA that finishes a row by asynchronous stores
                       // into its shared memory (1) instead of loads from the others' after a cluster barrier (0)
  int* err;            // error word for a wait that ran out (TMA variant), may be null
  // row scale: with row_sq the result rows are multiplied by rstd[m] = rsqrt(sum over tiles of
  // row_sq[m][tile] / K + eps) before bias, partial-sum output or activation (x then holds
  // bfloat16(h * gain) of the rows h whose squares were summed)
  const float* row_sq;   // [M, row_tiles] or null
  int row_tiles;
  float eps;
  // mode 4: residual[m][n] += sum over the cluster's K slices (+ bias);
  // sq[m][blockIdx.x] = sum of squares of the new residual[m][n0 .. n0 + BN)
  float* residual;     // [M, N]
  float* sq;           // [M, gridDim.x]
  // mode 4, optional: scaled[m][n] = bfloat16(new residual[m][n] * next_gain[n])
  bf16* scaled;        // [M, N] or null
  const float* next_gain;
  // mode 5: the product is the stacked q/k/v projection [M, (Hq + 2 Hkv) * D] of M tokens, q and k
  // rows in the paired layout (see paired_column in elementwise.cu)
  bf16* q_out;         // [M, q_stride]: rotated q, natural order
  int q_stride;
  const int* positions;          // [M]
  const int* request_of_token;   // [M]
  const int* table;              // [requests][table_width]
  int table_width, num_pages;
  bf16* k_pool;        // [pages][Hkv][page_size][D]
  bf16* v_pool;
  const float* inv_freq;         // [rot / 2]
  int q_heads, kv_heads, dim, rot, page_size, write_cache;
};

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

__device__ int timeout_sink;   // takes the time-out bit when the caller gave no error word

// rstd[m] = rsqrt(sum of row_sq[m][0 .. row_tiles) / K + eps) for the MP token rows, warp w taking
// rows w, w + warps, ...; a lane loads PER_LANE values per row at once (tiles beyond 32 * PER_LANE in
// a loop of their own).
template <int MP, int THREADS, int PER_LANE>
__device__ __forceinline__ void row_rstd(const StreamArgs& a, float* rstd_s, int warp, int lane) {
  constexpr int WARPS = THREADS / 32, ROWS = MP / WARPS;
  float vals[ROWS][PER_LANE];
#pragma unroll
  for (int i = 0; i < ROWS; ++i) {
    const int m = warp + i * WARPS;
#pragma unroll
    for (int j = 0; j < PER_LANE; ++j) {
      const int t = lane + 32 * j;
      vals[i][j] = (m < a.m && t < a.row_tiles) ? __ldg(a.row_sq + (size_t)m * a.row_tiles + t) : 0.f;
    }
  }
#pragma unroll
  for (int i = 0; i < ROWS; ++i) {
    const int m = warp + i * WARPS;
    float sum = 0.f;
#pragma unroll
    for (int j = 0; j < PER_LANE; ++j) sum += vals[i][j];
    if (m < a.m)
      for (int t = lane + 32 * PER_LANE; t < a.row_tiles; t += 32) sum += a.row_sq[(size_t)m * a.row_tiles + t];
    sum = warp_sum(sum);
    if (lane == 0) rstd_s[m] = m < a.m ? rsqrtf(sum / (float)a.k + a.eps) : 0.f;
  }
}

// Shared-memory layout.  cp.async variant: weight rows padded to WROW elements.  TMA variant: a
// weight stage is two boxes of [BN rows x 64 columns] as the copy leaves them (rows of 128 bytes,
// the 16-byte piece c of row r at position c ^ (r & 7)), stages 1024-byte aligned.
template <int BN, bool TMA>
constexpr int w_stage_elems() { return TMA ? BN * BK : BN * WROW; }

template <int MT, int BN, bool TMA>
__global__ void __launch_bounds__(BN * 2 * token_split_for<MT>() * k_split_for<MT>())
gemm_stream_kernel(const __grid_constant__ CUtensorMap w_map, const StreamArgs a) {
  constexpr int TS = token_split_for<MT>(), KS = k_split_for<MT>();
  constexpr int ROW_WARPS = BN / 16;
  constexpr int THREADS = BN * 2 * TS * KS;   // a warp per 16 weight rows, per token tile(s), per share of the k-steps
  constexpr int MTW = MT / TS;      // 8-token tiles of a warp
  constexpr int MP = MT * 8;        // padded token count
  constexpr int WSTAGE = w_stage_elems<BN, TMA>();
  constexpr int XSTAGE = MP * WROW * 2;
  constexpr int STAGES = stages_for<MT>();
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  unsigned char* smem_base = TMA ? reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023)
                                 : smem_raw;
  bf16* w_s = reinterpret_cast<bf16*>(smem_base);           // [STAGES][WSTAGE]
  unsigned char* x_s = reinterpret_cast<unsigned char*>(w_s + STAGES * WSTAGE);   // [STAGES][XSTAGE]
  __shared__ __align__(8) uint64_t full[STAGES];
  __shared__ float rstd_s[MP];
  // cluster epilogues with a.push: what the other CTAs of the cluster send of the rows this CTA
  // finishes, [peer, itself left out][row of this CTA][32 columns]; never more than MP rows
  __shared__ float inbox_s[MP * 32];
  __shared__ __align__(8) uint64_t inbox_bar;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  // which 16 weight rows, which token tiles and which k-steps of a tile this warp takes
  const int warp_row = warp % ROW_WARPS, warp_tok = (warp / ROW_WARPS) % TS, warp_k = warp / (ROW_WARPS * TS);
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
    bf16* wd = w_s + (step % STAGES) * WSTAGE;
    if constexpr (TMA) {
      // K slices end on a tile edge or at K itself, where the copy fills with zeros
      if (tid == 0) {
        bw::mbar_expect_tx(&full[step % STAGES], BN * BK * 2);
        bw::tma_load_2d(wd, &w_map, &full[step % STAGES], k0, n0);
        bw::tma_load_2d(wd + BN * 64, &w_map, &full[step % STAGES], k0 + 64, n0);
      }
    } else {
#pragma unroll
      for (int i = 0; i < (BN * 16) / THREADS; ++i) {   // BN rows x 16 pieces of 16 bytes
        const int e = tid + i * THREADS;
        const int r = e >> 4, c = e & 15;
        const int row = n0 + r, col = k0 + c * 8;
        const bool ok = row < a.n && col < k_end;
        cp_async16(wd + r * WROW + c * 8, ok ? a.w + (size_t)row * a.k + col : a.w, ok);
      }
    }
  };
  auto load_x = [&](int step) {
    int tile = step + rotate;
    if (tile >= steps) tile -= steps;
    const int k0 = k_begin + tile * BK;
    {
      bf16* xd = reinterpret_cast<bf16*>(x_s + (step % STAGES) * XSTAGE);
      for (int e = tid; e < MP * 16; e += THREADS) {
        const int r = e >> 4, c = e & 15;
        const int col = k0 + c * 8;
        const bool ok = r < a.m && col < k_end;
        cp_async16(xd + r * WROW + c * 8, ok ? a.x + (size_t)r * a.k + col : a.x, ok);
      }
    }
  };
  auto load_stage = [&](int step) {
    load_w(step);
    load_x(step);
  };

  // The weights do not depend on the kernel before this one: the CTA requests its first weight
  // tiles before waiting for it, so the weight stream overlaps the tail of that kernel.
  // (Asking L2 for the whole weight slice at this point was tried and made the step slower.)
  // the CTAs that share this block of weight rows (a cluster along grid.y), for the epilogues that
  // add their K slices up
  const bool gathers = (a.mode == kOutResidual || a.mode == kOutRope) && gridDim.y > 1;
  const bool pushes = gathers && a.push;
  const int size = gathers ? (int)gridDim.y : 1, rank = gathers ? (int)blockIdx.y : 0;
  if (TMA || pushes) {
    if (tid == 0) {
      if constexpr (TMA)
        for (int s = 0; s < STAGES; ++s) bw::mbar_init(&full[s], 1);
      if (pushes) bw::mbar_init(&inbox_bar, 1);
      bw::mbar_init_fence();
    }
    __syncthreads();
  }
  if (pushes) {
    // row m is finished by the CTA of rank m % size: this one expects the other CTAs' 32 values of
    // each of its rows, and tells the cluster that its inbox is ready (nobody waits here)
    const int rows_owned = rank < a.m ? (a.m - rank + size - 1) / size : 0;
    if (tid == 0 && rows_owned > 0) bw::mbar_expect_tx(&inbox_bar, (uint32_t)(rows_owned * (size - 1) * 32 * sizeof(float)));
    cluster_arrive();
  }
#pragma unroll
  for (int s = 0; s < STAGES - 1; ++s)
    if (s < steps) load_w(s);
  // A product with the residual epilogue may let the next kernel start already now, beside the
  // kernel before this one, if its caller says so (early_trigger): the caller knows that what
  // follows touches, before its own wait, only what no kernel of the same step writes (weight
  // tiles; key/value tiles of earlier steps), which is the rule for every kernel of this engine.
  const bool early = a.mode == kOutResidual && a.early_trigger;
  if (early) pdl_trigger();
  pdl_wait();
  if (!early) pdl_trigger();
#pragma unroll
  for (int s = 0; s < STAGES - 1; ++s) {
    if (s < steps) load_x(s);
    cp_async_commit();
  }
  if (a.row_sq) {
    // rstd of every token row from the partial sums of squares (used in the epilogue, behind
    // barriers); every load is issued before the first sum needs one
    if (a.row_tiles <= 64) row_rstd<MP, THREADS, 2>(a, rstd_s, warp, lane);
    else if (a.row_tiles <= 128) row_rstd<MP, THREADS, 4>(a, rstd_s, warp, lane);
    else row_rstd<MP, THREADS, 8>(a, rstd_s, warp, lane);
  }

  float acc[MTW][4];
#pragma unroll
  for (int i = 0; i < MTW; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;

  bool alive = true;
  for (int it = 0; it < steps; ++it) {
    cp_async_wait<STAGES - 2>();
    if constexpr (TMA) {
      // A wait that ran out has set the error bit.  The thread waits for nothing more but goes on
      // through the loop with the others (every barrier is still met; the result is void anyway).
      if (alive) alive = bw::mbar_wait(&full[it % STAGES], (it / STAGES) & 1, a.err ? a.err : &timeout_sink);
    }
    __syncthreads();
    if (it + STAGES - 1 < steps) load_stage(it + STAGES - 1);
    cp_async_commit();
    const bf16* ws = w_s + (it % STAGES) * WSTAGE;
    const unsigned char* xt_raw = x_s + (it % STAGES) * XSTAGE;
    const int wr = warp_row * 16 + (lane & 15);
#pragma unroll
    for (int kq = 0; kq < KSTEPS / 2 / KS; ++kq) {
      const int kp = kq * KS + warp_k;
      uint32_t a0[4], a1[4];
      if constexpr (TMA) {
        // 16-byte piece c of row wr: box c / 8, position (c % 8) ^ (wr % 8) in the 128-byte row
        const int c0 = (2 * kp) * 2 + (lane >> 4), c1 = c0 + 2;
        ldsm_x4(a0, ws + (c0 >> 3) * (BN * 64) + wr * 64 + (((c0 & 7) ^ (wr & 7)) << 3));
        ldsm_x4(a1, ws + (c1 >> 3) * (BN * 64) + wr * 64 + (((c1 & 7) ^ (wr & 7)) << 3));
      } else {
        ldsm_x4(a0, ws + wr * WROW + (2 * kp) * 16 + (lane >> 4) * 8);
        ldsm_x4(a1, ws + wr * WROW + (2 * kp + 1) * 16 + (lane >> 4) * 8);
      }
#pragma unroll
      for (int mt = 0; mt < MTW; ++mt) {
        uint32_t b[4];  // tokens (warp_tok * MTW + mt) * 8 .., k = kp*32 + {0, 8, 16, 24}
        {
          const bf16* xt = reinterpret_cast<const bf16*>(xt_raw);
          ldsm_x4(b, xt + ((warp_tok * MTW + mt) * 8 + (lane & 7)) * WROW + kp * 32 + (lane >> 3) * 8);
        }
        mma_bf16(acc[mt], a0, b[0], b[1]);
        mma_bf16(acc[mt], a1, b[2], b[3]);
      }
    }
  }
  cp_async_wait<0>();
  if constexpr (TMA) {
    // after a time-out copies may still be in flight: each stage gets one more bounded wait before
    // the shared memory they target is reused below or given up
    if (!alive && tid == 0)
      for (int late = max(0, steps - STAGES); late < steps; ++late)
        bw::mbar_wait(&full[late % STAGES], (late / STAGES) & 1, a.err ? a.err : &timeout_sink);
  }
  __syncthreads();

  // ---- epilogue through shared memory: out_s[token][weight row]
  float* out_s = reinterpret_cast<float*>(smem_base);  // [MP][BN + 1]
  const int g = lane >> 2, t4 = lane & 3;
  if constexpr (KS > 1) {
    // the warps with the other k-steps put their sums down first (a copy of the staging tile each);
    // the first ones add them to their own, in the order of the shares
    if (warp_k > 0) {
      float* mine = out_s + warp_k * (MP * (BN + 1));
#pragma unroll
      for (int mt = 0; mt < MTW; ++mt) {
        const int m0 = (warp_tok * MTW + mt) * 8 + 2 * t4, r0 = warp_row * 16 + g;
        mine[m0 * (BN + 1) + r0] = acc[mt][0];
        mine[(m0 + 1) * (BN + 1) + r0] = acc[mt][1];
        mine[m0 * (BN + 1) + r0 + 8] = acc[mt][2];
        mine[(m0 + 1) * (BN + 1) + r0 + 8] = acc[mt][3];
      }
    }
    __syncthreads();
    if (warp_k == 0) {
#pragma unroll
      for (int share = 1; share < KS; ++share) {
        const float* theirs = out_s + share * (MP * (BN + 1));
#pragma unroll
        for (int mt = 0; mt < MTW; ++mt) {
          const int m0 = (warp_tok * MTW + mt) * 8 + 2 * t4, r0 = warp_row * 16 + g;
          acc[mt][0] += theirs[m0 * (BN + 1) + r0];
          acc[mt][1] += theirs[(m0 + 1) * (BN + 1) + r0];
          acc[mt][2] += theirs[m0 * (BN + 1) + r0 + 8];
          acc[mt][3] += theirs[(m0 + 1) * (BN + 1) + r0 + 8];
        }
      }
    }
  }
  if (warp_k == 0) {
#pragma unroll
    for (int mt = 0; mt < MTW; ++mt) {
      const int m0 = (warp_tok * MTW + mt) * 8 + 2 * t4, r0 = warp_row * 16 + g;
      const float s0 = a.row_sq ? rstd_s[m0] : 1.f, s1 = a.row_sq ? rstd_s[m0 + 1] : 1.f;
      out_s[m0 * (BN + 1) + r0] = acc[mt][0] * s0;
      out_s[(m0 + 1) * (BN + 1) + r0] = acc[mt][1] * s1;
      out_s[m0 * (BN + 1) + r0 + 8] = acc[mt][2] * s0;
      out_s[(m0 + 1) * (BN + 1) + r0 + 8] = acc[mt][3] * s1;
    }
  }
  __syncthreads();
  const int rows_per_owner = (MP + size - 1) / size;
  if (pushes) {
    if constexpr (BN == 32) {
      // every row of this CTA's slice goes to the CTA that finishes it; then this CTA waits for the
      // others' slices of its own rows.  Nobody meets: a CTA whose rows are done may leave.
      cluster_wait();   // every inbox of the cluster is ready (they said so when they started)
      for (int m = warp; m < a.m; m += THREADS / 32) {
        const int owner = m % size;
        if (owner == rank) continue;
        const int slot = rank < owner ? rank : rank - 1;
        push_f32(map_to_rank(inbox_s + (slot * rows_per_owner + m / size) * 32 + lane, owner),
                 out_s[m * (BN + 1) + lane], map_to_rank(&inbox_bar, owner));
      }
      if (rank < a.m && !bw::mbar_wait(&inbox_bar, 0, a.err ? a.err : &timeout_sink)) return;
    }
  }
  // slice `r` of the 32 values of row m (a row this CTA finishes), r in rank order
  auto slice_of = [&](cg::cluster_group& cluster, int r, int m) -> float {
    if (r >= size) return 0.f;
    if (!pushes) return cluster.map_shared_rank(out_s, r)[m * (BN + 1) + lane];
    if (r == rank) return out_s[m * (BN + 1) + lane];
    return inbox_s[((r < rank ? r : r - 1) * rows_per_owner + m / size) * 32 + lane];
  };
  if (a.mode == kOutResidual) {
    if constexpr (BN == 32) {
      // the CTAs of the cluster hold the K slices of the same [M x 32] block; row m is finished by
      // the CTA of rank m % size, whose first warp adds the slices in rank order
      cg::cluster_group cluster = cg::this_cluster();
      // this CTA's rows are rank, rank + size, ...: warp w takes every (THREADS / 32)-th of them;
      // what does not depend on the other CTAs is fetched before the cluster meets
      const int col = n0 + lane;
      const int first = rank + warp * size, stride = size * (THREADS / 32);
      constexpr int MAX_ROWS = (MP + THREADS / 32 - 1) / (THREADS / 32);   // per warp, if size == 1
      float old[MAX_ROWS];
      const float bias = (a.bias && col < a.n) ? a.bias[col] : 0.f;
      const float next_gain = (a.scaled && col < a.n) ? a.next_gain[col] : 0.f;
#pragma unroll
      for (int i = 0; i < MAX_ROWS; ++i) {
        const int m = first + i * stride;
        old[i] = (m < a.m && col < a.n) ? a.residual[(size_t)m * a.n + col] : 0.f;
      }
      if (!pushes) cluster.sync();
#pragma unroll
      for (int i = 0; i < MAX_ROWS; ++i) {
        const int m = first + i * stride;
        if (m >= a.m) break;
        // all remote loads are issued before the first addition (a cluster has at most 8 CTAs)
        float part[8];
#pragma unroll
        for (int r = 0; r < 8; ++r) part[r] = slice_of(cluster, r, m);
        float v = 0.f;
#pragma unroll
        for (int r = 0; r < 8; ++r) v += part[r];
        float square = 0.f;
        if (col < a.n) {
          const float updated = old[i] + (v + bias);
          a.residual[(size_t)m * a.n + col] = updated;
          if (a.scaled) a.scaled[(size_t)m * a.n + col] = __float2bfloat16_rn(updated * next_gain);
          square = updated * updated;
        }
        square = warp_sum(square);
        if (lane == 0) a.sq[(size_t)m * gridDim.x + blockIdx.x] = square;
      }
      if (!pushes) cluster.sync();   // nobody leaves while its shared memory may still be read
    }
    return;
  }
  if (a.mode == kOutRope) {
    if constexpr (BN == 32) {
      cg::cluster_group cluster = cg::this_cluster();
      const int first = rank + warp * size, stride = size * (THREADS / 32);
      constexpr int MAX_ROWS = (MP + THREADS / 32 - 1) / (THREADS / 32);
      // the 32 columns of this CTA lie in one head (D is a multiple of 32)
      const int q_width = a.q_heads * a.dim, kv_width = a.kv_heads * a.dim;
      const int region = n0 < q_width ? 0 : n0 < q_width + kv_width ? 1 : 2;   // q, k, v
      const int local = n0 - (region == 0 ? 0 : region == 1 ? q_width : q_width + kv_width);
      const int head = local / a.dim, p0 = local % a.dim;
      const int half = a.rot / 2;
      const bool rotary = region < 2 && p0 < a.rot;
      // natural position of this lane's element inside its head, and its rotary frequency
      const int pair = (p0 >> 5) * 16 + (lane & 15);
      const int d_out = rotary ? (lane < 16 ? pair : half + pair) : p0 + lane;
      const float freq = rotary ? a.inv_freq[pair] : 0.f;
      const float bias = a.bias ? a.bias[n0 + lane] : 0.f;
      int pos[MAX_ROWS];
      long long slot[MAX_ROWS];   // element offset of (page, head 0, slot in page, 0), or -1
#pragma unroll
      for (int i = 0; i < MAX_ROWS; ++i) {
        const int m = first + i * stride;
        pos[i] = 0;
        slot[i] = -1;
        if (m < a.m) {
          pos[i] = a.positions[m];
          if (region > 0 && a.write_cache) {
            const int index = pos[i] / a.page_size;
            const int page = index < a.table_width ? a.table[(size_t)a.request_of_token[m] * a.table_width + index] : -1;
            if (page < 0 || page >= a.num_pages) {
              if (lane == 0) atomicOr(a.err ? a.err : &timeout_sink, kErrBadPage);
            } else {
              slot[i] = ((long long)page * a.kv_heads * a.page_size + pos[i] % a.page_size) * a.dim;
            }
          }
        }
      }
      if (!pushes) cluster.sync();
#pragma unroll
      for (int i = 0; i < MAX_ROWS; ++i) {
        const int m = first + i * stride;
        if (m >= a.m) break;
        float part[8];
#pragma unroll
        for (int r = 0; r < 8; ++r) part[r] = slice_of(cluster, r, m);
        float v = 0.f;
#pragma unroll
        for (int r = 0; r < 8; ++r) v += part[r];
        v += bias;
        float result = v;
        if (rotary) {
          float sn, cs;
          sincosf((float)pos[i] * freq, &sn, &cs);
          const float other = __shfl_xor_sync(0xffffffffu, v, 16);
          result = lane < 16 ? v * cs - other * sn : v * cs + other * sn;
        }
        const bf16 rounded = __float2bfloat16_rn(result);
        if (region == 0) {
          a.q_out[(size_t)m * a.q_stride + head * a.dim + d_out] = rounded;
        } else if (slot[i] >= 0) {
          bf16* pool = region == 1 ? a.k_pool : a.v_pool;
          pool[slot[i] + (long long)head * a.page_size * a.dim + d_out] = rounded;
        }
      }
      if (!pushes) cluster.sync();
    }
    return;
  }
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

template <int MT, int BN, bool TMA>
static int launch_variant(const CUtensorMap& w_map, const StreamArgs& a, int splits, cudaStream_t stream) {
  constexpr int MP = MT * 8;
  constexpr size_t pipeline = (size_t)stages_for<MT>() * (w_stage_elems<BN, TMA>() + MP * WROW) * sizeof(bf16);
  constexpr size_t staging = (size_t)k_split_for<MT>() * MP * (BN + 1) * sizeof(float);
  constexpr size_t smem = (pipeline > staging ? pipeline : staging) + (TMA ? 1024 : 0);
  static bool configured = false;
  if (!configured) {
    cudaError_t status = cudaFuncSetAttribute(gemm_stream_kernel<MT, BN, TMA>,
                                              cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (status != cudaSuccess) CIE_FAIL("gemm_stream: shared memory %zu: %s", smem, cudaGetErrorString(status));
    configured = true;
  }
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3((a.n + BN - 1) / BN, splits);
  config.blockDim = dim3(BN * 2 * token_split_for<MT>() * k_split_for<MT>());
  config.dynamicSmemBytes = smem;
  config.stream = stream;
  cudaLaunchAttribute attributes[2];
  int count = 0;
  if (pdl_enabled()) {
    attributes[count].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attributes[count].val.programmaticStreamSerializationAllowed = 1;
    ++count;
  }
  if ((a.mode == kOutResidual || a.mode == kOutRope) && splits > 1) {
    // the K slices of one block of weight rows are one thread-block cluster
    attributes[count].id = cudaLaunchAttributeClusterDimension;
    attributes[count].val.clusterDim.x = 1;
    attributes[count].val.clusterDim.y = splits;
    attributes[count].val.clusterDim.z = 1;
    ++count;
  }
  config.attrs = attributes;
  config.numAttrs = count;
  cudaError_t status = cudaLaunchKernelEx(&config, gemm_stream_kernel<MT, BN, TMA>, w_map, a);
  if (status != cudaSuccess) CIE_FAIL("gemm_stream: launch failed: %s", cudaGetErrorString(status));
  return 0;
}

// TMA needs the weight 16-byte aligned with rows of a multiple of 16 bytes (K % 8 == 0 is checked
// by the caller); CIE_STREAM_TMA=0 in the environment keeps cp.async.
template <int MT, int BN>
static int launch(const StreamArgs& a, int splits, cudaStream_t stream) {
  static const bool allowed = [] {
    const char* value = getenv("CIE_STREAM_TMA");
    return !(value && value[0] == '0');
  }();
  CUtensorMap w_map = {};
  if (allowed && (reinterpret_cast<uintptr_t>(a.w) & 15) == 0 && bw::tensor_map_bf16(a.w, a.n, a.k, BN, &w_map))
    return launch_variant<MT, BN, true>(w_map, a, splits, stream);
  return launch_variant<MT, BN, false>(w_map, a, splits, stream);
}

// CIE_STREAM_PUSH=0 in the environment keeps the cluster epilogues on loads from the peers' shared
// memory between two cluster barriers.
static int push_enabled() {
  static const int enabled = [] {
    const char* value = getenv("CIE_STREAM_PUSH");
    return !(value && value[0] == '0') ? 1 : 0;
  }();
  return enabled;
}

// Cuts K into `splits` slices of whole tiles and picks the kernel for the row count.
static int dispatch(StreamArgs& a, int splits, int block_rows, cudaStream_t s) {
  const int k_tiles = (a.k + BK - 1) / BK;
  a.k_per_split = ((k_tiles + splits - 1) / splits) * BK;
  if (block_rows != 32) CIE_FAIL("gemm_stream: weight rows per CTA must be 32, got %d", block_rows);
  if (a.m <= 8) return launch<1, 32>(a, splits, s);
  return launch<2, 32>(a, splits, s);
}

}  // namespace cie

using namespace cie;

// The general entry point.
//  input:  x (bfloat16 [M, K]).  With row_sq ([M, row_tiles] float32 sums of squares of the rows
//          that x was made from) every result row m is multiplied by
//          rsqrt(sum of row_sq[m] / K + eps) before anything else is done with it.
//  output: mode 0 bf16 out, 1 float32 out, 2 float32 partials [splits][M][N] (bias ignored),
//          3 SiLU(gate)*up with gate/up rows interleaved in blocks of block_rows/2 (one split),
//          4 residual[M, N] += product (+ bias), sq[M, ceil(N / 32)] = sums of squares of the new
//          rows per block of 32 columns and, with next_gain, scaled[M, N] = bfloat16(new row *
//          next_gain); splits must be 1, 2, 4 or 8 (the size of a cluster), block_rows 32;
//          early_trigger != 0 lets the kernel after this one start before this one has waited for
//          the kernel before it (see the kernel).
// block_rows: weight rows per CTA; 32 is the one size built.
extern "C" int cie_gemm_stream_ex(const void* x, const float* row_sq, int row_tiles, float eps, const void* w,
                                  const float* bias, void* out, float* residual, float* sq, void* scaled,
                                  const float* next_gain, int m, int n, int k, int splits, int mode,
                                  int block_rows, int early_trigger, int* err, void* stream) {
  if (m <= 0 || n <= 0) return 0;
  if (!x || !w) CIE_FAIL("gemm_stream: null operand");
  if (m > 16) CIE_FAIL("gemm_stream: takes at most 16 rows, got %d", m);
  if (k < 8 || k % 8) CIE_FAIL("gemm_stream: K must be a multiple of 8 (16-byte rows), got %d", k);
  if (splits < 1) CIE_FAIL("gemm_stream: splits %d", splits);
  if (mode < 0 || mode > kOutResidual) CIE_FAIL("gemm_stream: mode %d (the rotary epilogue has its own entry point)", mode);
  if (mode == kOutSiluMul && (splits != 1 || n % 2)) CIE_FAIL("gemm_stream: the SiLU epilogue needs one split and an even N");
  if (mode == kOutResidual) {
    if (splits != 1 && splits != 2 && splits != 4 && splits != 8) CIE_FAIL("gemm_stream: the residual epilogue takes 1, 2, 4 or 8 splits, got %d", splits);
    if (block_rows != 32 || !residual || !sq) CIE_FAIL("gemm_stream: the residual epilogue needs 32-row blocks, a residual and a place for the sums of squares");
    if ((scaled != nullptr) != (next_gain != nullptr)) CIE_FAIL("gemm_stream: the scaled copy needs both its buffer and the gain");
  } else if (mode != kOutPartial && splits != 1) {
    CIE_FAIL("gemm_stream: %d splits need the partial-sum or the residual output", splits);
  }
  if (row_sq && row_tiles < 1) CIE_FAIL("gemm_stream: %d tiles of sums of squares", row_tiles);
  StreamArgs a = {};
  a.x = (const bf16*)x; a.w = (const bf16*)w; a.bias = bias; a.out = out;
  a.m = m; a.n = n; a.k = k; a.mode = mode; a.err = err;
  a.row_sq = row_sq; a.row_tiles = row_tiles; a.eps = eps;
  a.residual = residual; a.sq = sq; a.scaled = (bf16*)scaled; a.next_gain = next_gain;
  a.early_trigger = early_trigger;
  a.push = push_enabled();
  return dispatch(a, splits, block_rows, (cudaStream_t)stream);
}

// The stacked q/k/v projection of at most 16 decode tokens with the rotary epilogue (mode 5): q is
// written, rotated, to q_out [M, q_stride]; k (rotated) and v go to the token's slot of the cache
// pages unless write_cache is 0.  The weight (and bias) rows of q and k heads are in the paired
// layout; head size and rotary size are multiples of 32; splits is 1, 2, 4 or 8.
extern "C" int cie_gemm_stream_rope(const void* x, const float* row_sq, int row_tiles, float eps, const void* w,
                                    const float* bias, void* q_out, int q_stride, const int* positions,
                                    const int* request_of_token, const int* table, int table_width,
                                    int num_pages, void* k_pool, void* v_pool, const float* inv_freq, int m,
                                    int q_heads, int kv_heads, int dim, int rot, int page_size,
                                    int write_cache, int k, int splits, int* err, void* stream) {
  if (m <= 0) return 0;
  if (!x || !w || !q_out || !positions || !inv_freq) CIE_FAIL("gemm_stream_rope: null operand");
  if (m > 16) CIE_FAIL("gemm_stream_rope: takes at most 16 rows, got %d", m);
  if (k < 8 || k % 8) CIE_FAIL("gemm_stream_rope: K must be a multiple of 8, got %d", k);
  if (splits != 1 && splits != 2 && splits != 4 && splits != 8) CIE_FAIL("gemm_stream_rope: 1, 2, 4 or 8 splits, got %d", splits);
  if (dim < 32 || dim % 32 || rot < 32 || rot % 32 || rot > dim)
    CIE_FAIL("gemm_stream_rope: head size %d and rotary size %d must be multiples of 32", dim, rot);
  if (q_heads < 1 || kv_heads < 1) CIE_FAIL("gemm_stream_rope: %d query and %d kv heads", q_heads, kv_heads);
  if (write_cache && (!request_of_token || !table || !k_pool || !v_pool || page_size < 1))
    CIE_FAIL("gemm_stream_rope: the cache write needs the block table and the pools");
  if (row_sq && row_tiles < 1) CIE_FAIL("gemm_stream_rope: %d tiles of sums of squares", row_tiles);
  StreamArgs a = {};
  a.x = (const bf16*)x; a.w = (const bf16*)w; a.bias = bias;
  a.m = m; a.n = (q_heads + 2 * kv_heads) * dim; a.k = k; a.mode = kOutRope; a.err = err;
  a.row_sq = row_sq; a.row_tiles = row_tiles; a.eps = eps;
  a.q_out = (bf16*)q_out; a.q_stride = q_stride; a.positions = positions; a.request_of_token = request_of_token;
  a.table = table; a.table_width = table_width; a.num_pages = num_pages;
  a.k_pool = (bf16*)k_pool; a.v_pool = (bf16*)v_pool; a.inv_freq = inv_freq;
  a.q_heads = q_heads; a.kv_heads = kv_heads; a.dim = dim; a.rot = rot; a.page_size = page_size;
  a.write_cache = write_cache;
  a.push = push_enabled();
  return dispatch(a, splits, 32, (cudaStream_t)stream);
}

// bfloat16 input, modes 0..3.
extern "C" int cie_gemm_stream(const void* x, const void* w, const float* bias, void* out, int m,
                               int n, int k, int splits, int mode, int block_rows, int* err, void* stream) {
  if (mode == kOutResidual) CIE_FAIL("gemm_stream: the residual epilogue is reached through cie_gemm_stream_ex");
  return cie_gemm_stream_ex(x, nullptr, 0, 0.f, w, bias, out, nullptr, nullptr, nullptr, nullptr, m, n, k, splits,
                            mode, block_rows, 0, err, stream);
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
  if (cie_gemm_stream(x, w, nullptr, scratch, m, n, k, splits, kOutPartial, 32, nullptr, stream) != 0) return 1;
  // ... and are added up, with the bias, by one more kernel (launched without programmatic
  // overlap, so it starts after the product has finished)
  const size_t total = (size_t)m * n;
  int blocks = (int)((total + 255) / 256);
  if (blocks > 1024) blocks = 1024;
  noalloc_reduce_kernel<<<blocks, 256, 0, (cudaStream_t)stream>>>(scratch, bias, (bf16*)out, m, n, splits);
  CIE_CHECK_LAUNCH("gemm_stream_noalloc");
  return 0;
}
