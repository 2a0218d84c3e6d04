// Device helpers shared by the tensor-core attention kernels of one head size (-DHEAD_DIM): fragment
// loads, mma.sync, the address of an element in a key/value tile as a TMA copy leaves it, the
// score and accumulate steps for 16-key blocks and the running-maximum softmax update.
#pragma once

#include "blackwell.cuh"
#include "common.cuh"

#include <cfloat>

#ifndef HEAD_DIM
#define HEAD_DIM 128
#endif

namespace cie {

using bf16 = __nv_bfloat16;
using bw::mbar_expect_tx;
using bw::mbar_init;
using bw::mbar_wait;
using bw::smem_u32;
using bw::tma_load_2d;
constexpr int D = HEAD_DIM;
static_assert(D % 16 == 0 && D >= 16 && D <= 256, "head size must be a multiple of 16 up to 256");
constexpr int ROW = D + 8;          // shared-memory row in elements: odd number of 16-byte units
constexpr int CHUNKS = D / 8;       // 16-byte pieces of a row
constexpr int KSTEPS = D / 16;
constexpr int NTILES_D = D / 8;
constexpr uint32_t ROW_BYTES = D * sizeof(__nv_bfloat16);

__device__ __forceinline__ void cp_async16(void* dst, const void* src, bool valid) {
  const int bytes = valid ? 16 : 0;  // 0: the 16 bytes are filled with zeros, nothing is read
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(smem_u32(dst)), "l"(src), "r"(bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

__device__ __forceinline__ void bulk_copy(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ float quad_max(float v) {
  v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 1));
  return fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 2));
}
__device__ __forceinline__ float quad_sum(float v) {
  v += __shfl_xor_sync(0xffffffffu, v, 1);
  return v + __shfl_xor_sync(0xffffffffu, v, 2);
}

struct Pools {
  const bf16* k;
  const bf16* v;
  const int* table;   // [requests][table_width]
  int table_width;
  int num_pages;
  int kv_heads;
  int page_size;
};

// Address of key `key` of request row `row` for kv head `kvh`, or nullptr (and an error bit) if
// the block table has no page there.
__device__ __forceinline__ long long kv_offset(const Pools& pools, const int* row, int key, int kvh, int* err) {
  const int index = key / pools.page_size;
  const int page = index < pools.table_width ? row[index] : -1;
  if (page < 0 || page >= pools.num_pages) {
    atomicOr(err, kErrBadPage);
    return -1;
  }
  return (((long long)page * pools.kv_heads + kvh) * pools.page_size + key % pools.page_size) * D;
}

// One 16-row block against NB*16 keys held in shared memory (rows of ROW elements).
// q_frag: A fragments of the 16 query rows.  s: NB*2 score tiles of 16 x 8.
// Address of element (row, col) of a key/value tile in shared memory, col a multiple of 8.
// SW == false: rows of ROW elements (padded).  SW == true: the layout a TMA tensor copy with
// 128-byte swizzle leaves: 16-row sub-tiles of 64 columns, 2 KB each, the 16-byte piece c of
// row r stored at piece position c ^ (r & 7).
// For head sizes 64 and 128 one TMA copy brings a whole 16-key tile (a 4-dimensional box, see
// tensor_map_bf16_row_blocks): every 8 rows are two swizzled 8 x 64 pieces side by side.
constexpr bool kBlockCopies = D == 64 || D == 128;
template <bool SW>
__device__ __forceinline__ const bf16* tile_ptr(const bf16* base, int row, int col) {
  if constexpr (!SW) return base + row * ROW + col;
  else if constexpr (kBlockCopies)
    return base + (row >> 3) * (D * 8) + (col >> 6) * 512 + (row & 7) * 64 + ((((col & 63) >> 3) ^ (row & 7)) << 3);
  else return base + (col >> 6) * 1024 + row * 64 + ((((col & 63) >> 3) ^ (row & 7)) << 3);
}

template <int NB, bool SW = false>
__device__ __forceinline__ void scores(const uint32_t (&q_frag)[KSTEPS][4], const bf16* k_tile,
                                       float (&s)[NB * 2][4], int lane) {
  static_assert(!SW || NB == 1, "swizzled tiles hold 16 keys");
  // two accumulator sets (even and odd k-steps) halve the chain of dependent tensor-core
  // instructions; they are added at the end
  float s2[NB * 2][4];
#pragma unroll
  for (int i = 0; i < NB * 2; ++i) {
    s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
    s2[i][0] = s2[i][1] = s2[i][2] = s2[i][3] = 0.f;
  }
  const int mi = lane >> 3, r = lane & 7;
#pragma unroll
  for (int kk = 0; kk < KSTEPS; ++kk) {
#pragma unroll
    for (int nb = 0; nb < NB; ++nb) {
      uint32_t b[4];
      ldsm_x4(b, tile_ptr<SW>(k_tile, nb * 16 + (mi >> 1) * 8 + r, kk * 16 + (mi & 1) * 8));
      if (kk & 1) {
        mma_bf16(s2[2 * nb], q_frag[kk], b[0], b[1]);
        mma_bf16(s2[2 * nb + 1], q_frag[kk], b[2], b[3]);
      } else {
        mma_bf16(s[2 * nb], q_frag[kk], b[0], b[1]);
        mma_bf16(s[2 * nb + 1], q_frag[kk], b[2], b[3]);
      }
    }
  }
#pragma unroll
  for (int i = 0; i < NB * 2; ++i) {
    s[i][0] += s2[i][0]; s[i][1] += s2[i][1]; s[i][2] += s2[i][2]; s[i][3] += s2[i][3];
  }
}

// o += P V for NB*16 keys; p: probabilities in the score-tile layout.
template <int NB, bool SW = false>
__device__ __forceinline__ void accumulate(const float (&p)[NB * 2][4], const bf16* v_tile,
                                           float (&o)[NTILES_D][4], int lane) {
  const int mi = lane >> 3, r = lane & 7;
#pragma unroll
  for (int kb = 0; kb < NB; ++kb) {
    uint32_t a[4];
    a[0] = pack_bf16(p[2 * kb][0], p[2 * kb][1]);
    a[1] = pack_bf16(p[2 * kb][2], p[2 * kb][3]);
    a[2] = pack_bf16(p[2 * kb + 1][0], p[2 * kb + 1][1]);
    a[3] = pack_bf16(p[2 * kb + 1][2], p[2 * kb + 1][3]);
#pragma unroll
    for (int db = 0; db < KSTEPS; ++db) {
      uint32_t b[4];
      ldsm_x4_trans(b, tile_ptr<SW>(v_tile, kb * 16 + (mi & 1) * 8 + r, db * 16 + (mi >> 1) * 8));
      mma_bf16(o[2 * db], a, b[0], b[1]);
      mma_bf16(o[2 * db + 1], a, b[2], b[3]);
    }
  }
}

// Running-maximum softmax update for the two rows (g, g + 8) a thread holds.
// s holds scores already multiplied by scale * log2(e); masked entries are -inf.
// HALVES == 1: rows 8..15 of the block are not in use (at most 8 heads share a kv head) and are
// skipped.  The accumulator is rescaled only when some row's maximum moved (a warp-wide vote).
template <int NT, int HALVES = 2>
__device__ __forceinline__ void softmax_update(float (&s)[NT][4], float (&m)[2], float (&l)[2],
                                               float (&o)[NTILES_D][4]) {
  float tile_max[2] = {-INFINITY, -INFINITY};
#pragma unroll
  for (int i = 0; i < NT; ++i) {
    tile_max[0] = fmaxf(tile_max[0], fmaxf(s[i][0], s[i][1]));
    if (HALVES == 2) tile_max[1] = fmaxf(tile_max[1], fmaxf(s[i][2], s[i][3]));
  }
  float alpha[2] = {1.f, 1.f};
  bool moved = false;
#pragma unroll
  for (int h = 0; h < HALVES; ++h) {
    const float m_new = fmaxf(m[h], quad_max(tile_max[h]));
    if (m_new != m[h]) {
      alpha[h] = (m[h] == -INFINITY) ? 0.f : exp2f(m[h] - m_new);
      moved = true;
    }
    m[h] = m_new;
  }
  float sum[2] = {0.f, 0.f};
#pragma unroll
  for (int i = 0; i < NT; ++i) {
    s[i][0] = (m[0] == -INFINITY) ? 0.f : exp2f(s[i][0] - m[0]);
    s[i][1] = (m[0] == -INFINITY) ? 0.f : exp2f(s[i][1] - m[0]);
    sum[0] += s[i][0] + s[i][1];
    if (HALVES == 2) {
      s[i][2] = (m[1] == -INFINITY) ? 0.f : exp2f(s[i][2] - m[1]);
      s[i][3] = (m[1] == -INFINITY) ? 0.f : exp2f(s[i][3] - m[1]);
      sum[1] += s[i][2] + s[i][3];
    } else {
      s[i][2] = s[i][3] = 0.f;
    }
  }
  l[0] = l[0] * alpha[0] + sum[0];
  if (HALVES == 2) l[1] = l[1] * alpha[1] + sum[1];
  if (__any_sync(0xffffffffu, moved)) {
#pragma unroll
    for (int i = 0; i < NTILES_D; ++i) {
      o[i][0] *= alpha[0];
      o[i][1] *= alpha[0];
      if (HALVES == 2) {
        o[i][2] *= alpha[1];
        o[i][3] *= alpha[1];
      }
    }
  }
}

}  // namespace cie
