// Small wrappers around the sm_100a instructions the tensor-memory kernels share: mbarriers with
// bounded waits, TMA tensor copies, tcgen05 (alloc, mma, commit, ld, st, fences) and the
// shared-memory matrix descriptors of 128-byte-swizzled tiles.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>

#include <cstdint>
#include <mutex>
#include <unordered_map>

namespace cie {
namespace bw {

constexpr int kErrTimeout = 8;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, int count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_init_fence() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
      : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
  return ok != 0;
}
// Bounded wait: after about two seconds of cycles it sets the time-out bit and returns false.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, int* err) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long start = clock64();
  while (!mbar_try_wait(bar, parity)) {
    if (clock64() - start > 4000000000ll) {
      atomicOr(err, kErrTimeout);
      return false;
    }
  }
  return true;
}

// x is the innermost coordinate: x * element size must be a multiple of 16 bytes.
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, uint64_t* bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void tma_load_3d(void* dst, const CUtensorMap* map, uint64_t* bar, int x, int y, int z) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(x), "r"(y), "r"(z) : "memory");
}
__device__ __forceinline__ void tma_load_4d(void* dst, const CUtensorMap* map, uint64_t* bar, int x, int y, int z, int w) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
      ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(x), "r"(y), "r"(z), "r"(w) : "memory");
}
__device__ __forceinline__ void tma_load_5d(void* dst, const CUtensorMap* map, uint64_t* bar, int x, int y, int z, int w, int v) {
  asm volatile(
      "cp.async.bulk.tensor.5d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6, %7}], [%2];"
      ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(x), "r"(y), "r"(z), "r"(w), "r"(v) : "memory");
}
// Orders this thread's ordinary shared-memory writes before later reads or writes of the same
// bytes by TMA or the tensor cores.
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// ---- tensor memory
template <int COLS>
__device__ __forceinline__ void tmem_alloc(uint32_t* slot) {   // whole warp
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(slot)), "n"(COLS));
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
}
template <int COLS>
__device__ __forceinline__ void tmem_free(uint32_t base) {     // whole warp
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(base), "n"(COLS));
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tc_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// Thread i of the warp receives 32 consecutive columns of tensor-memory lane (lane base + i).
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
      "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr));
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
      "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
      ::"r"(taddr),
        "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
        "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
        "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
        "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}

// Shared-memory matrix descriptor of a tile stored with 128-byte swizzle (what a TMA tensor copy
// with CU_TENSOR_MAP_SWIZZLE_128B leaves): rows of 128 bytes, groups of 8 rows 1024 bytes apart.
//  * reduction dimension contiguous ("K-major", rows are M or N indices): `leading` is not used;
//  * M/N dimension contiguous ("MN-major", rows are indices of the reduction dimension, 64
//    M/N elements per row): `leading` is the distance in bytes between blocks of 64 M/N elements.
// `stride`: distance in bytes between groups of 8 rows (1024 when the groups follow each other).
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t addr, uint32_t leading = 16, uint32_t stride = 1024) {
  uint64_t desc = 0;
  desc |= (uint64_t)((addr & 0x3FFFF) >> 4);
  desc |= (uint64_t)((leading >> 4) & 0x3FFF) << 16;
  desc |= (uint64_t)((stride >> 4) & 0x3FFF) << 32;
  desc |= (uint64_t)1 << 46;                   // descriptor version of sm_100
  desc |= (uint64_t)2 << 61;                   // SWIZZLE_128B
  return desc;
}
// Instruction descriptor of kind::f16 with bfloat16 operands and a float32 accumulator.
// b_mn_major: the B operand is stored with its N dimension contiguous.
__host__ __device__ constexpr uint32_t idesc_bf16(int m, int n, bool b_mn_major = false) {
  return (1u << 4) | (1u << 7) | (1u << 10) | (b_mn_major ? (1u << 16) : 0u) | ((uint32_t)(n >> 3) << 17) |
         ((uint32_t)(m >> 4) << 24);
}
__device__ __forceinline__ void umma_bf16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
      " tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}

// ---- host side: tensor maps
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_tiled() {
  static EncodeTiledFn encode = [] {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult status;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &status) != cudaSuccess ||
        status != cudaDriverEntryPointSuccess)
      fn = nullptr;
    return reinterpret_cast<EncodeTiledFn>(fn);
  }();
  return encode;
}

// Tensor map of a row-major bfloat16 matrix [rows, cols] (cols a multiple of 8, base 16-byte
// aligned) read in boxes of [box_rows, 64 columns] with 128-byte swizzle; what lies outside the
// matrix reads as zero.  Maps are kept by (address, shape, box) for the life of the process.
inline bool tensor_map_bf16(const void* ptr, long long rows, long long cols, int box_rows, CUtensorMap* out) {
  struct Key {
    const void* ptr; long long rows, cols; int box_rows;
    bool operator==(const Key& o) const { return ptr == o.ptr && rows == o.rows && cols == o.cols && box_rows == o.box_rows; }
  };
  struct Hash {
    size_t operator()(const Key& k) const {
      return std::hash<const void*>()(k.ptr) ^ (std::hash<long long>()(k.rows) * 31) ^
             (std::hash<long long>()(k.cols) * 131) ^ (size_t)k.box_rows;
    }
  };
  static std::unordered_map<Key, CUtensorMap, Hash> cache;
  static std::mutex lock;
  const Key key{ptr, rows, cols, box_rows};
  std::lock_guard<std::mutex> guard(lock);
  auto found = cache.find(key);
  if (found != cache.end()) { *out = found->second; return true; }
  EncodeTiledFn encode = encode_tiled();
  if (!encode) return false;
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)cols * 2};
  cuuint32_t box[2] = {64, (cuuint32_t)box_rows};
  cuuint32_t elem[2] = {1, 1};
  CUtensorMap map;
  if (encode(&map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, elem,
             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
    return false;
  if (cache.size() > 8192) cache.clear();
  cache.emplace(key, map);
  *out = map;
  return true;
}

// Tensor map of a row-major bfloat16 matrix [rows, cols] (rows a multiple of 8, cols 64 or 128)
// read in blocks of `block_rows` whole rows (a multiple of 8) by ONE copy each.  What a copy leaves
// in shared memory is, for every group of 8 rows, first the 8 x 64 left columns (1 KB, 128-byte
// swizzle) and then, if cols is 128, the 8 x 64 right columns: a layout the tensor core reads as a
// swizzled operand whose groups of 8 rows are cols * 16 bytes apart.  The coordinates of a copy
// are (0, 0, [0,] first row / 8).
inline bool tensor_map_bf16_row_blocks(const void* ptr, long long rows, int cols, int block_rows, CUtensorMap* out) {
  struct Key {
    const void* ptr; long long rows; int cols, block_rows;
    bool operator==(const Key& o) const { return ptr == o.ptr && rows == o.rows && cols == o.cols && block_rows == o.block_rows; }
  };
  struct Hash {
    size_t operator()(const Key& k) const {
      return std::hash<const void*>()(k.ptr) ^ (std::hash<long long>()(k.rows) * 31) ^ ((size_t)k.cols * 131) ^ (size_t)k.block_rows;
    }
  };
  static std::unordered_map<Key, CUtensorMap, Hash> cache;
  static std::mutex lock;
  if ((cols != 64 && cols != 128) || rows % 8 || block_rows % 8 || block_rows < 8 || block_rows > 256 * 8) return false;
  const Key key{ptr, rows, cols, block_rows};
  std::lock_guard<std::mutex> guard(lock);
  auto found = cache.find(key);
  if (found != cache.end()) { *out = found->second; return true; }
  EncodeTiledFn encode = encode_tiled();
  if (!encode) return false;
  const cuuint64_t row_bytes = (cuuint64_t)cols * 2;
  CUtensorMap map;
  CUresult status;
  cuuint32_t elem[4] = {1, 1, 1, 1};
  if (cols == 128) {
    cuuint64_t dims[4] = {64, 8, 2, (cuuint64_t)(rows / 8)};
    cuuint64_t strides[3] = {row_bytes, 128, 8 * row_bytes};
    cuuint32_t box[4] = {64, 8, 2, (cuuint32_t)(block_rows / 8)};
    status = encode(&map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(ptr), dims, strides, box, elem,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  } else {
    cuuint64_t dims[3] = {64, 8, (cuuint64_t)(rows / 8)};
    cuuint64_t strides[2] = {row_bytes, 8 * row_bytes};
    cuuint32_t box[3] = {64, 8, (cuuint32_t)(block_rows / 8)};
    status = encode(&map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(ptr), dims, strides, box, elem,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  }
  if (status != CUDA_SUCCESS) return false;
  if (cache.size() > 8192) cache.clear();
  cache.emplace(key, map);
  *out = map;
  return true;
}

// Tensor map of a paged key (or value) pool [pages][kv_heads][page_size][cols] (bfloat16, cols 64 or
// 128, page_size a multiple of 8) for copies that span `run_pages` consecutive pages of ONE kv head,
// `groups` groups of 8 rows from each: what a copy leaves in shared memory is the layout of
// tensor_map_bf16_row_blocks (per 8 rows the left 8 x 64 columns, then the right ones), page after
// page.  Coordinates of a copy: (0, 0, [0,] kv_head * page_size / 8 + first group in the page, first page).
inline bool tensor_map_bf16_page_runs(const void* ptr, long long num_pages, int kv_heads, int page_size, int cols,
                                      int groups, int run_pages, CUtensorMap* out) {
  struct Key {
    const void* ptr; long long pages; int heads, page, cols, groups, run;
    bool operator==(const Key& o) const {
      return ptr == o.ptr && pages == o.pages && heads == o.heads && page == o.page && cols == o.cols &&
             groups == o.groups && run == o.run;
    }
  };
  struct Hash {
    size_t operator()(const Key& k) const {
      return std::hash<const void*>()(k.ptr) ^ (std::hash<long long>()(k.pages) * 31) ^ ((size_t)k.heads * 131) ^
             ((size_t)k.page * 1031) ^ ((size_t)k.cols * 7) ^ ((size_t)k.groups * 8191) ^ ((size_t)k.run * 65537);
    }
  };
  static std::unordered_map<Key, CUtensorMap, Hash> cache;
  static std::mutex lock;
  if ((cols != 64 && cols != 128) || page_size % 8 || groups < 1 || groups > 256 || run_pages < 1 || run_pages > 256 ||
      groups > page_size / 8)
    return false;
  const Key key{ptr, num_pages, kv_heads, page_size, cols, groups, run_pages};
  std::lock_guard<std::mutex> guard(lock);
  auto found = cache.find(key);
  if (found != cache.end()) { *out = found->second; return true; }
  EncodeTiledFn encode = encode_tiled();
  if (!encode) return false;
  const cuuint64_t row_bytes = (cuuint64_t)cols * 2;
  const cuuint64_t groups_per_page = (cuuint64_t)kv_heads * (page_size / 8);
  CUtensorMap map;
  CUresult status;
  cuuint32_t elem[5] = {1, 1, 1, 1, 1};
  if (cols == 128) {
    cuuint64_t dims[5] = {64, 8, 2, groups_per_page, (cuuint64_t)num_pages};
    cuuint64_t strides[4] = {row_bytes, 128, 8 * row_bytes, groups_per_page * 8 * row_bytes};
    cuuint32_t box[5] = {64, 8, 2, (cuuint32_t)groups, (cuuint32_t)run_pages};
    status = encode(&map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 5, const_cast<void*>(ptr), dims, strides, box, elem,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  } else {
    cuuint64_t dims[4] = {64, 8, groups_per_page, (cuuint64_t)num_pages};
    cuuint64_t strides[3] = {row_bytes, 8 * row_bytes, groups_per_page * 8 * row_bytes};
    cuuint32_t box[4] = {64, 8, (cuuint32_t)groups, (cuuint32_t)run_pages};
    status = encode(&map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(ptr), dims, strides, box, elem,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  }
  if (status != CUDA_SUCCESS) return false;
  if (cache.size() > 8192) cache.clear();
  cache.emplace(key, map);
  *out = map;
  return true;
}

}  // namespace bw
}  // namespace cie
