// Building blocks of the kernels that use the 5th-generation tensor cores: mbarriers with bounded waits, TMA tile
// loads, tcgen05.mma / commit / ld, shared-memory matrix descriptors, and tensor maps made through the driver's
// entry point (no link against libcuda). Everything is for cta_group::1, operands in bfloat16, accumulation in
// float32 in tensor memory.
#pragma once
#include <cuda.h>

#include <mutex>
#include <unordered_map>

#include "common.cuh"

namespace tc5 {
#ifndef DLLM_WAIT_LIMIT_CYCLES
#define DLLM_WAIT_LIMIT_CYCLES 2000000000ll  // about a second; a test builds with a few microseconds instead
#endif
constexpr long long WAIT_LIMIT_CYCLES = DLLM_WAIT_LIMIT_CYCLES;

__device__ __forceinline__ unsigned smem_u32(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, unsigned count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, unsigned bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(unsigned addr, unsigned parity) {
  unsigned done;
  asm volatile(
      "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
      : "=r"(done) : "r"(addr), "r"(parity) : "memory");
  return done != 0;
}
// Bounded wait: false if the phase did not complete within the limit. (A phase that is already complete costs one
// look; the clock is read only from the second look on.)
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, unsigned parity) {
  unsigned addr = smem_u32(bar);
  if (mbar_try_wait(addr, parity)) return true;
  long long begin = clock64();
  for (;;) {
    if (mbar_try_wait(addr, parity)) return true;  // try_wait itself pauses between looks
    if (clock64() - begin > WAIT_LIMIT_CYCLES) return false;
  }
}
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, uint64_t* bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void tcgen05_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void fence_before_sync() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fence_after_sync() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// Shared-memory matrix descriptor of a tile whose rows are 128 bytes with the 128-byte swizzle (what a TMA box of
// 64 bfloat16 columns writes): start address / 16, stride between groups of 8 rows 1024 bytes, descriptor version 1,
// swizzle mode 2. For a K-major operand the rows are the M or N index and a product of K = 16 advances the start
// by 32 bytes; for an MN-major operand (B read as [K rows][N contiguous]) the rows are K and a product of K = 16
// advances by 16 rows = 2048 bytes.
__device__ __forceinline__ uint64_t smem_desc(unsigned addr) {
  uint64_t d = 0;
  d |= (uint64_t)((addr & 0x3FFFF) >> 4);
  d |= (uint64_t)1 << 16;                 // leading byte offset (not used while MN spans one 128-byte atom)
  d |= (uint64_t)(1024 >> 4) << 32;       // stride byte offset
  d |= (uint64_t)1 << 46;                 // descriptor version
  d |= (uint64_t)2 << 61;                 // 128-byte swizzle
  return d;
}
// Instruction descriptor, kind::f16: D float32 (bit 4), A and B bfloat16 (bits 7, 10), A K-major; B K-major, or
// MN-major with bit 16; N / 8 at bit 17, M / 16 at bit 24.
__host__ __device__ constexpr unsigned instr_desc(int m, int n, bool b_mn_major = false) {
  return (1u << 4) | (1u << 7) | (1u << 10) | (b_mn_major ? (1u << 16) : 0u) | ((unsigned)(n >> 3) << 17) |
         ((unsigned)(m >> 4) << 24);
}
__device__ __forceinline__ void umma(unsigned tmem_d, uint64_t adesc, uint64_t bdesc, unsigned idesc, unsigned acc) {
  asm volatile(
      "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
      " tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(acc) : "memory");
}
// 16 consecutive columns of this thread's lane; `tmem_wait_ld` before the registers are used.
__device__ __forceinline__ void tmem_load16_nowait(unsigned taddr, unsigned* v) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
        "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
      : "r"(taddr));
}
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_load16(unsigned taddr, unsigned* v) {
  tmem_load16_nowait(taddr, v);
  tmem_wait_ld();
}
// One warp allocates `columns` (a power of two, at least 32) and writes the base address to shared memory.
__device__ __forceinline__ void tmem_alloc(unsigned* base_in_smem, unsigned columns) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
               ::"r"(smem_u32(base_in_smem)), "r"(columns) : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(unsigned base, unsigned columns) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(base), "r"(columns) : "memory");
}

// ---- host side: tensor maps ------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static inline EncodeTiled encoder() {
  static EncodeTiled fn = nullptr;
  if (fn == nullptr) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult result;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &result) == cudaSuccess &&
        result == cudaDriverEntryPointSuccess)
      fn = (EncodeTiled)p;
  }
  return fn;
}

// A [rows, cols] bfloat16 row-major matrix, boxes of box_rows x 64 columns, 128-byte swizzle, zero fill outside.
// Encoded maps are kept (a map depends only on these five numbers, and the same weights and workspace buffers come
// again every step): a launch then costs a table lookup instead of two driver calls.
static inline bool make_map(CUtensorMap* map, const void* base, long long rows, long long cols, int box_rows) {
  struct Key {
    const void* base; long long rows, cols; int box_rows;
    bool operator==(const Key& o) const { return base == o.base && rows == o.rows && cols == o.cols && box_rows == o.box_rows; }
  };
  struct Hash {
    size_t operator()(const Key& k) const {
      size_t h = (size_t)(uintptr_t)k.base * 0x9E3779B97F4A7C15ull;
      h ^= (size_t)k.rows * 0xC2B2AE3D27D4EB4Full + (h << 6) + (h >> 2);
      h ^= (size_t)k.cols * 0x165667B19E3779F9ull + (h << 6) + (h >> 2);
      return h ^ (size_t)k.box_rows;
    }
  };
  static std::unordered_map<Key, CUtensorMap, Hash> cache;
  static std::mutex lock;
  Key key{base, rows, cols, box_rows};
  {
    std::lock_guard<std::mutex> guard(lock);
    auto found = cache.find(key);
    if (found != cache.end()) { *map = found->second; return true; }
  }
  EncodeTiled encode = encoder();
  if (encode == nullptr) return false;
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)cols * 2};
  cuuint32_t box[2] = {64u, (cuuint32_t)box_rows};
  cuuint32_t elem[2] = {1, 1};
  if (encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
    return false;
  std::lock_guard<std::mutex> guard(lock);
  if (cache.size() >= 8192) cache.clear();
  cache.emplace(key, *map);
  return true;
}
}  // namespace tc5
