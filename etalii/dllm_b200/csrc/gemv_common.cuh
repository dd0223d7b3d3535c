// What the weight-streaming products for decode-sized steps share: the tensor-core instruction with W as the 16-row
// operand, which rows of W make up a 16-row tile, and the requests to L2 for what later kernels of the step read.
#pragma once
#include "gemm_common.cuh"

namespace gemv {
typedef __nv_bfloat16 bf16;
constexpr int TILE = 16;  // rows of W per tile

__device__ __forceinline__ void mma_bf16(float* c, const unsigned* a, unsigned b0, unsigned b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ unsigned pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<unsigned*>(&v);
}

// The row of W behind tile row r (0..15) of block `item`. In the q/k/v projection a rotated head's tile holds eight
// dimensions and their rotary partners (r and r + 8 are a pair); everywhere else 16 consecutive rows.
template <int EPI>
__device__ __forceinline__ int tile_row(int item, int r, int N, const RopeArgs& rope, int& head, int& dim0,
                                        bool& paired) {
  if (EPI == EPI_QKV_ROPE) {
    int hd = rope.cache.head_dim, per_head = hd / TILE;
    head = item / per_head;
    int it = item % per_head;
    bool rotated = rope.table != nullptr && head < rope.heads + rope.cache.kv_heads;
    paired = rotated && it < rope.rotary_dim / TILE;
    if (paired) {
      dim0 = it * 8;
      return head * hd + dim0 + (r & 7) + (r >> 3) * (rope.rotary_dim / 2);
    }
    dim0 = it * TILE;
    return head * hd + dim0 + r;
  }
  head = 0; dim0 = 0; paired = false;
  return min(item * TILE + r, N - 1);
}

// Weights that a later kernel of the step will stream: every block asks the L2 cache for its share of them while
// its own loads are in flight, so that the later kernel reads from L2 instead of waiting on DRAM.
struct Prefetch {
  const char* ptr;
  size_t bytes;
};

__device__ __forceinline__ void prefetch_share(const Prefetch& pf) {
  if (pf.ptr == nullptr) return;
  size_t lines = (pf.bytes + 127) / 128;
  size_t per_block = (lines + gridDim.x - 1) / gridDim.x;
  size_t begin = (size_t)blockIdx.x * per_block, end = min(lines, begin + per_block);
  for (size_t line = begin + threadIdx.x; line < end; line += blockDim.x)
    asm volatile("prefetch.global.L2 [%0];" ::"l"(pf.ptr + line * 128));
}

// The q/k/v projection of a decode step asks L2 for the keys and values that the attention kernel behind it will
// read: the pages of every sequence in the step (a page is one contiguous piece: keys and values of all kv heads).
// They are nobody's output in this step (the step's own rows are written below and read through L2 anyway), so the
// request goes out before the wait on the previous kernel and the pages travel from HBM while this kernel and the
// launch of the next one run. A sequence's pages are dealt to warps in turn, a page's lines to the warp's lanes.
__device__ __forceinline__ void prefetch_cache_pages(const RopeArgs& rope, int M) {
  if (rope.prefetch_window < 0 || !rope.write_cache) return;
  const KvLayout& c = rope.cache;
  int lane = threadIdx.x & 31, warps = blockDim.x >> 5;
  int all_warps = (int)gridDim.x * warps, me = (int)blockIdx.x * warps + (threadIdx.x >> 5);
  int sharers = max(1, all_warps / M);  // warps that share one token's sequence; each takes every sharers-th page
  if (me >= sharers * M) return;
  int m = me % M, share = me / M;
  int seq = rope.tok_seq[m];
  if (m > 0 && rope.tok_seq[m - 1] == seq) return;  // (a sequence's first token in the step stands for it)
  int pos = rope.tok_pos[m];
  int first = (rope.prefetch_window > 0 && pos + 1 > rope.prefetch_window) ? pos + 1 - rope.prefetch_window : 0;
  const int* pages = c.page_table + (size_t)rope.slots[seq] * c.max_pages;
  int last_page = min(pos / c.page_size, c.max_pages - 1);
  size_t page_bytes = (size_t)2 * c.kv_heads * c.page_size * c.head_dim * sizeof(bf16);
  int lines = (int)((page_bytes + 127) / 128);
  for (int j = first / c.page_size + share; j <= last_page; j += sharers) {
    const char* at = (const char*)c.base + (size_t)pages[j] * page_bytes;
    for (int line = lane; line < lines; line += 32) asm volatile("prefetch.global.L2 [%0];" ::"l"(at + (size_t)line * 128));
  }
}
}  // namespace gemv
