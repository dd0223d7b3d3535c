// What the two fused decode kernels (feed-forward, attention + output projection) have in common: thread-block
// cluster helpers, and the tail that turns a block's slice of activations into its share of a projection that ends
// in the residual sum.
//
// The tail: a block holds, in shared memory, a slice W[rows of this block][k of this cluster] of a projection
// matrix (copied there with cp.async before the kernel waits for its predecessor) and the activations
// act[token][k of this cluster]. It multiplies them on the tensor cores (mma.sync m16n8k16, W as the 16-row
// operand), writes the partial sums to scratch [part][token][column], and takes a ticket for its group of columns.
// The block that takes the last ticket of a group adds the parts in part order to the residual: a fixed order, so a
// repeated run gives the same bits; nobody waits for anybody.
#pragma once
#include "gemm_common.cuh"

namespace fused {
typedef __nv_bfloat16 bf16;

__device__ __forceinline__ void cp_async_16(void* smem, const void* gmem) {
  unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(s), "l"(gmem));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;\n" ::: "memory"); }
__device__ __forceinline__ void ldmatrix_x4(unsigned* r, const void* p) {
  unsigned s = (unsigned)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
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

// ---- clusters ---------------------------------------------------------------------------------------------------
__device__ __forceinline__ void cluster_arrive() { asm volatile("barrier.cluster.arrive.release.aligned;\n" ::: "memory"); }
__device__ __forceinline__ void cluster_wait() { asm volatile("barrier.cluster.wait.acquire.aligned;\n" ::: "memory"); }
__device__ __forceinline__ void cluster_sync() { cluster_arrive(); cluster_wait(); }
// The address of `local` (a shared-memory location of this block) in block `rank` of the cluster.
__device__ __forceinline__ unsigned remote_address(const void* local, unsigned rank) {
  unsigned addr = (unsigned)__cvta_generic_to_shared(local), remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(addr), "r"(rank));
  return remote;
}
__device__ __forceinline__ void store_remote_b16(unsigned remote, bf16 v) {
  asm volatile("st.shared::cluster.b16 [%0], %1;" ::"r"(remote), "h"(*reinterpret_cast<unsigned short*>(&v)) : "memory");
}
__device__ __forceinline__ void store_remote_b32(unsigned remote, unsigned v) {
  asm volatile("st.shared::cluster.b32 [%0], %1;" ::"r"(remote), "r"(v) : "memory");
}

// ---- the tail -----------------------------------------------------------------------------------------------------
// Shared-memory row of a slice: `cols` values plus 8 of padding (16 bytes: ldmatrix rows then fall into different
// banks).
__host__ __device__ constexpr int padded(int cols) { return cols + 8; }

// Copies W[row0 .. row0+rows)[col0 .. col0+cols) (row-major, row length ld) into w_s[rows16][padded(cols)], zero
// rows from `rows` up to rows16 (a multiple of 16). cols is a multiple of 8; row0 * ld + col0 too (16-byte pieces).
__device__ __forceinline__ void stage_slice(bf16* w_s, const bf16* w, int row0, int rows, int rows16, int col0,
                                            int cols, size_t ld, int tid, int threads) {
  int pieces = cols >> 3;
  for (int i = tid; i < rows16 * pieces; i += threads) {
    int r = i / pieces, p = i % pieces;
    bf16* dst = w_s + (size_t)r * padded(cols) + p * 8;
    if (r < rows) cp_async_16(dst, w + (size_t)(row0 + r) * ld + col0 + p * 8);
    else *reinterpret_cast<uint4*>(dst) = make_uint4(0u, 0u, 0u, 0u);
  }
  cp_async_commit();
}

// partial[(part * tokens_ld + m) * out_ld + column0 + r] = sum_k w_s[r][k] * act_s[m][k] for the block's rows r and
// the tokens m < tokens (NT groups of 8). Warps take tiles of 16 rows in turn.
template <int NT>
__device__ __forceinline__ void slice_product(float* __restrict__ partial_row0, size_t token_stride,
                                              const bf16* w_s, const bf16* act_s, int rows, int rows16, int cols,
                                              int act_ld, int tokens, int warp, int warps, int lane) {
  int g = lane >> 2, t = lane & 3;
  for (int tile = warp; tile * 16 < rows16; tile += warps) {
    float acc[NT][4];
#pragma unroll
    for (int n = 0; n < NT; ++n)
#pragma unroll
      for (int i = 0; i < 4; ++i) acc[n][i] = 0.f;
    for (int k0 = 0; k0 < cols; k0 += 16) {
      unsigned a[4];
      int mat = lane >> 3;  // matrices: (rows 0-7, k 0-7), (rows 8-15, k 0-7), (rows 0-7, k 8-15), (rows 8-15, k 8-15)
      ldmatrix_x4(a, w_s + (size_t)(tile * 16 + (mat & 1) * 8 + (lane & 7)) * padded(cols) + k0 + (mat >> 1) * 8);
#pragma unroll
      for (int n = 0; n < NT; ++n) {
        const bf16* row = act_s + (size_t)(n * 8 + g) * act_ld + k0 + 2 * t;
        mma_bf16(acc[n], a, *reinterpret_cast<const unsigned*>(row), *reinterpret_cast<const unsigned*>(row + 8));
      }
    }
#pragma unroll
    for (int n = 0; n < NT; ++n)
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        int r = tile * 16 + g + (i >> 1) * 8, m = n * 8 + 2 * t + (i & 1);
        if (r < rows && m < tokens) partial_row0[(size_t)m * token_stride + r] = acc[n][i];
      }
  }
}

// After `slice_product`: the block takes a ticket of its column group; the block that takes the last of `parts`
// tickets adds the parts, in part order, to the residual rows and leaves the ticket at zero for the next launch.
// partial: [parts][tokens][out_ld] floats from column0 on; residual: [tokens][out_ld]. rows, column0, out_ld and
// part_stride are multiples of 4 and the buffers 16-byte aligned (vector loads).
__device__ __forceinline__ void combine_if_last(float* __restrict__ residual, const float* __restrict__ partial,
                                                int* ticket, int parts, int tokens, size_t part_stride,
                                                size_t out_ld, int column0, int rows, int tid, int threads,
                                                int* flag_s) {
  __threadfence();  // this block's partial sums are visible before its ticket is
  __syncthreads();
  if (tid == 0) {
    int taken = atomicAdd(ticket, 1);
    *flag_s = taken == parts - 1;
    if (taken == parts - 1) *ticket = 0;
  }
  __syncthreads();
  if (!*flag_s) return;
  __threadfence();  // the other blocks' partial sums are visible after their tickets
  // Four columns a thread; the loads of up to sixteen parts are all issued before the first sum (one round trip to
  // L2 instead of one per part), the sums run in part order. rows, column0 and out_ld are multiples of 4.
  constexpr int BATCH = 16;
  int quads = rows >> 2;
  for (int i = tid; i < tokens * quads; i += threads) {
    int m = i / quads, r = (i % quads) * 4;
    size_t at = (size_t)m * out_ld + column0 + r;
    float4 sum = *reinterpret_cast<const float4*>(residual + at);
    for (int p0 = 0; p0 < parts; p0 += BATCH) {
      float4 v[BATCH];
#pragma unroll
      for (int j = 0; j < BATCH; ++j)
        v[j] = p0 + j < parts ? __ldcg(reinterpret_cast<const float4*>(partial + (size_t)(p0 + j) * part_stride + at))
                              : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int j = 0; j < BATCH; ++j)
        if (p0 + j < parts) { sum.x += v[j].x; sum.y += v[j].y; sum.z += v[j].z; sum.w += v[j].w; }
    }
    *reinterpret_cast<float4*>(residual + at) = sum;
  }
}
}  // namespace fused
