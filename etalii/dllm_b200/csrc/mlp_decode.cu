// The whole SwiGLU feed-forward of a decode step in ONE kernel (at most 16 tokens, bfloat16 weights):
//   x += down( silu(gate(norm(x))) * up(norm(x)) )
// instead of two dependent kernels with the activations in global memory between them.
//
// The intermediate dimension is cut into slices: a block owns 16 of its values, a cluster of C blocks 16 C of them.
//   1. Every block computes its 16 activations for all tokens like the streaming product does: RMSNorm of the
//      float32 residual on the way in, 32 interleaved gate/up rows of W on the tensor cores (mma.sync, W as the
//      16-row operand), eight warps splitting the two row tiles and the reduction, SwiGLU on the sums.
//   2. It writes them, in bfloat16, into the shared memory of all blocks of its cluster (distributed shared
//      memory); one cluster barrier later every block holds the cluster's 16 C activations of every token.
//   3. Block r of the cluster multiplies them with its share of the down projection, W_down[columns of r][slice of
//      the cluster], which it copied into shared memory before it waited for the previous kernel, and writes the
//      partial sums to scratch.
//   4. The last block to finish a group of columns adds the clusters' partial sums to the residual in cluster order
//      (fused_tail.cuh): a fixed order, no waiting.
// The gate/up rows, the slice of W_down and the L2 prefetch of later weights are requested before
// griddepcontrol.wait, so they travel while the previous kernel still runs.
#include "fused_tail.cuh"

namespace {
using namespace fused;
constexpr int THREADS = 256, WARPS = 8, TILE = 16;
constexpr int ACT_PER_BLOCK = 16;  // SwiGLU outputs of a block = 32 interleaved rows of W_gate_up = two row tiles

struct Prefetch2 {
  const char* ptr[2];
  size_t bytes[2];
};

__device__ __forceinline__ void prefetch_share(const Prefetch2& pf) {
#pragma unroll
  for (int which = 0; which < 2; ++which) {
    if (pf.ptr[which] == nullptr) continue;
    size_t lines = (pf.bytes[which] + 127) / 128;
    size_t per_block = (lines + gridDim.x - 1) / gridDim.x;
    size_t begin = (size_t)blockIdx.x * per_block, end = min(lines, begin + per_block);
    for (size_t line = begin + threadIdx.x; line < end; line += blockDim.x)
      asm volatile("prefetch.global.L2 [%0];" ::"l"(pf.ptr[which] + line * 128));
  }
}

struct Sizes {
  int M, H, I;
  int columns_per_block;  // of the down projection: ceil(H / C) rounded up to 8
  int rows16;             // the same rounded up to 16 (rows of the shared-memory slice)
};

template <int NT, int C>
__global__ void __launch_bounds__(THREADS) mlp_decode_kernel(float* __restrict__ x, const float* __restrict__ norm_w,
                                                             float eps, const bf16* __restrict__ w_gu,
                                                             const bf16* __restrict__ w_d, float* __restrict__ partial,
                                                             int* __restrict__ tickets, Sizes sz, Prefetch2 pf) {
  constexpr int MAX_STEPS = NT == 1 ? 5 : 3;        // 32-value k steps whose loads are issued before the products
  constexpr int SLICE = ACT_PER_BLOCK * C;          // activations of a cluster
  constexpr int ACT_LD = padded(SLICE);
  extern __shared__ __align__(16) unsigned char smem_raw[];
  float (*red)[TILE][NT * 8 + 1] = reinterpret_cast<float (*)[TILE][NT * 8 + 1]>(smem_raw);
  float (*red_ss)[NT * 8] = reinterpret_cast<float (*)[NT * 8]>(smem_raw + sizeof(float) * WARPS * TILE * (NT * 8 + 1));
  bf16* act_s = reinterpret_cast<bf16*>(smem_raw + sizeof(float) * (WARPS * TILE * (NT * 8 + 1) + WARPS * NT * 8 + 8));
  bf16* wd_s = act_s + NT * 8 * ACT_LD;
  __shared__ int last_s;

  int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  int g = lane >> 2, t = lane & 3;
  unsigned rank = blockIdx.x % C;
  int cluster = blockIdx.x / C;
  int K = sz.H;
  pdl_launch_dependents();
  if (C > 1) cluster_arrive();  // (met again before the first write into a neighbour's shared memory)

  // ---- requests that depend on nobody: this block's slice of W_down, its gate/up rows, later weights into L2 ----
  int column0 = (int)rank * sz.columns_per_block;
  int columns = min(sz.columns_per_block, sz.H - column0);
  if (columns < 0) columns = 0;
  stage_slice(wd_s, w_d, column0, columns, sz.rows16, cluster * SLICE, SLICE, (size_t)sz.I, tid, THREADS);

  int tile = warp & 1, split = warp >> 1;
  int row_lo = blockIdx.x * (2 * ACT_PER_BLOCK) + tile * TILE + g, row_hi = row_lo + 8;
  const uint4* w_lo = (const uint4*)(w_gu + (size_t)row_lo * K);
  const uint4* w_hi = (const uint4*)(w_gu + (size_t)row_hi * K);
  int chunks = K >> 3, steps = (chunks + 3) >> 2;
  int per_split = (steps + WARPS / 2 - 1) / (WARPS / 2);
  int s_begin = split * per_split, s_end = min(steps, s_begin + per_split);
  const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
  uint4 wl[MAX_STEPS], wh[MAX_STEPS];
  auto load_weights = [&](int s0) {
#pragma unroll
    for (int i = 0; i < MAX_STEPS; ++i) {
      int ch = (s0 + i) * 4 + t;
      bool ok = s0 + i < s_end && ch < chunks;
      wl[i] = ok ? __ldg(w_lo + ch) : zero;
      wh[i] = ok ? __ldg(w_hi + ch) : zero;
    }
  };
  if (s_begin < s_end) load_weights(s_begin);
  prefetch_share(pf);
  pdl_wait();  // from here on: the residual, which the previous kernel wrote

  // ---- 1. gate/up of this block's 16 activations, RMSNorm on the way in ---------------------------------------
  float acc[NT][4], ss[NT];
#pragma unroll
  for (int n = 0; n < NT; ++n) {
    ss[n] = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) acc[n][i] = 0.f;
  }
  for (int s0 = s_begin; s0 < s_end; s0 += MAX_STEPS) {
    float4 xr[MAX_STEPS][NT][2], nr[MAX_STEPS][2];
#pragma unroll
    for (int i = 0; i < MAX_STEPS; ++i) {
      int ch = (s0 + i) * 4 + t;
      bool ok = s0 + i < s_end && ch < chunks;
      nr[i][0] = nr[i][1] = make_float4(0.f, 0.f, 0.f, 0.f);
      if (ok) {
        nr[i][0] = __ldg((const float4*)norm_w + 2 * ch);
        nr[i][1] = __ldg((const float4*)norm_w + 2 * ch + 1);
      }
#pragma unroll
      for (int n = 0; n < NT; ++n) {
        int m = n * 8 + g;
        xr[i][n][0] = xr[i][n][1] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (ok && m < sz.M) {
          const float4* xp = (const float4*)(x + (size_t)m * K) + 2 * ch;
          xr[i][n][0] = xp[0];
          xr[i][n][1] = xp[1];
        }
      }
    }
    // (all loads of the stretch above, then the arithmetic: a step's loads must not wait behind another step's sums)
    uint4 xb[MAX_STEPS][NT];
#pragma unroll
    for (int i = 0; i < MAX_STEPS; ++i) {
#pragma unroll
      for (int n = 0; n < NT; ++n) {
        float4 x0 = xr[i][n][0], x1 = xr[i][n][1], n0 = nr[i][0], n1 = nr[i][1];
        ss[n] = fmaf(x0.x, x0.x, ss[n]); ss[n] = fmaf(x0.y, x0.y, ss[n]);
        ss[n] = fmaf(x0.z, x0.z, ss[n]); ss[n] = fmaf(x0.w, x0.w, ss[n]);
        ss[n] = fmaf(x1.x, x1.x, ss[n]); ss[n] = fmaf(x1.y, x1.y, ss[n]);
        ss[n] = fmaf(x1.z, x1.z, ss[n]); ss[n] = fmaf(x1.w, x1.w, ss[n]);
        // (the k positions inside a 32-block are permuted the same way for W and x, which a sum does not see)
        xb[i][n] = make_uint4(pack_bf16(x0.x * n0.x, x0.y * n0.y), pack_bf16(x0.z * n0.z, x0.w * n0.w),
                              pack_bf16(x1.x * n1.x, x1.y * n1.y), pack_bf16(x1.z * n1.z, x1.w * n1.w));
      }
    }
#pragma unroll
    for (int i = 0; i < MAX_STEPS; ++i) {
      unsigned a0[4] = {wl[i].x, wh[i].x, wl[i].y, wh[i].y};
      unsigned a1[4] = {wl[i].z, wh[i].z, wl[i].w, wh[i].w};
#pragma unroll
      for (int n = 0; n < NT; ++n) {
        mma_bf16(acc[n], a0, xb[i][n].x, xb[i][n].y);
        mma_bf16(acc[n], a1, xb[i][n].z, xb[i][n].w);
      }
    }
    if (s0 + MAX_STEPS < s_end) load_weights(s0 + MAX_STEPS);
  }
#pragma unroll
  for (int n = 0; n < NT; ++n) {
    red[warp][g][n * 8 + 2 * t] = acc[n][0];
    red[warp][g][n * 8 + 2 * t + 1] = acc[n][1];
    red[warp][g + 8][n * 8 + 2 * t] = acc[n][2];
    red[warp][g + 8][n * 8 + 2 * t + 1] = acc[n][3];
    float v = ss[n];
    v += __shfl_xor_sync(0xffffffffu, v, 1);
    v += __shfl_xor_sync(0xffffffffu, v, 2);
    if (t == 0) red_ss[warp][n * 8 + g] = v;
  }
  __syncthreads();
  if (C > 1) cluster_wait();  // every block of the cluster runs: its shared memory may be written

  // ---- 2. SwiGLU, and the activations into every block of the cluster --------------------------------------------
  for (int idx = tid; idx < 2 * 8 * NT * 8; idx += THREADS) {
    int m = idx % (NT * 8), p = (idx / (NT * 8)) % 8, tl = idx / (NT * 8 * 8);
    float gate = 0.f, up = 0.f, sumsq = 0.f;
#pragma unroll
    for (int s = 0; s < WARPS / 2; ++s) {
      gate += red[2 * s + tl][2 * p][m];
      up += red[2 * s + tl][2 * p + 1][m];
      sumsq += red_ss[2 * s][m];  // (the warps of row tile 0 cover every k once)
    }
    float inv = 1.0f / sqrtf(sumsq / (float)K + eps);
    bf16 a = __float2bfloat16_rn(silu_fast(gate * inv) * (up * inv));
    bf16* slot = act_s + (size_t)m * ACT_LD + rank * ACT_PER_BLOCK + tl * 8 + p;
    if (C == 1) {
      *slot = a;
    } else {
#pragma unroll
      for (unsigned r = 0; r < C; ++r) store_remote_b16(remote_address(slot, r), a);
    }
  }
  cp_async_wait_all();  // this thread's pieces of the W_down slice
  if (C > 1) cluster_sync(); else __syncthreads();

  // ---- 3. this block's columns of the down projection over the cluster's slice; 4. the last block adds up -------
  size_t part_stride = (size_t)NT * 8 * sz.H;
  if (columns > 0) {
    slice_product<NT>(partial + (size_t)cluster * part_stride + column0, (size_t)sz.H, wd_s, act_s, columns,
                      sz.rows16, SLICE, ACT_LD, sz.M, warp, WARPS, lane);
    combine_if_last(x, partial, tickets + rank, sz.I / SLICE, sz.M, part_stride, (size_t)sz.H, column0, columns, tid,
                    THREADS, &last_s);
  }
}

template <int NT, int C>
int launch(float* x, const float* norm_w, float eps, const bf16* w_gu, const bf16* w_d, float* partial, int* tickets,
           const Sizes& sz, const Prefetch2& pf, cudaStream_t stream) {
  constexpr int SLICE = ACT_PER_BLOCK * C;
  size_t smem = sizeof(float) * (WARPS * TILE * (NT * 8 + 1) + WARPS * NT * 8 + 8) +
                sizeof(bf16) * ((size_t)NT * 8 * padded(SLICE) + (size_t)sz.rows16 * padded(SLICE));
  if (smem > 200 * 1024) return DLLM_UNSUPPORTED_SIZE;
  static size_t configured = 0;
  if (smem > configured) {
    if (cudaFuncSetAttribute(mlp_decode_kernel<NT, C>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) !=
        cudaSuccess)
      return DLLM_LAUNCH_FAILED;
    configured = smem;
  }
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3(sz.I / ACT_PER_BLOCK);
  config.blockDim = dim3(THREADS);
  config.dynamicSmemBytes = smem;
  config.stream = stream;
  cudaLaunchAttribute attributes[2];
  attributes[0].id = cudaLaunchAttributeClusterDimension;
  attributes[0].val.clusterDim.x = C;
  attributes[0].val.clusterDim.y = 1;
  attributes[0].val.clusterDim.z = 1;
  attributes[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attributes[1].val.programmaticStreamSerializationAllowed = 1;
  config.attrs = attributes;
  config.numAttrs = dllm_pdl_enabled() ? 2 : 1;
  return cudaLaunchKernelEx(&config, mlp_decode_kernel<NT, C>, x, norm_w, eps, w_gu, w_d, partial, tickets, sz, pf) ==
                 cudaSuccess
             ? DLLM_OK
             : DLLM_LAUNCH_FAILED;
}
}  // namespace

// Blocks per cluster for an intermediate size: the largest of 8, 4, 2, 1 whose slices (16 values a block) tile it.
// 0 if the size is no multiple of 16.
DLLM_EXPORT int dllm_mlp_decode_cluster(int intermediate) {
  if (intermediate <= 0 || intermediate % ACT_PER_BLOCK) return 0;
  for (int c = 8; c > 1; c >>= 1)
    if (intermediate % (ACT_PER_BLOCK * c) == 0) return c;
  return 1;
}

// Floats of scratch: one partial result [16 tokens at most][H] per cluster.
DLLM_EXPORT long long dllm_mlp_decode_scratch(int M, int H, int I) {
  int c = dllm_mlp_decode_cluster(I);
  if (c == 0 || M <= 0) return 0;
  return (long long)(I / (ACT_PER_BLOCK * c)) * (M <= 8 ? 8 : 16) * H;
}

// x[M,H] (float32 residual) += down(silu(gate(h)) * up(h)) with h = RMSNorm(x; norm_w, eps) rounded to bfloat16.
// w_gate_up: [2 I, H] bfloat16, rows interleaved (2i = gate_i, 2i+1 = up_i); w_down: [H, I] bfloat16.
// M at most 16; H a multiple of 8; I a multiple of 16. partial: `dllm_mlp_decode_scratch` floats; tickets: 8 ints,
// zero before the first launch (the kernel leaves them zero). prefetch_*: optional memory to bring into L2.
DLLM_EXPORT int dllm_mlp_decode(float* x, const float* norm_w, float eps, const void* w_gate_up, const void* w_down,
                                int M, int H, int I, float* partial, int* tickets, const void* prefetch_a,
                                long long prefetch_a_bytes, const void* prefetch_b, long long prefetch_b_bytes,
                                cudaStream_t stream) {
  if (M <= 0) return DLLM_OK;
  int c = dllm_mlp_decode_cluster(I);
  if (M > 16 || H <= 0 || (H & 7) || c == 0) return DLLM_UNSUPPORTED_SIZE;
  if (x == nullptr || norm_w == nullptr || partial == nullptr || tickets == nullptr) return DLLM_BAD_ARGUMENT;
  Sizes sz{M, H, I, 0, 0};
  sz.columns_per_block = (((H + c - 1) / c) + 7) & ~7;
  sz.rows16 = (sz.columns_per_block + 15) & ~15;
  Prefetch2 pf{{(const char*)prefetch_a, (const char*)prefetch_b},
               {prefetch_a ? (size_t)prefetch_a_bytes : 0, prefetch_b ? (size_t)prefetch_b_bytes : 0}};
  const bf16* gu = (const bf16*)w_gate_up;
  const bf16* wd = (const bf16*)w_down;
#define DLLM_GO(NT, C) return launch<NT, C>(x, norm_w, eps, gu, wd, partial, tickets, sz, pf, stream)
  if (M <= 8) {
    switch (c) { case 8: DLLM_GO(1, 8); case 4: DLLM_GO(1, 4); case 2: DLLM_GO(1, 2); default: DLLM_GO(1, 1); }
  }
  switch (c) { case 8: DLLM_GO(2, 8); case 4: DLLM_GO(2, 4); case 2: DLLM_GO(2, 2); default: DLLM_GO(2, 1); }
#undef DLLM_GO
  return DLLM_BAD_ARGUMENT;
}
