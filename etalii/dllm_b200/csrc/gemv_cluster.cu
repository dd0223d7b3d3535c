// Products of 17 to 64 rows of activations with small weights (a few megabytes: the layers of a narrow model), where
// neither reading W nor the arithmetic costs anything and the time goes into bringing the activations to the
// multiprocessors: the kernel that gives every 16 rows of W a block of their own reads all rows of X once per block.
// Here a thread-block CLUSTER owns 32 rows of W and splits the reduction (k) over all warps of its blocks, so X is
// read once per 32 rows of W, by up to eight multiprocessors together, and W exactly once:
//   - a warp takes a run of 32-value k steps, all 32 rows of W and all tokens: mma.sync m16n8k16 with W as the
//     16-row operand, the k positions inside a step permuted the same way for W and X (16-byte loads);
//   - the four warps' partial tiles meet in the block's shared memory and are summed in warp order;
//   - the blocks' sums go to the block that owns the token (tokens are dealt to the blocks in equal runs) with
//     st.shared::cluster, one barrier.cluster later the owner adds them in block order: fixed order, no atomics;
//   - the owner applies the epilogue: store, residual add, SwiGLU, or rotation and the write into the paged cache.
// In front, optionally, RMSNorm of the float32 residual rows (sums of squares travel with the partial tiles).
#include "gemv_common.cuh"

namespace {
using namespace gemv;
constexpr int WARPS = 4, ITEMS = 2, ROWS = ITEMS * TILE;  // 32 rows of W per cluster; row ROWS holds sums of squares
constexpr int RSTRIDE = ROWS + 4;                         // a token's received values: 16-byte pieces of four rows

__device__ __forceinline__ unsigned cluster_rank() {
  unsigned r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ unsigned cluster_size() {
  unsigned r;
  asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_arrive_relaxed() { asm volatile("barrier.cluster.arrive.relaxed.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_arrive_release() { asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_wait_acquire() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }
// Four floats to the same shared-memory place in block `rank` of the cluster.
__device__ __forceinline__ void store_to_block(float* local, unsigned rank, float4 v) {
  unsigned addr = (unsigned)__cvta_generic_to_shared(local), remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(addr), "r"(rank));
  asm volatile("st.shared::cluster.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(remote), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w)
               : "memory");
}

// One (pair of tile rows, token) of the owner's epilogue: where it goes and what it needs from memory besides the
// sums (old residual values; the token's position, rotation and cache page). Asked for right after the wait on the
// previous kernel, so that the loads run under the products. (Asking for the chains of dependent loads link by link
// at later places, each behind other work, was measured and changed nothing here; in `gemv.cu` it cost 5 %.)
template <int EPI>
struct Unit {
  int m = 0, item = 0, p = 0, head = 0, dim0 = 0;
  bool valid = false, paired = false;
  float r0 = 0.f, r1 = 0.f;
  int pos = 0, page = 0;
  float2 cs = make_float2(1.f, 0.f);
  __device__ __forceinline__ void prepare(const void* c, int m_, int item_, int p_, int M, int N, int items,
                                          const RopeArgs& rope) {
    m = m_; item = item_; p = p_;
    valid = m < M && item < items;
    if (!valid) return;
    tile_row<EPI>(item, p, N, rope, head, dim0, paired);
    if (EPI == EPI_RESIDUAL) {
      int n = item * TILE + 2 * p;
      const float* src = (const float*)c + (size_t)m * N + n;
      if (n < N) r0 = src[0];
      if (n + 1 < N) r1 = src[1];
    } else if (EPI == EPI_QKV_ROPE) {
      pos = rope.tok_pos[m];
      if (paired) cs = rope.table[(size_t)pos * (rope.rotary_dim / 2) + dim0 + p];
      if (head >= rope.heads && rope.write_cache) {
        int slot = rope.slots[rope.tok_seq[m]];
        page = rope.cache.page_table[(size_t)slot * rope.cache.max_pages + pos / rope.cache.page_size];
      }
    }
  }
  __device__ __forceinline__ void finish(void* c, int M, int N, const RopeArgs& rope, float v0, float v1) const {
    if (EPI == EPI_QKV_ROPE) {
      int hd = rope.cache.head_dim, nkv = rope.cache.kv_heads, heads = rope.heads;
      int d0 = dim0 + p, d1 = d0 + 8;
      if (paired) {
        d1 = d0 + rope.rotary_dim / 2;
        float x = v0, y = v1;
        v0 = fmaf(x, cs.x, -(y * cs.y));
        v1 = fmaf(x, cs.y, y * cs.x);
      }
      bf16* dst;
      if (head < heads) {
        dst = rope.q_out + ((size_t)m * heads + head) * hd;
      } else {
        if (!rope.write_cache) return;
        int which = head < heads + nkv ? 0 : 1;
        int kvh = head - heads - which * nkv;
        dst = (bf16*)rope.cache.base + kv_offset(rope.cache, page, which, kvh, pos % rope.cache.page_size);
      }
      dst[d0] = __float2bfloat16_rn(v0);
      dst[d1] = __float2bfloat16_rn(v1);
    } else if (EPI == EPI_RESIDUAL) {
      int n = item * TILE + 2 * p;
      float* dst = (float*)c + (size_t)m * N + n;
      if (n < N) dst[0] = r0 + v0;
      if (n + 1 < N) dst[1] = r1 + v1;
    } else {
      epilogue_pair<EPI, bf16>(c, m, item * TILE + 2 * p, M, N, v0, v1);
    }
  }
};

// NT: tiles of 8 tokens (the step has at most 8 NT rows). Launched as clusters of 1, 2, 4 or 8 blocks (at most 2 NT)
// along x; cluster j owns the tiles ITEMS j .. ITEMS j + ITEMS - 1 of 16 rows of W.
template <int NT, int EPI, bool NORM>
__global__ void __launch_bounds__(WARPS * 32) gemv_cluster_kernel(void* __restrict__ c, const void* __restrict__ a,
                                                                  const float* __restrict__ norm_w, float eps,
                                                                  const bf16* __restrict__ w, int M, int N, int K,
                                                                  RopeArgs rope, Prefetch pf, int items) {
  constexpr int COLS = NT * 8, STRIDE = COLS + 8;
  constexpr int STEPS = NORM ? 1 : 2;  // k steps whose loads are issued before the first product
  // [WARPS][ROWS + 1][STRIDE] partial tiles of the warps, then [blocks][tokens of this block][RSTRIDE] received sums
  extern __shared__ float space[];
  float* red = space;
  float* received = space + WARPS * (ROWS + 1) * STRIDE;
  int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  int g = lane >> 2, t = lane & 3;
  unsigned rank = cluster_rank(), blocks = cluster_size();
  int tokens_here = COLS / (int)blocks;  // tokens this block owns: rank * tokens_here ..
  int cluster = blockIdx.x / blocks;
  pdl_launch_dependents();
  cluster_arrive_relaxed();  // (every block of the cluster runs before anyone writes into its shared memory)

  const uint4* w_lo[ITEMS];
  const uint4* w_hi[ITEMS];
#pragma unroll
  for (int it = 0; it < ITEMS; ++it) {
    int item = min(cluster * ITEMS + it, items - 1), head, dim0;
    bool paired;
    w_lo[it] = (const uint4*)(w + (size_t)tile_row<EPI>(item, g, N, rope, head, dim0, paired) * K);
    w_hi[it] = (const uint4*)(w + (size_t)tile_row<EPI>(item, g + 8, N, rope, head, dim0, paired) * K);
  }
  int chunks = K >> 3;            // 16-byte pieces of a row
  int steps = (chunks + 3) >> 2;  // k steps of 32 values, dealt to the cluster's warps in runs
  int all_warps = WARPS * (int)blocks, me = (int)rank * WARPS + warp;
  int s_begin = (int)((long long)me * steps / all_warps), s_end = (int)((long long)(me + 1) * steps / all_warps);

  float acc[ITEMS][NT][4];
  float ss[NT];
#pragma unroll
  for (int n = 0; n < NT; ++n) {
    ss[n] = 0.f;
#pragma unroll
    for (int it = 0; it < ITEMS; ++it)
#pragma unroll
      for (int i = 0; i < 4; ++i) acc[it][n][i] = 0.f;
  }
  const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
  uint4 wl[STEPS][ITEMS], wh[STEPS][ITEMS];
  auto load_weights = [&](int s0) {
#pragma unroll
    for (int i = 0; i < STEPS; ++i) {
      int ch = (s0 + i) * 4 + t;
      bool ok = s0 + i < s_end && ch < chunks;
#pragma unroll
      for (int it = 0; it < ITEMS; ++it) {
        wl[i][it] = ok ? __ldg(w_lo[it] + ch) : zero;
        wh[i][it] = ok ? __ldg(w_hi[it] + ch) : zero;
      }
    }
  };
  if (s_begin < s_end) load_weights(s_begin);
  if (EPI == EPI_QKV_ROPE) prefetch_cache_pages(rope, M);
  prefetch_share(pf);
  pdl_wait();  // the weights are nobody's output; everything below may be the previous kernel's

  // the owner's first two units (pair p fastest, then tile, then token: neighbouring threads store side by side)
  int units = ITEMS * 8 * tokens_here;
  Unit<EPI> early[2];
#pragma unroll
  for (int j = 0; j < 2; ++j) {
    int idx = tid + j * WARPS * 32;
    if (idx < units)
      early[j].prepare(c, (int)rank * tokens_here + idx / (ITEMS * 8), cluster * ITEMS + (idx >> 3) % ITEMS, idx & 7, M,
                       N, items, rope);
  }

  for (int s0 = s_begin; s0 < s_end; s0 += STEPS) {
    uint4 xb[STEPS][NT];
    if (NORM) {
      float4 xr[STEPS][NT][2], nr[STEPS][2];
#pragma unroll
      for (int i = 0; i < STEPS; ++i) {
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
          if (ok && m < M) {
            const float4* xp = (const float4*)((const float*)a + (size_t)m * K) + 2 * ch;
            xr[i][n][0] = xp[0];
            xr[i][n][1] = xp[1];
          }
        }
      }
#pragma unroll
      for (int i = 0; i < STEPS; ++i) {
#pragma unroll
        for (int n = 0; n < NT; ++n) {
          float4 x0 = xr[i][n][0], x1 = xr[i][n][1], n0 = nr[i][0], n1 = nr[i][1];
          ss[n] = fmaf(x0.x, x0.x, ss[n]); ss[n] = fmaf(x0.y, x0.y, ss[n]);
          ss[n] = fmaf(x0.z, x0.z, ss[n]); ss[n] = fmaf(x0.w, x0.w, ss[n]);
          ss[n] = fmaf(x1.x, x1.x, ss[n]); ss[n] = fmaf(x1.y, x1.y, ss[n]);
          ss[n] = fmaf(x1.z, x1.z, ss[n]); ss[n] = fmaf(x1.w, x1.w, ss[n]);
          xb[i][n] = make_uint4(pack_bf16(x0.x * n0.x, x0.y * n0.y), pack_bf16(x0.z * n0.z, x0.w * n0.w),
                                pack_bf16(x1.x * n1.x, x1.y * n1.y), pack_bf16(x1.z * n1.z, x1.w * n1.w));
        }
      }
    } else {
#pragma unroll
      for (int i = 0; i < STEPS; ++i) {
        int ch = (s0 + i) * 4 + t;
        bool ok = s0 + i < s_end && ch < chunks;
#pragma unroll
        for (int n = 0; n < NT; ++n) {
          int m = n * 8 + g;
          xb[i][n] = (ok && m < M) ? *((const uint4*)((const bf16*)a + (size_t)m * K) + ch) : zero;
        }
      }
    }
#pragma unroll
    for (int i = 0; i < STEPS; ++i) {
#pragma unroll
      for (int it = 0; it < ITEMS; ++it) {
        unsigned a0[4] = {wl[i][it].x, wh[i][it].x, wl[i][it].y, wh[i][it].y};
        unsigned a1[4] = {wl[i][it].z, wh[i][it].z, wl[i][it].w, wh[i][it].w};
#pragma unroll
        for (int n = 0; n < NT; ++n) {
          mma_bf16(acc[it][n], a0, xb[i][n].x, xb[i][n].y);
          mma_bf16(acc[it][n], a1, xb[i][n].z, xb[i][n].w);
        }
      }
    }
    if (s0 + STEPS < s_end) load_weights(s0 + STEPS);
  }

  // the warp's partial tile (and sums of squares) to shared memory
  float* mine = red + warp * (ROWS + 1) * STRIDE;
#pragma unroll
  for (int n = 0; n < NT; ++n) {
#pragma unroll
    for (int it = 0; it < ITEMS; ++it) {
      *reinterpret_cast<float2*>(mine + (it * TILE + g) * STRIDE + n * 8 + 2 * t) =
          make_float2(acc[it][n][0], acc[it][n][1]);
      *reinterpret_cast<float2*>(mine + (it * TILE + g + 8) * STRIDE + n * 8 + 2 * t) =
          make_float2(acc[it][n][2], acc[it][n][3]);
    }
    if (NORM) {
      float v = ss[n];
      v += __shfl_xor_sync(0xffffffffu, v, 1);
      v += __shfl_xor_sync(0xffffffffu, v, 2);
      if (t == 0) mine[ROWS * STRIDE + n * 8 + g] = v;
    }
  }
  __syncthreads();
  cluster_wait_acquire();  // (pairs with the arrival at the top)

  // the block's sums, four rows of a token at a time, to the token's owner
  constexpr int QUADS = ROWS / 4 + (NORM ? 1 : 0);
  for (int u = tid; u < COLS * QUADS; u += WARPS * 32) {
    int m = u % COLS, quad = u / COLS;
    if (m >= M) continue;
    float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int wi = 0; wi < WARPS; ++wi) {
      const float* src = red + (wi * (ROWS + 1) + 4 * quad) * STRIDE + m;
      s.x += src[0];
      if (quad < ROWS / 4) { s.y += src[STRIDE]; s.z += src[2 * STRIDE]; s.w += src[3 * STRIDE]; }
    }
    int owner = m / tokens_here;
    float* dst = received + ((size_t)rank * tokens_here + m % tokens_here) * RSTRIDE + 4 * quad;
    if (blocks == 1) *reinterpret_cast<float4*>(dst) = s;
    else store_to_block(dst, (unsigned)owner, s);
  }
  if (blocks == 1) {
    __syncthreads();
  } else {
    cluster_arrive_release();
    cluster_wait_acquire();
  }

  // the owner's epilogue: the blocks' sums in block order
  auto finish = [&](int idx, const Unit<EPI>& unit) {
    if (!unit.valid) return;
    int local = idx / (ITEMS * 8), it = (idx >> 3) % ITEMS, p = idx & 7;
    int r0 = it * TILE + ((EPI == EPI_QKV_ROPE) ? p : 2 * p), r1 = it * TILE + ((EPI == EPI_QKV_ROPE) ? p + 8 : 2 * p + 1);
    float v0 = 0.f, v1 = 0.f, sumsq = 0.f;
    for (unsigned b = 0; b < blocks; ++b) {
      const float* src = received + ((size_t)b * tokens_here + local) * RSTRIDE;
      v0 += src[r0];
      v1 += src[r1];
      if (NORM) sumsq += src[ROWS];
    }
    if (NORM) {
      float inv = 1.0f / sqrtf(sumsq / (float)K + eps);
      v0 *= inv;
      v1 *= inv;
    }
    unit.finish(c, M, N, rope, v0, v1);
  };
  if (tid < units) finish(tid, early[0]);
  if (tid + WARPS * 32 < units) finish(tid + WARPS * 32, early[1]);
  for (int idx = tid + 2 * WARPS * 32; idx < units; idx += WARPS * 32) {
    Unit<EPI> late;
    late.prepare(c, (int)rank * tokens_here + idx / (ITEMS * 8), cluster * ITEMS + (idx >> 3) % ITEMS, idx & 7, M, N,
                 items, rope);
    finish(idx, late);
  }
}

// Blocks of a cluster (`asked`, or chosen): enough warps that each takes no more k steps than it asks for at once,
// at most eight blocks, no more than leaves every block four tokens to own, and no more than lets all clusters of
// the launch run at the same time (measured, 64 x 3072 x 576 with the norm: 7.4 µs with two blocks, 192 in all,
// 10.6 with four, 15.1 with eight).
template <int NT, int EPI, bool NORM>
int launch_one(void* c, const void* a, const float* norm_w, float eps, const bf16* w, int M, int N, int K,
               const RopeArgs& rope, const Prefetch& pf, int asked, cudaStream_t stream) {
  constexpr int COLS = NT * 8, MOST = 2 * NT < 8 ? 2 * NT : 8;
  size_t smem = (size_t)(WARPS * (ROWS + 1) * (COLS + 8) + COLS * RSTRIDE) * sizeof(float);
  static int resident = 0;  // blocks of this kernel that fit on the device at once
  if (resident == 0) {
    if (smem > 48 * 1024 &&
        cudaFuncSetAttribute(gemv_cluster_kernel<NT, EPI, NORM>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             (int)smem) != cudaSuccess)
      return DLLM_LAUNCH_FAILED;
    int device = 0, sms = 0, per_sm = 0;
    if (cudaGetDevice(&device) != cudaSuccess ||
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess ||
        cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, gemv_cluster_kernel<NT, EPI, NORM>, WARPS * 32,
                                                      smem) != cudaSuccess ||
        sms <= 0 || per_sm <= 0)
      return DLLM_LAUNCH_FAILED;
    resident = sms * per_sm;
  }
  int items = (N + TILE - 1) / TILE, clusters = (items + ITEMS - 1) / ITEMS;
  int blocks = asked;
  if (asked > 0) {
    if ((asked != 1 && asked != 2 && asked != 4 && asked != 8) || asked > MOST) return DLLM_BAD_ARGUMENT;
  } else {
    int steps = (K / 8 + 3) / 4, at_once = NORM ? 1 : 2;
    blocks = 1;
    while (blocks < MOST && blocks * WARPS * at_once < steps) blocks *= 2;
    while (blocks > 1 && (long long)clusters * blocks > resident) blocks /= 2;
  }
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3(clusters * blocks);
  config.blockDim = dim3(WARPS * 32);
  config.dynamicSmemBytes = smem;
  config.stream = stream;
  cudaLaunchAttribute attributes[2];
  attributes[0].id = cudaLaunchAttributeClusterDimension;
  attributes[0].val.clusterDim.x = blocks;
  attributes[0].val.clusterDim.y = 1;
  attributes[0].val.clusterDim.z = 1;
  attributes[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attributes[1].val.programmaticStreamSerializationAllowed = 1;
  config.attrs = attributes;
  config.numAttrs = dllm_pdl_enabled() ? 2 : 1;
  return cudaLaunchKernelEx(&config, gemv_cluster_kernel<NT, EPI, NORM>, c, a, norm_w, eps, w, M, N, K, rope, pf,
                            items) == cudaSuccess
             ? DLLM_OK
             : DLLM_LAUNCH_FAILED;
}

template <int EPI, bool NORM>
int launch(void* c, const void* a, const float* norm_w, float eps, const bf16* w, int M, int N, int K,
           const RopeArgs& rope, const Prefetch& pf, int blocks, cudaStream_t stream) {
  if (M <= 16) return launch_one<2, EPI, NORM>(c, a, norm_w, eps, w, M, N, K, rope, pf, blocks, stream);
  if (M <= 32) return launch_one<4, EPI, NORM>(c, a, norm_w, eps, w, M, N, K, rope, pf, blocks, stream);
  return launch_one<8, EPI, NORM>(c, a, norm_w, eps, w, M, N, K, rope, pf, blocks, stream);
}

template <bool NORM>
int dispatch(void* c, const void* a, const float* norm_w, float eps, const bf16* w, int M, int N, int K, int epilogue,
             const RopeArgs& rope, const Prefetch& pf, int blocks, cudaStream_t stream) {
  switch (epilogue) {
    case EPI_STORE_F32: return launch<EPI_STORE_F32, NORM>(c, a, norm_w, eps, w, M, N, K, rope, pf, blocks, stream);
    case EPI_STORE_T: return launch<EPI_STORE_T, NORM>(c, a, norm_w, eps, w, M, N, K, rope, pf, blocks, stream);
    case EPI_RESIDUAL: return launch<EPI_RESIDUAL, NORM>(c, a, norm_w, eps, w, M, N, K, rope, pf, blocks, stream);
    case EPI_SWIGLU: return launch<EPI_SWIGLU, NORM>(c, a, norm_w, eps, w, M, N, K, rope, pf, blocks, stream);
    case EPI_QKV_ROPE: return launch<EPI_QKV_ROPE, NORM>(c, a, norm_w, eps, w, M, N, K, rope, pf, blocks, stream);
    default: return DLLM_BAD_ARGUMENT;
  }
}
}  // namespace

// C = X[M,K] * W[N,K]^T for M <= 64, epilogues 0..3 as the tile kernels. With norm_w != null, X is the float32
// residual stream and is RMS-normed on the way in; else X is bfloat16. K a multiple of 8, N even for SwiGLU.
// `cluster`: blocks per cluster (1, 2, 4 or 8; 0 chooses). prefetch_ptr / prefetch_bytes: optional memory (weights a
// later kernel reads) to bring into L2 meanwhile.
DLLM_EXPORT int dllm_gemv_cluster(void* c, const void* a, const float* norm_w, float eps, const void* w, int M, int N,
                                  int K, int epilogue, int cluster, const void* prefetch_ptr, long long prefetch_bytes,
                                  cudaStream_t stream) {
  if (M <= 0 || N <= 0) return DLLM_OK;
  if (M > 64 || K <= 0 || (K & 7) || ((N & 1) && epilogue == EPI_SWIGLU) || epilogue < 0 || epilogue > EPI_SWIGLU)
    return DLLM_UNSUPPORTED_SIZE;
  if (cluster < 0) return DLLM_BAD_ARGUMENT;
  int blocks = cluster;
  RopeArgs rope{};
  Prefetch pf{(const char*)prefetch_ptr, prefetch_ptr ? (size_t)prefetch_bytes : 0};
  return norm_w ? dispatch<true>(c, a, norm_w, eps, (const bf16*)w, M, N, K, epilogue, rope, pf, blocks, stream)
                : dispatch<false>(c, a, nullptr, eps, (const bf16*)w, M, N, K, epilogue, rope, pf, blocks, stream);
}

// The q/k/v projection of a step of at most 64 tokens: optional RMSNorm in front, rotation of q and k by the table's
// angle for each token's position, q to q_out, k and v into the token's place in the paged cache.
// W is [(heads + 2 kv_heads) * head_dim, K]. head_dim and rotary_dim must be multiples of 16. prefetch_window: -1, or
// which cached keys the attention behind this kernel will read (0: all, w: the last w): their pages are asked into L2.
DLLM_EXPORT int dllm_gemv_cluster_qkv_rope(const void* a, const float* norm_w, float eps, const void* w, int M, int K,
                                           void* q_out, void* cache_base, const int* page_table, int max_pages,
                                           int page_size, int heads, int kv_heads, int head_dim, const float* table,
                                           int rotary_dim, const int* tok_seq, const int* tok_pos, const int* slots,
                                           int write_cache, int prefetch_window, int cluster,
                                           const void* prefetch_ptr, long long prefetch_bytes, cudaStream_t stream) {
  if (M <= 0) return DLLM_OK;
  if (M > 64 || K <= 0 || (K & 7) || heads <= 0 || kv_heads <= 0 || head_dim <= 0 || (head_dim & 15) ||
      rotary_dim < 0 || rotary_dim > head_dim || (rotary_dim & 15))
    return DLLM_UNSUPPORTED_SIZE;
  if (cluster < 0) return DLLM_BAD_ARGUMENT;
  int blocks = cluster;
  RopeArgs rope{(bf16*)q_out, KvLayout{cache_base, page_table, max_pages, page_size, kv_heads, head_dim},
                (const float2*)table, table ? rotary_dim : 0, heads, tok_seq, tok_pos, slots, write_cache,
                prefetch_window};
  int N = (heads + 2 * kv_heads) * head_dim;
  Prefetch pf{(const char*)prefetch_ptr, prefetch_ptr ? (size_t)prefetch_bytes : 0};
  return norm_w
             ? dispatch<true>(nullptr, a, norm_w, eps, (const bf16*)w, M, N, K, EPI_QKV_ROPE, rope, pf, blocks, stream)
             : dispatch<false>(nullptr, a, nullptr, eps, (const bf16*)w, M, N, K, EPI_QKV_ROPE, rope, pf, blocks, stream);
}
