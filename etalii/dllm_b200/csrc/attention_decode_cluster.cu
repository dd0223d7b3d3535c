// Decode attention (one new token per sequence, bfloat16 cache) with the split over the keys held inside a
// thread-block cluster: the 1, 2, 4 or 8 blocks of a cluster serve one (sequence, kv head); each warp of a block
// takes pages of 64 keys (tile t of the sequence goes to block (t / WARPS) % CLUSTER, warp t % WARPS), computes
// scores and output on the tensor cores (mma.sync m16n8k16; the 16 rows are the query heads of the kv group) with a
// running maximum and sum over its pages. The warps meet in shared memory, the blocks through distributed shared
// memory (mapa + ld.shared::cluster between two cluster barriers): no scratch in global memory, no atomics, and a
// launch shape (blocks per pair, kv heads, sequences) that does not depend on the context length; the number of
// blocks per pair follows from how many pairs there are. head_dim: a multiple of 16 up to 128.
#include "common.cuh"

namespace {
typedef __nv_bfloat16 bf16;
constexpr int TILE_KEYS = 64;

__device__ __forceinline__ void cp_async_16(void* smem, const void* gmem) {
  unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(s), "l"(gmem));
}
__device__ __forceinline__ void ldmatrix_x4(unsigned* r, const void* p) {
  unsigned s = (unsigned)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void ldmatrix_x4_trans(unsigned* r, const void* p) {
  unsigned s = (unsigned)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
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
__device__ __forceinline__ void cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n"
               "barrier.cluster.wait.acquire.aligned;\n" ::: "memory");
}
// A float at the same shared-memory offset in block `rank` of this cluster.
__device__ __forceinline__ float remote_float(const float* local, unsigned rank) {
  unsigned addr = (unsigned)__cvta_generic_to_shared(local), remote;
  float v;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(addr), "r"(rank));
  asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(remote) : "memory");
  return v;
}

// CLUSTER blocks of WARPS warps serve one (sequence, kv head). Few (sequence, kv head) pairs: many blocks per pair
// to fill the device and shorten every chain of pages; many pairs: one block per pair, no exchange between blocks.
template <int HD, int CLUSTER, int WARPS>
__global__ void __launch_bounds__(WARPS * 32) decode_attention_cluster_kernel(
    bf16* __restrict__ out, const bf16* __restrict__ q, KvLayout cache, const int* __restrict__ tok_pos,
    const int* __restrict__ slots, int heads, float scale_log2, int window) {
  constexpr int LD = HD + 8;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  bf16* kv_s = reinterpret_cast<bf16*>(smem_raw);        // per warp: K [64][LD], V [64][LD]
  constexpr int RLD = HD + 8;  // floats per row of the warps' partial outputs: the eight rows a warp writes with one
                               // instruction then lie in different banks (at a stride of HD they all met the same)
  float* red_o = reinterpret_cast<float*>(smem_raw);      // after the products: [WARPS][16][RLD]
  float* cta_o = red_o + WARPS * 16 * RLD;                // this block's partial output [16][HD]
  __shared__ float sm_ml[WARPS][16][2];
  __shared__ float cta_ml[16][2];
  int b = blockIdx.z, g = blockIdx.y;
  unsigned rank = blockIdx.x;  // cluster dims are (CLUSTER, 1, 1) and gridDim.x == CLUSTER
  int hd = cache.head_dim;
  int group = heads / cache.kv_heads;
  pdl_launch_dependents();
  int end = tok_pos[b] + 1;    // positions and slots are written only by the step's last kernel
  int first = (window > 0 && end > window) ? end - window : 0;
  int base = (first / TILE_KEYS) * TILE_KEYS;
  int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int gq = lane >> 2, tq = lane & 3;
  const int* pages = cache.page_table + (size_t)slots[b] * cache.max_pages;
  bf16* k_s = kv_s + (size_t)warp * 2 * TILE_KEYS * LD;
  bf16* v_s = k_s + TILE_KEYS * LD;
  int chunks16 = hd >> 3;
  int newest = end - 1;
  constexpr int ROUND = CLUSTER * WARPS * TILE_KEYS;

  auto copy_page = [&](int key0) {
    int page = pages[key0 / TILE_KEYS];
    const bf16* ksrc = (const bf16*)cache.base + kv_offset(cache, page, 0, g, 0);
    const bf16* vsrc = (const bf16*)cache.base + kv_offset(cache, page, 1, g, 0);
    if (hd == HD) {
#pragma unroll
      for (int i = 0; i < TILE_KEYS * (HD / 8) / 32; ++i) {
        int idx = lane + 32 * i;
        int dst = (idx / (HD / 8)) * LD + (idx % (HD / 8)) * 8;
        cp_async_16(k_s + dst, ksrc + idx * 8);
        cp_async_16(v_s + dst, vsrc + idx * 8);
      }
    } else {
      for (int idx = lane; idx < TILE_KEYS * (HD / 8); idx += 32) {
        int r = idx / (HD / 8), cc = idx % (HD / 8);
        if (cc < chunks16) {
          cp_async_16(k_s + r * LD + cc * 8, ksrc + (size_t)r * hd + cc * 8);
          cp_async_16(v_s + r * LD + cc * 8, vsrc + (size_t)r * hd + cc * 8);
        } else {
          *reinterpret_cast<uint4*>(k_s + r * LD + cc * 8) = make_uint4(0u, 0u, 0u, 0u);
          *reinterpret_cast<uint4*>(v_s + r * LD + cc * 8) = make_uint4(0u, 0u, 0u, 0u);
        }
      }
    }
    asm volatile("cp.async.commit_group;\n" ::);
    return page;
  };

  // this warp's first page: keys of earlier steps do not change any more, so it is copied before the wait on the
  // projection kernel; the row that kernel writes (position end - 1) is read again after the wait
  int my_first = base + ((int)rank * WARPS + warp) * TILE_KEYS;
  int page0 = 0;
  if (my_first < end) page0 = copy_page(my_first);
  // The tile that holds the newest key belongs to one warp of the cluster. That warp asks for the row right after
  // the wait, together with the queries, and puts it into its shared-memory page when the tile's turn comes: the
  // round trip runs under the wait for the page instead of after it.
  int newest_tile = (newest / TILE_KEYS) * TILE_KEYS;
  bool owns_newest = newest_tile >= my_first && (newest_tile - my_first) % ROUND == 0;
  uint4 newest_k = make_uint4(0u, 0u, 0u, 0u), newest_v = newest_k;
  pdl_wait();
  if (owns_newest && lane < chunks16) {
    int page = pages[newest / TILE_KEYS];
    int r = newest - newest_tile;
    newest_k = __ldcg(reinterpret_cast<const uint4*>((const bf16*)cache.base + kv_offset(cache, page, 0, g, r)) + lane);
    newest_v = __ldcg(reinterpret_cast<const uint4*>((const bf16*)cache.base + kv_offset(cache, page, 1, g, r)) + lane);
  }

  for (int h0 = 0; h0 < group; h0 += 16) {
    int nh = min(16, group - h0);
    float o_acc[HD / 8][4];
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
#pragma unroll
    for (int i = 0; i < HD / 8; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) o_acc[i][j] = 0.f;
    unsigned q_frag[HD / 16][4];
    {
      const bf16* q_lo = q + ((size_t)b * heads + g * group + h0 + gq) * hd;
      const bf16* q_hi = q_lo + (size_t)8 * hd;
#pragma unroll
      for (int ks = 0; ks < HD / 16; ++ks) {
        int col = ks * 16 + tq * 2;
        q_frag[ks][0] = (gq < nh && col < hd) ? *reinterpret_cast<const unsigned*>(q_lo + col) : 0u;
        q_frag[ks][1] = (gq + 8 < nh && col < hd) ? *reinterpret_cast<const unsigned*>(q_hi + col) : 0u;
        q_frag[ks][2] = (gq < nh && col + 8 < hd) ? *reinterpret_cast<const unsigned*>(q_lo + col + 8) : 0u;
        q_frag[ks][3] = (gq + 8 < nh && col + 8 < hd) ? *reinterpret_cast<const unsigned*>(q_hi + col + 8) : 0u;
      }
    }
    // (the very first page is already on its way; a later pass over the heads starts again at the first page)
    int page = page0;
    if (h0 != 0 && my_first < end) page = copy_page(my_first);
    for (int key0 = my_first; key0 < end; key0 += ROUND) {
      asm volatile("cp.async.wait_group 0;\n" ::);
      __syncwarp();
      if (key0 == newest_tile) {  // the row the projection kernel has just written (chunks16 <= 16 lanes hold it)
        int r = newest - key0;
        if (lane < chunks16) {
          *reinterpret_cast<uint4*>(k_s + r * LD + lane * 8) = newest_k;
          *reinterpret_cast<uint4*>(v_s + r * LD + lane * 8) = newest_v;
        }
        __syncwarp();
      }
      float s[TILE_KEYS / 8][4];
#pragma unroll
      for (int j = 0; j < TILE_KEYS / 8; ++j)
#pragma unroll
        for (int r = 0; r < 4; ++r) s[j][r] = 0.f;
#pragma unroll
      for (int ks = 0; ks < HD / 16; ++ks) {
#pragma unroll
        for (int jp = 0; jp < TILE_KEYS / 16; ++jp) {
          unsigned bfr[4];
          int mat = lane >> 3;
          ldmatrix_x4(bfr, k_s + (jp * 16 + (mat >> 1) * 8 + (lane & 7)) * LD + ks * 16 + (mat & 1) * 8);
          mma_bf16(s[2 * jp], q_frag[ks], bfr[0], bfr[1]);
          mma_bf16(s[2 * jp + 1], q_frag[ks], bfr[2], bfr[3]);
        }
      }
      if (key0 < first || key0 + TILE_KEYS > end) {  // a tile with an edge: keys outside [first, end) do not count
#pragma unroll
        for (int j = 0; j < TILE_KEYS / 8; ++j)
#pragma unroll
          for (int r = 0; r < 4; ++r) {
            int key = key0 + j * 8 + tq * 2 + (r & 1);
            if (key < first || key >= end) s[j][r] = -INFINITY;
          }
      }
      float tile_max[2] = {-INFINITY, -INFINITY};
#pragma unroll
      for (int j = 0; j < TILE_KEYS / 8; ++j)
#pragma unroll
        for (int r = 0; r < 4; ++r) tile_max[r >> 1] = fmaxf(tile_max[r >> 1], s[j][r]);
      float corr[2], neg_max[2];
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        tile_max[i] = fmaxf(tile_max[i], __shfl_xor_sync(0xffffffffu, tile_max[i], 1));
        tile_max[i] = fmaxf(tile_max[i], __shfl_xor_sync(0xffffffffu, tile_max[i], 2));
        float m_new = fmaxf(m_run[i], tile_max[i] * scale_log2);  // maxima live in the scaled log2 domain
        corr[i] = fast_exp2(m_run[i] - m_new);
        m_run[i] = m_new;
        neg_max[i] = -m_new;
      }
      float row_sum[2] = {0.f, 0.f};
      unsigned p_frag[TILE_KEYS / 16][4];
#pragma unroll
      for (int j = 0; j < TILE_KEYS / 8; ++j) {
        float p0 = fast_exp2(fmaf(s[j][0], scale_log2, neg_max[0])), p1 = fast_exp2(fmaf(s[j][1], scale_log2, neg_max[0]));
        float p2 = fast_exp2(fmaf(s[j][2], scale_log2, neg_max[1])), p3 = fast_exp2(fmaf(s[j][3], scale_log2, neg_max[1]));
        row_sum[0] += p0 + p1;
        row_sum[1] += p2 + p3;
        p_frag[j >> 1][(j & 1) * 2 + 0] = pack_bf16(p0, p1);
        p_frag[j >> 1][(j & 1) * 2 + 1] = pack_bf16(p2, p3);
      }
#pragma unroll
      for (int i = 0; i < 2; ++i) l_run[i] = l_run[i] * corr[i] + row_sum[i];
#pragma unroll
      for (int i = 0; i < HD / 8; ++i) {
        o_acc[i][0] *= corr[0]; o_acc[i][1] *= corr[0];
        o_acc[i][2] *= corr[1]; o_acc[i][3] *= corr[1];
      }
#pragma unroll
      for (int kk = 0; kk < TILE_KEYS / 16; ++kk) {
#pragma unroll
        for (int np = 0; np < HD / 16; ++np) {
          unsigned bfr[4];
          int mat = lane >> 3;
          ldmatrix_x4_trans(bfr, v_s + (kk * 16 + (mat & 1) * 8 + (lane & 7)) * LD + np * 16 + (mat >> 1) * 8);
          mma_bf16(o_acc[2 * np], p_frag[kk], bfr[0], bfr[1]);
          mma_bf16(o_acc[2 * np + 1], p_frag[kk], bfr[2], bfr[3]);
        }
      }
      __syncwarp();  // the page's space is free for the next copy
      if (key0 + ROUND < end) page = copy_page(key0 + ROUND);
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      l_run[i] += __shfl_xor_sync(0xffffffffu, l_run[i], 1);
      l_run[i] += __shfl_xor_sync(0xffffffffu, l_run[i], 2);
    }
    __syncthreads();  // every warp is done with its keys and values: the space becomes the exchange buffer
    if (tq == 0) {
      sm_ml[warp][gq][0] = m_run[0]; sm_ml[warp][gq][1] = l_run[0];
      sm_ml[warp][gq + 8][0] = m_run[1]; sm_ml[warp][gq + 8][1] = l_run[1];
    }
#pragma unroll
    for (int i = 0; i < HD / 8; ++i) {
      int d = i * 8 + tq * 2;
      *reinterpret_cast<float2*>(red_o + ((size_t)warp * 16 + gq) * RLD + d) = make_float2(o_acc[i][0], o_acc[i][1]);
      *reinterpret_cast<float2*>(red_o + ((size_t)warp * 16 + gq + 8) * RLD + d) = make_float2(o_acc[i][2], o_acc[i][3]);
    }
    __syncthreads();
    // the block's partial result: warps in warp order
    for (int idx = threadIdx.x; idx < nh * HD; idx += WARPS * 32) {
      int h = idx / HD, d = idx % HD;
      float m = -INFINITY;
#pragma unroll
      for (int w = 0; w < WARPS; ++w) m = fmaxf(m, sm_ml[w][h][0]);
      float o = 0.f, l = 0.f;
#pragma unroll
      for (int w = 0; w < WARPS; ++w) {
        float f = sm_ml[w][h][0] == -INFINITY ? 0.f : fast_exp2(sm_ml[w][h][0] - m);
        o = fmaf(red_o[((size_t)w * 16 + h) * RLD + d], f, o);
        l = fmaf(sm_ml[w][h][1], f, l);
      }
      cta_o[h * HD + d] = o;
      if (d == 0) { cta_ml[h][0] = m; cta_ml[h][1] = l; }
    }
    if (CLUSTER == 1) {
      __syncthreads();
      for (int idx = threadIdx.x; idx < nh * hd; idx += WARPS * 32) {
        int h = idx / hd, d = idx % hd;
        out[((size_t)b * heads + g * group + h0 + h) * hd + d] = __float2bfloat16_rn(cta_o[h * HD + d] / cta_ml[h][1]);
      }
    } else {
      cluster_sync();  // every block's partial result is in its shared memory
      // The outputs (head, dimension) are dealt out to the blocks of the cluster in equal runs; a thread asks for all
      // blocks' values of its output before it touches the first (one round trip through distributed shared memory,
      // not one per block), then sums in rank order.
      int total = nh * hd, per = (total + CLUSTER - 1) / CLUSTER;
      int stop = min(total, ((int)rank + 1) * per);
      for (int idx = (int)rank * per + threadIdx.x; idx < stop; idx += WARPS * 32) {
        int h = idx / hd, d = idx % hd;
        float mr[CLUSTER], lr[CLUSTER], orr[CLUSTER];
#pragma unroll
        for (unsigned r = 0; r < CLUSTER; ++r) {
          mr[r] = remote_float(&cta_ml[h][0], r);
          lr[r] = remote_float(&cta_ml[h][1], r);
          orr[r] = remote_float(&cta_o[h * HD + d], r);
        }
        float m = -INFINITY;
#pragma unroll
        for (unsigned r = 0; r < CLUSTER; ++r) m = fmaxf(m, mr[r]);
        float o = 0.f, l = 0.f;
#pragma unroll
        for (unsigned r = 0; r < CLUSTER; ++r) {
          float f = mr[r] == -INFINITY ? 0.f : fast_exp2(mr[r] - m);
          o = fmaf(orr[r], f, o);
          l = fmaf(lr[r], f, l);
        }
        out[((size_t)b * heads + g * group + h0 + h) * hd + d] = __float2bfloat16_rn(o / l);
      }
    }
    if (CLUSTER > 1) cluster_sync();  // nobody leaves (or reuses the space) while others still read its partial result
    else __syncthreads();
  }
}

template <int HD, int WARPS>
constexpr size_t block_smem() {
  size_t kv_bytes = (size_t)WARPS * 2 * TILE_KEYS * (HD + 8) * sizeof(bf16);
  size_t red_bytes = (size_t)(WARPS * 16 * (HD + 8) + 16 * HD) * sizeof(float);
  return kv_bytes > red_bytes ? kv_bytes : red_bytes;
}

template <int HD, int CLUSTER, int WARPS>
int launch(void* out, const void* q, const KvLayout& cache, const int* tok_pos, const int* slots, int heads,
           int sequences, float scale, int window, cudaStream_t stream) {
  constexpr size_t smem = block_smem<HD, WARPS>();
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(decode_attention_cluster_kernel<HD, CLUSTER, WARPS>,
                             cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
      return DLLM_LAUNCH_FAILED;
    configured = true;
  }
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3(CLUSTER, cache.kv_heads, sequences);
  config.blockDim = dim3(WARPS * 32);
  config.dynamicSmemBytes = smem;
  config.stream = stream;
  cudaLaunchAttribute attributes[2];
  attributes[0].id = cudaLaunchAttributeClusterDimension;
  attributes[0].val.clusterDim.x = CLUSTER;
  attributes[0].val.clusterDim.y = 1;
  attributes[0].val.clusterDim.z = 1;
  attributes[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attributes[1].val.programmaticStreamSerializationAllowed = 1;
  config.attrs = attributes;
  config.numAttrs = dllm_pdl_enabled() ? 2 : 1;
  return cudaLaunchKernelEx(&config, decode_attention_cluster_kernel<HD, CLUSTER, WARPS>, (bf16*)out, (const bf16*)q,
                            cache, tok_pos, slots, heads, scale * 1.4426950408889634f, window) == cudaSuccess
             ? DLLM_OK
             : DLLM_LAUNCH_FAILED;
}

// What bounds this kernel is how many pages are on their way into shared memory at once: blocks are kept small
// (4 warps, 2 where a page of head_dim above 64 is twice as large) so that three of them share a multiprocessor,
// and the number of blocks per (sequence, kv head) pair is the smallest power of two that fills those places.
// Launch shapes 0..3: 1, 2, 4, 8 blocks per pair; shape 4: 8 blocks of 4 warps at any head_dim (for very few pairs,
// where every block has a multiprocessor of its own anyway).
constexpr int SHAPES = 5;
constexpr size_t SMEM_PER_SM = 227 * 1024;

template <int HD>
int launch_shape(int shape, void* out, const void* q, const KvLayout& cache, const int* tok_pos, const int* slots,
                 int heads, int sequences, float scale, int window, cudaStream_t stream) {
  constexpr int NW = HD > 64 ? 2 : 4;
  if (shape < 0) {
    static int sms = 0;
    if (sms == 0) {
      int device = 0;
      if (cudaGetDevice(&device) != cudaSuccess ||
          cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || sms <= 0)
        sms = 148;
    }
    long long pairs = (long long)sequences * cache.kv_heads;
    size_t per_sm = SMEM_PER_SM / (block_smem<HD, NW>() + 1024);
    long long places = (long long)sms * (long long)(per_sm > 8 ? 8 : per_sm);
    if (pairs * 8 <= sms) shape = 4;
    else for (shape = 0; shape < 3 && (pairs << shape) * 20 < places * 17; ++shape) {}
    // (heads above 64: a block is two warps, and two blocks a pair even out contexts of unequal length better than
    // one; measured with 32 query and 8 kv heads of 128, contexts 128 to 2,304: 64 sequences 62.5 µs against 69.0,
    // 128 sequences 129.3 against 134.0)
    if (HD > 64 && shape == 0 && pairs <= 4 * places) shape = 1;
  }
#define DLLM_GO(CL, WARPS) \
  return launch<HD, CL, WARPS>(out, q, cache, tok_pos, slots, heads, sequences, scale, window, stream)
  switch (shape) {
    case 0: DLLM_GO(1, NW);
    case 1: DLLM_GO(2, NW);
    case 2: DLLM_GO(4, NW);
    case 3: DLLM_GO(8, NW);
    case 4: DLLM_GO(8, 4);
  }
#undef DLLM_GO
  return DLLM_BAD_ARGUMENT;
}
}  // namespace

// out, q: [sequences, heads * head_dim] bfloat16; sequence b's query is the token at tok_pos[b], whose key and value
// are already in the cache. head_dim a multiple of 16 up to 128, pages of 64 positions, at most 65,535 sequences.
// shape: -1 chooses by the number of (sequence, kv head) pairs; 0..4 name a launch shape (see above).
DLLM_EXPORT int dllm_attention_decode_cluster(void* out, const void* q, void* cache_base, const int* page_table,
                                              int max_pages, int page_size, int heads, int kv_heads, int head_dim,
                                              const int* tok_pos, const int* slots, int sequences, float scale,
                                              int window, int shape, cudaStream_t stream) {
  if (sequences <= 0) return DLLM_OK;
  if (heads <= 0 || kv_heads <= 0 || heads % kv_heads || shape < -1 || shape >= SHAPES) return DLLM_BAD_ARGUMENT;
  if (head_dim <= 0 || head_dim > 128 || (head_dim & 15) || page_size != TILE_KEYS || sequences > 65535 ||
      kv_heads > 65535)
    return DLLM_UNSUPPORTED_SIZE;
  KvLayout cache{cache_base, page_table, max_pages, page_size, kv_heads, head_dim};
  if (head_dim <= 32) return launch_shape<32>(shape, out, q, cache, tok_pos, slots, heads, sequences, scale, window, stream);
  if (head_dim <= 64) return launch_shape<64>(shape, out, q, cache, tok_pos, slots, heads, sequences, scale, window, stream);
  return launch_shape<128>(shape, out, q, cache, tok_pos, slots, heads, sequences, scale, window, stream);
}
