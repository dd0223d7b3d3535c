// Prefill attention over the paged cache (bfloat16), blockwise with an online softmax, on the tensor cores
// (mma.sync m16n8k16). A block takes 64 consecutive new tokens of one sequence and one query head. Its eight warps
// form two groups of four; in a group every warp owns 16 queries, and the two groups take alternate key/value tiles
// (the longest query tile's serial chain of tiles is halved) and are merged at the end. Key/value tiles are whole
// cache pages (64 positions), copied to shared memory with cp.async, double buffered per group. Scores, the running maximum and sum and the output accumulate in float32; probabilities are
// rounded to bfloat16 only as the operand of the second product. Causal and window masks are applied per element.
// Tiles of queries never straddle sequences: the host lists (sequence, first token) per tile.
//
// head_dim: any multiple of 16 up to 128 (the kernel is instantiated for 32, 64 and 128 and pads with zeros).
// The page size must be 64.
#include "common.cuh"

namespace {
typedef __nv_bfloat16 bf16;
constexpr int BM = 64, BN = 64, WARPS = 4, GROUPS = 2, THREADS = GROUPS * WARPS * 32;
constexpr int MAX_TILES = 512;  // page indices kept in shared memory (32,768 positions); beyond: read as needed

__device__ __forceinline__ void cp_async_16(void* smem, const void* gmem, bool valid) {
  unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  int bytes = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(s), "l"(gmem), "r"(bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }
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

template <int HD>
__global__ void __launch_bounds__(THREADS) prefill_kernel(
    bf16* __restrict__ out, const bf16* __restrict__ q, KvLayout cache, const int* __restrict__ tile_seq,
    const int* __restrict__ tile_first, const int* __restrict__ cu_seqlens, const int* __restrict__ start,
    const int* __restrict__ slots, int heads, float scale_log2, int window) {
  constexpr int LD = HD + 8;  // padded row, keeps 16-byte alignment
  extern __shared__ __align__(16) unsigned char smem_raw[];
  bf16* q_s = reinterpret_cast<bf16*>(smem_raw);            // [BM][LD]
  int group = threadIdx.x / (WARPS * 32);                    // which half of the key tiles this warp works on
  bf16* k_s = q_s + BM * LD + (size_t)group * 4 * BN * LD;   // per group: [2][BN][LD]
  bf16* v_s = k_s + 2 * BN * LD;                             // per group: [2][BN][LD]
  int tile = blockIdx.x, h = blockIdx.y;
  int b = tile_seq[tile], q0 = tile_first[tile];
  int hd = cache.head_dim;
  int g = h / (heads / cache.kv_heads);
  int n_new = cu_seqlens[b + 1] - cu_seqlens[b];
  int tok0 = cu_seqlens[b] + q0;           // first token row of this tile in the packed batch
  int rows = min(BM, n_new - q0);          // queries of this tile that exist
  int pos0 = start[b] + q0;                // absolute position of the tile's first query
  const int* pages = cache.page_table + (size_t)slots[b] * cache.max_pages;
  const bf16* base = (const bf16*)cache.base;
  int tid = threadIdx.x % (WARPS * 32), lane = tid & 31, warp = tid >> 5;  // within the group
  int chunks = hd >> 3;                    // 16-byte pieces of a real row
  auto group_sync = [&]() { asm volatile("bar.sync %0, %1;" ::"r"(group + 1), "r"(WARPS * 32) : "memory"); };

  // queries -> shared memory (rows beyond the tile and dims beyond head_dim are zero)
  for (int idx = threadIdx.x; idx < BM * (HD / 8); idx += THREADS) {
    int r = idx / (HD / 8), c = idx % (HD / 8);
    bool ok = r < rows && c < chunks;
    const bf16* src = ok ? q + ((size_t)(tok0 + r) * heads + h) * hd + c * 8 : q;
    cp_async_16(q_s + r * LD + c * 8, src, ok);
  }
  int last_pos = pos0 + rows - 1;                                   // last query's position
  int kt_end = last_pos / BN;                                       // last key tile any query of the tile sees
  int kt_begin = (window > 0 && pos0 + 1 > window) ? (pos0 + 1 - window) / BN : 0;
  // the pages of the key tiles this block will read, fetched once (not one dependent load per tile)
  __shared__ int page_s[MAX_TILES];
  for (int i = threadIdx.x; i <= kt_end - kt_begin && i < MAX_TILES; i += THREADS) page_s[i] = pages[kt_begin + i];
  __syncthreads();

  const int flat_dst = (tid / (HD / 8)) * LD + (tid % (HD / 8)) * 8, flat_src = tid * 8;
  auto load_kv = [&](int stage, int kt) {
    int page = kt - kt_begin < MAX_TILES ? page_s[kt - kt_begin] : pages[kt];
    const bf16* ksrc = base + kv_offset(cache, page, 0, g, 0);
    const bf16* vsrc = base + kv_offset(cache, page, 1, g, 0);
    if (hd == HD) {
      // the page is one flat piece; each thread's pieces sit at fixed offsets (computed once, below)
#pragma unroll
      for (int i = 0; i < BN * (HD / 8) / (WARPS * 32); ++i) {
        int dst = stage * BN * LD + flat_dst + i * ((WARPS * 32) / (HD / 8)) * LD;
        int src = flat_src + i * (WARPS * 32) * 8;
        cp_async_16(k_s + dst, ksrc + src, true);
        cp_async_16(v_s + dst, vsrc + src, true);
      }
    } else {
      for (int idx = tid; idx < BN * (HD / 8); idx += WARPS * 32) {
        int r = idx / (HD / 8), c = idx % (HD / 8);
        bool ok = c < chunks;
        cp_async_16(k_s + (stage * BN + r) * LD + c * 8, ok ? ksrc + (size_t)r * hd + c * 8 : ksrc, ok);
        cp_async_16(v_s + (stage * BN + r) * LD + c * 8, ok ? vsrc + (size_t)r * hd + c * 8 : vsrc, ok);
      }
    }
  };
  int kt_first = kt_begin + group;          // this group's tiles: kt_first, kt_first + GROUPS, ...
  if (kt_first <= kt_end) load_kv(0, kt_first);
  cp_async_commit();
  cp_async_wait<0>();
  __syncthreads();  // the queries were copied by all threads of the block: both groups may read them from here on

  float o_acc[HD / 8][4];
#pragma unroll
  for (int i = 0; i < HD / 8; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) o_acc[i][j] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
  unsigned q_frag[HD / 16][4];
  int gq = lane >> 2, tq = lane & 3;
  int row_pos[2] = {pos0 + warp * 16 + gq, pos0 + warp * 16 + gq + 8};  // positions of this thread's two rows

  bool have_q = false;
  for (int kt = kt_first; kt <= kt_end; kt += GROUPS) {
    int stage = ((kt - kt_first) / GROUPS) & 1;
    if (kt + GROUPS <= kt_end) load_kv(stage ^ 1, kt + GROUPS);
    cp_async_commit();
    cp_async_wait<1>();
    group_sync();
    if (!have_q) {
      have_q = true;
#pragma unroll
      for (int ks = 0; ks < HD / 16; ++ks)
        ldmatrix_x4(q_frag[ks], q_s + (warp * 16 + (lane & 15)) * LD + ks * 16 + (lane >> 4) * 8);
    }
    // scores of 16 queries x 64 keys
    float s[BN / 8][4];
#pragma unroll
    for (int j = 0; j < BN / 8; ++j)
#pragma unroll
      for (int r = 0; r < 4; ++r) s[j][r] = 0.f;
    const bf16* kb = k_s + stage * BN * LD;
#pragma unroll
    for (int ks = 0; ks < HD / 16; ++ks) {
#pragma unroll
      for (int jp = 0; jp < BN / 16; ++jp) {
        unsigned bfr[4];
        int mat = lane >> 3;
        ldmatrix_x4(bfr, kb + (jp * 16 + (mat >> 1) * 8 + (lane & 7)) * LD + ks * 16 + (mat & 1) * 8);
        mma_bf16(s[2 * jp], q_frag[ks], bfr[0], bfr[1]);
        mma_bf16(s[2 * jp + 1], q_frag[ks], bfr[2], bfr[3]);
      }
    }
    // scale (log2 domain), masks, running maximum
    int key0 = kt * BN;
    bool need_mask = key0 + BN - 1 > pos0 + warp * 16 || (window > 0 && key0 < pos0 + warp * 16 + 16 - window);
    float tile_max[2] = {-INFINITY, -INFINITY};
    if (need_mask) {
#pragma unroll
      for (int j = 0; j < BN / 8; ++j)
#pragma unroll
        for (int r = 0; r < 4; ++r) {
          int key = key0 + j * 8 + tq * 2 + (r & 1);
          int qp = row_pos[r >> 1];
          if (key > qp || (window > 0 && key < qp + 1 - window)) s[j][r] = -INFINITY;
        }
    }
#pragma unroll
    for (int j = 0; j < BN / 8; ++j)
#pragma unroll
      for (int r = 0; r < 4; ++r) tile_max[r >> 1] = fmaxf(tile_max[r >> 1], s[j][r]);
    float corr[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      tile_max[i] = fmaxf(tile_max[i], __shfl_xor_sync(0xffffffffu, tile_max[i], 1));
      tile_max[i] = fmaxf(tile_max[i], __shfl_xor_sync(0xffffffffu, tile_max[i], 2));
      tile_max[i] *= scale_log2;  // maxima live in the scaled log2 domain; the scores are scaled inside the exponent
      float m_new = fmaxf(m_run[i], tile_max[i]);
      float m_use = m_new == -INFINITY ? 0.f : m_new;  // a row that sees nothing in this tile (and nothing before)
      corr[i] = fast_exp2(m_run[i] - m_use);
      m_run[i] = m_new;
      tile_max[i] = m_use;
    }
    float row_sum[2] = {0.f, 0.f};
    unsigned p_frag[BN / 16][4];
#pragma unroll
    for (int j = 0; j < BN / 8; ++j) {
      float p0 = fast_exp2(fmaf(s[j][0], scale_log2, -tile_max[0])), p1 = fast_exp2(fmaf(s[j][1], scale_log2, -tile_max[0]));
      float p2 = fast_exp2(fmaf(s[j][2], scale_log2, -tile_max[1])), p3 = fast_exp2(fmaf(s[j][3], scale_log2, -tile_max[1]));
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
    // output += probabilities x values
    const bf16* vb = v_s + stage * BN * LD;
#pragma unroll
    for (int kk = 0; kk < BN / 16; ++kk) {
#pragma unroll
      for (int np = 0; np < HD / 16; ++np) {
        unsigned bfr[4];
        int mat = lane >> 3;
        ldmatrix_x4_trans(bfr, vb + (kk * 16 + (mat & 1) * 8 + (lane & 7)) * LD + np * 16 + (mat >> 1) * 8);
        mma_bf16(o_acc[2 * np], p_frag[kk], bfr[0], bfr[1]);
        mma_bf16(o_acc[2 * np + 1], p_frag[kk], bfr[2], bfr[3]);
      }
    }
    group_sync();  // the stage is free for the load after next
  }
  cp_async_wait<0>();
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    l_run[i] += __shfl_xor_sync(0xffffffffu, l_run[i], 1);
    l_run[i] += __shfl_xor_sync(0xffffffffu, l_run[i], 2);
  }
  // merge the second group into the first through shared memory (the key/value space is free now)
  __syncthreads();
  float* ex_o = reinterpret_cast<float*>(q_s + BM * LD);          // [WARPS*32 threads][HD/8*4] outputs
  float* ex_ml = ex_o + (size_t)WARPS * 32 * (HD / 2);            // [threads][4]: m0, m1, l0, l1
  if (group == 1) {
#pragma unroll
    for (int i = 0; i < HD / 8; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) ex_o[(size_t)(i * 4 + j) * (WARPS * 32) + tid] = o_acc[i][j];
    ex_ml[0 * WARPS * 32 + tid] = m_run[0]; ex_ml[1 * WARPS * 32 + tid] = m_run[1];
    ex_ml[2 * WARPS * 32 + tid] = l_run[0]; ex_ml[3 * WARPS * 32 + tid] = l_run[1];
  }
  __syncthreads();
  if (group == 1) return;
  {
    float other_m[2] = {ex_ml[0 * WARPS * 32 + tid], ex_ml[1 * WARPS * 32 + tid]};
    float other_l[2] = {ex_ml[2 * WARPS * 32 + tid], ex_ml[3 * WARPS * 32 + tid]};
    float mine[2], theirs[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      float m = fmaxf(m_run[i], other_m[i]);
      float m_use = m == -INFINITY ? 0.f : m;
      mine[i] = fast_exp2(m_run[i] - m_use);
      theirs[i] = fast_exp2(other_m[i] - m_use);
      l_run[i] = l_run[i] * mine[i] + other_l[i] * theirs[i];
    }
#pragma unroll
    for (int i = 0; i < HD / 8; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j)
        o_acc[i][j] = o_acc[i][j] * mine[j >> 1] + ex_o[(size_t)(i * 4 + j) * (WARPS * 32) + tid] * theirs[j >> 1];
  }
  // normalise and store
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    int r = warp * 16 + gq + half * 8;
    if (r >= rows) continue;
    float inv = 1.0f / l_run[half];
    bf16* dst = out + ((size_t)(tok0 + r) * heads + h) * hd;
#pragma unroll
    for (int i = 0; i < HD / 8; ++i) {
      int d = i * 8 + tq * 2;
      if (d < hd) *reinterpret_cast<__nv_bfloat162*>(dst + d) =
          __floats2bfloat162_rn(o_acc[i][half * 2] * inv, o_acc[i][half * 2 + 1] * inv);
    }
  }
}

template <int HD>
int launch(void* out, const void* q, const KvLayout& cache, const int* tile_seq, const int* tile_first,
           const int* cu_seqlens, const int* start, const int* slots, int tiles, int heads, float scale, int window,
           cudaStream_t stream) {
  size_t smem = (size_t)(BM + GROUPS * 4 * BN) * (HD + 8) * sizeof(bf16);
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(prefill_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
      return DLLM_LAUNCH_FAILED;
    configured = true;
  }
  dim3 grid(tiles, heads);
  prefill_kernel<HD><<<grid, THREADS, smem, stream>>>((bf16*)out, (const bf16*)q, cache, tile_seq, tile_first,
                                                      cu_seqlens, start, slots, heads,
                                                      scale * 1.4426950408889634f, window);
  return dllm_launch_status();
}
}  // namespace

// out, q: [tokens, heads * head_dim] bfloat16. tile_seq / tile_first: for each tile of up to 64 new tokens, its
// sequence and the index of its first token among the sequence's new tokens. The keys and values of the new tokens
// are already in the cache.
DLLM_EXPORT int dllm_attention_prefill(void* out, const void* q, void* cache_base, const int* page_table,
                                       int max_pages, int page_size, int heads, int kv_heads, int head_dim,
                                       const int* tile_seq, const int* tile_first, const int* cu_seqlens,
                                       const int* start, const int* slots, int tiles, float scale, int window,
                                       cudaStream_t stream) {
  if (tiles <= 0) return DLLM_OK;
  if (heads <= 0 || kv_heads <= 0 || heads % kv_heads) return DLLM_BAD_ARGUMENT;
  if (head_dim <= 0 || head_dim > 128 || (head_dim & 15) || page_size != BN || heads > 65535)
    return DLLM_UNSUPPORTED_SIZE;
  KvLayout cache{cache_base, page_table, max_pages, page_size, kv_heads, head_dim};
  if (head_dim <= 32)
    return launch<32>(out, q, cache, tile_seq, tile_first, cu_seqlens, start, slots, tiles, heads, scale, window, stream);
  if (head_dim <= 64)
    return launch<64>(out, q, cache, tile_seq, tile_first, cu_seqlens, start, slots, tiles, heads, scale, window, stream);
  return launch<128>(out, q, cache, tile_seq, tile_first, cu_seqlens, start, slots, tiles, heads, scale, window, stream);
}
