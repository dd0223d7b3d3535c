// Weight-streaming products for decode (at most 64 rows of activations, bfloat16 weights): C = X * W^T where reading
// W once is the whole cost. A block owns 16 output columns (16 rows of W) and splits the reduction over its warps.
// The products run on the tensor cores with W as the 16-row operand (mma.sync m16n8k16, "swap A and B"): a thread
// loads 16 bytes of two rows of W and 16 bytes of one row of X per 32 values of k, all loads of a warp are issued
// before the first product, and no shuffle reduction is needed; the warps' partial tiles meet in shared memory in
// warp order. The k positions inside a 32-block are permuted the same way for W and X, which a sum does not see.
//
// Fused around the product, to save kernels and memory traffic in the decode step:
//   - in front: RMSNorm of the float32 residual stream (the block sums x^2 itself; x * norm_weight is rounded to
//     bfloat16 as the product's operand and 1/rms is applied to the float32 result);
//   - behind: store (float32 or bfloat16), residual add in float32, SwiGLU on interleaved gate/up rows, or rotary
//     position encoding of q/k and the write of k and v into the paged cache (q/k/v projection).
#include "gemv_common.cuh"

namespace {
using namespace gemv;

// What a thread's first epilogue item needs from memory besides the product: fetched right after the wait on the
// previous kernel, so that the latency runs under the products instead of after them.
template <int EPI, int NT>
struct Early {
  float r0 = 0.f, r1 = 0.f;   // residual values (EPI_RESIDUAL)
  int have = 0;
  int pos = 0, page = 0;      // position and cache page of the token (EPI_QKV_ROPE)
  float2 cs = make_float2(1.f, 0.f);
  __device__ __forceinline__ void load(const void* c, int tid, int M, int N, int item, const RopeArgs& rope,
                                       bool paired, int dim0) {
    int p = tid / (NT * 8), m = tid % (NT * 8);
    if (p >= 8 || m >= M) return;
    if (EPI == EPI_RESIDUAL) {
      int n = item * TILE + 2 * p;
      if (n < N) {
        const float* src = (const float*)c + (size_t)m * N + n;
        r0 = src[0];
        have = 1;
        if (n + 1 < N) { r1 = src[1]; have = 2; }
      }
    } else if (EPI == EPI_QKV_ROPE) {
      pos = rope.tok_pos[m];
      if (paired) cs = rope.table[(size_t)pos * (rope.rotary_dim / 2) + dim0 + p];
      int slot = rope.slots[rope.tok_seq[m]];
      page = rope.cache.page_table[(size_t)slot * rope.cache.max_pages + pos / rope.cache.page_size];
    }
  }
};

template <int WARPS, int NT, int EPI, bool NORM, bool PIPE>
__global__ void __launch_bounds__(WARPS * 32) gemv_kernel(void* __restrict__ c, const void* __restrict__ a,
                                                          const float* __restrict__ norm_w, float eps,
                                                          const bf16* __restrict__ w, int M, int N, int K,
                                                          RopeArgs rope, Prefetch pf, int items) {
  // 32-value k steps whose loads a warp issues before the first product (fewer when more tokens need registers)
  constexpr int MAX_STEPS = NORM ? (NT == 1 ? 6 : (NT == 2 ? 3 : 1)) : (NT == 1 ? 8 : (NT == 2 ? 4 : 2));
  // exchange space of the warps: [WARPS][TILE][NT * 8 + 1] partial tiles, then [WARPS][NT * 8] sums of squares
  extern __shared__ float exchange[];
  float (*red)[TILE][NT * 8 + 1] = reinterpret_cast<float (*)[TILE][NT * 8 + 1]>(exchange);
  float (*red_ss)[NT * 8] = reinterpret_cast<float (*)[NT * 8]>(exchange + WARPS * TILE * (NT * 8 + 1));
  int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  int g = lane >> 2, t = lane & 3;
  // A block takes the tiles blockIdx.x, blockIdx.x + gridDim.x, ... of the `items` tiles of 16 rows of W. (Launched
  // with one block per tile, the loop below runs once.)
  int item = blockIdx.x;
  int head, dim0;
  bool paired;
  int row_lo = tile_row<EPI>(item, g, N, rope, head, dim0, paired);
  int row_hi = tile_row<EPI>(item, g + 8, N, rope, head, dim0, paired);
  const uint4* w_lo = (const uint4*)(w + (size_t)row_lo * K);
  const uint4* w_hi = (const uint4*)(w + (size_t)row_hi * K);
  int chunks = K >> 3;                   // 16-byte pieces of a row
  int steps = (chunks + 3) >> 2;         // k steps of 32 values
  int per_warp = (steps + WARPS - 1) / WARPS;
  int s_begin = warp * per_warp, s_end = min(steps, s_begin + per_warp);

  float acc[NT][4];
  float ss[NT];
#pragma unroll
  for (int n = 0; n < NT; ++n) {
    ss[n] = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) acc[n][i] = 0.f;
  }
  const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
  Early<EPI, NT> early;
  pdl_launch_dependents();
  // A stretch is MAX_STEPS k steps. Every load of a stretch is issued before its first product. For long rows
  // (PIPE: a warp has more than one stretch) the weights of the NEXT stretch are requested before this stretch's
  // products start, so that the row streams without pauses.
  uint4 wl[MAX_STEPS], wh[MAX_STEPS];
  auto load_weights = [&](int s0, uint4* lo, uint4* hi) {
#pragma unroll
    for (int i = 0; i < MAX_STEPS; ++i) {
      int ch = (s0 + i) * 4 + t;
      bool ok = s0 + i < s_end && ch < chunks;
      lo[i] = ok ? __ldg(w_lo + ch) : zero;
      hi[i] = ok ? __ldg(w_hi + ch) : zero;
    }
  };
  if (s_begin < s_end) load_weights(s_begin, wl, wh);
  if (EPI == EPI_QKV_ROPE) prefetch_cache_pages(rope, M);
  bool waited = false;
  for (;;) {
    for (int s0 = s_begin; s0 < s_end; s0 += MAX_STEPS) {
      uint4 xb[MAX_STEPS][NT];
      if (s0 == s_begin) {
        if (!PIPE || !waited) {
          prefetch_share(pf);
          pdl_wait();  // the weights above are nobody's output; everything below may be the previous kernel's
          waited = true;
        }
        early.load(c, tid, M, N, item, rope, paired, dim0);
      }
      if (NORM) {
        // all loads of the stretch first (activations and norm weights), then the arithmetic: a step's loads must
        // not wait behind the previous step's sums
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
            if (ok && m < M) {
              const float4* xp = (const float4*)((const float*)a + (size_t)m * K) + 2 * ch;
              xr[i][n][0] = xp[0];
              xr[i][n][1] = xp[1];
            }
          }
        }
#pragma unroll
        for (int i = 0; i < MAX_STEPS; ++i) {
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
        for (int i = 0; i < MAX_STEPS; ++i) {
          int ch = (s0 + i) * 4 + t;
          bool ok = s0 + i < s_end && ch < chunks;
#pragma unroll
          for (int n = 0; n < NT; ++n) {
            int m = n * 8 + g;
            xb[i][n] = (ok && m < M) ? *((const uint4*)((const bf16*)a + (size_t)m * K) + ch) : zero;
          }
        }
      }
      uint4 wl_next[PIPE ? MAX_STEPS : 1], wh_next[PIPE ? MAX_STEPS : 1];
      bool more = PIPE && s0 + MAX_STEPS < s_end;
      if (PIPE && more) load_weights(s0 + MAX_STEPS, wl_next, wh_next);
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
      if (PIPE) {
        if (more) {
#pragma unroll
          for (int i = 0; i < MAX_STEPS; ++i) { wl[i] = wl_next[PIPE ? i : 0]; wh[i] = wh_next[PIPE ? i : 0]; }
        }
      } else if (s0 + MAX_STEPS < s_end) {
        load_weights(s0 + MAX_STEPS, wl, wh);
      }
    }
    if (s_begin >= s_end) {  // a warp without work has not waited yet
      if (!PIPE || !waited) {
        pdl_wait();
        waited = true;
      }
      early.load(c, tid, M, N, item, rope, paired, dim0);
    }
    // the block's next tile: its first weights are requested now and travel while this tile is summed and stored
    // (only the variants for long rows walk over several tiles; the others are launched with a block per tile)
    int next = PIPE ? item + (int)gridDim.x : items, next_head = 0, next_dim0 = 0;
    bool next_paired = false;
    if (PIPE && next < items) {
      row_lo = tile_row<EPI>(next, g, N, rope, next_head, next_dim0, next_paired);
      row_hi = tile_row<EPI>(next, g + 8, N, rope, next_head, next_dim0, next_paired);
      w_lo = (const uint4*)(w + (size_t)row_lo * K);
      w_hi = (const uint4*)(w + (size_t)row_hi * K);
      if (s_begin < s_end) load_weights(s_begin, wl, wh);
    }
    // partial tiles and partial sums of squares to shared memory
#pragma unroll
    for (int n = 0; n < NT; ++n) {
      red[warp][g][n * 8 + 2 * t] = acc[n][0];
      red[warp][g][n * 8 + 2 * t + 1] = acc[n][1];
      red[warp][g + 8][n * 8 + 2 * t] = acc[n][2];
      red[warp][g + 8][n * 8 + 2 * t + 1] = acc[n][3];
      if (NORM) {
        float v = ss[n];
        v += __shfl_xor_sync(0xffffffffu, v, 1);
        v += __shfl_xor_sync(0xffffffffu, v, 2);
        if (t == 0) red_ss[warp][n * 8 + g] = v;
      }
    }
    __syncthreads();

    float best_value = -INFINITY;  // EPI_ARGMAX: the larger of this thread's two features (the lower on a tie)
    int best_feature = 0x7fffffff;
    // one thread per (pair of tile rows, token): rows (2p, 2p+1), or (p, p + 8) for rotary pairs
    for (int idx = tid; idx < 8 * NT * 8; idx += WARPS * 32) {
      int p = idx / (NT * 8), m = idx % (NT * 8);
      if (m >= M) continue;
      int r0 = (EPI == EPI_QKV_ROPE) ? p : 2 * p, r1 = (EPI == EPI_QKV_ROPE) ? p + 8 : 2 * p + 1;
      float v0 = 0.f, v1 = 0.f, sumsq = 0.f;
#pragma unroll
      for (int wi = 0; wi < WARPS; ++wi) {
        v0 += red[wi][r0][m];
        v1 += red[wi][r1][m];
        if (NORM) sumsq += red_ss[wi][m];
      }
      if (NORM) {
        float inv = 1.0f / sqrtf(sumsq / (float)K + eps);
        v0 *= inv;
        v1 *= inv;
      }
      bool first_item = idx == tid;  // what `early` fetched belongs to each thread's first item
      if (EPI == EPI_QKV_ROPE) {
        int hd = rope.cache.head_dim, nkv = rope.cache.kv_heads, heads = rope.heads;
        int pos = first_item ? early.pos : rope.tok_pos[m];
        int d0, d1;
        if (paired) {
          int half = rope.rotary_dim / 2;
          d0 = dim0 + p;
          d1 = d0 + half;
          float2 cs = first_item ? early.cs : rope.table[(size_t)pos * half + d0];
          float x = v0, y = v1;
          v0 = fmaf(x, cs.x, -(y * cs.y));
          v1 = fmaf(x, cs.y, y * cs.x);
        } else {
          d0 = dim0 + p;
          d1 = d0 + 8;
        }
        bf16* dst;
        if (head < heads) {
          dst = rope.q_out + ((size_t)m * heads + head) * hd;
        } else {
          if (!rope.write_cache) continue;
          int which = head < heads + nkv ? 0 : 1;
          int kvh = head - heads - which * nkv;
          int page = first_item ? early.page
                                : rope.cache.page_table[(size_t)rope.slots[rope.tok_seq[m]] * rope.cache.max_pages +
                                                        pos / rope.cache.page_size];
          dst = (bf16*)rope.cache.base + kv_offset(rope.cache, page, which, kvh, pos % rope.cache.page_size);
        }
        dst[d0] = __float2bfloat16_rn(v0);
        dst[d1] = __float2bfloat16_rn(v1);
      } else if (EPI == EPI_RESIDUAL && first_item && early.have) {
        float* dst = (float*)c + (size_t)m * N + item * TILE + 2 * p;
        dst[0] = early.r0 + v0;
        if (early.have > 1) dst[1] = early.r1 + v1;
      } else if (EPI == EPI_ARGMAX) {
        int n = item * TILE + 2 * p;  // (a value that is not a number is never larger: it is never chosen)
        if (n < N && v0 > best_value) { best_value = v0; best_feature = n; }
        if (n + 1 < N && v1 > best_value) { best_value = v1; best_feature = n + 1; }
      } else {
        epilogue_pair<EPI, bf16>(c, m, item * TILE + 2 * p, M, N, v0, v1);
      }
    }
    if (EPI == EPI_ARGMAX) {  // (at most one item a thread: the launch gives 8 * NT * 8 threads or more)
      __syncthreads();        // every partial tile has been read: the space now takes the threads' candidates
      float* values = exchange;
      int* features = reinterpret_cast<int*>(exchange + 8 * NT * 8);
      if (tid < 8 * NT * 8) { values[tid] = best_value; features[tid] = best_feature; }
      __syncthreads();
      if (tid < NT * 8 && tid < M) {  // pairs in ascending order of their features: the first largest wins
        float best = -INFINITY;
        int feature = 0x7fffffff;
#pragma unroll
        for (int q = 0; q < 8; ++q) {
          float v = values[q * (NT * 8) + tid];
          if (v > best) { best = v; feature = features[q * (NT * 8) + tid]; }
        }
        float* out = (float*)c + ((size_t)tid * items + item) * 2;
        out[0] = best;
        out[1] = __int_as_float(feature);
      }
    }
    if (!PIPE || next >= items) break;
    __syncthreads();  // the exchange space is written again by the next tile
    item = next;
    head = next_head;
    dim0 = next_dim0;
    paired = next_paired;
    early = Early<EPI, NT>();
#pragma unroll
    for (int n = 0; n < NT; ++n) {
      ss[n] = 0.f;
#pragma unroll
      for (int i = 0; i < 4; ++i) acc[n][i] = 0.f;
    }
  }
}

template <int WARPS, int NT, int EPI, bool NORM, bool PIPE>
int launch_one(int items, void* c, const void* a, const float* norm_w, float eps, const bf16* w, int M, int N, int K,
               const RopeArgs& rope, const Prefetch& pf, cudaStream_t stream) {
  size_t smem = (size_t)(WARPS * TILE * (NT * 8 + 1) + WARPS * NT * 8) * sizeof(float);
  static int resident = 0;  // blocks of this kernel that fit on the device at once
  if (resident == 0) {
    if (smem > 48 * 1024 &&
        cudaFuncSetAttribute(gemv_kernel<WARPS, NT, EPI, NORM, PIPE>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             (int)smem) != cudaSuccess)
      return DLLM_LAUNCH_FAILED;
    int device = 0, sms = 0, per_sm = 0;
    if (cudaGetDevice(&device) != cudaSuccess ||
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess ||
        cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, gemv_kernel<WARPS, NT, EPI, NORM, PIPE>, WARPS * 32,
                                                      smem) != cudaSuccess ||
        sms <= 0 || per_sm <= 0)
      return DLLM_LAUNCH_FAILED;
    resident = sms * per_sm;
  }
  // long rows (measured: from K = 4096 on): as many blocks as fit at once, each walking over its tiles with the next
  // tile's weights on their way during the sum and store of this one; shorter rows: a block a tile (there the loop
  // costs more than the overlap brings)
  int blocks = (PIPE && items > resident) ? resident : items;
  return dllm_launch_pdl(gemv_kernel<WARPS, NT, EPI, NORM, PIPE>, dim3(blocks), dim3(WARPS * 32), smem, stream, c, a,
                         norm_w, eps, w, M, N, K, rope, pf, items);
}

template <int EPI, bool NORM>
int launch(void* c, const void* a, const float* norm_w, float eps, const bf16* w, int M, int N, int K,
           const RopeArgs& rope, const Prefetch& pf, cudaStream_t stream) {
  int items = (N + TILE - 1) / TILE;
  bool wide = K >= 1024;
  bool longrows = K > 2048;  // a warp has more than one stretch of k steps: stream the next stretch early
#define DLLM_GO(WARPS, NT, PIPE)                                                                          \
  return launch_one<WARPS, NT, EPI, NORM, PIPE>(items, c, a, norm_w, eps, w, M, N, K, rope, pf, stream)
#define DLLM_PICK(NT)                    \
  if (longrows) DLLM_GO(8, NT, true);    \
  else if (wide) DLLM_GO(8, NT, false);  \
  else DLLM_GO(4, NT, false)
  // many tokens leave few registers for loads in flight: sixteen warps split the reduction instead
#define DLLM_PICK_MANY(NT)               \
  if (longrows) DLLM_GO(16, NT, true);   \
  else DLLM_GO(16, NT, false)
  if (M <= 8) { DLLM_PICK(1); }
  else if (M <= 16) { DLLM_PICK(2); }
  else if (M <= 32) { DLLM_PICK_MANY(4); }
  else { DLLM_PICK_MANY(8); }
#undef DLLM_PICK_MANY
#undef DLLM_PICK
#undef DLLM_GO
}

template <bool NORM>
int dispatch(void* c, const void* a, const float* norm_w, float eps, const bf16* w, int M, int N, int K, int epilogue,
             const RopeArgs& rope, const Prefetch& pf, cudaStream_t stream) {
  switch (epilogue) {
    case EPI_STORE_F32: return launch<EPI_STORE_F32, NORM>(c, a, norm_w, eps, w, M, N, K, rope, pf, stream);
    case EPI_STORE_T: return launch<EPI_STORE_T, NORM>(c, a, norm_w, eps, w, M, N, K, rope, pf, stream);
    case EPI_RESIDUAL: return launch<EPI_RESIDUAL, NORM>(c, a, norm_w, eps, w, M, N, K, rope, pf, stream);
    case EPI_SWIGLU: return launch<EPI_SWIGLU, NORM>(c, a, norm_w, eps, w, M, N, K, rope, pf, stream);
    case EPI_QKV_ROPE: return launch<EPI_QKV_ROPE, NORM>(c, a, norm_w, eps, w, M, N, K, rope, pf, stream);
    case EPI_ARGMAX: return launch<EPI_ARGMAX, NORM>(c, a, norm_w, eps, w, M, N, K, rope, pf, stream);
    default: return DLLM_BAD_ARGUMENT;
  }
}
}  // namespace

// C = X[M,K] * W[N,K]^T for M <= 64. With norm_w != null, X is the float32 residual stream and is RMS-normed on
// the way in; else X is bfloat16. Epilogues 0..3 as the tile kernels; K a multiple of 8, N even for SwiGLU.
// prefetch_ptr / prefetch_bytes: optional memory (weights a later kernel reads) to bring into L2 meanwhile.
DLLM_EXPORT int dllm_gemv_bf16(void* c, const void* a, const float* norm_w, float eps, const void* w, int M, int N,
                               int K, int epilogue, const void* prefetch_ptr, long long prefetch_bytes,
                               cudaStream_t stream) {
  if (M <= 0 || N <= 0) return DLLM_OK;
  if (M > 64 || K <= 0 || (K & 7) || ((N & 1) && epilogue == EPI_SWIGLU) || epilogue < 0 ||
      (epilogue > EPI_SWIGLU && epilogue != EPI_ARGMAX))
    return DLLM_UNSUPPORTED_SIZE;
  RopeArgs rope{};
  Prefetch pf{(const char*)prefetch_ptr, prefetch_ptr ? (size_t)prefetch_bytes : 0};
  return norm_w ? dispatch<true>(c, a, norm_w, eps, (const bf16*)w, M, N, K, epilogue, rope, pf, stream)
                : dispatch<false>(c, a, nullptr, eps, (const bf16*)w, M, N, K, epilogue, rope, pf, stream);
}

// The second stage of the greedy head product (epilogue EPI_ARGMAX above): token r's winner among its `tiles`
// candidates (value, feature), the lowest feature on ties; a token without a candidate (no value above -inf) gets 0.
namespace {
__global__ void __launch_bounds__(256) argmax_candidates_kernel(int* __restrict__ out_tokens,
                                                                const float* __restrict__ candidates, int tiles) {
  __shared__ float values[8];
  __shared__ int features[8];
  pdl_launch_dependents();
  pdl_wait();
  const float* row = candidates + (size_t)blockIdx.x * tiles * 2;
  float best = -INFINITY;
  int feature = 0x7fffffff;
  for (int i = threadIdx.x; i < tiles; i += 256) {
    float v = row[2 * i];
    int f = __float_as_int(row[2 * i + 1]);
    if (v > best || (v == best && f < feature)) { best = v; feature = f; }
  }
  for (int o = 16; o > 0; o >>= 1) {
    float ov = __shfl_xor_sync(0xffffffffu, best, o);
    int of = __shfl_xor_sync(0xffffffffu, feature, o);
    if (ov > best || (ov == best && of < feature)) { best = ov; feature = of; }
  }
  if ((threadIdx.x & 31) == 0) { values[threadIdx.x >> 5] = best; features[threadIdx.x >> 5] = feature; }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int i = 1; i < 8; ++i)
      if (values[i] > best || (values[i] == best && features[i] < feature)) { best = values[i]; feature = features[i]; }
    out_tokens[blockIdx.x] = feature == 0x7fffffff ? 0 : feature;
  }
}
}  // namespace

// out_tokens[r] = the feature of the largest candidate of token r; candidates: [rows][tiles](value, feature).
DLLM_EXPORT int dllm_argmax_candidates(int* out_tokens, const float* candidates, int rows, int tiles,
                                       cudaStream_t stream) {
  if (rows <= 0) return DLLM_OK;
  if (tiles <= 0 || out_tokens == nullptr || candidates == nullptr) return DLLM_BAD_ARGUMENT;
  return dllm_launch_pdl(argmax_candidates_kernel, dim3(rows), dim3(256), 0, stream, out_tokens, candidates, tiles);
}

// The q/k/v projection of a decode step in one kernel: optional RMSNorm in front, rotation of q and k by the
// table's angle for each token's position, q to q_out, k and v into the token's place in the paged cache.
// W is [(heads + 2 kv_heads) * head_dim, K]. head_dim and rotary_dim must be multiples of 16.
// prefetch_window: -1, or which cached keys the attention behind this kernel will read (0: all, w: the last w), whose
// pages this kernel then asks into L2.
DLLM_EXPORT int dllm_gemv_qkv_rope(const void* a, const float* norm_w, float eps, const void* w, int M, int K,
                                   void* q_out, void* cache_base, const int* page_table, int max_pages, int page_size,
                                   int heads, int kv_heads, int head_dim, const float* table, int rotary_dim,
                                   const int* tok_seq, const int* tok_pos, const int* slots, int write_cache,
                                   int prefetch_window, const void* prefetch_ptr, long long prefetch_bytes,
                                   cudaStream_t stream) {
  if (M <= 0) return DLLM_OK;
  if (M > 64 || K <= 0 || (K & 7) || heads <= 0 || kv_heads <= 0 || head_dim <= 0 || (head_dim & 15) ||
      rotary_dim < 0 || rotary_dim > head_dim || (rotary_dim & 15))
    return DLLM_UNSUPPORTED_SIZE;
  RopeArgs rope{(bf16*)q_out, KvLayout{cache_base, page_table, max_pages, page_size, kv_heads, head_dim},
                (const float2*)table, table ? rotary_dim : 0, heads, tok_seq, tok_pos, slots, write_cache,
                prefetch_window};
  int N = (heads + 2 * kv_heads) * head_dim;
  Prefetch pf{(const char*)prefetch_ptr, prefetch_ptr ? (size_t)prefetch_bytes : 0};
  return norm_w ? dispatch<true>(nullptr, a, norm_w, eps, (const bf16*)w, M, N, K, EPI_QKV_ROPE, rope, pf, stream)
                : dispatch<false>(nullptr, a, nullptr, eps, (const bf16*)w, M, N, K, EPI_QKV_ROPE, rope, pf, stream);
}
