// Attention over the paged cache, general form: one warp per (token, query head). The warp walks the visible keys
// of the token's own sequence in tiles of 32 (one key per lane for the scores, one value dimension per lane for the
// weighted sum) with a running maximum and sum in float32. It serves whole prompts and single decoded tokens alike
// and any head size that is a multiple of 8 up to 256, any number of heads and groups, with or without a window.
// A (token, head) result depends only on that token's query and the keys it may see, so it is the same bits
// however the tokens were cut into steps or batched.
#include "common.cuh"

namespace {
constexpr int WARPS = 4;
constexpr int MAX_HEAD_DIM = 256;

template <typename T> struct Vec;  // 16-byte vectors of the element type
template <> struct Vec<float> { static constexpr int N = 4; };
template <> struct Vec<__nv_bfloat16> { static constexpr int N = 8; };

__device__ __forceinline__ float dot_vec(const float* q, const float* k) {
  float4 v = *(const float4*)k;
  return fmaf(q[3], v.w, fmaf(q[2], v.z, fmaf(q[1], v.y, q[0] * v.x)));
}
__device__ __forceinline__ float dot_vec(const float* q, const __nv_bfloat16* k) {
  uint4 raw = *(const uint4*)k;
  const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&raw);
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 x = __bfloat1622float2(p[i]);
    s = fmaf(q[2 * i], x.x, s);
    s = fmaf(q[2 * i + 1], x.y, s);
  }
  return s;
}

// The same sums from a vector that is already in registers (one load of a key for several queries).
__device__ __forceinline__ float4 load_vec(const float* k) { return *(const float4*)k; }
__device__ __forceinline__ uint4 load_vec(const __nv_bfloat16* k) { return *(const uint4*)k; }
__device__ __forceinline__ float dot_loaded(const float* q, float4 v) {
  return fmaf(q[3], v.w, fmaf(q[2], v.z, fmaf(q[1], v.y, q[0] * v.x)));
}
__device__ __forceinline__ float dot_loaded(const float* q, uint4 raw) {
  const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&raw);
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 x = __bfloat1622float2(p[i]);
    s = fmaf(q[2 * i], x.x, s);
    s = fmaf(q[2 * i + 1], x.y, s);
  }
  return s;
}

template <typename T>
__global__ void __launch_bounds__(WARPS * 32) attention_warp_kernel(
    T* __restrict__ out, const T* __restrict__ q, KvLayout cache, const int* __restrict__ tok_seq,
    const int* __restrict__ tok_pos, const int* __restrict__ slots, int tokens, int heads, float scale, int window) {
  __shared__ float q_s[WARPS][MAX_HEAD_DIM];
  int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  long long item = (long long)blockIdx.x * WARPS + warp;
  if (item >= (long long)tokens * heads) return;
  int t = (int)(item / heads), h = (int)(item % heads);
  int hd = cache.head_dim, ps = cache.page_size;
  int g = h / (heads / cache.kv_heads);
  int pos = tok_pos[t];
  const int* pages = cache.page_table + (size_t)slots[tok_seq[t]] * cache.max_pages;
  const T* qrow = q + ((size_t)t * heads + h) * hd;
  for (int d = lane; d < hd; d += 32) q_s[warp][d] = to_float(qrow[d]);
  __syncwarp();

  int end = pos + 1;
  int first = (window > 0 && end > window) ? end - window : 0;
  float m_run = -INFINITY, l_run = 0.f;
  float acc[MAX_HEAD_DIM / 32];
#pragma unroll
  for (int i = 0; i < MAX_HEAD_DIM / 32; ++i) acc[i] = 0.f;
  const T* base = (const T*)cache.base;

  for (int j0 = first; j0 < end; j0 += 32) {
    int j = j0 + lane;
    bool valid = j < end;
    int page = valid ? pages[j / ps] : 0;
    float s = -INFINITY;
    if (valid) {
      const T* krow = base + kv_offset(cache, page, 0, g, j % ps);
      float dot = 0.f;
      for (int d = 0; d < hd; d += Vec<T>::N) dot += dot_vec(&q_s[warp][d], krow + d);
      s = dot * scale;
    }
    float m_new = fmaxf(m_run, warp_max(s));
    float p = valid ? expf(s - m_new) : 0.f;
    float corr = expf(m_run - m_new);  // 0 on the first tile (m_run = -inf)
    l_run = l_run * corr + warp_sum(p);
#pragma unroll
    for (int i = 0; i < MAX_HEAD_DIM / 32; ++i) acc[i] *= corr;
    m_run = m_new;
    int count = min(32, end - j0);
    for (int jj = 0; jj < count; ++jj) {
      float pj = __shfl_sync(0xffffffffu, p, jj);
      int pg = __shfl_sync(0xffffffffu, page, jj);
      const T* vrow = base + kv_offset(cache, pg, 1, g, (j0 + jj) % ps);
#pragma unroll
      for (int i = 0; i < MAX_HEAD_DIM / 32; ++i) {
        int d = lane + 32 * i;
        if (d < hd) acc[i] = fmaf(pj, to_float(vrow[d]), acc[i]);
      }
    }
  }
  float inv = 1.0f / l_run;
  T* orow = out + ((size_t)t * heads + h) * hd;
#pragma unroll
  for (int i = 0; i < MAX_HEAD_DIM / 32; ++i) {
    int d = lane + 32 * i;
    if (d < hd) orow[d] = from_float<T>(acc[i] * inv);
  }
}

// ---- the same attention, blockwise ------------------------------------------------------------------------------
// A block serves one kv head and a run of consecutive tokens of the step; its warps are the (token, query head)
// pairs of that run, R tokens a warp. The block copies the keys and values of the kv head page by page (64
// positions) into shared memory, with the next page on its way (cp.async) while the warps work on this one, and
// every warp walks the page's two tiles of 32 keys exactly as the kernel above walks its tiles: one key a lane for
// the scores, one value dimension a lane for the weighted sum, the same running maximum and sum in the same order.
// Tiles start at multiples of 32 from position 0, so without a window a (token, head) result has the same bits as
// the kernel above gives (with a window the first tile is cut differently: same formula, other rounding), and it
// depends only on the token's own query and visible keys: not on its tile mates, the cut of the steps or the batch.
// Tokens of several sequences in one block are served sequence by sequence.
template <typename T> struct Pad { static constexpr int N = 16 / sizeof(T); };  // 16 bytes: rows in different banks

template <typename T>
__device__ __forceinline__ void stage_page(T* k_s, T* v_s, const KvLayout& cache, int page, int g, int hd, int ld,
                                           int tid, int threads) {
  const T* ksrc = (const T*)cache.base + kv_offset(cache, page, 0, g, 0);
  const T* vsrc = (const T*)cache.base + kv_offset(cache, page, 1, g, 0);
  constexpr int VN = Vec<T>::N;
  int pieces = hd / VN;  // 16-byte pieces of a row
  for (int i = tid; i < 64 * pieces; i += threads) {
    int r = i / pieces, c = (i % pieces) * VN;
    unsigned kd = (unsigned)__cvta_generic_to_shared(k_s + r * ld + c);
    unsigned vd = (unsigned)__cvta_generic_to_shared(v_s + r * ld + c);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(kd), "l"(ksrc + (size_t)r * hd + c));
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(vd), "l"(vsrc + (size_t)r * hd + c));
  }
  asm volatile("cp.async.commit_group;\n" ::);
}

template <typename T, int R, int CHUNKS>  // CHUNKS: head_dim / 32 rounded up (value dimensions a lane owns)
__global__ void __launch_bounds__(512) attention_block_kernel(
    T* __restrict__ out, const T* __restrict__ q, KvLayout cache, const int* __restrict__ tok_seq,
    const int* __restrict__ tok_pos, const int* __restrict__ slots, int tokens, int heads, float scale, int window,
    int heads_per_pass, int stages) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  int hd = cache.head_dim, ld = hd + Pad<T>::N;
  int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
  int token_slots = warps / heads_per_pass;       // warps = token_slots * heads_per_pass
  int block_tokens = token_slots * R;
  int slot_of_warp = warp / heads_per_pass, head_of_warp = warp % heads_per_pass;
  T* kv_s = reinterpret_cast<T*>(smem_raw);       // [stages][k|v][64][ld]
  float* q_all = reinterpret_cast<float*>(smem_raw + (size_t)stages * 2 * 64 * ld * sizeof(T));
  float* q_s = q_all + (size_t)warp * R * hd;                        // this warp's R queries
  float* p_s = q_all + (size_t)warps * R * hd + (size_t)warp * R * 32;  // and their weights for the tile at hand
  int g = blockIdx.y, group = heads / cache.kv_heads;
  // (the last tokens of a prompt see the most keys: their blocks go first, the short ones fill the gaps behind)
  int t0 = (int)(gridDim.x - 1 - blockIdx.x) * block_tokens, t_stop = min(tokens, t0 + block_tokens);

  for (int pass = 0; pass < group; pass += heads_per_pass) {
    int h = g * group + pass + head_of_warp;
    bool head_ok = pass + head_of_warp < group;
    for (int run_begin = t0; run_begin < t_stop;) {
      // a run: the block's tokens of one sequence (positions ascend inside it)
      int seq = tok_seq[run_begin], run_end = run_begin + 1;
      while (run_end < t_stop && tok_seq[run_end] == seq) ++run_end;
      const int* pages = cache.page_table + (size_t)slots[seq] * cache.max_pages;
      int run_last = tok_pos[run_end - 1] + 1;   // keys [run_first, run_last) are read by somebody of the run
      int first_end = tok_pos[run_begin] + 1;
      int run_first = (window > 0 && first_end > window) ? first_end - window : 0;

      // this warp's tokens of the run
      int end[R], first[R];
      float m_run[R], l_run[R], acc[R][CHUNKS];
#pragma unroll
      for (int r = 0; r < R; ++r) {
        int t = t0 + slot_of_warp * R + r;
        bool mine = head_ok && t >= run_begin && t < run_end;
        end[r] = mine ? tok_pos[t] + 1 : 0;
        first[r] = (window > 0 && end[r] > window) ? end[r] - window : 0;
        m_run[r] = -INFINITY;
        l_run[r] = 0.f;
#pragma unroll
        for (int i = 0; i < CHUNKS; ++i) acc[r][i] = 0.f;
        if (mine) {
          const T* qrow = q + ((size_t)t * heads + h) * hd;
          for (int d = lane; d < hd; d += 32) q_s[r * hd + d] = to_float(qrow[d]);
        }
      }
      __syncwarp();

      int page_first = run_first / 64, page_last = (run_last - 1) / 64;
      __syncthreads();  // (the stages may still be read by a warp that is behind in the run before)
      stage_page(kv_s, kv_s + 64 * ld, cache, pages[page_first], g, hd, ld, threadIdx.x, blockDim.x);
      for (int p = page_first; p <= page_last; ++p) {
        int stage = stages == 2 ? ((p - page_first) & 1) : 0;
        T* k_s = kv_s + (size_t)stage * 2 * 64 * ld;
        T* v_s = k_s + 64 * ld;
        if (stages == 2 && p < page_last) {
          T* next = kv_s + (size_t)(stage ^ 1) * 2 * 64 * ld;
          stage_page(next, next + 64 * ld, cache, pages[p + 1], g, hd, ld, threadIdx.x, blockDim.x);
          asm volatile("cp.async.wait_group 1;\n" ::: "memory");
        } else {
          asm volatile("cp.async.wait_group 0;\n" ::: "memory");
        }
        __syncthreads();
        // The warp's R tokens walk the tile together: a key is loaded once for the R scores and a value once for the
        // R weighted sums (what a token computes, and in which order, is what it would compute alone).
        for (int j0 = p * 64; j0 < p * 64 + 64; j0 += 32) {
          bool active[R], any = false, whole = hd == CHUNKS * 32;
#pragma unroll
          for (int r = 0; r < R; ++r) {
            active[r] = j0 < end[r] && j0 + 32 > first[r];  // (warp-uniform) a visible key in this tile
            any = any || active[r];
            whole = whole && (!active[r] || (first[r] <= j0 && j0 + 32 <= end[r]));
          }
          if (!any) continue;
          int j = j0 + lane;
          const T* krow = k_s + (j - p * 64) * ld;
          float dot[R];
#pragma unroll
          for (int r = 0; r < R; ++r) dot[r] = 0.f;
          if (hd == CHUNKS * 32) {
#pragma unroll
            for (int d = 0; d < CHUNKS * 32; d += Vec<T>::N) {
              auto key = load_vec(krow + d);
#pragma unroll
              for (int r = 0; r < R; ++r) dot[r] += dot_loaded(&q_s[r * hd + d], key);
            }
          } else {
            for (int d = 0; d < hd; d += Vec<T>::N) {
              auto key = load_vec(krow + d);
#pragma unroll
              for (int r = 0; r < R; ++r) dot[r] += dot_loaded(&q_s[r * hd + d], key);
            }
          }
          // (a single token a warp, as in decoding, hands its weights from lane to lane by shuffles; several go
          // through shared memory, four weights a load)
          float weight[R];
          if (R > 1) __syncwarp();  // (the weights of the tile before have been read by every lane)
#pragma unroll
          for (int r = 0; r < R; ++r) {
            weight[r] = 0.f;
            if (!active[r]) continue;
            bool valid = j >= first[r] && j < end[r];
            float sc = valid ? dot[r] * scale : -INFINITY;
            float m_new = fmaxf(m_run[r], warp_max(sc));
            float pr = valid ? expf(sc - m_new) : 0.f;
            float corr = expf(m_run[r] - m_new);  // 0 on the first tile (m_run = -inf)
            l_run[r] = l_run[r] * corr + warp_sum(pr);
#pragma unroll
            for (int i = 0; i < CHUNKS; ++i) acc[r][i] *= corr;
            m_run[r] = m_new;
            weight[r] = pr;
            if (R > 1) p_s[r * 32 + lane] = pr;
          }
          if (R > 1) __syncwarp();
          const T* vtile = v_s + (j0 - p * 64) * ld + lane;
          if (whole) {  // whole tiles of a whole head for every token that sees the tile: no bounds in the loop
#pragma unroll 4
            for (int jj = 0; jj < 32; jj += 4) {
              float v[4][CHUNKS];
#pragma unroll
              for (int u = 0; u < 4; ++u)
#pragma unroll
                for (int i = 0; i < CHUNKS; ++i) v[u][i] = to_float(vtile[(jj + u) * ld + 32 * i]);
#pragma unroll
              for (int r = 0; r < R; ++r) {
                if (!active[r]) continue;  // (a token that does not see the tile must not meet what lies there)
                float4 pj;
                if (R > 1) {
                  pj = *reinterpret_cast<const float4*>(&p_s[r * 32 + jj]);
                } else {
                  pj.x = __shfl_sync(0xffffffffu, weight[r], jj);
                  pj.y = __shfl_sync(0xffffffffu, weight[r], jj + 1);
                  pj.z = __shfl_sync(0xffffffffu, weight[r], jj + 2);
                  pj.w = __shfl_sync(0xffffffffu, weight[r], jj + 3);
                }
#pragma unroll
                for (int i = 0; i < CHUNKS; ++i) {
                  acc[r][i] = fmaf(pj.x, v[0][i], acc[r][i]);
                  acc[r][i] = fmaf(pj.y, v[1][i], acc[r][i]);
                  acc[r][i] = fmaf(pj.z, v[2][i], acc[r][i]);
                  acc[r][i] = fmaf(pj.w, v[3][i], acc[r][i]);
                }
              }
            }
          } else {
#pragma unroll
            for (int r = 0; r < R; ++r) {
              if (!active[r]) continue;
              int from = max(0, first[r] - j0), to = min(32, end[r] - j0);
              for (int jj = from; jj < to; ++jj) {
                float pj = R > 1 ? p_s[r * 32 + jj] : __shfl_sync(0xffffffffu, weight[r], jj);
#pragma unroll
                for (int i = 0; i < CHUNKS; ++i)
                  if (lane + 32 * i < hd) acc[r][i] = fmaf(pj, to_float(vtile[jj * ld + 32 * i]), acc[r][i]);
              }
            }
          }
        }
        if (stages != 2) {
          __syncthreads();  // one stage: it is free only when every warp is done with it
          if (p < page_last) stage_page(kv_s, kv_s + 64 * ld, cache, pages[p + 1], g, hd, ld, threadIdx.x, blockDim.x);
        } else {
          __syncthreads();  // the stage read now is the one the copy after next writes
        }
      }
#pragma unroll
      for (int r = 0; r < R; ++r) {
        int t = t0 + slot_of_warp * R + r;
        if (head_ok && t >= run_begin && t < run_end) {
          float inv = 1.0f / l_run[r];
          T* orow = out + ((size_t)t * heads + h) * hd;
#pragma unroll
          for (int i = 0; i < CHUNKS; ++i) {
            int d = lane + 32 * i;
            if (d < hd) orow[d] = from_float<T>(acc[r][i] * inv);
          }
        }
      }
      run_begin = run_end;
    }
  }
}

template <typename T, int R, int CHUNKS>
int launch_blocks(void* out, const void* q, const KvLayout& cache, const int* tok_seq, const int* tok_pos,
                  const int* slots, int tokens, int heads, float scale, int window, cudaStream_t stream) {
  int group = heads / cache.kv_heads;
  int heads_per_pass = group < 16 ? group : 16;
  int token_slots = R == 1 ? 1 : (16 / heads_per_pass > 0 ? 16 / heads_per_pass : 1);
  int warps = token_slots * heads_per_pass;
  int ld = cache.head_dim + Pad<T>::N;
  size_t stage_bytes = (size_t)2 * 64 * ld * sizeof(T);
  size_t q_bytes = (size_t)warps * R * (cache.head_dim + 32) * sizeof(float);  // queries and a tile's weights
  int stages = 2 * stage_bytes + q_bytes <= 200 * 1024 ? 2 : 1;
  size_t smem = stages * stage_bytes + q_bytes;
  static size_t configured = 0;
  if (smem > configured) {
    if (cudaFuncSetAttribute(attention_block_kernel<T, R, CHUNKS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) !=
        cudaSuccess)
      return DLLM_LAUNCH_FAILED;
    configured = smem;
  }
  int block_tokens = token_slots * R;
  dim3 grid((tokens + block_tokens - 1) / block_tokens, cache.kv_heads);
  attention_block_kernel<T, R, CHUNKS><<<grid, warps * 32, smem, stream>>>((T*)out, (const T*)q, cache, tok_seq, tok_pos,
                                                                  slots, tokens, heads, scale, window,
                                                                  heads_per_pass, stages);
  return dllm_launch_status();
}
}  // namespace

DLLM_EXPORT int dllm_attention_general(void* out, const void* q, void* cache_base, const int* page_table,
                                       int max_pages, int page_size, int heads, int kv_heads, int head_dim,
                                       const int* tok_seq, const int* tok_pos, const int* slots, int tokens,
                                       float scale, int window, int dtype, cudaStream_t stream) {
  if (tokens <= 0) return DLLM_OK;
  if (heads <= 0 || kv_heads <= 0 || heads % kv_heads) return DLLM_BAD_ARGUMENT;
  if (head_dim <= 0 || head_dim > MAX_HEAD_DIM || (head_dim & 7)) return DLLM_UNSUPPORTED_SIZE;
  KvLayout cache{cache_base, page_table, max_pages, page_size, kv_heads, head_dim};
  long long items = (long long)tokens * heads;
  unsigned blocks = (unsigned)((items + WARPS - 1) / WARPS);
  if (dtype == DLLM_F32)
    attention_warp_kernel<float><<<blocks, WARPS * 32, 0, stream>>>((float*)out, (const float*)q, cache, tok_seq,
                                                                    tok_pos, slots, tokens, heads, scale, window);
  else if (dtype == DLLM_BF16)
    attention_warp_kernel<__nv_bfloat16><<<blocks, WARPS * 32, 0, stream>>>(
        (__nv_bfloat16*)out, (const __nv_bfloat16*)q, cache, tok_seq, tok_pos, slots, tokens, heads, scale, window);
  else
    return DLLM_BAD_ARGUMENT;
  return dllm_launch_status();
}

// The same attention with the same arguments, blockwise (see attention_block_kernel). `max_new`: the most new
// tokens a sequence brings in this step: with one each (decoding) a block serves one token's heads, else runs of
// tokens with two tokens a warp. Pages of 64 positions, at most 65,535 kv heads.
DLLM_EXPORT int dllm_attention_blocks(void* out, const void* q, void* cache_base, const int* page_table,
                                      int max_pages, int page_size, int heads, int kv_heads, int head_dim,
                                      const int* tok_seq, const int* tok_pos, const int* slots, int tokens,
                                      int max_new, float scale, int window, int dtype, cudaStream_t stream) {
  if (tokens <= 0) return DLLM_OK;
  if (heads <= 0 || kv_heads <= 0 || heads % kv_heads) return DLLM_BAD_ARGUMENT;
  if (head_dim <= 0 || head_dim > MAX_HEAD_DIM || (head_dim & 7) || page_size != 64 || kv_heads > 65535)
    return DLLM_UNSUPPORTED_SIZE;
  KvLayout cache{cache_base, page_table, max_pages, page_size, kv_heads, head_dim};
  bool runs = max_new > 1;
  int chunks = (head_dim + 31) / 32;
#define DLLM_GO(T, R, CHUNKS) \
  return launch_blocks<T, R, CHUNKS>(out, q, cache, tok_seq, tok_pos, slots, tokens, heads, scale, window, stream)
#define DLLM_BY_WIDTH(T, R)                   \
  if (chunks <= 1) DLLM_GO(T, R, 1);          \
  else if (chunks == 2) DLLM_GO(T, R, 2);     \
  else if (chunks <= 4) DLLM_GO(T, R, 4);     \
  else DLLM_GO(T, R, 8)
  if (dtype == DLLM_F32) {
    if (runs) { DLLM_BY_WIDTH(float, 4); }
    DLLM_BY_WIDTH(float, 1);
  }
  if (dtype == DLLM_BF16) {
    if (runs) { DLLM_BY_WIDTH(__nv_bfloat16, 4); }
    DLLM_BY_WIDTH(__nv_bfloat16, 1);
  }
#undef DLLM_BY_WIDTH
#undef DLLM_GO
  return DLLM_BAD_ARGUMENT;
}
