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
