// Decode attention over the paged cache for sequences that bring ONE new token each (bfloat16 cache).
//
// Work is split over (key chunk, kv head, sequence): a block reads the keys and values of its chunk once and serves
// every query head of the group from them (grouped-query sharing), keeping a running maximum and sum in float32.
// Chunks start at fixed multiples of the chunk size, so a sequence's split does not depend on its batch mates. Each
// block writes a partial result (unnormalised output, maximum, sum) to scratch; a second kernel combines a
// sequence's chunks in chunk order. Blocks whose chunk lies beyond the sequence's length (or before its window)
// return at once, so one launch shape serves every length up to the bound it was sized for (CUDA graphs).
//
// Inside a warp, TPR = pow2ceil(head_dim / 8) lanes share one key row (16 bytes each), so 32 / TPR rows are read at
// once as one contiguous piece of a page. Any head_dim that is a multiple of 8 up to 256 works.
#include "common.cuh"

namespace {
typedef __nv_bfloat16 bf16;
constexpr int WARPS = 4;
constexpr int MAX_GROUP = 8;  // most query heads served per pass over the keys

__device__ __forceinline__ void unpack8(const uint4& v, float* f) {
  const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 x = __bfloat1622float2(p[i]);
    f[2 * i] = x.x;
    f[2 * i + 1] = x.y;
  }
}

// partial layout: o[(seq * heads + head) * chunks + chunk][head_dim], ml[... ][2]
template <int TPR, int G>
__global__ void __launch_bounds__(WARPS * 32) decode_partial_kernel(
    float* __restrict__ part_o, float* __restrict__ part_ml, const bf16* __restrict__ q, KvLayout cache,
    const int* __restrict__ tok_pos, const int* __restrict__ slots, int heads, int chunk, int chunks, float scale,
    int window) {
  constexpr int ROWS = 32 / TPR;  // key rows a warp reads at once
  __shared__ float sm_o[WARPS][G][256];
  __shared__ float sm_ml[WARPS][G][2];
  int b = blockIdx.z, g = blockIdx.y, c = blockIdx.x;
  int hd = cache.head_dim, ps = cache.page_size;
  int group = heads / cache.kv_heads;
  int end = tok_pos[b] + 1;
  int first = (window > 0 && end > window) ? end - window : 0;
  int lo = max(c * chunk, first), hi = min((c + 1) * chunk, end);
  if (lo >= hi) return;
  int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int sub = lane % TPR, rgroup = lane / TPR;
  bool lane_on = sub * 8 < hd;
  const int* pages = cache.page_table + (size_t)slots[b] * cache.max_pages;
  const bf16* base = (const bf16*)cache.base;
  // this warp's keys: a contiguous quarter of the chunk
  int per_warp = chunk / WARPS;
  int wlo = max(c * chunk + warp * per_warp, lo), whi = min(c * chunk + (warp + 1) * per_warp, hi);

  for (int h0 = 0; h0 < group; h0 += G) {
    int nh = min(G, group - h0);
    float qf[G][8], acc[G][8], m_run[G], l_run[G];
#pragma unroll
    for (int h = 0; h < G; ++h) {
      m_run[h] = -INFINITY;
      l_run[h] = 0.f;
#pragma unroll
      for (int i = 0; i < 8; ++i) { acc[h][i] = 0.f; qf[h][i] = 0.f; }
      if (h < nh && lane_on) {
        uint4 raw = *(const uint4*)(q + ((size_t)b * heads + g * group + h0 + h) * hd + sub * 8);
        unpack8(raw, qf[h]);
      }
    }
    for (int j0 = wlo; j0 < whi; j0 += ROWS) {
      int j = j0 + rgroup;
      bool valid = j < whi;
      float kf[8], vf[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) { kf[i] = 0.f; vf[i] = 0.f; }
      if (valid && lane_on) {
        int page = pages[j / ps];
        const bf16* krow = base + kv_offset(cache, page, 0, g, j % ps) + sub * 8;
        const bf16* vrow = base + kv_offset(cache, page, 1, g, j % ps) + sub * 8;
        uint4 kraw = *(const uint4*)krow;
        uint4 vraw = *(const uint4*)vrow;
        unpack8(kraw, kf);
        unpack8(vraw, vf);
      }
#pragma unroll
      for (int h = 0; h < G; ++h) {
        if (h >= nh) break;
        float s = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) s = fmaf(qf[h][i], kf[i], s);
#pragma unroll
        for (int o = TPR / 2; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
        s = valid ? s * scale : -INFINITY;
        float tile_max = s;
#pragma unroll
        for (int o = 16; o >= TPR; o >>= 1) tile_max = fmaxf(tile_max, __shfl_xor_sync(0xffffffffu, tile_max, o));
        float m_new = fmaxf(m_run[h], tile_max);
        float p = valid ? __expf(s - m_new) : 0.f;
        float corr = __expf(m_run[h] - m_new);
        float psum = p;
#pragma unroll
        for (int o = 16; o >= TPR; o >>= 1) psum += __shfl_xor_sync(0xffffffffu, psum, o);
        l_run[h] = l_run[h] * corr + psum;
        m_run[h] = m_new;
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[h][i] = fmaf(p, vf[i], acc[h][i] * corr);
      }
    }
    // add up the row groups of the warp (each holds different keys, the same dimensions)
#pragma unroll
    for (int h = 0; h < G; ++h) {
      if (h >= nh) break;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        float v = acc[h][i];
#pragma unroll
        for (int o = 16; o >= TPR; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
        acc[h][i] = v;
      }
      if (rgroup == 0 && lane_on) {
#pragma unroll
        for (int i = 0; i < 8; ++i) sm_o[warp][h][sub * 8 + i] = acc[h][i];
      }
      if (lane == 0) { sm_ml[warp][h][0] = m_run[h]; sm_ml[warp][h][1] = l_run[h]; }
    }
    __syncthreads();
    // combine the warps in warp order and write the chunk's partial result
    for (int idx = threadIdx.x; idx < nh * hd; idx += WARPS * 32) {
      int h = idx / hd, d = idx % hd;
      float m = -INFINITY;
#pragma unroll
      for (int w = 0; w < WARPS; ++w) m = fmaxf(m, sm_ml[w][h][0]);
      float o = 0.f, l = 0.f;
#pragma unroll
      for (int w = 0; w < WARPS; ++w) {
        float f = sm_ml[w][h][0] == -INFINITY ? 0.f : __expf(sm_ml[w][h][0] - m);
        o = fmaf(sm_o[w][h][d], f, o);
        l = fmaf(sm_ml[w][h][1], f, l);
      }
      size_t row = ((size_t)b * heads + g * group + h0 + h) * chunks + c;
      part_o[row * hd + d] = o;
      if (d == 0) { part_ml[row * 2] = m; part_ml[row * 2 + 1] = l; }
    }
    __syncthreads();
  }
}

__global__ void decode_combine_kernel(bf16* __restrict__ out, const float* __restrict__ part_o,
                                      const float* __restrict__ part_ml, const int* __restrict__ tok_pos, int heads,
                                      int head_dim, int chunk, int chunks, int window) {
  int b = blockIdx.y, h = blockIdx.x;
  int end = tok_pos[b] + 1;
  int first = (window > 0 && end > window) ? end - window : 0;
  int c_lo = first / chunk, c_hi = (end + chunk - 1) / chunk;
  size_t row0 = ((size_t)b * heads + h) * chunks;
  float m = -INFINITY;
  for (int c = c_lo; c < c_hi; ++c) m = fmaxf(m, part_ml[(row0 + c) * 2]);
  float l = 0.f;
  for (int c = c_lo; c < c_hi; ++c) l = fmaf(part_ml[(row0 + c) * 2 + 1], __expf(part_ml[(row0 + c) * 2] - m), l);
  float inv = 1.0f / l;
  for (int d = threadIdx.x; d < head_dim; d += blockDim.x) {
    float o = 0.f;
    for (int c = c_lo; c < c_hi; ++c)
      o = fmaf(part_o[(row0 + c) * head_dim + d], __expf(part_ml[(row0 + c) * 2] - m), o);
    out[((size_t)b * heads + h) * head_dim + d] = __float2bfloat16_rn(o * inv);
  }
}

int pow2ceil(int v) {
  int p = 1;
  while (p < v) p <<= 1;
  return p;
}
}  // namespace

// Scratch the two kernels share, in floats: sequences * heads * chunks * (head_dim + 2).
DLLM_EXPORT long long dllm_attention_decode_scratch(int sequences, int heads, int head_dim, int chunks) {
  return (long long)sequences * heads * chunks * (head_dim + 2);
}

// out, q: [sequences, heads * head_dim] bfloat16; sequence b's query is the token at tok_pos[b], whose key and value
// are already in the cache. `chunk` keys per block (a multiple of 16, at most 1024); `max_context` bounds the
// lengths this launch must serve (the grid covers max_context / chunk chunks).
DLLM_EXPORT int dllm_attention_decode(void* out, const void* q, void* cache_base, const int* page_table,
                                      int max_pages, int page_size, int heads, int kv_heads, int head_dim,
                                      const int* tok_pos, const int* slots, int sequences, float scale, int window,
                                      int chunk, int max_context, float* scratch, cudaStream_t stream) {
  if (sequences <= 0) return DLLM_OK;
  if (heads <= 0 || kv_heads <= 0 || heads % kv_heads) return DLLM_BAD_ARGUMENT;
  if (head_dim <= 0 || head_dim > 256 || (head_dim & 7)) return DLLM_UNSUPPORTED_SIZE;
  if (chunk < 16 || chunk > 1024 || chunk % 16 || max_context <= 0 || scratch == nullptr) return DLLM_BAD_ARGUMENT;
  int chunks = (max_context + chunk - 1) / chunk;
  if (sequences > 65535 || kv_heads > 65535) return DLLM_UNSUPPORTED_SIZE;
  KvLayout cache{cache_base, page_table, max_pages, page_size, kv_heads, head_dim};
  float* part_o = scratch;
  float* part_ml = scratch + (size_t)sequences * heads * chunks * head_dim;
  dim3 grid(chunks, kv_heads, sequences);
  int tpr = pow2ceil(head_dim / 8);
  int group = heads / kv_heads;
#define DLLM_LAUNCH_G(T, G)                                                                                     \
  decode_partial_kernel<T, G><<<grid, WARPS * 32, 0, stream>>>(part_o, part_ml, (const bf16*)q, cache, tok_pos, \
                                                                slots, heads, chunk, chunks, scale, window)
#define DLLM_LAUNCH(T)                        \
  if (group <= 1) DLLM_LAUNCH_G(T, 1);        \
  else if (group <= 2) DLLM_LAUNCH_G(T, 2);   \
  else if (group <= 4) DLLM_LAUNCH_G(T, 4);   \
  else DLLM_LAUNCH_G(T, MAX_GROUP)
  switch (tpr) {
    case 1: DLLM_LAUNCH(1); break;
    case 2: DLLM_LAUNCH(2); break;
    case 4: DLLM_LAUNCH(4); break;
    case 8: DLLM_LAUNCH(8); break;
    case 16: DLLM_LAUNCH(16); break;
    case 32: DLLM_LAUNCH(32); break;
    default: return DLLM_UNSUPPORTED_SIZE;
  }
#undef DLLM_LAUNCH
#undef DLLM_LAUNCH_G
  if (cudaGetLastError() != cudaSuccess) return DLLM_LAUNCH_FAILED;
  decode_combine_kernel<<<dim3(heads, sequences), 64, 0, stream>>>((bf16*)out, part_o, part_ml, tok_pos, heads,
                                                                   head_dim, chunk, chunks, window);
  return dllm_launch_status();
}
