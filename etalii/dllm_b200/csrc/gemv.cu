// Weight-streaming products for decode (at most 16 rows of activations, bfloat16 weights): C = X * W^T where reading
// W once is the whole cost. A block owns four output columns (rows of W) and splits the reduction over its threads:
// every thread loads 16 bytes of each of the four rows, so a matrix with few rows still spreads over the whole
// device and each row is in flight at once; partial sums meet in shared memory in a fixed order.
//
// Fused around the product, to save kernels and memory traffic in the decode step:
//   - in front: RMSNorm of the float32 residual stream (the block sums x^2 itself; the normed activations never
//     touch memory): x' = x * rsqrt(mean(x^2) + eps) * norm_weight, in float32;
//   - behind: store (float32 or bfloat16), residual add in float32, SwiGLU on interleaved gate/up rows, or rotary
//     position encoding of q/k and the write of k and v into the paged cache (q/k/v projection).
#include "gemm_common.cuh"

#define EPI_QKV_ROPE 4

namespace {
typedef __nv_bfloat16 bf16;
constexpr int THREADS = 128, WARPS = THREADS / 32, ROWS = 4;

struct RopeArgs {
  bf16* q_out;           // [tokens, heads * head_dim]
  KvLayout cache;
  const float2* table;   // [positions, rotary_dim / 2] (cos, sin) or null
  int rotary_dim, heads;
  const int* tok_seq;
  const int* tok_pos;
  const int* slots;
  int write_cache;
};

__device__ __forceinline__ void unpack8(const uint4& v, float* f) {
  const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 x = __bfloat1622float2(p[i]);
    f[2 * i] = x.x;
    f[2 * i + 1] = x.y;
  }
}

// The four rows of W a block owns. For the q/k/v projection with rotation, a block of a rotated head owns two
// rotary pairs: dims (j, j+1) and (j + half, j+1 + half); elsewhere four consecutive rows.
template <int EPI>
__device__ __forceinline__ void block_rows(int item, int N, const RopeArgs& r, int* rows, int& head, int& dim0,
                                           bool& paired) {
  paired = false;
  head = 0;
  dim0 = 0;
  if (EPI == EPI_QKV_ROPE) {
    int hd = r.cache.head_dim, per_head = hd / 4;
    head = item / per_head;
    int it = item % per_head;
    bool rotated = r.table != nullptr && head < r.heads + r.cache.kv_heads;
    int half = r.rotary_dim / 2;
    if (rotated && it < r.rotary_dim / 4) {
      paired = true;
      dim0 = it * 2;
      rows[0] = head * hd + dim0; rows[1] = rows[0] + 1; rows[2] = rows[0] + half; rows[3] = rows[2] + 1;
    } else {
      dim0 = it * 4;
      for (int i = 0; i < 4; ++i) rows[i] = head * hd + dim0 + i;
    }
  } else {
    for (int i = 0; i < 4; ++i) rows[i] = min(item * ROWS + i, N - 1);
  }
}

template <int MT, int EPI, bool NORM>
__global__ void __launch_bounds__(THREADS) gemv_kernel(void* __restrict__ c, const void* __restrict__ a,
                                                       const float* __restrict__ norm_w, float eps,
                                                       const bf16* __restrict__ w, int M, int N, int K, RopeArgs rope) {
  __shared__ float red[WARPS][ROWS + 1][MT];
  int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  int rows[ROWS], head, dim0;
  bool paired;
  block_rows<EPI>(blockIdx.x, N, rope, rows, head, dim0, paired);
  float acc[ROWS][MT], ss[MT];
#pragma unroll
  for (int m = 0; m < MT; ++m) {
    ss[m] = 0.f;
#pragma unroll
    for (int r = 0; r < ROWS; ++r) acc[r][m] = 0.f;
  }
  int chunks = K >> 3;
  for (int ch = tid; ch < chunks; ch += THREADS) {
    float wf[ROWS][8];
#pragma unroll
    for (int r = 0; r < ROWS; ++r) {
      uint4 v = __ldg((const uint4*)(w + (size_t)rows[r] * K) + ch);
      unpack8(v, wf[r]);
    }
    float nw[8];
    if (NORM) {
      float4 n0 = __ldg((const float4*)(norm_w) + 2 * ch), n1 = __ldg((const float4*)(norm_w) + 2 * ch + 1);
      nw[0] = n0.x; nw[1] = n0.y; nw[2] = n0.z; nw[3] = n0.w; nw[4] = n1.x; nw[5] = n1.y; nw[6] = n1.z; nw[7] = n1.w;
    }
#pragma unroll
    for (int m = 0; m < MT; ++m) {
      if (m >= M) break;
      float xf[8];
      if (NORM) {
        const float4* xp = (const float4*)((const float*)a + (size_t)m * K) + 2 * ch;
        float4 x0 = xp[0], x1 = xp[1];
        xf[0] = x0.x; xf[1] = x0.y; xf[2] = x0.z; xf[3] = x0.w; xf[4] = x1.x; xf[5] = x1.y; xf[6] = x1.z; xf[7] = x1.w;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          ss[m] = fmaf(xf[i], xf[i], ss[m]);
          xf[i] *= nw[i];
        }
      } else {
        uint4 v = *((const uint4*)((const bf16*)a + (size_t)m * K) + ch);
        unpack8(v, xf);
      }
#pragma unroll
      for (int r = 0; r < ROWS; ++r)
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[r][m] = fmaf(xf[i], wf[r][i], acc[r][m]);
    }
  }
  // warp sums, then the warps in order
#pragma unroll
  for (int m = 0; m < MT; ++m) {
#pragma unroll
    for (int r = 0; r < ROWS; ++r) acc[r][m] = warp_sum(acc[r][m]);
    if (NORM) ss[m] = warp_sum(ss[m]);
  }
  if (lane == 0) {
#pragma unroll
    for (int m = 0; m < MT; ++m) {
#pragma unroll
      for (int r = 0; r < ROWS; ++r) red[warp][r][m] = acc[r][m];
      red[warp][ROWS][m] = ss[m];
    }
  }
  __syncthreads();
  if (tid >= MT || tid >= M) return;
  int m = tid;
  float out[ROWS], sumsq = 0.f;
#pragma unroll
  for (int r = 0; r < ROWS; ++r) out[r] = 0.f;
#pragma unroll
  for (int wi = 0; wi < WARPS; ++wi) {
#pragma unroll
    for (int r = 0; r < ROWS; ++r) out[r] += red[wi][r][m];
    sumsq += red[wi][ROWS][m];
  }
  if (NORM) {
    float inv = 1.0f / sqrtf(sumsq / (float)K + eps);
#pragma unroll
    for (int r = 0; r < ROWS; ++r) out[r] *= inv;
  }
  if (EPI == EPI_QKV_ROPE) {
    int hd = rope.cache.head_dim, nkv = rope.cache.kv_heads, heads = rope.heads;
    int pos = rope.tok_pos[m];
    int dims[ROWS];
    if (paired) {
      int half = rope.rotary_dim / 2;
      float2 cs0 = rope.table[(size_t)pos * half + dim0], cs1 = rope.table[(size_t)pos * half + dim0 + 1];
      float a0 = out[0], a1 = out[1], b0 = out[2], b1 = out[3];
      out[0] = fmaf(a0, cs0.x, -(b0 * cs0.y)); out[2] = fmaf(a0, cs0.y, b0 * cs0.x);
      out[1] = fmaf(a1, cs1.x, -(b1 * cs1.y)); out[3] = fmaf(a1, cs1.y, b1 * cs1.x);
      dims[0] = dim0; dims[1] = dim0 + 1; dims[2] = dim0 + half; dims[3] = dim0 + half + 1;
    } else {
      for (int i = 0; i < ROWS; ++i) dims[i] = dim0 + i;
    }
    bf16* dst;
    if (head < heads) {
      dst = rope.q_out + ((size_t)m * heads + head) * hd;
    } else {
      if (!rope.write_cache) return;
      int which = head < heads + nkv ? 0 : 1;
      int g = head - heads - which * nkv;
      int slot = rope.slots[rope.tok_seq[m]];
      int page = rope.cache.page_table[(size_t)slot * rope.cache.max_pages + pos / rope.cache.page_size];
      dst = (bf16*)rope.cache.base + kv_offset(rope.cache, page, which, g, pos % rope.cache.page_size);
    }
#pragma unroll
    for (int i = 0; i < ROWS; ++i) dst[dims[i]] = __float2bfloat16_rn(out[i]);
  } else {
    int n0 = blockIdx.x * ROWS;
    epilogue_pair<EPI, bf16>(c, m, n0, M, N, out[0], out[1]);
    epilogue_pair<EPI, bf16>(c, m, n0 + 2, M, N, out[2], out[3]);
  }
}

template <int EPI, bool NORM>
int launch(void* c, const void* a, const float* norm_w, float eps, const bf16* w, int M, int N, int K,
           const RopeArgs& rope, cudaStream_t stream) {
  int items = (N + ROWS - 1) / ROWS;
#define DLLM_GO(MT) gemv_kernel<MT, EPI, NORM><<<items, THREADS, 0, stream>>>(c, a, norm_w, eps, w, M, N, K, rope)
  if (M <= 1) DLLM_GO(1);
  else if (M <= 2) DLLM_GO(2);
  else if (M <= 4) DLLM_GO(4);
  else if (M <= 8) DLLM_GO(8);
  else DLLM_GO(16);
#undef DLLM_GO
  return dllm_launch_status();
}

template <bool NORM>
int dispatch(void* c, const void* a, const float* norm_w, float eps, const bf16* w, int M, int N, int K, int epilogue,
             const RopeArgs& rope, cudaStream_t stream) {
  switch (epilogue) {
    case EPI_STORE_F32: return launch<EPI_STORE_F32, NORM>(c, a, norm_w, eps, w, M, N, K, rope, stream);
    case EPI_STORE_T: return launch<EPI_STORE_T, NORM>(c, a, norm_w, eps, w, M, N, K, rope, stream);
    case EPI_RESIDUAL: return launch<EPI_RESIDUAL, NORM>(c, a, norm_w, eps, w, M, N, K, rope, stream);
    case EPI_SWIGLU: return launch<EPI_SWIGLU, NORM>(c, a, norm_w, eps, w, M, N, K, rope, stream);
    case EPI_QKV_ROPE: return launch<EPI_QKV_ROPE, NORM>(c, a, norm_w, eps, w, M, N, K, rope, stream);
    default: return DLLM_BAD_ARGUMENT;
  }
}
}  // namespace

// C = X[M,K] * W[N,K]^T for M <= 16. With norm_w != null, X is the float32 residual stream and is RMS-normed on
// the way in; else X is bfloat16. Epilogues 0..3 as the tile kernels; K a multiple of 8, N even.
DLLM_EXPORT int dllm_gemv_bf16(void* c, const void* a, const float* norm_w, float eps, const void* w, int M, int N,
                               int K, int epilogue, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return DLLM_OK;
  if (M > 16 || K <= 0 || (K & 7) || (N & 1) || epilogue < 0 || epilogue > EPI_SWIGLU) return DLLM_UNSUPPORTED_SIZE;
  RopeArgs rope{};
  return norm_w ? dispatch<true>(c, a, norm_w, eps, (const bf16*)w, M, N, K, epilogue, rope, stream)
                : dispatch<false>(c, a, nullptr, eps, (const bf16*)w, M, N, K, epilogue, rope, stream);
}

// The q/k/v projection of a decode step in one kernel: optional RMSNorm in front, rotation of q and k by the
// table's angle for each token's position, q to q_out, k and v into the token's place in the paged cache.
// W is [(heads + 2 kv_heads) * head_dim, K]. head_dim and rotary_dim must be multiples of 4.
DLLM_EXPORT int dllm_gemv_qkv_rope(const void* a, const float* norm_w, float eps, const void* w, int M, int K,
                                   void* q_out, void* cache_base, const int* page_table, int max_pages, int page_size,
                                   int heads, int kv_heads, int head_dim, const float* table, int rotary_dim,
                                   const int* tok_seq, const int* tok_pos, const int* slots, int write_cache,
                                   cudaStream_t stream) {
  if (M <= 0) return DLLM_OK;
  if (M > 16 || K <= 0 || (K & 7) || heads <= 0 || kv_heads <= 0 || head_dim <= 0 || (head_dim & 3) ||
      rotary_dim < 0 || rotary_dim > head_dim || (rotary_dim & 3))
    return DLLM_UNSUPPORTED_SIZE;
  RopeArgs rope{(bf16*)q_out, KvLayout{cache_base, page_table, max_pages, page_size, kv_heads, head_dim},
                (const float2*)table, table ? rotary_dim : 0, heads, tok_seq, tok_pos, slots, write_cache};
  int N = (heads + 2 * kv_heads) * head_dim;
  return norm_w ? dispatch<true>(nullptr, a, norm_w, eps, (const bf16*)w, M, N, K, EPI_QKV_ROPE, rope, stream)
                : dispatch<false>(nullptr, a, nullptr, eps, (const bf16*)w, M, N, K, EPI_QKV_ROPE, rope, stream);
}
