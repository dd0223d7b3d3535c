// Epilogues shared by the matrix-product kernels. C = A[M,K] * W[N,K]^T with float32 accumulation, then:
//   EPI_STORE_F32   C float32 [M,N]
//   EPI_STORE_T     C in the activation type [M,N]
//   EPI_RESIDUAL    C float32 [M,N] += product  (the residual sum, in float32)
//   EPI_SWIGLU      W's rows interleave gate and up (row 2i = gate_i, row 2i+1 = up_i);
//                   C in the activation type [M,N/2] = float32(silu(gate)) * up
#pragma once
#include "common.cuh"

#define EPI_STORE_F32 0
#define EPI_STORE_T 1
#define EPI_RESIDUAL 2
#define EPI_SWIGLU 3
#define EPI_QKV_ROPE 4  // q/k/v projection: rotate q and k, q to its buffer, k and v into the paged cache
// The same four for a product computed the other way round (the accumulator tile is C^T: its rows are output
// features, its columns tokens), used when the tokens are few and W is the 128-row operand of the tensor cores:
#define EPI_T_STORE_F32 5
#define EPI_T_STORE_T 6
#define EPI_T_RESIDUAL 7
#define EPI_T_SWIGLU 8
// The head product of a greedy step (weight-streaming kernel only): no logits are stored; every tile of 16 output
// features writes its largest value per token and the feature that has it (the lowest on ties) as a candidate,
// C = [tokens][tiles](value, feature as an int's bits); a second small kernel picks each token's winner.
#define EPI_ARGMAX 9

// What the q/k/v epilogue needs: where queries go, where the cache is, the rotation table, who the tokens are.
struct RopeArgs {
  __nv_bfloat16* q_out;  // [tokens, heads * head_dim]
  KvLayout cache;
  const float2* table;   // [positions, rotary_dim / 2] (cos, sin) or null
  int rotary_dim, heads;
  const int* tok_seq;
  const int* tok_pos;
  const int* slots;
  int write_cache;
  int prefetch_window;   // -1: no prefetch; 0: every page of the tokens' sequences; w > 0: the pages of the last w keys
  int table_positions;   // the tile product only: its table is [rotary_dim / 2][table_positions] (see gemm_tcgen05.cu)
};

// RMSNorm around the tile product of prefill-sized steps, without a kernel of its own. The product that writes the
// residual stream (`x += A W^T`) also writes a bfloat16 copy of the new rows and, per row and tile of columns, the
// sum of the squares of what it wrote; the product that reads the residual next takes the bfloat16 copy as its
// operand (its weights carry the norm's weight in their columns) and scales every row of its result by
// 1 / sqrt(sum of the parts / width + eps): norm(x) W^T = (x W'^T) / rms(x). The parts are summed in tile order by
// every reader, so the scale has the same bits everywhere.
struct NormArgs {
  const float* ssq_in;      // [parts_in][rows] sums of squares of the rows of the operand, or null (no scaling)
  int parts_in;
  float inv_width, eps;     // 1 / (width of the normed rows), the norm's eps
  float* ssq_out;           // [column tiles of this product][rows], or null
  __nv_bfloat16* copy_out;  // [rows][N] bfloat16 copy of the new residual rows, or null
};

// (The parts of a row lie `M` floats apart, so the 32 rows of a warp read 128 contiguous bytes per part; up to
// sixteen parts are asked for before the first is summed: one round trip, not one per part.)
__device__ __forceinline__ float row_scale(const NormArgs& norm, int m, int M) {
  if (norm.ssq_in == nullptr || m >= M) return 1.0f;
  float sum = 0.f;
  for (int j0 = 0; j0 < norm.parts_in; j0 += 16) {
    float v[16];
#pragma unroll
    for (int j = 0; j < 16; ++j) v[j] = j0 + j < norm.parts_in ? norm.ssq_in[(size_t)(j0 + j) * M + m] : 0.f;
#pragma unroll
    for (int j = 0; j < 16; ++j) sum += v[j];
  }
  return 1.0f / sqrtf(sum * norm.inv_width + norm.eps);
}

// silu(g) = g * sigmoid(g), sigmoid as 1/(1+e^-g) for g >= 0 and e^g/(1+e^g) below, in float32; the product with
// `up` is a separate float32 multiply of the rounded activation.
__device__ __forceinline__ float silu_f32(float g) {
  float s;
  if (g >= 0.f) {
    s = 1.0f / (1.0f + expf(-g));
  } else {
    float e = expf(g);
    s = e / (1.0f + e);
  }
  return g * s;
}

// The same function with the hardware's approximate exponential and reciprocal (relative error about 2^-21, far
// below bfloat16's 2^-9): used where the result is rounded to bfloat16 anyway. Large negative g gives -0, never NaN.
// (ex2.approx and rcp.approx: two special-function instructions; the correctly rounded reciprocal this replaced cost
// about ten instructions more per value, and the SwiGLU epilogue of a prefill product is nothing but this function.)
__device__ __forceinline__ float silu_fast(float g) {
  float e = fast_exp2(g * -1.4426950408889634f);  // e^-g
  float r;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(1.0f + e));
  return g * r;
}

template <typename T> __device__ __forceinline__ float silu_for(float g) { return silu_f32(g); }
template <> __device__ __forceinline__ float silu_for<__nv_bfloat16>(float g) { return silu_fast(g); }

// Stores the pair of adjacent columns (n, n+1) of row m. n is even.
template <int EPI, typename T>
__device__ __forceinline__ void epilogue_pair(void* __restrict__ c, int m, int n, int M, int N, float v0, float v1) {
  if (m >= M || n >= N) return;
  bool second = n + 1 < N;
  if (EPI == EPI_STORE_F32) {
    float* dst = (float*)c + (size_t)m * N + n;
    dst[0] = v0;
    if (second) dst[1] = v1;
  } else if (EPI == EPI_STORE_T) {
    T* dst = (T*)c + (size_t)m * N + n;
    dst[0] = from_float<T>(v0);
    if (second) dst[1] = from_float<T>(v1);
  } else if (EPI == EPI_RESIDUAL) {
    float* dst = (float*)c + (size_t)m * N + n;
    dst[0] += v0;
    if (second) dst[1] += v1;
  } else {
    T* dst = (T*)c + (size_t)m * (N / 2) + (n >> 1);
    dst[0] = from_float<T>(silu_for<T>(v0) * v1);
  }
}

// Sixteen consecutive columns n .. n+15 of row m held by one thread (n a multiple of 16): vector stores when the
// row piece is whole and 16-byte aligned, else the pairwise path.
template <int EPI, typename T>
__device__ __forceinline__ void epilogue_row16(void* __restrict__ c, int m, int n, int M, int N, const float* v) {
  if (m >= M || n >= N) return;
  bool whole = n + 16 <= N;
  if (EPI == EPI_STORE_F32 || EPI == EPI_RESIDUAL) {
    float* dst = (float*)c + (size_t)m * N + n;
    if (whole && (N & 3) == 0) {
      // (load, add, store per 16 bytes, as written: with the loads of a piece gathered in front of its stores the
      // 256-wide tile's epilogue, sixteen pieces a row, ran 3.5 times slower; the compiler pipelines this form)
#pragma unroll
      for (int i = 0; i < 16; i += 4) {
        float4 o = make_float4(v[i], v[i + 1], v[i + 2], v[i + 3]);
        if (EPI == EPI_RESIDUAL) {
          float4 r = *reinterpret_cast<float4*>(dst + i);
          o.x += r.x; o.y += r.y; o.z += r.z; o.w += r.w;
        }
        *reinterpret_cast<float4*>(dst + i) = o;
      }
      return;
    }
  } else if (EPI == EPI_STORE_T) {
    if (whole && (N & 7) == 0 && sizeof(T) == 2) {
      uint4 lo, hi;
      __nv_bfloat162* pl = reinterpret_cast<__nv_bfloat162*>(&lo);
      __nv_bfloat162* ph = reinterpret_cast<__nv_bfloat162*>(&hi);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        pl[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
        ph[i] = __floats2bfloat162_rn(v[8 + 2 * i], v[8 + 2 * i + 1]);
      }
      uint4* dst = reinterpret_cast<uint4*>((__nv_bfloat16*)c + (size_t)m * N + n);
      dst[0] = lo;
      dst[1] = hi;
      return;
    }
  } else {  // SwiGLU: eight outputs
    if (whole && (N & 15) == 0 && sizeof(T) == 2) {
      uint4 o;
      __nv_bfloat162* po = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
      for (int i = 0; i < 4; ++i)
        po[i] = __floats2bfloat162_rn(silu_for<T>(v[4 * i]) * v[4 * i + 1], silu_for<T>(v[4 * i + 2]) * v[4 * i + 3]);
      *reinterpret_cast<uint4*>((__nv_bfloat16*)c + (size_t)m * (N / 2) + (n >> 1)) = o;
      return;
    }
  }
#pragma unroll
  for (int i = 0; i < 16; i += 2) epilogue_pair<EPI, T>(c, m, n + i, M, N, v[i], v[i + 1]);
}

// Sixteen consecutive tokens token0 .. token0+15 of one output feature held by one thread, the lanes of the warp
// holding consecutive features (the accumulator is C^T). C is [tokens, features] as always, so a warp's stores for
// one token are contiguous. Every lane of the warp must call this (the SwiGLU pairs sit in neighbouring lanes).
template <int EPI, typename T>
__device__ __forceinline__ void epilogue_col16(void* __restrict__ c, int feature, int token0, int features, int tokens,
                                               const float* v) {
  if (EPI == EPI_T_SWIGLU) {
    T* out = (T*)c;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      float up = __shfl_xor_sync(0xffffffffu, v[i], 1);  // the odd lane's value: up_i beside gate_i
      if (!(feature & 1) && feature + 1 < features && token0 + i < tokens)
        out[(size_t)(token0 + i) * (features / 2) + (feature >> 1)] = from_float<T>(silu_for<T>(v[i]) * up);
    }
    return;
  }
  if (feature >= features) return;
  if (EPI == EPI_T_RESIDUAL) {  // all sixteen loads first: one round trip, not sixteen
    float old[16];
#pragma unroll
    for (int i = 0; i < 16; ++i)
      old[i] = token0 + i < tokens ? ((const float*)c)[(size_t)(token0 + i) * features + feature] : 0.f;
#pragma unroll
    for (int i = 0; i < 16; ++i)
      if (token0 + i < tokens) ((float*)c)[(size_t)(token0 + i) * features + feature] = old[i] + v[i];
    return;
  }
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    if (token0 + i >= tokens) break;
    size_t at = (size_t)(token0 + i) * features + feature;
    if (EPI == EPI_T_STORE_F32) ((float*)c)[at] = v[i];
    else ((T*)c)[at] = from_float<T>(v[i]);
  }
}
