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
    dst[0] = from_float<T>(silu_f32(v0) * v1);
  }
}
