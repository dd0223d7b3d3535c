// The true 32-bit matrix product: float32 operands, one fused multiply-add chain per output over k ascending, on
// the CUDA cores. No tensor cores, no reduced-precision mode, no split of the reduction, so an output's bits depend
// only on its own row of A and row of W: not on M, on the tile it falls in, or on what else is in the batch.
#include "gemm_common.cuh"

namespace {
constexpr int BM = 64, BN = 64, BK = 16, THREADS = 256;

template <int EPI>
__global__ void __launch_bounds__(THREADS) gemm_f32_kernel(void* __restrict__ c, const float* __restrict__ a,
                                                           const float* __restrict__ w, int M, int N, int K) {
  __shared__ float as[BK][BM + 4];
  __shared__ float ws[BK][BN + 4];
  int tid = threadIdx.x;
  int tx = tid & 15, ty = tid >> 4;
  int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  int lrow = tid >> 2, lk = (tid & 3) * 4;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

  for (int k0 = 0; k0 < K; k0 += BK) {
    float4 va = make_float4(0.f, 0.f, 0.f, 0.f), vw = va;
    if (m0 + lrow < M && k0 + lk < K) va = *(const float4*)(a + (size_t)(m0 + lrow) * K + k0 + lk);
    if (n0 + lrow < N && k0 + lk < K) vw = *(const float4*)(w + (size_t)(n0 + lrow) * K + k0 + lk);
    as[lk + 0][lrow] = va.x; as[lk + 1][lrow] = va.y; as[lk + 2][lrow] = va.z; as[lk + 3][lrow] = va.w;
    ws[lk + 0][lrow] = vw.x; ws[lk + 1][lrow] = vw.y; ws[lk + 2][lrow] = vw.z; ws[lk + 3][lrow] = vw.w;
    __syncthreads();
#pragma unroll
    for (int k = 0; k < BK; ++k) {
      float4 ra = *(const float4*)&as[k][ty * 4];
      float4 rw = *(const float4*)&ws[k][tx * 4];
      float av[4] = {ra.x, ra.y, ra.z, ra.w}, wv[4] = {rw.x, rw.y, rw.z, rw.w};
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], wv[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    int m = m0 + ty * 4 + i, n = n0 + tx * 4;
    epilogue_pair<EPI, float>(c, m, n, M, N, acc[i][0], acc[i][1]);
    epilogue_pair<EPI, float>(c, m, n + 2, M, N, acc[i][2], acc[i][3]);
  }
}
}  // namespace

// C = A[M,K] * W[N,K]^T in float32; K a multiple of 4 (16-byte rows); N even for the SwiGLU epilogue (column pairs).
DLLM_EXPORT int dllm_gemm_f32(void* c, const float* a, const float* w, int M, int N, int K, int epilogue,
                              cudaStream_t stream) {
  if (M <= 0 || N <= 0) return DLLM_OK;
  if (K <= 0 || (K & 3) || ((N & 1) && epilogue == EPI_SWIGLU)) return DLLM_UNSUPPORTED_SIZE;
  dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
  if (grid.y > 65535) return DLLM_UNSUPPORTED_SIZE;
  switch (epilogue) {
    case EPI_STORE_F32: gemm_f32_kernel<EPI_STORE_F32><<<grid, THREADS, 0, stream>>>(c, a, w, M, N, K); break;
    case EPI_STORE_T: gemm_f32_kernel<EPI_STORE_F32><<<grid, THREADS, 0, stream>>>(c, a, w, M, N, K); break;
    case EPI_RESIDUAL: gemm_f32_kernel<EPI_RESIDUAL><<<grid, THREADS, 0, stream>>>(c, a, w, M, N, K); break;
    case EPI_SWIGLU: gemm_f32_kernel<EPI_SWIGLU><<<grid, THREADS, 0, stream>>>(c, a, w, M, N, K); break;
    default: return DLLM_BAD_ARGUMENT;
  }
  return dllm_launch_status();
}
