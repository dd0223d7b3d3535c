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

// ---- the same product for many rows: 128 x 128 tiles, 8 x 8 outputs a thread ---------------------------------------
// Two stages of shared memory; the next k tile travels from global memory into registers while this one is
// multiplied. A thread's 64 outputs are 2 x 2 groups of 4 x 4, so its shared-memory reads are four 16-byte loads per
// k. Every output is still one chain of fused multiply-adds over k ascending from zero: the same bits as above.
constexpr int LM = 128, LN = 128, LK = 16, LTHREADS = 256;

template <int EPI>
__global__ void __launch_bounds__(LTHREADS) gemm_f32_large_kernel(void* __restrict__ c, const float* __restrict__ a,
                                                                  const float* __restrict__ w, int M, int N, int K) {
  __shared__ __align__(16) float as[2][LK][LM + 4];
  __shared__ __align__(16) float ws[2][LK][LN + 4];
  int tid = threadIdx.x;
  int tx = tid & 15, ty = tid >> 4;             // 16 x 16 threads; outputs rows ty*4 + {0..3, 64..67}, cols likewise
  int m0 = blockIdx.y * LM, n0 = blockIdx.x * LN;
  int lrow = tid >> 2, lk = (tid & 3) * 4;      // a thread fetches rows lrow and lrow + 64, k lk .. lk + 3
  float acc[8][8];
#pragma unroll
  for (int i = 0; i < 8; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[i][j] = 0.f;
  float4 va[2], vw[2];
  auto fetch = [&](int k0) {
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      int r = lrow + 64 * h;
      va[h] = vw[h] = make_float4(0.f, 0.f, 0.f, 0.f);
      if (m0 + r < M && k0 + lk < K) va[h] = *(const float4*)(a + (size_t)(m0 + r) * K + k0 + lk);
      if (n0 + r < N && k0 + lk < K) vw[h] = *(const float4*)(w + (size_t)(n0 + r) * K + k0 + lk);
    }
  };
  auto stash = [&](int buf) {
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      int r = lrow + 64 * h;
      as[buf][lk + 0][r] = va[h].x; as[buf][lk + 1][r] = va[h].y; as[buf][lk + 2][r] = va[h].z; as[buf][lk + 3][r] = va[h].w;
      ws[buf][lk + 0][r] = vw[h].x; ws[buf][lk + 1][r] = vw[h].y; ws[buf][lk + 2][r] = vw[h].z; ws[buf][lk + 3][r] = vw[h].w;
    }
  };
  fetch(0);
  stash(0);
  __syncthreads();
  int tiles = (K + LK - 1) / LK;
  for (int t = 0; t < tiles; ++t) {
    int buf = t & 1;
    if (t + 1 < tiles) fetch((t + 1) * LK);
#pragma unroll
    for (int k = 0; k < LK; ++k) {
      float4 a0 = *(const float4*)&as[buf][k][ty * 4], a1 = *(const float4*)&as[buf][k][64 + ty * 4];
      float4 w0 = *(const float4*)&ws[buf][k][tx * 4], w1 = *(const float4*)&ws[buf][k][64 + tx * 4];
      float av[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
      float wv[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
      for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[i][j] = fmaf(av[i], wv[j], acc[i][j]);
    }
    if (t + 1 < tiles) {
      stash(buf ^ 1);  // (the other stage was last read before the barrier that ended the step before)
      __syncthreads();
    }
  }
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    int m = m0 + (i >> 2) * 64 + ty * 4 + (i & 3);
#pragma unroll
    for (int j = 0; j < 8; j += 2) {
      int n = n0 + (j >> 2) * 64 + tx * 4 + (j & 3);
      epilogue_pair<EPI, float>(c, m, n, M, N, acc[i][j], acc[i][j + 1]);
    }
  }
}

// ---- and for a few rows (decode steps): 32 columns a block, the reduction streamed through three stages -------------
// A thread owns one column and four rows; W and A tiles of 32 values of k arrive by cp.async. Again one chain of
// fused multiply-adds per output over k ascending from zero: a token's bits are the ones it gets in a long prompt.
constexpr int SN = 32, SK = 32, SM_ROWS = 16, STHREADS = 128, SSTAGES = 3, SLD = SK + 4;

__device__ __forceinline__ void cp_async_f4(float* smem, const float* gmem, bool ok) {
  unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  int bytes = ok ? 16 : 0;  // (a copy of no bytes fills the 16 bytes with zeros)
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(s), "l"(gmem), "r"(bytes));
}

template <int EPI>
__global__ void __launch_bounds__(STHREADS) gemm_f32_small_kernel(void* __restrict__ c, const float* __restrict__ a,
                                                                  const float* __restrict__ w, int M, int N, int K) {
  __shared__ __align__(16) float w_s[SSTAGES][SN][SLD];
  __shared__ __align__(16) float a_s[SSTAGES][SM_ROWS][SLD];
  int tid = threadIdx.x, col = tid & 31, rows0 = (tid >> 5) * 4;
  int n0 = blockIdx.x * SN;
  int tiles = (K + SK - 1) / SK;
  auto issue = [&](int t) {
    if (t < tiles) {
      int buf = t % SSTAGES, k0 = t * SK;
      for (int i = tid; i < (SN + SM_ROWS) * (SK / 4); i += STHREADS) {
        int r = i / (SK / 4), k = (i % (SK / 4)) * 4;
        if (r < SN) {
          bool ok = n0 + r < N && k0 + k < K;
          cp_async_f4(&w_s[buf][r][k], ok ? w + (size_t)(n0 + r) * K + k0 + k : w, ok);
        } else {
          int m = r - SN;
          bool ok = m < M && k0 + k < K;
          cp_async_f4(&a_s[buf][m][k], ok ? a + (size_t)m * K + k0 + k : a, ok);
        }
      }
    }
    asm volatile("cp.async.commit_group;\n" ::);
  };
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
  issue(0);
  issue(1);
  for (int t = 0; t < tiles; ++t) {
    issue(t + 2);
    asm volatile("cp.async.wait_group 2;\n" ::: "memory");
    __syncthreads();
    int buf = t % SSTAGES;
#pragma unroll
    for (int k = 0; k < SK; k += 4) {
      float4 wv = *(const float4*)&w_s[buf][col][k];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        float4 av = *(const float4*)&a_s[buf][rows0 + i][k];
        acc[i] = fmaf(av.x, wv.x, acc[i]);
        acc[i] = fmaf(av.y, wv.y, acc[i]);
        acc[i] = fmaf(av.z, wv.z, acc[i]);
        acc[i] = fmaf(av.w, wv.w, acc[i]);
      }
    }
    __syncthreads();  // the stage is free for the copy after next
  }
  // pairs of columns are stored by the even lane (the SwiGLU epilogue needs gate and up together)
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float other = __shfl_down_sync(0xffffffffu, acc[i], 1);
    if (!(col & 1)) epilogue_pair<EPI, float>(c, rows0 + i, n0 + col, M, N, acc[i], other);
  }
}
}  // namespace

// C = A[M,K] * W[N,K]^T in float32; K a multiple of 4 (16-byte rows); N even for the SwiGLU epilogue (column pairs).
// Up to 16 rows take the kernel that streams the reduction, 17 to 64 the 64 x 64 tiles, more the 128 x 128 tiles;
// the three give an output the same bits.
DLLM_EXPORT int dllm_gemm_f32(void* c, const float* a, const float* w, int M, int N, int K, int epilogue,
                              cudaStream_t stream) {
  if (M <= 0 || N <= 0) return DLLM_OK;
  if (K <= 0 || (K & 3) || ((N & 1) && epilogue == EPI_SWIGLU)) return DLLM_UNSUPPORTED_SIZE;
  if (epilogue < 0 || epilogue > EPI_SWIGLU) return DLLM_BAD_ARGUMENT;
  if (epilogue == EPI_STORE_T) epilogue = EPI_STORE_F32;  // (the activation type is float32 here)
#define DLLM_BY_EPILOGUE(KERNEL, GRID, THREADS_)                                                      \
  switch (epilogue) {                                                                                 \
    case EPI_STORE_F32: KERNEL<EPI_STORE_F32><<<GRID, THREADS_, 0, stream>>>(c, a, w, M, N, K); break; \
    case EPI_RESIDUAL: KERNEL<EPI_RESIDUAL><<<GRID, THREADS_, 0, stream>>>(c, a, w, M, N, K); break;   \
    default: KERNEL<EPI_SWIGLU><<<GRID, THREADS_, 0, stream>>>(c, a, w, M, N, K); break;               \
  }
  if (M <= SM_ROWS) {
    dim3 grid((N + SN - 1) / SN);
    DLLM_BY_EPILOGUE(gemm_f32_small_kernel, grid, STHREADS)
  } else if (M <= 64) {
    dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
    DLLM_BY_EPILOGUE(gemm_f32_kernel, grid, THREADS)
  } else {
    dim3 grid((N + LN - 1) / LN, (M + LM - 1) / LM);
    if (grid.y > 65535) return DLLM_UNSUPPORTED_SIZE;
    DLLM_BY_EPILOGUE(gemm_f32_large_kernel, grid, LTHREADS)
  }
#undef DLLM_BY_EPILOGUE
  return dllm_launch_status();
}
