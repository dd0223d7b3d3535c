// bfloat16 matrix product with float32 accumulation on the tensor cores (mma.sync m16n8k16, cp.async 3-stage
// pipeline), for any M, ending in the shared epilogues (store, residual add in float32, SwiGLU). K must be a
// multiple of 8 (16-byte rows), and N even for the SwiGLU epilogue; anything else is refused. (Decode-sized products run in gemv.cu.)
#include "gemm_common.cuh"

namespace {
typedef __nv_bfloat16 bf16;

// ---------------------------------------------------------------------------------------------------------------
// tensor-core tile kernel
// ---------------------------------------------------------------------------------------------------------------
constexpr int BM = 128, BN = 64, BK = 32, STAGES = 3, THREADS = 256;
constexpr int LDS = BK + 8;  // row stride in elements: 80 bytes, keeps 16-byte alignment and spreads banks

__device__ __forceinline__ void cp_async_16(void* smem, const void* gmem, bool valid) {
  unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  int bytes = valid ? 16 : 0;  // 0 bytes read: the 16 bytes of shared memory are filled with zeros
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(s), "l"(gmem), "r"(bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}
__device__ __forceinline__ void ldmatrix_x4(unsigned& r0, unsigned& r1, unsigned& r2, unsigned& r3, const void* p) {
  unsigned s = (unsigned)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(s));
}
__device__ __forceinline__ void mma_bf16(float* c, const unsigned* a, unsigned b0, unsigned b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

template <int EPI>
__global__ void __launch_bounds__(THREADS) gemm_bf16_mma_kernel(void* __restrict__ c, const bf16* __restrict__ a,
                                                                const bf16* __restrict__ w, int M, int N, int K) {
  __shared__ __align__(16) bf16 as[STAGES][BM][LDS];
  __shared__ __align__(16) bf16 ws[STAGES][BN][LDS];
  int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  int wm = warp >> 1, wn = warp & 1;  // 4 x 2 warps, each 32 x 32
  int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  int ktiles = (K + BK - 1) / BK;

  auto load_stage = [&](int stage, int kt) {
    int k0 = kt * BK;
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      int chunk = tid + i * THREADS;  // 512 chunks of A
      int row = chunk >> 2, kc = (chunk & 3) * 8;
      bool ok = m0 + row < M && k0 + kc < K;
      const bf16* src = ok ? a + (size_t)(m0 + row) * K + k0 + kc : a;
      cp_async_16(&as[stage][row][kc], src, ok);
    }
    {
      int row = tid >> 2, kc = (tid & 3) * 8;  // 256 chunks of W
      bool ok = n0 + row < N && k0 + kc < K;
      const bf16* src = ok ? w + (size_t)(n0 + row) * K + k0 + kc : w;
      cp_async_16(&ws[stage][row][kc], src, ok);
    }
  };

  float acc[2][4][4];
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
      for (int r = 0; r < 4; ++r) acc[i][j][r] = 0.f;

#pragma unroll
  for (int s = 0; s < STAGES - 1; ++s) {
    if (s < ktiles) load_stage(s, s);
    cp_async_commit();
  }
  for (int kt = 0; kt < ktiles; ++kt) {
    cp_async_wait<STAGES - 2>();
    __syncthreads();
    int next = kt + STAGES - 1;
    if (next < ktiles) load_stage(next % STAGES, next);
    cp_async_commit();
    int stage = kt % STAGES;
#pragma unroll
    for (int kk = 0; kk < BK; kk += 16) {
      unsigned af[2][4], bfr[4][2];
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        const bf16* p = &as[stage][wm * 32 + i * 16 + (lane & 15)][kk + (lane >> 4) * 8];
        ldmatrix_x4(af[i][0], af[i][1], af[i][2], af[i][3], p);
      }
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        int mat = lane >> 3;
        const bf16* p = &ws[stage][wn * 32 + j * 16 + (mat >> 1) * 8 + (lane & 7)][kk + (mat & 1) * 8];
        ldmatrix_x4(bfr[2 * j][0], bfr[2 * j][1], bfr[2 * j + 1][0], bfr[2 * j + 1][1], p);
      }
#pragma unroll
      for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) mma_bf16(acc[i][j], af[i], bfr[j][0], bfr[j][1]);
    }
  }
  cp_async_wait<0>();

  int g = lane >> 2, t = lane & 3;
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      int m = m0 + wm * 32 + i * 16 + g, n = n0 + wn * 32 + j * 8 + t * 2;
      epilogue_pair<EPI, bf16>(c, m, n, M, N, acc[i][j][0], acc[i][j][1]);
      epilogue_pair<EPI, bf16>(c, m + 8, n, M, N, acc[i][j][2], acc[i][j][3]);
    }
}

template <int EPI>
int launch_mma(void* c, const bf16* a, const bf16* w, int M, int N, int K, cudaStream_t stream) {
  dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
  if (grid.y > 65535) return DLLM_UNSUPPORTED_SIZE;
  gemm_bf16_mma_kernel<EPI><<<grid, THREADS, 0, stream>>>(c, a, w, M, N, K);
  return dllm_launch_status();
}
}  // namespace

// C = A[M,K] * W[N,K]^T, bfloat16 operands, float32 accumulation.
DLLM_EXPORT int dllm_gemm_bf16(void* c, const void* a, const void* w, int M, int N, int K, int epilogue,
                               cudaStream_t stream) {
  if (M <= 0 || N <= 0) return DLLM_OK;
  if (K <= 0 || (K & 7) || ((N & 1) && epilogue == EPI_SWIGLU)) return DLLM_UNSUPPORTED_SIZE;
  const bf16 *ap = (const bf16*)a, *wp = (const bf16*)w;
  switch (epilogue) {
    case EPI_STORE_F32: return launch_mma<EPI_STORE_F32>(c, ap, wp, M, N, K, stream);
    case EPI_STORE_T: return launch_mma<EPI_STORE_T>(c, ap, wp, M, N, K, stream);
    case EPI_RESIDUAL: return launch_mma<EPI_RESIDUAL>(c, ap, wp, M, N, K, stream);
    case EPI_SWIGLU: return launch_mma<EPI_SWIGLU>(c, ap, wp, M, N, K, stream);
    default: return DLLM_BAD_ARGUMENT;
  }
}
