// Weight-streaming products for decode on large matrices (at most 16 rows of activations, bfloat16): C = X * W^T
// where reading W once from HBM is the whole cost, so what counts is how many bytes are on their way at any time.
// Here they travel into shared memory, not into registers: a producer warp issues bulk copies (cp.async.bulk, 2 KB
// of one row of W or X per copy, completion counted by an mbarrier) into a ring of stages that holds about 200 KB
// per multiprocessor, and two consumer warps multiply out of shared memory on the tensor cores (mma.sync m16n8k16
// with W as the 16-row operand, ldmatrix from rows padded by 16 bytes so that no two rows share a bank).
// Blocks are persistent: a block walks over its tiles of 16 or 32 rows of W and the ring runs on across tiles.
//   ROWS = 32: each consumer warp owns 16 rows of W over the whole reduction (no exchange between warps);
//   ROWS = 16: the two warps share the rows and take alternate 16-value steps; the second hands its sums to the
//              first.
// Epilogues as the tile kernels: store (float32 / bfloat16), residual add in float32, SwiGLU on interleaved rows.
// K must be a multiple of 64. Every wait on an mbarrier is bounded; a role that gives up records a status word.
#include "gemm_common.cuh"
#include "tcgen05.cuh"

namespace {
using namespace tc5;
typedef __nv_bfloat16 bf16;
constexpr int KC = 1024;                   // values of k per stage: 2 KB of every row (a bulk copy costs its
                                           // issuer about as much whatever its size, so copies are long)
constexpr int ROW_BYTES = KC * 2;
constexpr int PITCH = ROW_BYTES + 16;      // rows in shared memory: 16 bytes of padding (ldmatrix without conflicts)
constexpr int THREADS = 96;                // warp 0 copies, warps 1 and 2 multiply
constexpr int RING_BYTES = 216 * 1024;

__device__ __forceinline__ void bulk_copy(void* dst, const void* src, unsigned bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void ldmatrix_x4(unsigned* r, unsigned addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x2(unsigned* r, unsigned addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];\n" : "=r"(r[0]), "=r"(r[1]) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float* c, const unsigned* a, unsigned b0, unsigned b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

template <int ROWS, int NT> struct Shape {
  static constexpr int TOKENS = NT * 8;                          // token rows of a stage (those beyond M stay unused)
  static constexpr int STAGE_BYTES = (ROWS + TOKENS) * PITCH;
  static constexpr int STAGES = RING_BYTES / STAGE_BYTES;
  static constexpr int SCRATCH_FLOATS = 2 * 16 * (TOKENS + 1);   // a 16 x TOKENS tile per consumer warp
  static constexpr size_t SMEM = (size_t)STAGES * STAGE_BYTES + SCRATCH_FLOATS * sizeof(float) + 128;
};

template <int ROWS, int NT, int EPI>
__global__ void __launch_bounds__(THREADS, 1) gemv_tma_kernel(void* __restrict__ c, const bf16* __restrict__ x,
                                                              const bf16* __restrict__ w, int M, int N, int K,
                                                              int tiles, int* __restrict__ status) {
  typedef Shape<ROWS, NT> S;
  extern __shared__ __align__(128) unsigned char smem_raw[];
  unsigned char* ring = (unsigned char*)(((uintptr_t)smem_raw + 127) & ~(uintptr_t)127);
  float* scratch = reinterpret_cast<float*>(ring + (size_t)S::STAGES * S::STAGE_BYTES);
  __shared__ uint64_t full_bar[S::STAGES], empty_bar[S::STAGES];
  int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  int chunks = K / KC + (K % KC ? 1 : 0);  // stages per tile; the last may be shorter (K is a multiple of 64)
  pdl_launch_dependents();
  if (threadIdx.x == 0) {
    for (int s = 0; s < S::STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 2); }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();

  if (warp == 0) {
    // ---- producer: lane r copies row r of the tile's W; lanes also copy the token rows of X. The weights are
    // nobody's output: the first trip round the ring asks for them before the wait on the kernel before, and adds
    // the rows of X (which that kernel may have written) after it.
    auto fill = [&](int it, int tile, int ch, bool weights, bool tokens) {
      int s = it % S::STAGES;
      int row0 = tile * ROWS, rows_valid = min(ROWS, N - row0), k0 = ch * KC;
      unsigned bytes = (unsigned)min(KC, K - k0) * 2u;
      unsigned char* stage = ring + (size_t)s * S::STAGE_BYTES;
      if (weights) {
        if (lane == 0) mbar_expect_tx(&full_bar[s], bytes * (unsigned)(rows_valid + M));
        __syncwarp();
        for (int r = lane; r < rows_valid; r += 32)
          bulk_copy(stage + r * PITCH, w + (size_t)(row0 + r) * K + k0, bytes, &full_bar[s]);
      }
      if (tokens)
        for (int m = lane; m < M; m += 32)
          bulk_copy(stage + (ROWS + m) * PITCH, x + (size_t)m * K + k0, bytes, &full_bar[s]);
    };
    int it = 0, tile = blockIdx.x, ch = 0;
    for (; it < S::STAGES && tile < tiles; ++it) {  // the first trip: weights only
      fill(it, tile, ch, true, false);
      if (++ch == chunks) { ch = 0; tile += gridDim.x; }
    }
    pdl_wait();
    {
      int it2 = 0, tile2 = blockIdx.x, ch2 = 0;
      for (; it2 < it; ++it2) {  // their rows of X
        fill(it2, tile2, ch2, false, true);
        if (++ch2 == chunks) { ch2 = 0; tile2 += gridDim.x; }
      }
    }
    for (; tile < tiles; ++it) {
      int s = it % S::STAGES;
      if (!mbar_wait(&empty_bar[s], ((it / S::STAGES) - 1) & 1)) {
        if (lane == 0) *(volatile int*)status = 32;
        break;
      }
      fill(it, tile, ch, true, true);
      if (++ch == chunks) { ch = 0; tile += gridDim.x; }
    }
  } else {
    // ---- consumers
    pdl_wait();  // C (for the residual) may come from the kernel before
    int cw = warp - 1;                       // 0 or 1
    int g = lane >> 2, t = lane & 3;
    int row_base = ROWS == 32 ? cw * 16 : 0;  // first of this warp's 16 rows within the tile
    // ldmatrix addresses inside a stage: W rows (lane & 15), k offset 8 for the upper lanes; X rows (lane & 7),
    // k offset 8 for lanes 8..15 (and the second eight tokens for lanes 16..31 when NT == 2)
    unsigned a_off = (unsigned)((row_base + (lane & 15)) * PITCH + (lane >> 4) * 16);
    unsigned b_off =
        (unsigned)((ROWS + (lane & 7) + (NT == 2 ? (lane >> 4) * 8 : 0)) * PITCH + ((lane >> 3) & 1) * 16);
    float* mine = scratch + cw * 16 * (S::TOKENS + 1);
    int it = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < tiles && ok; tile += gridDim.x) {
      float acc[2][NT][4];  // two sets on alternate steps: a step does not wait for the one before
#pragma unroll
      for (int e = 0; e < 2; ++e)
#pragma unroll
        for (int n = 0; n < NT; ++n)
#pragma unroll
          for (int i = 0; i < 4; ++i) acc[e][n][i] = 0.f;
      for (int ch = 0; ch < chunks; ++ch, ++it) {
        int s = it % S::STAGES;
        if (!mbar_wait(&full_bar[s], (it / S::STAGES) & 1)) {
          if (lane == 0) *(volatile int*)status = 33;
          ok = false;
          break;
        }
        unsigned stage = smem_u32(ring + (size_t)s * S::STAGE_BYTES);
        int ksteps = min(KC, K - ch * KC) / 16;
        // ROWS == 32: every step; ROWS == 16: this warp's alternate steps
        constexpr int STRIDE = ROWS == 32 ? 1 : 2;
        int first = ROWS == 32 ? 0 : cw;
        // (a stage holds a multiple of four steps, so a warp's steps come in pairs: one for each set of sums)
#pragma unroll 2
        for (int ks = first; ks < ksteps; ks += 2 * STRIDE) {
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            unsigned a[4], b[4];
            unsigned at = (unsigned)(ks + e * STRIDE) * 32u;
            ldmatrix_x4(a, stage + a_off + at);
            if (NT == 2) ldmatrix_x4(b, stage + b_off + at);
            else ldmatrix_x2(b, stage + b_off + at);
            mma_bf16(acc[e][0], a, b[0], b[1]);
            if (NT == 2) mma_bf16(acc[e][NT - 1], a, b[2], b[3]);
          }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty_bar[s]);  // this warp is done with the stage
      }
      if (!ok) break;
      // the warp's 16 x TOKENS tile to shared memory, then one (pair of rows, token) per thread and turn
#pragma unroll
      for (int n = 0; n < NT; ++n) {
        mine[g * (S::TOKENS + 1) + n * 8 + 2 * t] = acc[0][n][0] + acc[1][n][0];
        mine[g * (S::TOKENS + 1) + n * 8 + 2 * t + 1] = acc[0][n][1] + acc[1][n][1];
        mine[(g + 8) * (S::TOKENS + 1) + n * 8 + 2 * t] = acc[0][n][2] + acc[1][n][2];
        mine[(g + 8) * (S::TOKENS + 1) + n * 8 + 2 * t + 1] = acc[0][n][3] + acc[1][n][3];
      }
      if (ROWS == 16) asm volatile("bar.sync 1, 64;" ::: "memory");  // both halves of the reduction are there
      else __syncwarp();
      if (ROWS == 32 || cw == 0) {
        const float* other = scratch + 16 * (S::TOKENS + 1);
        int n0 = tile * ROWS + row_base;
        for (int idx = lane; idx < 8 * S::TOKENS; idx += 32) {
          int p = idx / S::TOKENS, m = idx % S::TOKENS;
          if (m >= M) continue;
          float v0 = mine[(2 * p) * (S::TOKENS + 1) + m], v1 = mine[(2 * p + 1) * (S::TOKENS + 1) + m];
          if (ROWS == 16) {
            v0 += other[(2 * p) * (S::TOKENS + 1) + m];
            v1 += other[(2 * p + 1) * (S::TOKENS + 1) + m];
          }
          epilogue_pair<EPI, bf16>(c, m, n0 + 2 * p, M, N, v0, v1);
        }
      }
      if (ROWS == 16) asm volatile("bar.sync 1, 64;" ::: "memory");  // the scratch is free for the next tile
      else __syncwarp();
    }
  }
}

template <int ROWS, int NT, int EPI>
int launch(void* c, const bf16* x, const bf16* w, int M, int N, int K, int* status, cudaStream_t stream) {
  typedef Shape<ROWS, NT> S;
  static int sms = 0;
  if (sms == 0) {
    int device = 0;
    if (cudaFuncSetAttribute(gemv_tma_kernel<ROWS, NT, EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             (int)S::SMEM) != cudaSuccess ||
        cudaGetDevice(&device) != cudaSuccess ||
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || sms <= 0) {
      sms = 0;
      return DLLM_LAUNCH_FAILED;
    }
  }
  int tiles = (N + ROWS - 1) / ROWS;
  int blocks = tiles < sms ? tiles : sms;
  return dllm_launch_pdl(gemv_tma_kernel<ROWS, NT, EPI>, dim3(blocks), dim3(THREADS), S::SMEM, stream, c, x, w, M, N,
                         K, tiles, status);
}

template <int ROWS, int NT>
int dispatch(void* c, const bf16* x, const bf16* w, int M, int N, int K, int epilogue, int* status,
             cudaStream_t stream) {
  switch (epilogue) {
    case EPI_STORE_F32: return launch<ROWS, NT, EPI_STORE_F32>(c, x, w, M, N, K, status, stream);
    case EPI_STORE_T: return launch<ROWS, NT, EPI_STORE_T>(c, x, w, M, N, K, status, stream);
    case EPI_RESIDUAL: return launch<ROWS, NT, EPI_RESIDUAL>(c, x, w, M, N, K, status, stream);
    case EPI_SWIGLU: return launch<ROWS, NT, EPI_SWIGLU>(c, x, w, M, N, K, status, stream);
    default: return DLLM_BAD_ARGUMENT;
  }
}
}  // namespace

// C = X[M,K] * W[N,K]^T for M <= 16, bfloat16 X and W, K a multiple of 64, N even for SwiGLU; X and W 16-byte
// aligned. `status` is a word the device can write; the kernel sets it non-zero if a bounded wait ran out
// (32: producer, 33: consumer).
DLLM_EXPORT int dllm_gemv_tma(void* c, const void* x, const void* w, int M, int N, int K, int epilogue, int* status,
                              cudaStream_t stream) {
  if (M <= 0 || N <= 0) return DLLM_OK;
  if (M > 16 || K <= 0 || (K & 63) || ((N & 1) && epilogue == EPI_SWIGLU) || ((uintptr_t)x & 15) ||
      ((uintptr_t)w & 15) || status == nullptr)
    return DLLM_UNSUPPORTED_SIZE;
  static int sms = 0;
  if (sms == 0) {
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess ||
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || sms <= 0)
      return DLLM_LAUNCH_FAILED;
  }
  // the tile height that leaves the busiest multiprocessor the fewest rows
  long long rows32 = (long long)((((N + 31) / 32) + sms - 1) / sms) * 32;
  long long rows16 = (long long)((((N + 15) / 16) + sms - 1) / sms) * 16;
  bool tall = rows32 <= rows16;
  const bf16* xp = (const bf16*)x;
  const bf16* wp = (const bf16*)w;
  if (M <= 8) return tall ? dispatch<32, 1>(c, xp, wp, M, N, K, epilogue, status, stream)
                          : dispatch<16, 1>(c, xp, wp, M, N, K, epilogue, status, stream);
  return tall ? dispatch<32, 2>(c, xp, wp, M, N, K, epilogue, status, stream)
              : dispatch<16, 2>(c, xp, wp, M, N, K, epilogue, status, stream);
}
