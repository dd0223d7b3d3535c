// Shared helpers of the sm_100a kernels: element types, conversions, warp reductions, status codes.
//
// Every exported entry point is `extern "C"`, takes raw device pointers, sizes and a stream, launches
// asynchronously and returns 0 or a negative status for arguments it refuses (never a wrong result).
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdlib.h>

#define DLLM_OK 0
#define DLLM_BAD_ARGUMENT (-1)
#define DLLM_UNSUPPORTED_SIZE (-2)
#define DLLM_LAUNCH_FAILED (-3)

#define DLLM_F32 0
#define DLLM_BF16 1

#define DLLM_EXPORT extern "C" __attribute__((visibility("default")))

static inline int dllm_launch_status() {
  return cudaGetLastError() == cudaSuccess ? DLLM_OK : DLLM_LAUNCH_FAILED;
}

// ---- programmatic dependent launch ----------------------------------------------------------------------------
// Kernels of the decode step are launched so that the next kernel's blocks may start while this one still runs:
// a kernel first lets its dependents go (`pdl_launch_dependents`), may read what no earlier kernel of the step
// writes (weights, tables), and must call `pdl_wait` before it touches anything an earlier kernel produced and
// before its own first write. Launched without the attribute both calls do nothing. DLLM_B200_PDL=0 turns the
// attribute off.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

static inline bool dllm_pdl_enabled() {
  static int enabled = -1;
  if (enabled < 0) {
    const char* v = getenv("DLLM_B200_PDL");
    enabled = (v && v[0] == '0') ? 0 : 1;
  }
  return enabled == 1;
}

template <typename... KArgs, typename... Args>
static inline int dllm_launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                  Args... args) {
  cudaLaunchConfig_t config = {};
  config.gridDim = grid;
  config.blockDim = block;
  config.dynamicSmemBytes = smem;
  config.stream = stream;
  cudaLaunchAttribute attribute[1];
  attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attribute[0].val.programmaticStreamSerializationAllowed = 1;
  config.attrs = attribute;
  config.numAttrs = dllm_pdl_enabled() ? 1 : 0;
  return cudaLaunchKernelEx(&config, kernel, KArgs(args)...) == cudaSuccess ? DLLM_OK : DLLM_LAUNCH_FAILED;
}

__device__ __forceinline__ float to_float(float v) { return v; }
__device__ __forceinline__ float to_float(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T from_float(float v);
template <> __device__ __forceinline__ float from_float<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// 2^x with the hardware approximation (one instruction; 2^-inf = 0), for softmax weights in float32.
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Where the keys and values of one cache entry (one layer's cache) live. A page holds `page_size` positions of
// every kv head: [page][k|v][kv_head][page_size][head_dim]. `page_table[slot * max_pages + i]` is the page that
// holds positions i*page_size .. of the sequence in `slot`.
struct KvLayout {
  void* base;            // this cache entry's storage
  const int* page_table;
  int max_pages;         // page table row length
  int page_size;
  int kv_heads;
  int head_dim;
};

__device__ __forceinline__ size_t kv_offset(const KvLayout& c, int page, int which, int kv_head, int row) {
  return ((((size_t)page * 2 + which) * c.kv_heads + kv_head) * c.page_size + row) * (size_t)c.head_dim;
}
