// Decode attention without any allocation: one entry point whose scratch memory is a fixed array inside the
// library. This entry point is an addition of this library; the reference project has no counterpart.
//
// Who it is for: callers that must not or cannot allocate device memory. A plugin inside a host program that owns
// the whole device through its own pool and hands out nothing but input and output buffers; a control loop that
// cannot afford the device-wide synchronisation a cudaMalloc or cudaFree may bring; bindings that can pass raw
// pointers but have no allocator of their own. They pass inputs and outputs exactly as for `dllm_attention_decode`
// and nothing else.
//
// Limits and rules:
//   - The scratch is `DLLM_STATIC_SCRATCH_FLOATS` floats (8 MiB) plus `DLLM_STATIC_TICKETS` counters, held by every
//     device that loads this library until the process ends. A call that needs more returns
//     DLLM_STATIC_TOO_LARGE (-4) and prints the sizes to standard error; nothing is launched.
//     Needed: sequences * heads * ceil(max_context / chunk) * (head_dim + 2) floats, sequences * kv_heads counters.
//   - The first call on a device looks up the array's device address (cudaGetSymbolAddress, once per device, with
//     that device current). Make that first call outside any stream capture, and from one thread: the look-up is
//     not synchronised, so two threads must not both make a device's first call at the same time. The address is
//     kept for the life of the device's context; after cudaDeviceReset the library must be loaded afresh.
//   - It calls no cudaMalloc, no cudaFree and no library routine that allocates.
//   - All calls share the one array and it keeps what the last call left. The counters are cleared on the stream
//     before every launch; partial results are overwritten before they are read. Two calls that overlap on the
//     device (different streams, no ordering) race on it: order them.
#pragma once
#include <cuda_runtime.h>

#define DLLM_STATIC_SCRATCH_FLOATS (2 * 1024 * 1024)
#define DLLM_STATIC_TICKETS 4096
#define DLLM_STATIC_TOO_LARGE (-4)

#ifdef __cplusplus
extern "C" {
#endif

// Same arguments and result as `dllm_attention_decode` (attention_decode.cu) without `scratch` and `tickets`.
int dllm_attention_decode_static(void* out, const void* q, void* cache_base, const int* page_table, int max_pages,
                                 int page_size, int heads, int kv_heads, int head_dim, const int* tok_pos,
                                 const int* slots, int sequences, float scale, int window, int chunk,
                                 int max_context, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
