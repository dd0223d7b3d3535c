// The allocation-free variant of decode attention (see attention_decode_static.h for who needs it and its rules).
// The kernels are those of attention_decode.cu, compiled into this library as they are; only the scratch differs:
// it is the file-scope device array below instead of memory the caller brings.
#include "attention_decode_static.h"

#include <stdio.h>

#include "attention_decode.cu"

namespace {
constexpr int MAX_DEVICES = 64;

// Scratch for the partial results and the ticket counters. In host code these names are only stand-ins for the
// device objects; the host gets their device addresses from cudaGetSymbolAddress.
static __device__ __align__(256) float static_scratch[DLLM_STATIC_SCRATCH_FLOATS];
static __device__ __align__(256) unsigned static_tickets[DLLM_STATIC_TICKETS];

struct DeviceAddresses {
  float* scratch;
  unsigned* tickets;
  bool ready;
};
DeviceAddresses addresses[MAX_DEVICES];

// Once per device, with that device current: the device addresses of the two arrays.
int addresses_of_current_device(DeviceAddresses** found) {
  int device = -1;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= MAX_DEVICES) return DLLM_LAUNCH_FAILED;
  DeviceAddresses& entry = addresses[device];
  if (!entry.ready) {
    float* scratch = nullptr;
    unsigned* tickets = nullptr;
    if (cudaGetSymbolAddress((void**)&scratch, static_scratch) != cudaSuccess || scratch == nullptr)
      return DLLM_LAUNCH_FAILED;
    if (cudaGetSymbolAddress((void**)&tickets, static_tickets) != cudaSuccess || tickets == nullptr)
      return DLLM_LAUNCH_FAILED;
    entry.scratch = scratch;
    entry.tickets = tickets;
    entry.ready = true;
  }
  *found = &entry;
  return DLLM_OK;
}
}  // namespace

DLLM_EXPORT int dllm_attention_decode_static(void* out, const void* q, void* cache_base, const int* page_table,
                                             int max_pages, int page_size, int heads, int kv_heads, int head_dim,
                                             const int* tok_pos, const int* slots, int sequences, float scale,
                                             int window, int chunk, int max_context, cudaStream_t stream) {
  if (sequences <= 0) return DLLM_OK;
  if (heads <= 0 || kv_heads <= 0 || head_dim <= 0 || chunk < 16 || max_context <= 0) return DLLM_BAD_ARGUMENT;
  long long chunks = ((long long)max_context + chunk - 1) / chunk;
  long long need_floats = (long long)sequences * heads * chunks * (head_dim + 2);
  long long need_tickets = (long long)sequences * kv_heads;
  if (need_floats > DLLM_STATIC_SCRATCH_FLOATS || need_tickets > DLLM_STATIC_TICKETS) {
    fprintf(stderr,
            "dllm_attention_decode_static: the built-in scratch is too small for this call: it needs %lld floats and "
            "%lld counters, the library holds %d floats and %d counters (fewer sequences, a larger chunk or a smaller "
            "max_context fit)\n",
            need_floats, need_tickets, DLLM_STATIC_SCRATCH_FLOATS, DLLM_STATIC_TICKETS);
    return DLLM_STATIC_TOO_LARGE;
  }
  DeviceAddresses* device = nullptr;
  int status = addresses_of_current_device(&device);
  if (status != DLLM_OK) return status;
  // the counters must start at zero whatever an earlier (perhaps aborted) call left in them
  if (cudaMemsetAsync(device->tickets, 0, (size_t)need_tickets * sizeof(unsigned), stream) != cudaSuccess)
    return DLLM_LAUNCH_FAILED;
  return dllm_attention_decode(out, q, cache_base, page_table, max_pages, page_size, heads, kv_heads, head_dim, tok_pos,
                               slots, sequences, scale, window, chunk, max_context, device->scratch, device->tickets,
                               stream);
}
