// A test's own kernel: one thread waits, with the library's bounded wait, on an mbarrier that nobody ever arrives
// at. Built with a wait limit of a few tens of microseconds (-DDLLM_WAIT_LIMIT_CYCLES=...), the wait runs out, the
// thread records a status word the way the library's kernels do, and the kernel returns: nothing hangs and the
// context stays usable.
#include "tcgen05.cuh"

namespace {
__global__ void wait_that_runs_out(int* status, long long* cycles) {
  __shared__ uint64_t bar;
  if (threadIdx.x == 0) {
    tc5::mbar_init(&bar, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    long long begin = clock64();
    bool completed = tc5::mbar_wait(&bar, 0);
    *cycles = clock64() - begin;
    if (!completed) *(volatile int*)status = 3;  // the tile product's code for "operands never arrived"
  }
}
}  // namespace

// The limit this file was built with, so the test can see that its flag took effect.
DLLM_EXPORT long long probe_wait_limit() { return tc5::WAIT_LIMIT_CYCLES; }

DLLM_EXPORT int probe_wait_that_runs_out(int* status, long long* cycles, cudaStream_t stream) {
  wait_that_runs_out<<<1, 32, 0, stream>>>(status, cycles);
  return dllm_launch_status();
}
