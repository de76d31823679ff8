// Self-test of the bounded device-side waits.
//
// Every mbarrier wait of the contraction kernels gives up after a time limit,
// records a code in the per-device status word, raises its CTA's abort flag
// and lets all roles fall through to the teardown (ptx::mbar_wait, gemm.cuh).
// That path only runs when something is wrong, so this entry point runs it on
// purpose in the one harmless way there is: a one-block kernel whose barrier
// nobody ever arrives at, with a limit of the caller's choosing (a millisecond
// or so). Nothing traps, nothing faults, the kernel returns by itself and the
// context stays usable; the host then reads the code with
// nb200_take_device_status exactly as after a real contraction.
#include "gemm.cuh"

namespace nb200 {
namespace {

__global__ void __launch_bounds__(64) wait_timeout_kernel(uint64_t limit_ns, int *status, int *observed) {
  __shared__ uint64_t bar;
  __shared__ int abort_word;
  volatile int *abort_flag = &abort_word;
  if (threadIdx.x == 0) {
    ptx::mbar_init(&bar, 1);
    abort_word = 0;
    ptx::mbar_fence_init();
  }
  __syncthreads();
  const int warp = threadIdx.x >> 5;
  if (warp == 0) {
    // the role that gives up first: same bookkeeping as the producer of the contraction kernel
    if (ptx::elect_one()) {
      if (!ptx::mbar_wait(&bar, 0u, abort_flag, limit_ns)) {
        if (*abort_flag == 0)
          atomicCAS(status, 0, kStatusProducerTimeout);
        *abort_flag = 1;
      }
    }
  } else {
    // a second role with a much longer limit: it must leave because of the abort flag, not its own clock
    const uint64_t t0 = ptx::globaltimer_ns();
    const bool got = ptx::mbar_wait_backoff(&bar, 0u, abort_flag, 200, limit_ns * 1000ull + 1000000000ull);
    if (threadIdx.x == 32) {
      observed[0] = got ? 1 : 0;
      observed[1] = (int)((ptx::globaltimer_ns() - t0) / 1000ull); // microseconds until it left
    }
  }
  __syncthreads();
}

} // namespace
} // namespace nb200

using namespace nb200;

extern "C" int nb200_selftest_wait_timeout(int limit_us, int *waited_us, void *stream) {
  NB_CHECK(limit_us > 0 && limit_us <= 100000, NB200_EVALUE, "limit_us must be in 1..100000 (got %d)", limit_us);
  int *status = nullptr;
  NB_TRY(device_status_word(&status));
  cudaStream_t st = as_stream(stream);
  AsyncScratch scratch(st);
  NB_TRY(scratch.alloc(2 * sizeof(int)));
  int *observed = static_cast<int *>(scratch.p);
  NB_CUDA(cudaMemsetAsync(observed, 0xff, 2 * sizeof(int), st));
  wait_timeout_kernel<<<1, 64, 0, st>>>((uint64_t)limit_us * 1000ull, status, observed);
  NB_LAUNCH_CHECK();
  int host[2] = {-1, -1};
  NB_CUDA(cudaMemcpyAsync(host, observed, sizeof(host), cudaMemcpyDeviceToHost, st));
  NB_CUDA(cudaStreamSynchronize(st));
  NB_CHECK(host[0] == 0, NB200_ECUDA, "the second role did not leave through the abort flag (observed %d)", host[0]);
  if (waited_us)
    *waited_us = host[1];
  return NB200_OK;
}
