// Programmatic dependent launch: a kernel launched with launch_dependent() may be scheduled while the
// kernel before it in the stream is still draining; its blocks become resident as that kernel's blocks
// retire and stop at pdl_wait() until the predecessor has completed and its writes are visible. At a few
// dozen images per GPU a network is a chain of kernels of a few microseconds each, and the gap between two
// kernels (launch processing, grid start) is a large part of the step; this hides most of it.
//
// Rules that keep it correct: (1) every kernel launched this way executes pdl_wait() as its first
// statement, in every thread, before any global-memory access (so its completion implies the
// predecessor's, and ordering stays transitive along the stream); (2) pdl_trigger() only says "my
// successor may be scheduled", it orders nothing. Kernels launched the ordinary way in between serialize
// fully, as before. NNABLA_B200_PDL=0 turns the attribute off (ordinary launches; the waits are no-ops).
#pragma once
#include <cuda_runtime.h>

#include <cstdlib>

namespace nb200 {

__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

inline bool pdl_enabled() {
  static const bool on = []() {
    const char *e = std::getenv("NNABLA_B200_PDL");
    return !(e && e[0] == '0');
  }();
  return on;
}

template <typename... KArgs, typename... Args>
inline cudaError_t launch_dependent(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st,
                                    Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

} // namespace nb200
