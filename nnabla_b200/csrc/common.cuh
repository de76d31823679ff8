// Shared host/device helpers of the nnabla_b200 library (sm_100a only).
#pragma once
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

#include "nnabla_b200.h"

namespace nb200 {

// Records a message for nb200_last_error() on this thread and returns `code`.
int fail(int code, const char *fmt, ...) __attribute__((format(printf, 2, 3)));
void clear_error();

// Number of SMs of the current device (cached per device).
int sm_count();

inline cudaStream_t as_stream(void *s) { return reinterpret_cast<cudaStream_t>(s); }

#define NB_CUDA(expr)                                                                              \
  do {                                                                                             \
    cudaError_t nb_e_ = (expr);                                                                    \
    if (nb_e_ != cudaSuccess)                                                                      \
      return ::nb200::fail(NB200_ECUDA, "%s: %s (%s:%d)", #expr, cudaGetErrorString(nb_e_),        \
                           __FILE__, __LINE__);                                                    \
  } while (0)

#define NB_CHECK(cond, code, ...)                                                                  \
  do {                                                                                             \
    if (!(cond))                                                                                   \
      return ::nb200::fail(code, __VA_ARGS__);                                                     \
  } while (0)

#define NB_TRY(expr)                                                                               \
  do {                                                                                             \
    int nb_rc_ = (expr);                                                                           \
    if (nb_rc_ != NB200_OK)                                                                        \
      return nb_rc_;                                                                               \
  } while (0)

// Launch-error check that does not synchronise.
#define NB_LAUNCH_CHECK() NB_CUDA(cudaGetLastError())

// Streaming (evict-first) 128-bit global accesses for data touched once.
__device__ __forceinline__ float4 ld_stream(const float4 *p) { return __ldcs(p); }
__device__ __forceinline__ void st_stream(float4 *p, float4 v) { __stcs(p, v); }

// Channel of a grid-stride walker over an [outer, C, S] tensor (item i belongs
// to channel (i / S) % C): two 64-bit divisions when the walk starts, additions
// afterwards (a 64-bit division per item costs more than the item's arithmetic).
struct ChannelWalk {
  unsigned off, c, ds, dc, S, C;
  __device__ __forceinline__ ChannelWalk(size_t first, size_t stride, unsigned S_, unsigned C_) : S(S_), C(C_) {
    const size_t plane = first / S_, dplane = stride / S_;
    off = (unsigned)(first - plane * S_);
    c = (unsigned)(plane % C_);
    ds = (unsigned)(stride - dplane * S_);
    dc = (unsigned)(dplane % C_);
  }
  __device__ __forceinline__ void next() {
    off += ds;
    const unsigned carry = off >= S ? 1u : 0u;
    off -= carry ? S : 0u;
    c += dc + carry;
    c -= c >= C ? C : 0u;
  }
};

// Stream-ordered scratch for one call: allocated from the device's default
// memory pool (whose release threshold is raised on first use so that the pool
// keeps its memory across synchronisations instead of returning it to the
// driver), freed in stream order when the object goes out of scope.
int scratch_alloc(void **p, size_t bytes, cudaStream_t st);
struct AsyncScratch {
  void *p = nullptr;
  cudaStream_t st;
  explicit AsyncScratch(cudaStream_t s) : st(s) {}
  AsyncScratch(const AsyncScratch &) = delete;
  AsyncScratch &operator=(const AsyncScratch &) = delete;
  int alloc(size_t bytes) { return scratch_alloc(&p, bytes, st); }
  ~AsyncScratch() {
    if (p)
      cudaFreeAsync(p, st);
  }
};

// Host-buffer pipeline shared by the _host entry points: copies `n` floats
// from hx to the device in chunks, runs `launch(dx, dy, count, offset, stream)`
// on each chunk and copies the result to hy, overlapping the three stages
// across chunks. Returns after hy is complete.
typedef int (*chunk_fn)(const float *dx, float *dy, size_t count, size_t offset, cudaStream_t st, void *user);
int host_pipeline(const float *hx, float *hy, size_t n, chunk_fn fn, void *user);

} // namespace nb200
