// Runtime entry points of the C ABI: error reporting, device selection,
// memory, copies, streams. These are what nnabla's backend layer (Memory,
// Array synchronizers, BackendBase) needs from a device; see the citations in
// include/nnabla_b200.h.
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <string>

#include "common.cuh"

namespace nb200 {

static thread_local std::string g_error;

int fail(int code, const char *fmt, ...) {
  char buf[1024];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof(buf), fmt, ap);
  va_end(ap);
  g_error = buf;
  return code;
}

void clear_error() { g_error.clear(); }

int sm_count() {
  static int cached[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64)
    return 148;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
      n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

int scratch_alloc(void **p, size_t bytes, cudaStream_t st) {
  static std::mutex m;
  static bool pool_ready[64];
  int dev = 0;
  NB_CUDA(cudaGetDevice(&dev));
  NB_CHECK(dev >= 0 && dev < 64, NB200_EVALUE, "device index %d out of range", dev);
  {
    std::lock_guard<std::mutex> lock(m);
    if (!pool_ready[dev]) {
      cudaMemPool_t pool;
      NB_CUDA(cudaDeviceGetDefaultMemPool(&pool, dev));
      uint64_t keep = UINT64_MAX;
      NB_CUDA(cudaMemPoolSetAttribute(pool, cudaMemPoolAttrReleaseThreshold, &keep));
      pool_ready[dev] = true;
    }
  }
  cudaError_t e = cudaMallocAsync(p, bytes ? bytes : 1, st);
  if (e == cudaErrorMemoryAllocation) {
    cudaGetLastError();
    return fail(NB200_EMEMORY, "stream-ordered allocation of %zu bytes of scratch failed: out of device memory", bytes);
  }
  NB_CUDA(e);
  return NB200_OK;
}

// ---- host pipeline ---------------------------------------------------------

namespace {
constexpr int kSlots = 4;
constexpr size_t kChunkElems = size_t(16) << 20; // 64 MiB of fp32 per chunk

struct PipeState {
  bool ready = false;
  cudaStream_t st[kSlots];
  float *dx[kSlots];
  float *dy[kSlots];
};
std::mutex g_pipe_mutex;
PipeState g_pipe[64];
} // namespace

int host_pipeline(const float *hx, float *hy, size_t n, chunk_fn fn, void *user) {
  if (n == 0)
    return NB200_OK;
  int dev = 0;
  NB_CUDA(cudaGetDevice(&dev));
  NB_CHECK(dev >= 0 && dev < 64, NB200_EVALUE, "device index %d out of range", dev);
  // One pipeline per device; calls on the same device are serialised.
  std::lock_guard<std::mutex> lock(g_pipe_mutex);
  PipeState &p = g_pipe[dev];
  if (!p.ready) {
    for (int s = 0; s < kSlots; ++s) {
      NB_CUDA(cudaStreamCreateWithFlags(&p.st[s], cudaStreamNonBlocking));
      NB_CUDA(cudaMalloc(&p.dx[s], kChunkElems * sizeof(float)));
      NB_CUDA(cudaMalloc(&p.dy[s], kChunkElems * sizeof(float)));
    }
    p.ready = true;
  }
  size_t off = 0;
  for (int c = 0; off < n; ++c) {
    const int s = c % kSlots;
    const size_t cnt = (n - off < kChunkElems) ? (n - off) : kChunkElems;
    NB_CUDA(cudaMemcpyAsync(p.dx[s], hx + off, cnt * sizeof(float), cudaMemcpyHostToDevice, p.st[s]));
    NB_TRY(fn(p.dx[s], p.dy[s], cnt, off, p.st[s], user));
    NB_CUDA(cudaMemcpyAsync(hy + off, p.dy[s], cnt * sizeof(float), cudaMemcpyDeviceToHost, p.st[s]));
    off += cnt;
  }
  for (int s = 0; s < kSlots; ++s)
    NB_CUDA(cudaStreamSynchronize(p.st[s]));
  return NB200_OK;
}

__global__ void fill_kernel(float *p, size_t n, float v) {
  size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (; i < n; i += stride)
    p[i] = v;
}

} // namespace nb200

using namespace nb200;

extern "C" {

const char *nb200_last_error(void) { return g_error.c_str(); }

int nb200_abi_version(void) { return 1; }

int nb200_device_count(int *count) {
  NB_CHECK(count != nullptr, NB200_EVALUE, "count is NULL");
  NB_CUDA(cudaGetDeviceCount(count));
  return NB200_OK;
}

int nb200_set_device(int device) {
  NB_CUDA(cudaSetDevice(device));
  return NB200_OK;
}

int nb200_get_device(int *device) {
  NB_CHECK(device != nullptr, NB200_EVALUE, "device is NULL");
  NB_CUDA(cudaGetDevice(device));
  return NB200_OK;
}

int nb200_check_device(void) {
  int dev = 0, major = 0;
  NB_CUDA(cudaGetDevice(&dev));
  NB_CUDA(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev));
  NB_CHECK(major == 10, NB200_ENOTIMPL,
           "device %d has compute capability %d.x; this library is built for sm_100a only and has no fallback",
           dev, major);
  return NB200_OK;
}

int nb200_malloc(void **dev_ptr, size_t bytes) {
  NB_CHECK(dev_ptr != nullptr, NB200_EVALUE, "dev_ptr is NULL");
  *dev_ptr = nullptr;
  if (bytes == 0)
    return NB200_OK;
  cudaError_t e = cudaMalloc(dev_ptr, bytes);
  if (e == cudaErrorMemoryAllocation) {
    cudaGetLastError();
    return fail(NB200_EMEMORY, "cudaMalloc of %zu bytes failed: out of device memory", bytes);
  }
  NB_CUDA(e);
  return NB200_OK;
}

int nb200_free(void *dev_ptr) {
  if (dev_ptr)
    NB_CUDA(cudaFree(dev_ptr));
  return NB200_OK;
}

static_assert(sizeof(cudaIpcMemHandle_t) == NB200_IPC_HANDLE_BYTES, "handle size of the C ABI");

int nb200_ipc_export(const void *dev_ptr, void *handle) {
  NB_CHECK(dev_ptr != nullptr && handle != nullptr, NB200_EVALUE, "null pointer");
  cudaIpcMemHandle_t h;
  NB_CUDA(cudaIpcGetMemHandle(&h, const_cast<void *>(dev_ptr)));
  std::memcpy(handle, &h, sizeof(h));
  return NB200_OK;
}

int nb200_ipc_open(const void *handle, void **peer_ptr) {
  NB_CHECK(handle != nullptr && peer_ptr != nullptr, NB200_EVALUE, "null pointer");
  *peer_ptr = nullptr;
  cudaIpcMemHandle_t h;
  std::memcpy(&h, handle, sizeof(h));
  NB_CUDA(cudaIpcOpenMemHandle(peer_ptr, h, cudaIpcMemLazyEnablePeerAccess));
  return NB200_OK;
}

int nb200_ipc_close(void *peer_ptr) {
  if (peer_ptr)
    NB_CUDA(cudaIpcCloseMemHandle(peer_ptr));
  return NB200_OK;
}

int nb200_malloc_host(void **host_ptr, size_t bytes) {
  NB_CHECK(host_ptr != nullptr, NB200_EVALUE, "host_ptr is NULL");
  *host_ptr = nullptr;
  if (bytes == 0)
    return NB200_OK;
  cudaError_t e = cudaMallocHost(host_ptr, bytes);
  if (e == cudaErrorMemoryAllocation) {
    cudaGetLastError();
    return fail(NB200_EMEMORY, "cudaMallocHost of %zu bytes failed", bytes);
  }
  NB_CUDA(e);
  return NB200_OK;
}

int nb200_free_host(void *host_ptr) {
  if (host_ptr)
    NB_CUDA(cudaFreeHost(host_ptr));
  return NB200_OK;
}

int nb200_memcpy_h2d(void *dev_dst, const void *host_src, size_t bytes, void *stream) {
  if (bytes)
    NB_CUDA(cudaMemcpyAsync(dev_dst, host_src, bytes, cudaMemcpyHostToDevice, as_stream(stream)));
  return NB200_OK;
}

int nb200_memcpy_d2h(void *host_dst, const void *dev_src, size_t bytes, void *stream) {
  if (bytes)
    NB_CUDA(cudaMemcpyAsync(host_dst, dev_src, bytes, cudaMemcpyDeviceToHost, as_stream(stream)));
  return NB200_OK;
}

int nb200_memcpy_d2d(void *dev_dst, const void *dev_src, size_t bytes, void *stream) {
  if (bytes)
    NB_CUDA(cudaMemcpyAsync(dev_dst, dev_src, bytes, cudaMemcpyDeviceToDevice, as_stream(stream)));
  return NB200_OK;
}

int nb200_memset_zero(void *dev_ptr, size_t bytes, void *stream) {
  if (bytes)
    NB_CUDA(cudaMemsetAsync(dev_ptr, 0, bytes, as_stream(stream)));
  return NB200_OK;
}

int nb200_fill_f32(float *dev_ptr, size_t n, float value, void *stream) {
  if (n == 0)
    return NB200_OK;
  if (value == 0.0f) {
    NB_CUDA(cudaMemsetAsync(dev_ptr, 0, n * sizeof(float), as_stream(stream)));
    return NB200_OK;
  }
  size_t blocks = (n + 255) / 256;
  const size_t cap = (size_t)sm_count() * 16;
  if (blocks > cap)
    blocks = cap;
  fill_kernel<<<(unsigned)blocks, 256, 0, as_stream(stream)>>>(dev_ptr, n, value);
  NB_LAUNCH_CHECK();
  return NB200_OK;
}

int nb200_stream_create(void **stream) {
  NB_CHECK(stream != nullptr, NB200_EVALUE, "stream is NULL");
  cudaStream_t s;
  NB_CUDA(cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking));
  *stream = s;
  return NB200_OK;
}

int nb200_stream_destroy(void *stream) {
  if (stream)
    NB_CUDA(cudaStreamDestroy(as_stream(stream)));
  return NB200_OK;
}

int nb200_stream_synchronize(void *stream) {
  NB_CUDA(cudaStreamSynchronize(as_stream(stream)));
  return NB200_OK;
}

int nb200_scratch_pool_stats(int64_t *used_now, int64_t *used_high, int reset_high) {
  int dev = 0;
  NB_CUDA(cudaGetDevice(&dev));
  cudaMemPool_t pool;
  NB_CUDA(cudaDeviceGetDefaultMemPool(&pool, dev));
  uint64_t v = 0;
  if (reset_high) {
    NB_CUDA(cudaMemPoolSetAttribute(pool, cudaMemPoolAttrUsedMemHigh, &v)); // the watermark can only be set to 0
  }
  if (used_now) {
    NB_CUDA(cudaMemPoolGetAttribute(pool, cudaMemPoolAttrUsedMemCurrent, &v));
    *used_now = (int64_t)v;
  }
  if (used_high) {
    NB_CUDA(cudaMemPoolGetAttribute(pool, cudaMemPoolAttrUsedMemHigh, &v));
    *used_high = (int64_t)v;
  }
  return NB200_OK;
}

int nb200_device_synchronize(void) {
  NB_CUDA(cudaDeviceSynchronize());
  return NB200_OK;
}
}
