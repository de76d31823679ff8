// The weight update inside INQAffine / INQConvolution (incremental network quantization,
// src/nbla/function/generic/inq_affine.cpp:82-203): weights that were fixed keep their value, and every
// fixed weight is snapped to a power of two inside a window below the largest magnitude, or pruned to zero.
//
//   restore  (:101-105)  w[i] = old_w[i] where old_indicator[i] == 1
//   select   (:108-148)  at the iterations the user lists, half of the still learnable weights become fixed
//                        (largest magnitude first, or a Bernoulli draw each); the caller does this step,
//                        it is a sort or a random stream a few times per training run
//   quantize (:150-203)  n1 from max |w|, n2 = n1 + 1 - 2^(bits - 2); fixed weights below 2^(n2 - 1) become 0,
//                        the others sign * 2^e with e = floor(log2 |w|) + (frac >= log2 1.5) clipped to
//                        [n2, n1]; weights and indicators are copied to the function's state.
//
// The exponent rule is written with the host's log2f in the reference, and its result at a mantissa of
// 1.5 depends on how that logarithm rounds in each binade. As for Pow2Quantize, the library therefore asks
// the host libm once where the step lies in every binade (bisection, monotonicity checked around the step)
// and the kernel compares mantissa bits with that table; if the libm does not behave as one step per binade
// the entry point refuses to run.
#include <cmath>
#include <cstdio>
#include <mutex>

#include "common.cuh"

namespace nb200 {
namespace {

constexpr int kThreads = 256;
constexpr int kMinExp = -149, kNumBinades = 127 - kMinExp + 1;

// mantissa bits (left-aligned to 23) above which the exponent is e + 1, for the two ways the reference writes
// the rule: [0] for the weights (inq_affine.cpp:173-177, the threshold is a float variable), [1] for the largest
// magnitude (:152-154, the threshold is the double std::log2(1.5)); they differ exactly at 1.5 * 2^e
struct InqTables {
  uint32_t cut[2][kNumBinades];
};

inline int host_inq_exponent(float a, int of_max) {
  const float b = log2f(a);
  if (of_max)
    return (int)(std::floor(b) + ((b - std::floor(b)) >= std::log2(1.5)));
  const float d = 0.58496250072115619;
  return (int)(std::floor(b) + ((b - std::floor(b)) >= d));
}
// the value of binade e (p fraction bits) with fraction f
inline float binade_value(int e, int p, uint32_t f) { return ldexpf((float)((1u << p) + f), e - p); }

bool build_inq_tables(InqTables *T, char *why, size_t why_len) {
  for (int which = 0; which < 2; ++which)
  for (int e = kMinExp; e <= 127; ++e) {
    const int p = (e >= -126) ? 23 : e + 149;
    const uint32_t fmax = (p == 0) ? 0u : ((1u << p) - 1u);
    if (host_inq_exponent(binade_value(e, p, 0), which) != e) {
      snprintf(why, why_len, "libm: the INQ exponent of 2^%d is not %d", e, e);
      return false;
    }
    uint32_t lo = 0, hi = fmax;
    if (host_inq_exponent(binade_value(e, p, fmax), which) == e) {
      lo = fmax; // no step inside this binade
    } else {
      if (host_inq_exponent(binade_value(e, p, fmax), which) != e + 1) {
        snprintf(why, why_len, "libm: unexpected INQ exponent at the top of binade %d", e);
        return false;
      }
      while (hi - lo > 1) {
        const uint32_t mid = lo + (hi - lo) / 2;
        if (host_inq_exponent(binade_value(e, p, mid), which) == e)
          lo = mid;
        else
          hi = mid;
      }
      for (int d = -64; d <= 64; ++d) {
        const int64_t f = (int64_t)lo + d;
        if (f < 0 || f > (int64_t)fmax)
          continue;
        if (host_inq_exponent(binade_value(e, p, (uint32_t)f), which) != (f <= (int64_t)lo ? e : e + 1)) {
          snprintf(why, why_len, "libm: log2f is not monotone around the INQ step of binade %d", e);
          return false;
        }
      }
    }
    T->cut[which][e - kMinExp] = lo << (23 - p);
  }
  return true;
}

std::mutex g_inq_mutex;
InqTables g_inq_host;
int g_inq_state = 0; // 0 = not built, 1 = ok, -1 = unusable
char g_inq_why[160];
InqTables *g_inq_dev[64];

int inq_tables_for_current_device(const InqTables **out) {
  int dev = 0;
  NB_CUDA(cudaGetDevice(&dev));
  NB_CHECK(dev >= 0 && dev < 64, NB200_EVALUE, "device index %d out of range", dev);
  std::lock_guard<std::mutex> lock(g_inq_mutex);
  if (g_inq_state == 0)
    g_inq_state = build_inq_tables(&g_inq_host, g_inq_why, sizeof(g_inq_why)) ? 1 : -1;
  NB_CHECK(g_inq_state == 1, NB200_ENOTIMPL, "INQ: cannot reproduce the host libm (%s)", g_inq_why);
  if (g_inq_dev[dev] == nullptr) {
    NB_CUDA(cudaMalloc(&g_inq_dev[dev], sizeof(InqTables)));
    NB_CUDA(cudaMemcpy(g_inq_dev[dev], &g_inq_host, sizeof(InqTables), cudaMemcpyHostToDevice));
  }
  *out = g_inq_dev[dev];
  return NB200_OK;
}

// the reference's exponent of a finite a > 0
__device__ __forceinline__ int inq_exponent(float a, const uint32_t *cut) {
  const uint32_t bits = __float_as_uint(a);
  const uint32_t E = bits >> 23;
  uint32_t frac = bits & 0x7fffffu;
  int e;
  if (E == 0u) {
    const int p = 31 - __clz(frac);
    e = p - 149;
    frac = (frac << (23 - p)) & 0x7fffffu;
  } else {
    e = (int)E - 127;
  }
  return e + (frac > cut[e - kMinExp] ? 1 : 0);
}

__global__ void __launch_bounds__(kThreads) inq_restore_kernel(float *__restrict__ w, const float *__restrict__ old_w,
                                                               const int32_t *__restrict__ old_ind, size_t n) {
  const size_t stride = (size_t)gridDim.x * kThreads;
  for (size_t i = (size_t)blockIdx.x * kThreads + threadIdx.x; i < n; i += stride)
    if (old_ind[i] == 1)
      w[i] = old_w[i];
}

__global__ void __launch_bounds__(kThreads) inq_absmax_kernel(const float *__restrict__ w, size_t n,
                                                              uint32_t *__restrict__ maxbits) {
  uint32_t m = 0;
  const size_t stride = (size_t)gridDim.x * kThreads;
  for (size_t i = (size_t)blockIdx.x * kThreads + threadIdx.x; i < n; i += stride) {
    const float a = fabsf(w[i]);
    if (a > __uint_as_float(m)) // the reference's strict compare: a NaN never becomes the maximum
      m = __float_as_uint(a);
  }
  m = __reduce_max_sync(0xffffffffu, m);
  if ((threadIdx.x & 31) == 0 && m != 0)
    atomicMax(maxbits, m);
}

__global__ void __launch_bounds__(kThreads)
    inq_quantize_kernel(float *__restrict__ w, int32_t *__restrict__ ind, float *__restrict__ old_w,
                        int32_t *__restrict__ old_ind, size_t n, int num_bits, int fix_all,
                        const InqTables *__restrict__ tables, const uint32_t *__restrict__ maxbits) {
  __shared__ uint32_t s_cut[kNumBinades], s_cut_max[kNumBinades];
  for (int t = threadIdx.x; t < kNumBinades; t += kThreads) {
    s_cut[t] = tables->cut[0][t];
    s_cut_max[t] = tables->cut[1][t];
  }
  __syncthreads();
  float max_absval = __uint_as_float(*maxbits);
  if (max_absval == 0.0f)
    max_absval = 1.0f;
  // an infinite maximum: log2f gives +inf and the reference's conversion to int is undefined; 128 here
  const int n1 = max_absval > 3.4028234e38f ? 128 : inq_exponent(max_absval, s_cut_max);
  const int window = num_bits >= 2 ? (num_bits - 2 < 30 ? 1 << (num_bits - 2) : 1 << 30) : 0; // (int)pow(2, bits - 2)
  const int n2 = n1 + 1 - window;
  const float threshold = ldexpf(1.0f, n2 - 1); // (float)pow(2, n2 - 1)
  const size_t stride = (size_t)gridDim.x * kThreads;
  for (size_t i = (size_t)blockIdx.x * kThreads + threadIdx.x; i < n; i += stride) {
    const int fixed = fix_all ? 1 : ind[i];
    float v = w[i];
    if (fixed == 1) {
      const float a = fabsf(v);
      if (a < threshold) {
        v = 0.0f;
      } else if (a <= 3.4028234e38f) {
        int e = a > 0.0f ? inq_exponent(a, s_cut) : n2;
        e = e > n1 ? n1 : e;
        e = e < n2 ? n2 : e;
        v = ldexpf(v < 0.0f ? -1.0f : 1.0f, e);
      } else if (a == a) {
        v = ldexpf(v < 0.0f ? -1.0f : 1.0f, n1); // infinite weight: the largest power of the window
      }
      w[i] = v;
    }
    if (fix_all)
      ind[i] = 1;
    old_w[i] = v;
    old_ind[i] = fixed;
  }
}

inline unsigned grid_for(size_t n) {
  size_t b = (n + kThreads - 1) / kThreads;
  const size_t cap = (size_t)sm_count() * 16;
  return (unsigned)(b < 1 ? 1 : (b > cap ? cap : b));
}

} // namespace
} // namespace nb200

using namespace nb200;

extern "C" {

int nb200_inq_restore_f32(float *weights, const float *old_weights, const int32_t *old_indicators, size_t size,
                          void *stream) {
  if (size == 0)
    return NB200_OK;
  NB_CHECK(weights && old_weights && old_indicators, NB200_EVALUE, "null data pointer");
  inq_restore_kernel<<<grid_for(size), kThreads, 0, as_stream(stream)>>>(weights, old_weights, old_indicators, size);
  NB_LAUNCH_CHECK();
  return NB200_OK;
}

int nb200_inq_quantize_f32(float *weights, int32_t *indicators, float *old_weights, int32_t *old_indicators,
                           size_t size, int num_bits, int fix_all, void *stream) {
  if (size == 0)
    return NB200_OK;
  NB_CHECK(weights && indicators && old_weights && old_indicators, NB200_EVALUE, "null data pointer");
  NB_CHECK(num_bits >= 0 && num_bits <= 32, NB200_EVALUE, "num_bits out of range");
  const InqTables *tables = nullptr;
  NB_TRY(inq_tables_for_current_device(&tables));
  cudaStream_t st = as_stream(stream);
  AsyncScratch scratch(st);
  NB_TRY(scratch.alloc(256));
  uint32_t *maxbits = static_cast<uint32_t *>(scratch.p);
  NB_CUDA(cudaMemsetAsync(maxbits, 0, 4, st));
  inq_absmax_kernel<<<grid_for(size), kThreads, 0, st>>>(weights, size, maxbits);
  NB_LAUNCH_CHECK();
  inq_quantize_kernel<<<grid_for(size), kThreads, 0, st>>>(weights, indicators, old_weights, old_indicators, size,
                                                           num_bits, fix_all, tables, maxbits);
  NB_LAUNCH_CHECK();
  return NB200_OK;
}

} // extern "C"
