// Training side of the companion functions of a binary-weight ResNet:
// batch-statistics BatchNormalization (forward), and the backward passes of
// BatchNormalization, ReLU, Add2, MaxPooling and GlobalAveragePooling.
//
// The elementwise parts follow the reference's operation order, every operation
// rounded separately, so that given the same per-channel statistics the results
// are bit-identical to its CPU code. The per-channel SUMS (batch mean and
// variance, parameter gradients) are block partials added in a fixed order in
// double precision: deterministic, and closer to the exact sums than the
// reference's sequential fp32 accumulation, so those agree to rounding only.
#include <cmath>

#include "common.cuh"

namespace nb200 {
namespace {

constexpr int kThreads = 256;

inline unsigned grid_for(size_t items, int per_thread = 1) {
  size_t b = (items + (size_t)kThreads * per_thread - 1) / ((size_t)kThreads * per_thread);
  const size_t cap = (size_t)sm_count() * 64;
  if (b > cap)
    b = cap;
  return (unsigned)(b < 1 ? 1 : b);
}

// ---------------------------------------------------------------- elementwise backward passes

// relu.cpp:41-49: dx (+)= y > 0 ? dy : 0; add2.cpp: dx (+)= dy.
template <int kOp, bool kAccum>
__global__ void __launch_bounds__(kThreads) grad_pass_kernel(const float *__restrict__ y, const float *__restrict__ dy,
                                                             float *__restrict__ dx, size_t total, bool vec) {
  const size_t stride = (size_t)gridDim.x * kThreads;
  const size_t first = (size_t)blockIdx.x * kThreads + threadIdx.x;
  auto one = [](float yv, float g, float old) {
    const float v = kOp == 0 ? (yv > 0.0f ? g : 0.0f) : g;
    return kAccum ? __fadd_rn(old, v) : v;
  };
  const size_t total4 = vec ? total / 4 : 0;
  for (size_t i = first; i < total4; i += stride) {
    const float4 g = __ldcs(reinterpret_cast<const float4 *>(dy) + i);
    float4 yv = make_float4(0, 0, 0, 0), o = make_float4(0, 0, 0, 0);
    if (kOp == 0)
      yv = __ldcs(reinterpret_cast<const float4 *>(y) + i);
    if (kAccum)
      o = reinterpret_cast<const float4 *>(dx)[i];
    reinterpret_cast<float4 *>(dx)[i] = make_float4(one(yv.x, g.x, o.x), one(yv.y, g.y, o.y), one(yv.z, g.z, o.z),
                                                    one(yv.w, g.w, o.w));
  }
  for (size_t i = total4 * 4 + first; i < total; i += stride)
    dx[i] = one(kOp == 0 ? y[i] : 0.0f, dy[i], kAccum ? dx[i] : 0.0f);
}

// global_average_pooling.cpp:75-117: every pixel of map m receives dy[m] / (H W).
template <bool kAccum>
__global__ void __launch_bounds__(kThreads) gap_backward_kernel(const float *__restrict__ dy, float *__restrict__ dx,
                                                                size_t total, unsigned S) {
  const size_t stride = (size_t)gridDim.x * kThreads;
  for (size_t i = (size_t)blockIdx.x * kThreads + threadIdx.x; i < total; i += stride) {
    const float g = __fdiv_rn(__ldg(dy + i / S), (float)S);
    dx[i] = kAccum ? __fadd_rn(dx[i], g) : g;
  }
}

// max_pooling.cpp:44-77, :134-139, :194-228. The reference stores the index of the first maximum of
// every clipped window and then runs dx[index] += dy over the outputs in order. Two passes here: the
// first writes that index map (one thread per output, the reference's scan with its strict compare);
// in the second every INPUT pixel walks the windows that contain it in ascending output order and adds
// dy of those whose index is its own: the same additions in the same order, without atomics.
__global__ void __launch_bounds__(kThreads)
    max_pooling_index_kernel(const float *__restrict__ x, int *__restrict__ index, size_t outputs, int H, int W,
                             int Ho, int Wo, int kh, int kw, int sh, int sw, int ph, int pw) {
  const size_t stride = (size_t)gridDim.x * kThreads;
  for (size_t o = (size_t)blockIdx.x * kThreads + threadIdx.x; o < outputs; o += stride) {
    const int ox = (int)(o % Wo);
    const size_t t = o / Wo;
    const int oy = (int)(t % Ho);
    const float *xm = x + (t / Ho) * H * W;
    int y0 = oy * sh - ph, x0 = ox * sw - pw;
    const int y1 = min(y0 + kh, H), x1 = min(x0 + kw, W);
    y0 = max(y0, 0);
    x0 = max(x0, 0);
    int best_i = y0 * W + x0;
    float best = __ldg(xm + best_i);
    for (int yy = y0; yy < y1; ++yy)
      for (int xx = x0; xx < x1; ++xx) {
        const float v = __ldg(xm + yy * W + xx);
        if (best < v) {
          best = v;
          best_i = yy * W + xx;
        }
      }
    index[o] = best_i;
  }
}

template <bool kAccum>
__global__ void __launch_bounds__(kThreads)
    max_pooling_backward_kernel(const int *__restrict__ index, const float *__restrict__ dy, float *__restrict__ dx,
                                size_t total, int H, int W, int Ho, int Wo, int kh, int kw, int sh, int sw, int ph,
                                int pw) {
  const size_t stride = (size_t)gridDim.x * kThreads;
  for (size_t i = (size_t)blockIdx.x * kThreads + threadIdx.x; i < total; i += stride) {
    const int ix = (int)(i % W);
    const size_t t = i / W;
    const int iy = (int)(t % H);
    const size_t m = t / H;
    const int *im = index + m * Ho * Wo;
    const float *dym = dy + m * Ho * Wo;
    float acc = kAccum ? dx[i] : 0.0f;
    // windows oy with oy * sh - ph <= iy < oy * sh - ph + kh
    int oy0 = iy + ph - kh + 1;
    oy0 = oy0 <= 0 ? 0 : (oy0 + sh - 1) / sh;
    int oy1 = (iy + ph) / sh;
    oy1 = oy1 < Ho - 1 ? oy1 : Ho - 1;
    int ox0 = ix + pw - kw + 1;
    ox0 = ox0 <= 0 ? 0 : (ox0 + sw - 1) / sw;
    int ox1 = (ix + pw) / sw;
    ox1 = ox1 < Wo - 1 ? ox1 : Wo - 1;
    const int mine = iy * W + ix;
    for (int oy = oy0; oy <= oy1; ++oy)
      for (int ox = ox0; ox <= ox1; ++ox)
        if (__ldg(im + oy * Wo + ox) == mine)
          acc = __fadd_rn(acc, __ldg(dym + oy * Wo + ox));
    dx[i] = acc;
  }
}

// ---------------------------------------------------------------- per-channel sums

// Walks the values of channel c of an [N, C, S] tensor: item j of the channel (j = n * S + s, counted in
// units of kW values) lives at ((n * C + c) * S + s). Start and step are split once; no division per item.
struct ChannelItems {
  unsigned n, s, dn, ds, S, N;
  __device__ __forceinline__ ChannelItems(size_t first, size_t step, unsigned S_, unsigned N_) : S(S_), N(N_) {
    n = (unsigned)(first / S_);
    s = (unsigned)(first - (size_t)n * S_);
    dn = (unsigned)(step / S_);
    ds = (unsigned)(step - (size_t)dn * S_);
  }
  __device__ __forceinline__ bool valid() const { return n < N; }
  __device__ __forceinline__ void next() {
    s += ds;
    const unsigned carry = s >= S ? 1u : 0u;
    s -= carry ? S : 0u;
    n += dn + carry;
  }
};

// (v)^-0.5 and (v)^-1.5 rounded from double precision: what a correctly rounded powf returns
__device__ __forceinline__ float inv_sqrt_rn(float v) { return (float)(1.0 / sqrt((double)v)); }
__device__ __forceinline__ float inv_sqrt_cubed_rn(float v) { return (float)(1.0 / ((double)v * sqrt((double)v))); }

template <int K> __device__ __forceinline__ void block_sums(float (&v)[K], float *out) {
  __shared__ float part[K][kThreads / 32];
#pragma unroll
  for (int k = 0; k < K; ++k) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
      v[k] += __shfl_xor_sync(0xffffffffu, v[k], o);
    if ((threadIdx.x & 31) == 0)
      part[k][threadIdx.x >> 5] = v[k];
  }
  __syncthreads();
  if (threadIdx.x < K) {
    float t = 0.0f;
    for (int w = 0; w < kThreads / 32; ++w)
      t += part[threadIdx.x][w];
    out[threadIdx.x] = t;
  }
}

// partial sums of x and x^2 of channel blockIdx.y over the items of block blockIdx.x: partial[c][p][2]
template <bool kVec>
__global__ void __launch_bounds__(kThreads) bn_stats_kernel(const float *__restrict__ x, unsigned N, unsigned C,
                                                            unsigned S, float *__restrict__ partial) {
  const unsigned c = blockIdx.y, P = gridDim.x;
  const unsigned Su = kVec ? S / 4 : S;
  float v[2] = {0.0f, 0.0f};
  ChannelItems it((size_t)blockIdx.x * kThreads + threadIdx.x, (size_t)P * kThreads, Su, N);
  for (; it.valid(); it.next()) {
    const size_t base = ((size_t)it.n * C + c) * S;
    if (kVec) {
      const float4 a = __ldg(reinterpret_cast<const float4 *>(x + base) + it.s);
      v[0] += (a.x + a.y) + (a.z + a.w);
      v[1] += (a.x * a.x + a.y * a.y) + (a.z * a.z + a.w * a.w);
    } else {
      const float a = __ldg(x + base + it.s);
      v[0] += a;
      v[1] += a * a;
    }
  }
  block_sums<2>(v, partial + ((size_t)c * P + blockIdx.x) * 2);
}

// batch_normalization.cpp:191-205 given the channel's sums: mean, variance, running statistics.
__global__ void bn_stats_finish_kernel(const float *__restrict__ partial, unsigned P, unsigned C, float count,
                                       float decay, int update, float *__restrict__ m, float *__restrict__ v,
                                       float *__restrict__ rm, float *__restrict__ rv) {
  const unsigned c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C)
    return;
  double s = 0.0, q = 0.0;
  for (unsigned p = 0; p < P; ++p) {
    s += (double)partial[((size_t)c * P + p) * 2];
    q += (double)partial[((size_t)c * P + p) * 2 + 1];
  }
  const float mean = __fdiv_rn((float)s, count);
  const float var = __fsub_rn(__fdiv_rn((float)q, count), __fmul_rn(mean, mean));
  m[c] = mean;
  v[c] = var;
  if (update) {
    const float keep = __fsub_rn(1.0f, decay);
    rm[c] = __fadd_rn(__fmul_rn(decay, rm[c]), __fmul_rn(keep, mean));
    rv[c] = __fadd_rn(__fmul_rn(decay, rv[c]),
                      __fdiv_rn(__fmul_rn(__fmul_rn(keep, var), count), __fsub_rn(count, 1.0f)));
  }
}

// partial[c][p][5]: sum dy*scale*(x-m), sum dy*scale, sum (x-m), sum dy, sum dy*(x-m)/sqrt(v+eps)   (batch)
//                   -, -, -, sum dy, sum dy*((x-m)*rstd_inv)                                          (global)
template <bool kVec, bool kBatch>
__global__ void __launch_bounds__(kThreads)
    bn_backward_sums_kernel(const float *__restrict__ x, const float *__restrict__ dy, const float *__restrict__ gamma,
                            const float *__restrict__ mean, const float *__restrict__ var, float eps, unsigned N,
                            unsigned C, unsigned S, float *__restrict__ partial) {
  const unsigned c = blockIdx.y, P = gridDim.x;
  const unsigned Su = kVec ? S / 4 : S;
  const float m = mean[c], scale = gamma ? gamma[c] : 1.0f;
  const float sd = __fsqrt_rn(__fadd_rn(var[c], eps));
  const float rstd_inv = kBatch ? 0.0f : inv_sqrt_rn(__fadd_rn(var[c], eps));
  float v[5] = {0.0f, 0.0f, 0.0f, 0.0f, 0.0f};
  auto one = [&](float xv, float g) {
    const float cx = __fsub_rn(xv, m);
    if (kBatch) {
      const float dxh = __fmul_rn(g, scale);
      v[0] += __fmul_rn(dxh, cx);
      v[1] += dxh;
      v[2] += cx;
      v[4] += __fdiv_rn(__fmul_rn(g, cx), sd);
    } else {
      v[4] += __fmul_rn(g, __fmul_rn(cx, rstd_inv));
    }
    v[3] += g;
  };
  ChannelItems it((size_t)blockIdx.x * kThreads + threadIdx.x, (size_t)P * kThreads, Su, N);
  for (; it.valid(); it.next()) {
    const size_t base = ((size_t)it.n * C + c) * S;
    if (kVec) {
      const float4 a = __ldg(reinterpret_cast<const float4 *>(x + base) + it.s);
      const float4 g = __ldg(reinterpret_cast<const float4 *>(dy + base) + it.s);
      one(a.x, g.x);
      one(a.y, g.y);
      one(a.z, g.z);
      one(a.w, g.w);
    } else {
      one(__ldg(x + base + it.s), __ldg(dy + base + it.s));
    }
  }
  block_sums<5>(v, partial + ((size_t)c * P + blockIdx.x) * 5);
}

// coef[c][4] for the dx pass: {dvar * 2, dmean / n, gamma * (v + eps)^-0.5, -}. Batch mode
// (batch_normalization.cpp:326-334): dvar = s0 * -0.5 * (v + eps)^-1.5 + dv;
// dmean = s1 * (-1 / sqrt(v + eps)) + dvar * -2 * s2 / n + dm. `partial` may be NULL (no sums were needed).
__global__ void bn_backward_finish_kernel(const float *__restrict__ partial, unsigned P, unsigned C, float count,
                                          const float *__restrict__ gamma, const float *__restrict__ var, float eps,
                                          const float *__restrict__ dm, const float *__restrict__ dv, int batch,
                                          float *__restrict__ coef, float *__restrict__ dbeta, int accum_dbeta,
                                          float *__restrict__ dgamma, int accum_dgamma) {
  const unsigned c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C)
    return;
  double s[5] = {0, 0, 0, 0, 0};
  if (partial)
    for (unsigned p = 0; p < P; ++p)
      for (int k = 0; k < 5; ++k)
        s[k] += (double)partial[((size_t)c * P + p) * 5 + k];
  const float ve = __fadd_rn(var[c], eps);
  {
    const float r = inv_sqrt_rn(ve);
    coef[c * 4 + 2] = gamma ? __fmul_rn(gamma[c], r) : r;
  }
  if (batch) {
    const float dvar = __fadd_rn(__fmul_rn(__fmul_rn((float)s[0], -0.5f), inv_sqrt_cubed_rn(ve)), dv ? dv[c] : 0.0f);
    float dmean = __fmul_rn((float)s[1], __fdiv_rn(-1.0f, __fsqrt_rn(ve)));
    dmean = __fadd_rn(dmean, __fdiv_rn(__fmul_rn(__fmul_rn(dvar, -2.0f), (float)s[2]), count));
    dmean = __fadd_rn(dmean, dm ? dm[c] : 0.0f);
    coef[c * 4 + 0] = __fmul_rn(dvar, 2.0f);
    coef[c * 4 + 1] = __fdiv_rn(dmean, count);
  }
  if (dbeta)
    dbeta[c] = accum_dbeta ? __fadd_rn(dbeta[c], (float)s[3]) : (float)s[3];
  if (dgamma)
    dgamma[c] = accum_dgamma ? __fadd_rn(dgamma[c], (float)s[4]) : (float)s[4];
}

// batch (batch_normalization.cpp:336-349): dx (+)= dy * scale / sqrt(v + eps) + dvar * 2 * (x - m) / n + dmean / n
// global (:413-440):                       dx (+)= dy * (gamma * (v + eps)^-0.5)
template <bool kBatch, bool kAccum>
__global__ void __launch_bounds__(kThreads)
    bn_backward_dx_kernel(const float *__restrict__ x, const float *__restrict__ dy, const float *__restrict__ gamma,
                          const float *__restrict__ mean, const float *__restrict__ var, float eps,
                          const float *__restrict__ coef, float count, size_t total, unsigned C, unsigned S,
                          float *__restrict__ dx) {
  const size_t stride = (size_t)gridDim.x * kThreads;
  const size_t first = (size_t)blockIdx.x * kThreads + threadIdx.x;
  ChannelWalk walk(first, stride, S, C);
  for (size_t i = first; i < total; i += stride, walk.next()) {
    const unsigned c = walk.c;
    const float scale = gamma ? __ldg(gamma + c) : 1.0f;
    const float ve = __fadd_rn(__ldg(var + c), eps);
    float g;
    if (kBatch) {
      const float a = __fdiv_rn(__fmul_rn(dy[i], scale), __fsqrt_rn(ve));
      const float b = __fdiv_rn(__fmul_rn(__ldg(coef + c * 4), __fsub_rn(x[i], __ldg(mean + c))), count);
      g = __fadd_rn(__fadd_rn(a, b), __ldg(coef + c * 4 + 1));
    } else {
      g = __fmul_rn(dy[i], __ldg(coef + c * 4 + 2));
    }
    dx[i] = kAccum ? __fadd_rn(dx[i], g) : g;
  }
}

// The same for planes of whole float4: one block per (plane, chunk), the channel's constants taken once.
template <bool kBatch, bool kAccum>
__global__ void __launch_bounds__(kThreads)
    bn_backward_dx_plane_kernel(const float *__restrict__ x, const float *__restrict__ dy,
                                const float *__restrict__ gamma, const float *__restrict__ mean,
                                const float *__restrict__ var, float eps, const float *__restrict__ coef, float count,
                                int C, int S4, float *__restrict__ dx) {
  const unsigned plane = blockIdx.x;
  const int c = (int)(plane % (unsigned)C);
  const float scale = gamma ? __ldg(gamma + c) : 1.0f;
  const float sd = __fsqrt_rn(__fadd_rn(__ldg(var + c), eps));
  const float m = __ldg(mean + c), k0 = __ldg(coef + c * 4), k1 = __ldg(coef + c * 4 + 1), k2 = __ldg(coef + c * 4 + 2);
  const float4 *xp = reinterpret_cast<const float4 *>(x) + (size_t)plane * S4;
  const float4 *gp = reinterpret_cast<const float4 *>(dy) + (size_t)plane * S4;
  float4 *op = reinterpret_cast<float4 *>(dx) + (size_t)plane * S4;
  auto one = [&](float xv, float g, float old) {
    float r;
    if (kBatch) {
      const float a = __fdiv_rn(__fmul_rn(g, scale), sd);
      const float b = __fdiv_rn(__fmul_rn(k0, __fsub_rn(xv, m)), count);
      r = __fadd_rn(__fadd_rn(a, b), k1);
    } else {
      r = __fmul_rn(g, k2);
    }
    return kAccum ? __fadd_rn(old, r) : r;
  };
  for (int i = blockIdx.y * kThreads + threadIdx.x; i < S4; i += gridDim.y * kThreads) {
    const float4 g = __ldcs(gp + i);
    float4 xv = make_float4(0, 0, 0, 0), o = make_float4(0, 0, 0, 0);
    if (kBatch)
      xv = __ldcs(xp + i);
    if (kAccum)
      o = op[i];
    op[i] = make_float4(one(xv.x, g.x, o.x), one(xv.y, g.y, o.y), one(xv.z, g.z, o.z), one(xv.w, g.w, o.w));
  }
}

int channel_blocks(int64_t outer, int64_t channels, int64_t inner, bool vec) {
  const int64_t items = outer * (vec ? inner / 4 : inner);
  int64_t p = (8ll * sm_count() + channels - 1) / channels;
  const int64_t most = (items + kThreads - 1) / kThreads;
  p = p > most ? most : p;
  return (int)(p < 1 ? 1 : p);
}

} // namespace
} // namespace nb200

using namespace nb200;

extern "C" {

int nb200_batch_normalization_inference_f32(const float *x, const float *beta, const float *gamma, const float *mean,
                                            const float *var, float *y, int64_t outer, int64_t channels,
                                            int64_t inner, float eps, void *stream);

int nb200_batch_normalization_batch_f32(const float *x, const float *beta, const float *gamma, float *running_mean,
                                        float *running_var, float *y, float *batch_mean, float *batch_var,
                                        int64_t outer, int64_t channels, int64_t inner, float eps, float decay_rate,
                                        int update_running, void *stream) {
  NB_CHECK(outer > 0 && channels > 0 && inner > 0, NB200_EVALUE, "bad extents");
  NB_CHECK(channels <= 65535 && inner < (1ll << 31) && outer < (1ll << 31), NB200_EVALUE, "extent too large");
  NB_CHECK(x && y && batch_mean && batch_var, NB200_EVALUE, "null data pointer");
  NB_CHECK(!update_running || (running_mean && running_var), NB200_EVALUE, "running statistics are needed");
  cudaStream_t st = as_stream(stream);
  const bool vec = (inner % 4 == 0) && (reinterpret_cast<uintptr_t>(x) & 15) == 0;
  const int P = channel_blocks(outer, channels, inner, vec);
  AsyncScratch scratch(st);
  NB_TRY(scratch.alloc((size_t)channels * P * 2 * sizeof(float)));
  float *partial = static_cast<float *>(scratch.p);
  const dim3 grid((unsigned)P, (unsigned)channels);
  if (vec)
    bn_stats_kernel<true><<<grid, kThreads, 0, st>>>(x, (unsigned)outer, (unsigned)channels, (unsigned)inner, partial);
  else
    bn_stats_kernel<false><<<grid, kThreads, 0, st>>>(x, (unsigned)outer, (unsigned)channels, (unsigned)inner, partial);
  NB_LAUNCH_CHECK();
  bn_stats_finish_kernel<<<(unsigned)((channels + 127) / 128), 128, 0, st>>>(
      partial, (unsigned)P, (unsigned)channels, (float)(outer * inner), decay_rate, update_running, batch_mean,
      batch_var, running_mean, running_var);
  NB_LAUNCH_CHECK();
  return nb200_batch_normalization_inference_f32(x, beta, gamma, batch_mean, batch_var, y, outer, channels, inner,
                                                 eps, stream);
}

int nb200_batch_normalization_backward_f32(const float *x, const float *dy, const float *gamma, const float *mean,
                                           const float *var, const float *dmean, const float *dvar, float *dx,
                                           float *dbeta, float *dgamma, int64_t outer, int64_t channels,
                                           int64_t inner, float eps, int batch_stat, int accum_dx, int accum_dbeta,
                                           int accum_dgamma, void *stream) {
  NB_CHECK(outer > 0 && channels > 0 && inner > 0, NB200_EVALUE, "bad extents");
  NB_CHECK(channels <= 65535 && inner < (1ll << 31) && outer < (1ll << 31), NB200_EVALUE, "extent too large");
  NB_CHECK(x && dy && mean && var, NB200_EVALUE, "null data pointer");
  if (!dx && !dbeta && !dgamma)
    return NB200_OK;
  cudaStream_t st = as_stream(stream);
  const bool vec = (inner % 4 == 0) && ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(dy)) & 15) == 0;
  const int P = channel_blocks(outer, channels, inner, vec);
  AsyncScratch scratch(st);
  NB_TRY(scratch.alloc((size_t)channels * (P * 5 + 4) * sizeof(float)));
  float *partial = static_cast<float *>(scratch.p);
  float *coef = partial + (size_t)channels * P * 5;
  const bool sums = (batch_stat && dx) || dbeta || dgamma;
  if (sums) {
    const dim3 grid((unsigned)P, (unsigned)channels);
#define NB_BN_SUMS(V, B)                                                                                               \
  bn_backward_sums_kernel<V, B><<<grid, kThreads, 0, st>>>(x, dy, gamma, mean, var, eps, (unsigned)outer,              \
                                                            (unsigned)channels, (unsigned)inner, partial)
    if (vec && batch_stat)
      NB_BN_SUMS(true, true);
    else if (vec)
      NB_BN_SUMS(true, false);
    else if (batch_stat)
      NB_BN_SUMS(false, true);
    else
      NB_BN_SUMS(false, false);
#undef NB_BN_SUMS
    NB_LAUNCH_CHECK();
  }
  bn_backward_finish_kernel<<<(unsigned)((channels + 127) / 128), 128, 0, st>>>(
      sums ? partial : nullptr, (unsigned)P, (unsigned)channels, (float)(outer * inner), gamma, var, eps, dmean, dvar,
      batch_stat, coef, sums ? dbeta : nullptr, accum_dbeta, sums ? dgamma : nullptr, accum_dgamma);
  NB_LAUNCH_CHECK();
  if (dx) {
    const size_t total = (size_t)outer * channels * inner;
    const unsigned grid = grid_for(total, 4);
    const bool planes = vec && inner >= 4 * kThreads && outer * channels < (1ll << 31) &&
                        (reinterpret_cast<uintptr_t>(dx) & 15) == 0;
    if (planes) {
      const int S4 = (int)(inner / 4);
      int chunks = (S4 + 2 * kThreads - 1) / (2 * kThreads);
      chunks = chunks > 64 ? 64 : chunks;
      const dim3 pgrid((unsigned)(outer * channels), (unsigned)chunks);
#define NB_BN_DXP(B, A)                                                                                                \
  bn_backward_dx_plane_kernel<B, A><<<pgrid, kThreads, 0, st>>>(x, dy, gamma, mean, var, eps, coef,                    \
                                                                (float)(outer * inner), (int)channels, S4, dx)
      if (batch_stat && accum_dx)
        NB_BN_DXP(true, true);
      else if (batch_stat)
        NB_BN_DXP(true, false);
      else if (accum_dx)
        NB_BN_DXP(false, true);
      else
        NB_BN_DXP(false, false);
#undef NB_BN_DXP
      NB_LAUNCH_CHECK();
      return NB200_OK;
    }
#define NB_BN_DX(B, A)                                                                                                 \
  bn_backward_dx_kernel<B, A><<<grid, kThreads, 0, st>>>(x, dy, gamma, mean, var, eps, coef, (float)(outer * inner),   \
                                                          total, (unsigned)channels, (unsigned)inner, dx)
    if (batch_stat && accum_dx)
      NB_BN_DX(true, true);
    else if (batch_stat)
      NB_BN_DX(true, false);
    else if (accum_dx)
      NB_BN_DX(false, true);
    else
      NB_BN_DX(false, false);
#undef NB_BN_DX
    NB_LAUNCH_CHECK();
  }
  return NB200_OK;
}

int nb200_relu_backward_f32(const float *y, const float *dy, float *dx, size_t size, int accum, void *stream) {
  if (size == 0)
    return NB200_OK;
  NB_CHECK(y && dy && dx, NB200_EVALUE, "null data pointer");
  const bool vec =
      ((reinterpret_cast<uintptr_t>(y) | reinterpret_cast<uintptr_t>(dy) | reinterpret_cast<uintptr_t>(dx)) & 15) == 0;
  const unsigned grid = grid_for(size / 4 + 1, 2);
  if (accum)
    grad_pass_kernel<0, true><<<grid, kThreads, 0, as_stream(stream)>>>(y, dy, dx, size, vec);
  else
    grad_pass_kernel<0, false><<<grid, kThreads, 0, as_stream(stream)>>>(y, dy, dx, size, vec);
  NB_LAUNCH_CHECK();
  return NB200_OK;
}

int nb200_add2_backward_f32(const float *dy, float *dx, size_t size, int accum, void *stream) {
  if (size == 0)
    return NB200_OK;
  NB_CHECK(dy && dx, NB200_EVALUE, "null data pointer");
  const bool vec = ((reinterpret_cast<uintptr_t>(dy) | reinterpret_cast<uintptr_t>(dx)) & 15) == 0;
  const unsigned grid = grid_for(size / 4 + 1, 2);
  if (accum)
    grad_pass_kernel<1, true><<<grid, kThreads, 0, as_stream(stream)>>>(nullptr, dy, dx, size, vec);
  else
    grad_pass_kernel<1, false><<<grid, kThreads, 0, as_stream(stream)>>>(nullptr, dy, dx, size, vec);
  NB_LAUNCH_CHECK();
  return NB200_OK;
}

int nb200_global_average_pooling_backward_f32(const float *dy, float *dx, int64_t maps, int64_t spatial, int accum,
                                              void *stream) {
  NB_CHECK(maps >= 0 && spatial > 0 && spatial < (1ll << 31), NB200_EVALUE, "bad extents");
  const size_t total = (size_t)maps * spatial;
  if (total == 0)
    return NB200_OK;
  NB_CHECK(dy && dx, NB200_EVALUE, "null data pointer");
  if (accum)
    gap_backward_kernel<true><<<grid_for(total, 4), kThreads, 0, as_stream(stream)>>>(dy, dx, total, (unsigned)spatial);
  else
    gap_backward_kernel<false><<<grid_for(total, 4), kThreads, 0, as_stream(stream)>>>(dy, dx, total, (unsigned)spatial);
  NB_LAUNCH_CHECK();
  return NB200_OK;
}

int nb200_max_pooling_backward_f32(const float *x, const float *dy, float *dx, int64_t maps, int height, int width,
                                   int kernel_h, int kernel_w, int stride_h, int stride_w, int pad_h, int pad_w,
                                   int ignore_border, int accum, void *stream) {
  NB_CHECK(maps >= 0 && height > 0 && width > 0 && kernel_h > 0 && kernel_w > 0 && stride_h > 0 && stride_w > 0 &&
               pad_h >= 0 && pad_w >= 0,
           NB200_EVALUE, "bad pooling geometry");
  // Output extent: src/nbla/function/utils/base_pooling.cpp:59.
  const int Ho = (height + pad_h - (ignore_border ? kernel_h - pad_h : 1)) / stride_h + 1;
  const int Wo = (width + pad_w - (ignore_border ? kernel_w - pad_w : 1)) / stride_w + 1;
  NB_CHECK(Ho > 0 && Wo > 0, NB200_EVALUE, "pooling output would be empty");
  const size_t total = (size_t)maps * height * width;
  if (total == 0)
    return NB200_OK;
  NB_CHECK(x && dy && dx, NB200_EVALUE, "null data pointer");
  NB_CHECK((int64_t)height * width < (1ll << 31), NB200_EVALUE, "map larger than 2^31 pixels");
  cudaStream_t st = as_stream(stream);
  const size_t outputs = (size_t)maps * Ho * Wo;
  AsyncScratch scratch(st);
  NB_TRY(scratch.alloc(outputs * sizeof(int)));
  int *index = static_cast<int *>(scratch.p);
  max_pooling_index_kernel<<<grid_for(outputs, 1), kThreads, 0, st>>>(x, index, outputs, height, width, Ho, Wo,
                                                                       kernel_h, kernel_w, stride_h, stride_w, pad_h,
                                                                       pad_w);
  NB_LAUNCH_CHECK();
  if (accum)
    max_pooling_backward_kernel<true><<<grid_for(total, 1), kThreads, 0, st>>>(
        index, dy, dx, total, height, width, Ho, Wo, kernel_h, kernel_w, stride_h, stride_w, pad_h, pad_w);
  else
    max_pooling_backward_kernel<false><<<grid_for(total, 1), kThreads, 0, st>>>(
        index, dy, dx, total, height, width, Ho, Wo, kernel_h, kernel_w, stride_h, stride_w, pad_h, pad_w);
  NB_LAUNCH_CHECK();
  return NB200_OK;
}

} // extern "C"
