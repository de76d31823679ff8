// The functions a binary-weight ResNet-18 graph needs next to the quantized
// layers, so that the whole graph runs under one context with no CPU
// fallback: BatchNormalization (inference), ReLU, Add2, MaxPooling,
// GlobalAveragePooling and a full-precision Convolution for the network stem.
// All but the convolution are HBM-bound single passes whose arithmetic follows
// the reference's operation order, so their results are bit-identical to its
// CPU code; the convolution accumulates with fused multiply-adds (tolerance
// parity, like the other contractions).
#include <cmath>

#include "common.cuh"
#include "narrow_conv.cuh"
#include "pdl.cuh"

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

// BatchNormalization<T>::forward_impl_global
// (src/nbla/function/generic/batch_normalization.cpp:228-260), channel axis 1:
// y = (x - mean) * gamma / sqrt(var + eps) + beta, each operation rounded.
// x is [N, C, S]; when S % 4 == 0 a thread handles one float4 (one channel).
template <bool kVec>
__global__ void __launch_bounds__(kThreads) bn_inference_kernel(const float *__restrict__ x, const float *beta,
                                                                const float *gamma, const float *mean,
                                                                const float *var, size_t total, int C, int S,
                                                                float eps, float *__restrict__ y) {
  pdl_wait();
  pdl_trigger();
  const size_t stride = (size_t)gridDim.x * kThreads;
  if (kVec) {
    const size_t total4 = total / 4;
    const int S4 = S / 4;
    const size_t first = (size_t)blockIdx.x * kThreads + threadIdx.x;
    ChannelWalk walk(first, stride, (unsigned)S4, (unsigned)C);
    for (size_t i = first; i < total4; i += stride, walk.next()) {
      const int c = (int)walk.c;
      const float m = __ldg(mean + c);
      const float sd = __fsqrt_rn(__fadd_rn(__ldg(var + c), eps));
      const float g = gamma ? __ldg(gamma + c) : 1.0f;
      const float b = beta ? __ldg(beta + c) : 0.0f;
      const float4 v = __ldcs(reinterpret_cast<const float4 *>(x) + i);
      float4 r;
      r.x = __fadd_rn(__fdiv_rn(__fmul_rn(__fsub_rn(v.x, m), g), sd), b);
      r.y = __fadd_rn(__fdiv_rn(__fmul_rn(__fsub_rn(v.y, m), g), sd), b);
      r.z = __fadd_rn(__fdiv_rn(__fmul_rn(__fsub_rn(v.z, m), g), sd), b);
      r.w = __fadd_rn(__fdiv_rn(__fmul_rn(__fsub_rn(v.w, m), g), sd), b);
      __stcs(reinterpret_cast<float4 *>(y) + i, r);
    }
  } else {
    const size_t first = (size_t)blockIdx.x * kThreads + threadIdx.x;
    ChannelWalk walk(first, stride, (unsigned)S, (unsigned)C);
    for (size_t i = first; i < total; i += stride, walk.next()) {
      const int c = (int)walk.c;
      const float sd = __fsqrt_rn(__fadd_rn(var[c], eps));
      const float g = gamma ? gamma[c] : 1.0f;
      const float b = beta ? beta[c] : 0.0f;
      y[i] = __fadd_rn(__fdiv_rn(__fmul_rn(__fsub_rn(x[i], mean[c]), g), sd), b);
    }
  }
}

// The same for planes of at least a few hundred float4: one block per (plane, chunk of the plane), so the
// channel's four parameters and the square root are taken once per thread and the loop is loads, four
// rounded operations per value and stores. blockIdx.x = plane (n * C + c), blockIdx.y = chunk.
__global__ void __launch_bounds__(kThreads) bn_inference_plane_kernel(const float *__restrict__ x, const float *beta,
                                                                      const float *gamma, const float *mean,
                                                                      const float *var, int C, int S4, float eps,
                                                                      float *__restrict__ y) {
  pdl_wait();
  pdl_trigger();
  const unsigned plane = blockIdx.x;
  const int c = (int)(plane % (unsigned)C);
  const float4 *xp = reinterpret_cast<const float4 *>(x) + (size_t)plane * S4;
  float4 *yp = reinterpret_cast<float4 *>(y) + (size_t)plane * S4;
  // the data loads go out first: they do not depend on the channel's constants, whose own loads, square
  // root and reciprocal would otherwise stand in front of them in every (short) block
  constexpr int kPer = 4;
  const int step = gridDim.y * kThreads;
  int i = blockIdx.y * kThreads + threadIdx.x;
  float4 v[kPer];
#pragma unroll
  for (int u = 0; u < kPer; ++u)
    if (i + u * step < S4)
      v[u] = __ldcs(xp + i + u * step);
  const float m = __ldg(mean + c);
  const float sd = __fsqrt_rn(__fadd_rn(__ldg(var + c), eps));
  const float g = gamma ? __ldg(gamma + c) : 1.0f;
  const float b = beta ? __ldg(beta + c) : 0.0f;
  auto one = [&](float4 a) {
    float4 r;
    r.x = __fadd_rn(__fdiv_rn(__fmul_rn(__fsub_rn(a.x, m), g), sd), b);
    r.y = __fadd_rn(__fdiv_rn(__fmul_rn(__fsub_rn(a.y, m), g), sd), b);
    r.z = __fadd_rn(__fdiv_rn(__fmul_rn(__fsub_rn(a.z, m), g), sd), b);
    r.w = __fadd_rn(__fdiv_rn(__fmul_rn(__fsub_rn(a.w, m), g), sd), b);
    return r;
  };
#pragma unroll
  for (int u = 0; u < kPer; ++u)
    if (i + u * step < S4)
      __stcs(yp + i + u * step, one(v[u]));
  for (i += kPer * step; i < S4; i += step)
    __stcs(yp + i, one(__ldcs(xp + i)));
}

// Planes of 32 to 1023 values (the later stages of a network: 28 x 28, 14 x 14, 7 x 7): one WARP per plane,
// eight planes per block. The channel's constants are taken once per lane instead of once per value, the
// data loads go out before them, and nothing divides by the plane size. kVec: S % 4 == 0 and 16-byte
// aligned tensors (float4 lanes), otherwise scalar lanes (a 7 x 7 plane is 49 values).
template <bool kVec>
__global__ void __launch_bounds__(kThreads) bn_inference_warp_kernel(const float *__restrict__ x, const float *beta,
                                                                     const float *gamma, const float *mean,
                                                                     const float *var, unsigned planes, int C, int S,
                                                                     float eps, float *__restrict__ y) {
  pdl_wait();
  pdl_trigger();
  const unsigned plane = blockIdx.x * (kThreads / 32) + (threadIdx.x >> 5);
  if (plane >= planes)
    return;
  const int lane = threadIdx.x & 31;
  const int c = (int)(plane % (unsigned)C);
  constexpr int kPer = kVec ? 7 : 4; // a 28 x 28 plane is 196 float4: seven per lane, all in flight at once
  if (kVec) {
    const int S4 = S / 4;
    const float4 *xp = reinterpret_cast<const float4 *>(x) + (size_t)plane * S4;
    float4 *yp = reinterpret_cast<float4 *>(y) + (size_t)plane * S4;
    float4 v[kPer];
#pragma unroll
    for (int u = 0; u < kPer; ++u)
      if (lane + 32 * u < S4)
        v[u] = __ldcs(xp + lane + 32 * u);
    const float m = __ldg(mean + c);
    const float sd = __fsqrt_rn(__fadd_rn(__ldg(var + c), eps));
    const float g = gamma ? __ldg(gamma + c) : 1.0f;
    const float b = beta ? __ldg(beta + c) : 0.0f;
    auto one = [&](float4 a) {
      float4 r;
      r.x = __fadd_rn(__fdiv_rn(__fmul_rn(__fsub_rn(a.x, m), g), sd), b);
      r.y = __fadd_rn(__fdiv_rn(__fmul_rn(__fsub_rn(a.y, m), g), sd), b);
      r.z = __fadd_rn(__fdiv_rn(__fmul_rn(__fsub_rn(a.z, m), g), sd), b);
      r.w = __fadd_rn(__fdiv_rn(__fmul_rn(__fsub_rn(a.w, m), g), sd), b);
      return r;
    };
#pragma unroll
    for (int u = 0; u < kPer; ++u)
      if (lane + 32 * u < S4)
        __stcs(yp + lane + 32 * u, one(v[u]));
    for (int i = lane + 32 * kPer; i < S4; i += 32)
      __stcs(yp + i, one(__ldcs(xp + i)));
  } else {
    const float *xp = x + (size_t)plane * S;
    float *yp = y + (size_t)plane * S;
    float v[kPer];
#pragma unroll
    for (int u = 0; u < kPer; ++u)
      if (lane + 32 * u < S)
        v[u] = __ldcs(xp + lane + 32 * u);
    const float m = __ldg(mean + c);
    const float sd = __fsqrt_rn(__fadd_rn(__ldg(var + c), eps));
    const float g = gamma ? __ldg(gamma + c) : 1.0f;
    const float b = beta ? __ldg(beta + c) : 0.0f;
#pragma unroll
    for (int u = 0; u < kPer; ++u)
      if (lane + 32 * u < S)
        __stcs(yp + lane + 32 * u, __fadd_rn(__fdiv_rn(__fmul_rn(__fsub_rn(v[u], m), g), sd), b));
    for (int i = lane + 32 * kPer; i < S; i += 32)
      __stcs(yp + i, __fadd_rn(__fdiv_rn(__fmul_rn(__fsub_rn(__ldcs(xp + i), m), g), sd), b));
  }
}

// Planes whose size is not a multiple of 4 (7 x 7 = 49 values): four consecutive planes are S float4, 16-byte
// aligned when the plane count is a multiple of 4, and a warp takes such a group. Lanes 0..3 hold the constants of
// the group's four channels; a float4 lies in one channel or across two neighbours (S >= 32), whose constants come
// by shuffle. A quarter of the load / store instructions of the scalar form, the same rounded operations.
__global__ void __launch_bounds__(kThreads) bn_inference_warp4_kernel(const float *__restrict__ x, const float *beta,
                                                                      const float *gamma, const float *mean,
                                                                      const float *var, unsigned groups, int C, int S,
                                                                      float eps, float *__restrict__ y) {
  pdl_wait();
  pdl_trigger();
  const unsigned group = blockIdx.x * (kThreads / 32) + (threadIdx.x >> 5);
  if (group >= groups)
    return;
  const int lane = threadIdx.x & 31;
  const float4 *xp = reinterpret_cast<const float4 *>(x) + (size_t)group * S;
  float4 *yp = reinterpret_cast<float4 *>(y) + (size_t)group * S;
  constexpr int kPer = 2;
  float4 v[kPer];
#pragma unroll
  for (int u = 0; u < kPer; ++u)
    if (lane + 32 * u < S)
      v[u] = __ldcs(xp + lane + 32 * u);
  const int c = (int)((group * 4u + (unsigned)(lane & 3)) % (unsigned)C);
  const float m = __ldg(mean + c);
  const float sd = __fsqrt_rn(__fadd_rn(__ldg(var + c), eps));
  const float g = gamma ? __ldg(gamma + c) : 1.0f;
  const float b = beta ? __ldg(beta + c) : 0.0f;
  auto one = [&](int j, float4 a) { // all lanes of the warp call this together (shuffles)
    const int e = 4 * j;
    const int k0 = (e >= S) + (e >= 2 * S) + (e >= 3 * S);
    const int k1 = k0 < 3 ? k0 + 1 : 3;
    const float m0 = __shfl_sync(0xffffffffu, m, k0), m1 = __shfl_sync(0xffffffffu, m, k1);
    const float g0 = __shfl_sync(0xffffffffu, g, k0), g1 = __shfl_sync(0xffffffffu, g, k1);
    const float s0 = __shfl_sync(0xffffffffu, sd, k0), s1 = __shfl_sync(0xffffffffu, sd, k1);
    const float b0 = __shfl_sync(0xffffffffu, b, k0), b1 = __shfl_sync(0xffffffffu, b, k1);
    const int edge = (k0 + 1) * S; // first element of the next plane
    auto el = [&](float t, int idx) {
      const bool nx = idx >= edge;
      return __fadd_rn(__fdiv_rn(__fmul_rn(__fsub_rn(t, nx ? m1 : m0), nx ? g1 : g0), nx ? s1 : s0), nx ? b1 : b0);
    };
    return make_float4(el(a.x, e), el(a.y, e + 1), el(a.z, e + 2), el(a.w, e + 3));
  };
  const int rounds = (S + 31) / 32;
#pragma unroll
  for (int u = 0; u < kPer; ++u) {
    if (u < rounds) { // warp-uniform
      const int j = lane + 32 * u;
      const float4 r = one(j < S ? j : 0, j < S ? v[u] : make_float4(0.f, 0.f, 0.f, 0.f));
      if (j < S)
        __stcs(yp + j, r);
    }
  }
  for (int u = kPer; u < rounds; ++u) {
    const int j = lane + 32 * u;
    const float4 a = j < S ? __ldcs(xp + j) : make_float4(0.f, 0.f, 0.f, 0.f);
    const float4 r = one(j < S ? j : 0, a);
    if (j < S)
      __stcs(yp + j, r);
  }
}

// ReLU (src/nbla/function/generic/relu.cpp): y = max(0, x); Add2 (add2.cpp): y = a + b.
template <int kOp, bool kVec>
__global__ void __launch_bounds__(kThreads) unary_binary_kernel(const float *__restrict__ a,
                                                                const float *__restrict__ b, size_t total,
                                                                float *__restrict__ y) {
  pdl_wait();
  pdl_trigger();
  const size_t stride = (size_t)gridDim.x * kThreads;
  if (kVec) {
    const size_t total4 = total / 4;
    for (size_t i = (size_t)blockIdx.x * kThreads + threadIdx.x; i < total4; i += stride) {
      const float4 v = __ldcs(reinterpret_cast<const float4 *>(a) + i);
      float4 r;
      if (kOp == 0) {
        r.x = v.x > 0.0f ? v.x : 0.0f;
        r.y = v.y > 0.0f ? v.y : 0.0f;
        r.z = v.z > 0.0f ? v.z : 0.0f;
        r.w = v.w > 0.0f ? v.w : 0.0f;
      } else {
        const float4 w = __ldcs(reinterpret_cast<const float4 *>(b) + i);
        r.x = __fadd_rn(v.x, w.x);
        r.y = __fadd_rn(v.y, w.y);
        r.z = __fadd_rn(v.z, w.z);
        r.w = __fadd_rn(v.w, w.w);
      }
      __stcs(reinterpret_cast<float4 *>(y) + i, r);
    }
    for (size_t i = total4 * 4 + (size_t)blockIdx.x * kThreads + threadIdx.x; i < total; i += stride)
      y[i] = (kOp == 0) ? (a[i] > 0.0f ? a[i] : 0.0f) : __fadd_rn(a[i], b[i]);
  } else {
    for (size_t i = (size_t)blockIdx.x * kThreads + threadIdx.x; i < total; i += stride)
      y[i] = (kOp == 0) ? (a[i] > 0.0f ? a[i] : 0.0f) : __fadd_rn(a[i], b[i]);
  }
}

// MaxPooling forward_map (src/nbla/function/generic/max_pooling.cpp:60-84):
// window clipped to the input, first maximum wins under "<".
__global__ void __launch_bounds__(kThreads) max_pooling_kernel(const float *__restrict__ x, size_t maps, int H, int W,
                                                               int Ho, int Wo, int kh, int kw, int sh, int sw, int ph,
                                                               int pw, float *__restrict__ y) {
  pdl_wait();
  pdl_trigger();
  const size_t total = maps * Ho * Wo;
  const size_t stride = (size_t)gridDim.x * kThreads;
  for (size_t i = (size_t)blockIdx.x * kThreads + threadIdx.x; i < total; i += stride) {
    const int ox = (int)(i % Wo);
    const int oy = (int)((i / Wo) % Ho);
    const size_t m = i / ((size_t)Wo * Ho);
    int y0 = oy * sh - ph, x0 = ox * sw - pw;
    int y1 = min(y0 + kh, H + ph), x1 = min(x0 + kw, W + pw);
    y0 = max(y0, 0);
    x0 = max(x0, 0);
    y1 = min(y1, H);
    x1 = min(x1, W);
    const float *xm = x + m * (size_t)H * W;
    float best = xm[(size_t)y0 * W + x0];
    for (int iy = y0; iy < y1; ++iy)
      for (int ix = x0; ix < x1; ++ix) {
        const float v = xm[(size_t)iy * W + ix];
        if (best < v)
          best = v;
      }
    y[i] = best;
  }
}

// The same for the 3 x 3 window, stride 2, padding 1 of residual networks when
// W and Wo are multiples of 4 (16-byte aligned rows): one thread produces four
// adjacent outputs from nine input columns per row (one scalar + two 128-bit
// loads), scanning every window in the reference's order (rows outer, columns
// inner, first maximum wins) so that ties between +0 and -0 resolve alike.
__global__ void __launch_bounds__(kThreads) max_pooling_3x3s2_kernel(const float *__restrict__ x, size_t maps, int H,
                                                                     int W, int Ho, int Wo, float *__restrict__ y) {
  pdl_wait();
  pdl_trigger();
  const int Wo4 = Wo / 4;
  const size_t total = maps * Ho * Wo4;
  const size_t stride = (size_t)gridDim.x * kThreads;
  for (size_t i = (size_t)blockIdx.x * kThreads + threadIdx.x; i < total; i += stride) {
    const int ox4 = (int)(i % Wo4);
    const int oy = (int)((i / Wo4) % Ho);
    const size_t m = i / ((size_t)Wo4 * Ho);
    const int y0 = max(2 * oy - 1, 0), y1 = min(2 * oy + 2, H);
    const float *xm = x + m * (size_t)H * W + 8 * ox4;
    float best[4];
    bool first = true;
    for (int iy = y0; iy < y1; ++iy) {
      const float *row = xm + (size_t)iy * W;
      float r[9];
      r[0] = ox4 > 0 ? __ldg(row - 1) : 0.0f;
      const float4 a = __ldcs(reinterpret_cast<const float4 *>(row));
      const float4 b = __ldcs(reinterpret_cast<const float4 *>(row) + 1);
      r[1] = a.x, r[2] = a.y, r[3] = a.z, r[4] = a.w, r[5] = b.x, r[6] = b.y, r[7] = b.z, r[8] = b.w;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
#pragma unroll
        for (int t = 0; t < 3; ++t) {
          if (j == 0 && t == 0 && ox4 == 0)
            continue; // column -1 is padding
          const float v = r[2 * j + t];
          // the first element of a window initialises it (for j = 0 at the left edge that is t = 1)
          const bool starts = first && (t == 0 || (j == 0 && t == 1 && ox4 == 0));
          if (starts)
            best[j] = v;
          else if (best[j] < v)
            best[j] = v;
        }
      }
      first = false;
    }
    __stcs(reinterpret_cast<float4 *>(y + (m * Ho + oy) * (size_t)Wo) + ox4, make_float4(best[0], best[1], best[2], best[3]));
  }
}

// GlobalAveragePooling (src/nbla/function/generic/global_average_pooling.cpp):
// std::accumulate in ascending order, then one division; one thread per map
// keeps that order.
__global__ void __launch_bounds__(kThreads) global_average_pooling_kernel(const float *__restrict__ x, size_t maps,
                                                                          int S, float *__restrict__ y) {
  pdl_wait();
  pdl_trigger();
  const size_t stride = (size_t)gridDim.x * kThreads;
  for (size_t m = (size_t)blockIdx.x * kThreads + threadIdx.x; m < maps; m += stride) {
    const float *xm = x + m * (size_t)S;
    float s = 0.0f;
    for (int i = 0; i < S; ++i)
      s = __fadd_rn(s, xm[i]);
    y[m] = __fdiv_rn(s, (float)S);
  }
}

// Full-precision Convolution (src/nbla/function/generic/convolution.cpp:160-197)
// for the few-channel network stem: direct convolution on the fp32 pipes.
// Each thread owns PX consecutive output pixels of one output row for OT
// output maps (OT * PX accumulators in registers); the OT filters are staged
// in shared memory tap-major so that one 128-bit broadcast load yields four
// output maps' weights for a tap. Products are accumulated with fused
// multiply-adds in the order of the reference's im2col rows (channel, kernel
// row, kernel column), i.e. at least as accurately as its fp32 product.
template <int OT, int PX>
__global__ void __launch_bounds__(kThreads) direct_conv_kernel(const float *__restrict__ x, const float *__restrict__ w,
                                                               const float *__restrict__ bias, int C, int H, int W,
                                                               int Ko, int kh, int kw, int ph, int pw, int sh, int sw,
                                                               int dh, int dw, int Ho, int Wo, float *__restrict__ y) {
  extern __shared__ float4 s_w4[]; // [C*kh*kw][OT/4] float4: weights of OT maps per tap
  float *s_w = reinterpret_cast<float *>(s_w4);
  const int n = blockIdx.z;
  const int o0 = blockIdx.y * OT;
  const int Kd = C * kh * kw;
  for (int i = threadIdx.x; i < OT * Kd; i += kThreads) {
    const int t = i / Kd, k = i - t * Kd; // read filter-major (coalesced), store tap-major
    s_w[k * OT + t] = (o0 + t < Ko) ? w[(size_t)(o0 + t) * Kd + k] : 0.0f;
  }
  __syncthreads();
  const int groups_x = (Wo + PX - 1) / PX;
  const int g = blockIdx.x * kThreads + threadIdx.x;
  if (g >= Ho * groups_x)
    return;
  const int oy = g / groups_x, ox0 = (g - oy * groups_x) * PX;
  float acc[OT][PX];
#pragma unroll
  for (int t = 0; t < OT; ++t)
#pragma unroll
    for (int p = 0; p < PX; ++p)
      acc[t][p] = 0.0f;
  const float *xn = x + (size_t)n * C * H * W;
  int k = 0;
  for (int c = 0; c < C; ++c)
    for (int ky = 0; ky < kh; ++ky) {
      const int iy = oy * sh - ph + ky * dh;
      const bool row_in = iy >= 0 && iy < H;
      const float *xrow = xn + ((size_t)c * H + (row_in ? iy : 0)) * W;
      for (int kx = 0; kx < kw; ++kx, ++k) {
        float v[PX];
#pragma unroll
        for (int p = 0; p < PX; ++p) {
          const int ix = (ox0 + p) * sw - pw + kx * dw;
          v[p] = (row_in && ix >= 0 && ix < W) ? __ldg(xrow + ix) : 0.0f;
        }
#pragma unroll
        for (int q = 0; q < OT / 4; ++q) {
          const float4 wv = s_w4[k * (OT / 4) + q];
#pragma unroll
          for (int p = 0; p < PX; ++p) {
            acc[4 * q + 0][p] = fmaf(wv.x, v[p], acc[4 * q + 0][p]);
            acc[4 * q + 1][p] = fmaf(wv.y, v[p], acc[4 * q + 1][p]);
            acc[4 * q + 2][p] = fmaf(wv.z, v[p], acc[4 * q + 2][p]);
            acc[4 * q + 3][p] = fmaf(wv.w, v[p], acc[4 * q + 3][p]);
          }
        }
      }
    }
#pragma unroll
  for (int t = 0; t < OT; ++t) {
    const int o = o0 + t;
    if (o >= Ko)
      continue;
    const float b = bias ? bias[o] : 0.0f;
    float *yo = y + (((size_t)n * Ko + o) * Ho + oy) * Wo + ox0;
#pragma unroll
    for (int p = 0; p < PX; ++p)
      if (ox0 + p < Wo)
        yo[p] = bias ? __fadd_rn(acc[t][p], b) : acc[t][p];
  }
}

// The same convolution specialised at compile time for a KW-wide filter with
// horizontal stride SW and no dilation (the ResNet stem: 7 x 7, stride 2): the
// (PX - 1) * SW + KW input values a thread needs from one input row are loaded
// once into registers and reused by every filter column, so the inner loop is
// almost purely fused multiply-adds.
template <int OT, int PX, int KW, int SW>
__global__ void __launch_bounds__(kThreads) direct_conv_window_kernel(const float *__restrict__ x,
                                                                      const float *__restrict__ w,
                                                                      const float *__restrict__ bias, int C, int H,
                                                                      int W, int Ko, int kh, int ph, int pw, int sh,
                                                                      int dh, int Ho, int Wo, float *__restrict__ y) {
  constexpr int WIN = (PX - 1) * SW + KW;
  extern __shared__ float4 s_w4[]; // [C*kh*KW][OT/4]
  float *s_w = reinterpret_cast<float *>(s_w4);
  const int n = blockIdx.z;
  const int o0 = blockIdx.y * OT;
  const int Kd = C * kh * KW;
  for (int i = threadIdx.x; i < OT * Kd; i += kThreads) {
    const int t = i / Kd, k = i - t * Kd;
    s_w[k * OT + t] = (o0 + t < Ko) ? w[(size_t)(o0 + t) * Kd + k] : 0.0f;
  }
  __syncthreads();
  const int groups_x = (Wo + PX - 1) / PX;
  const int g = blockIdx.x * kThreads + threadIdx.x;
  if (g >= Ho * groups_x)
    return;
  const int oy = g / groups_x, ox0 = (g - oy * groups_x) * PX;
  const int ix0 = ox0 * SW - pw;
  float acc[OT][PX];
#pragma unroll
  for (int t = 0; t < OT; ++t)
#pragma unroll
    for (int p = 0; p < PX; ++p)
      acc[t][p] = 0.0f;
  const float *xn = x + (size_t)n * C * H * W;
  int k = 0;
  for (int c = 0; c < C; ++c)
    for (int ky = 0; ky < kh; ++ky, k += KW) {
      const int iy = oy * sh - ph + ky * dh;
      const bool row_in = iy >= 0 && iy < H;
      const float *xrow = xn + ((size_t)c * H + (row_in ? iy : 0)) * W;
      float v[WIN];
#pragma unroll
      for (int i = 0; i < WIN; ++i) {
        const int ix = ix0 + i;
        v[i] = (row_in && ix >= 0 && ix < W) ? __ldg(xrow + ix) : 0.0f;
      }
#pragma unroll
      for (int kx = 0; kx < KW; ++kx) {
#pragma unroll
        for (int q = 0; q < OT / 4; ++q) {
          const float4 wv = s_w4[(k + kx) * (OT / 4) + q];
#pragma unroll
          for (int p = 0; p < PX; ++p) {
            const float xv = v[p * SW + kx];
            acc[4 * q + 0][p] = fmaf(wv.x, xv, acc[4 * q + 0][p]);
            acc[4 * q + 1][p] = fmaf(wv.y, xv, acc[4 * q + 1][p]);
            acc[4 * q + 2][p] = fmaf(wv.z, xv, acc[4 * q + 2][p]);
            acc[4 * q + 3][p] = fmaf(wv.w, xv, acc[4 * q + 3][p]);
          }
        }
      }
    }
#pragma unroll
  for (int t = 0; t < OT; ++t) {
    const int o = o0 + t;
    if (o >= Ko)
      continue;
    const float b = bias ? bias[o] : 0.0f;
    float *yo = y + (((size_t)n * Ko + o) * Ho + oy) * Wo + ox0;
#pragma unroll
    for (int p = 0; p < PX; ++p)
      if (ox0 + p < Wo)
        yo[p] = bias ? __fadd_rn(acc[t][p], b) : acc[t][p];
  }
}

// Tile-staged form of the window kernel for a whole output-row band: the block
// first copies the input rows its band needs into shared memory with coalesced
// loads and explicit zero padding (so the inner loop has no bounds checks and
// no scattered global loads: with per-thread windows the 14-float stride
// between lanes made every load touch 32 sectors and the load/store unit, not
// the FMA pipes, set the pace), then loops over the output maps OT at a time,
// reusing the staged input for all of them. Threads are (band row, pixel
// phase): a thread's PX pixels are Wo / PX apart so that a warp's store covers
// runs of consecutive pixels; weights of all maps sit in shared memory as
// [map group][k][OT].
template <int OT, int PX, int KW, int SW, bool kPairs>
__global__ void __launch_bounds__(kThreads) direct_conv_tile_kernel(const float *__restrict__ x,
                                                                    const float *__restrict__ w,
                                                                    const float *__restrict__ bias, int C, int H, int W,
                                                                    int Ko, int kh, int ph, int pw, int sh, int Ho,
                                                                    int Wo, int rows, int in_rows, int Wp,
                                                                    float *__restrict__ y) {
  constexpr int kLeft = 4;
  extern __shared__ float4 s_all4[];
  float *s_w = reinterpret_cast<float *>(s_all4);   // [Ko / OT][C * kh * KW][OT]
  const int Kd = C * kh * KW;
  const int o_groups = (Ko + OT - 1) / OT;
  float *s_x = s_w + (size_t)o_groups * Kd * OT;     // [C][in_rows][Wp]
  const int n = blockIdx.z;
  const int oy0 = blockIdx.x * rows;
  for (int i = threadIdx.x; i < o_groups * OT * Kd; i += blockDim.x) {
    const int o = i / Kd, k = i - o * Kd;
    s_w[((size_t)(o / OT) * Kd + k) * OT + (o % OT)] = (o < Ko) ? w[(size_t)o * Kd + k] : 0.0f;
  }
  // Input band: image column ix sits at shared column ix + kLeft (kLeft = 4 keeps the
  // 128-bit stores aligned; Wp is a multiple of 4); everything outside the image is zero.
  const float *xn = x + (size_t)n * C * H * W;
  const int iy_base = oy0 * sh - ph;
  const int W4 = W / 4, edge = Wp - kLeft - W; // zero columns right of the image
  for (int i = threadIdx.x; i < C * in_rows * (kLeft + edge); i += blockDim.x) {
    const int e = i % (kLeft + edge), rr = i / (kLeft + edge);
    s_x[(size_t)rr * Wp + (e < kLeft ? e : W + e)] = 0.0f;
  }
#pragma unroll 4
  for (int i = threadIdx.x; i < C * in_rows * W4; i += blockDim.x) {
    const int q = i % W4, rr = i / W4;
    const int r = rr % in_rows, c = rr / in_rows;
    const int iy = iy_base + r;
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (iy >= 0 && iy < H)
      v = __ldg(reinterpret_cast<const float4 *>(xn + ((size_t)c * H + iy) * W) + q);
    *reinterpret_cast<float4 *>(s_x + (size_t)rr * Wp + kLeft + 4 * q) = v;
  }
  __syncthreads();
  // A thread owns the pixels gx, gx + groups_x, gx + 2 groups_x, ... of its row, so
  // that neighbouring lanes store neighbouring pixels (whole sectors per store).
  const int groups_x = Wo / PX;
  const int row_local = threadIdx.x / groups_x, gx = threadIdx.x - row_local * groups_x;
  const int oy = oy0 + row_local;
  if (row_local >= rows || oy >= Ho)
    return;
  for (int og = 0; og < o_groups; ++og) {
    float acc[OT][PX];
#pragma unroll
    for (int t = 0; t < OT; ++t)
#pragma unroll
      for (int p = 0; p < PX; ++p)
        acc[t][p] = 0.0f;
    const float4 *wg = reinterpret_cast<const float4 *>(s_w + (size_t)og * Kd * OT);
    int k = 0;
    for (int c = 0; c < C; ++c)
      for (int ky = 0; ky < kh; ++ky, k += KW) {
        // first input column of pixel ox is ox * SW - pw, i.e. shared column ox * SW + kLeft - pw
        const float *srow = s_x + ((size_t)c * in_rows + row_local * sh + ky) * Wp + gx * SW + (kLeft - pw);
        float v[PX][KW];
#pragma unroll
        for (int p = 0; p < PX; ++p) {
          const float *sp = srow + p * groups_x * SW;
          if (kPairs) {
            // (kLeft - pw) odd and SW even: sp + 1 is 8-byte aligned, so taps 1.. load in pairs
            v[p][0] = sp[0];
#pragma unroll
            for (int kx = 1; kx + 1 < KW; kx += 2) {
              const float2 t2 = *reinterpret_cast<const float2 *>(sp + kx);
              v[p][kx] = t2.x;
              v[p][kx + 1] = t2.y;
            }
            if (KW % 2 == 0)
              v[p][KW - 1] = sp[KW - 1];
          } else {
#pragma unroll
            for (int kx = 0; kx < KW; ++kx)
              v[p][kx] = sp[kx];
          }
        }
#pragma unroll
        for (int kx = 0; kx < KW; ++kx) {
#pragma unroll
          for (int q = 0; q < OT / 4; ++q) {
            const float4 wv = wg[(k + kx) * (OT / 4) + q];
#pragma unroll
            for (int p = 0; p < PX; ++p) {
              const float xv = v[p][kx];
              acc[4 * q + 0][p] = fmaf(wv.x, xv, acc[4 * q + 0][p]);
              acc[4 * q + 1][p] = fmaf(wv.y, xv, acc[4 * q + 1][p]);
              acc[4 * q + 2][p] = fmaf(wv.z, xv, acc[4 * q + 2][p]);
              acc[4 * q + 3][p] = fmaf(wv.w, xv, acc[4 * q + 3][p]);
            }
          }
        }
      }
#pragma unroll
    for (int t = 0; t < OT; ++t) {
      const int o = og * OT + t;
      if (o >= Ko)
        continue;
      const float b = bias ? bias[o] : 0.0f;
      float *yo = y + (((size_t)n * Ko + o) * Ho + oy) * Wo + gx;
#pragma unroll
      for (int p = 0; p < PX; ++p)
        yo[p * groups_x] = bias ? __fadd_rn(acc[t][p], b) : acc[t][p];
    }
  }
}

} // namespace
} // namespace nb200

using namespace nb200;

extern "C" {

int nb200_batch_normalization_inference_f32(const float *x, const float *beta, const float *gamma, const float *mean,
                                            const float *var, float *y, int64_t outer, int64_t channels,
                                            int64_t inner, float eps, void *stream) {
  NB_CHECK(outer >= 0 && channels > 0 && inner > 0, NB200_EVALUE, "bad extents");
  NB_CHECK(channels < (1ll << 31) && inner < (1ll << 31), NB200_EVALUE, "extent exceeds 2^31");
  const size_t total = (size_t)outer * channels * inner;
  if (total == 0)
    return NB200_OK;
  NB_CHECK(x && y && mean && var, NB200_EVALUE, "null data pointer");
  const bool vec = (inner % 4 == 0) && ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y)) & 15) == 0;
  if (vec && inner >= 4 * kThreads && outer * channels < (1ll << 31)) {
    const int S4 = (int)(inner / 4);
    int chunks = (S4 + 4 * kThreads - 1) / (4 * kThreads); // about four float4 per thread
    chunks = chunks > 64 ? 64 : chunks;
    NB_CUDA(launch_dependent(bn_inference_plane_kernel, dim3((unsigned)(outer * channels), (unsigned)chunks),
                             dim3(kThreads), 0, as_stream(stream), x, beta, gamma, mean, var, (int)channels, S4, eps,
                             y));
  } else if (inner >= 32 && inner < 4 * kThreads && outer * channels < (1ll << 31)) {
    const unsigned planes = (unsigned)(outer * channels);
    const dim3 grid((planes + kThreads / 32 - 1) / (kThreads / 32));
    const bool aligned = ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y)) & 15) == 0;
    if (vec)
      NB_CUDA(launch_dependent(bn_inference_warp_kernel<true>, grid, dim3(kThreads), 0, as_stream(stream), x, beta, gamma,
                               mean, var, planes, (int)channels, (int)inner, eps, y));
    else if (aligned && planes % 4 == 0)
      NB_CUDA(launch_dependent(bn_inference_warp4_kernel, dim3((planes / 4 + kThreads / 32 - 1) / (kThreads / 32)),
                               dim3(kThreads), 0, as_stream(stream), x, beta, gamma, mean, var, planes / 4,
                               (int)channels, (int)inner, eps, y));
    else
      NB_CUDA(launch_dependent(bn_inference_warp_kernel<false>, grid, dim3(kThreads), 0, as_stream(stream), x, beta,
                               gamma, mean, var, planes, (int)channels, (int)inner, eps, y));
  } else if (vec)
    NB_CUDA(launch_dependent(bn_inference_kernel<true>, dim3(grid_for(total / 4, 2)), dim3(kThreads), 0,
                             as_stream(stream), x, beta, gamma, mean, var, total, (int)channels, (int)inner, eps, y));
  else
    NB_CUDA(launch_dependent(bn_inference_kernel<false>, dim3(grid_for(total, 4)), dim3(kThreads), 0,
                             as_stream(stream), x, beta, gamma, mean, var, total, (int)channels, (int)inner, eps, y));
  return NB200_OK;
}

int nb200_relu_f32(const float *x, float *y, size_t size, void *stream) {
  if (size == 0)
    return NB200_OK;
  NB_CHECK(x && y, NB200_EVALUE, "null data pointer");
  const bool vec = ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y)) & 15) == 0;
  const float *none = nullptr;
  if (vec)
    NB_CUDA(launch_dependent(unary_binary_kernel<0, true>, dim3(grid_for(size / 4 + 1, 2)), dim3(kThreads), 0,
                             as_stream(stream), x, none, size, y));
  else
    NB_CUDA(launch_dependent(unary_binary_kernel<0, false>, dim3(grid_for(size, 4)), dim3(kThreads), 0,
                             as_stream(stream), x, none, size, y));
  return NB200_OK;
}

namespace nb200 {
namespace {
__global__ void __launch_bounds__(kThreads) scale_kernel(float *__restrict__ x, size_t total, float factor) {
  const size_t stride = (size_t)gridDim.x * kThreads;
  for (size_t i = (size_t)blockIdx.x * kThreads + threadIdx.x; i < total; i += stride)
    x[i] = __fmul_rn(x[i], factor);
}
} // namespace
} // namespace nb200

int nb200_scale_f32(float *x, size_t size, float factor, void *stream) {
  if (size == 0)
    return NB200_OK;
  NB_CHECK(x != nullptr, NB200_EVALUE, "null data pointer");
  scale_kernel<<<grid_for(size, 4), kThreads, 0, as_stream(stream)>>>(x, size, factor);
  NB_LAUNCH_CHECK();
  return NB200_OK;
}

int nb200_add2_f32(const float *a, const float *b, float *y, size_t size, void *stream) {
  if (size == 0)
    return NB200_OK;
  NB_CHECK(a && b && y, NB200_EVALUE, "null data pointer");
  const bool vec =
      ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b) | reinterpret_cast<uintptr_t>(y)) & 15) == 0;
  if (vec)
    NB_CUDA(launch_dependent(unary_binary_kernel<1, true>, dim3(grid_for(size / 4 + 1, 2)), dim3(kThreads), 0,
                             as_stream(stream), a, b, size, y));
  else
    NB_CUDA(launch_dependent(unary_binary_kernel<1, false>, dim3(grid_for(size, 4)), dim3(kThreads), 0,
                             as_stream(stream), a, b, size, y));
  return NB200_OK;
}

int nb200_max_pooling_f32(const float *x, float *y, int64_t maps, int height, int width, int kernel_h, int kernel_w,
                          int stride_h, int stride_w, int pad_h, int pad_w, int ignore_border, void *stream) {
  NB_CHECK(maps >= 0 && height > 0 && width > 0 && kernel_h > 0 && kernel_w > 0 && stride_h > 0 && stride_w > 0 &&
               pad_h >= 0 && pad_w >= 0,
           NB200_EVALUE, "bad pooling geometry");
  // Output extent: src/nbla/function/utils/base_pooling.cpp:59.
  const int Ho = (height + pad_h - (ignore_border ? kernel_h - pad_h : 1)) / stride_h + 1;
  const int Wo = (width + pad_w - (ignore_border ? kernel_w - pad_w : 1)) / stride_w + 1;
  NB_CHECK(Ho > 0 && Wo > 0, NB200_EVALUE, "pooling output would be empty");
  const size_t total = (size_t)maps * Ho * Wo;
  if (total == 0)
    return NB200_OK;
  NB_CHECK(x && y, NB200_EVALUE, "null data pointer");
  const bool fast = kernel_h == 3 && kernel_w == 3 && stride_h == 2 && stride_w == 2 && pad_h == 1 && pad_w == 1 &&
                    width % 4 == 0 && Wo % 4 == 0 && 2 * Wo == width &&
                    ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y)) & 15) == 0;
  if (fast)
    NB_CUDA(launch_dependent(max_pooling_3x3s2_kernel, dim3(grid_for(total / 4, 1)), dim3(kThreads), 0,
                             as_stream(stream), x, (size_t)maps, height, width, Ho, Wo, y));
  else
    NB_CUDA(launch_dependent(max_pooling_kernel, dim3(grid_for(total, 2)), dim3(kThreads), 0, as_stream(stream), x,
                             (size_t)maps, height, width, Ho, Wo, kernel_h, kernel_w, stride_h, stride_w, pad_h, pad_w,
                             y));
  return NB200_OK;
}

int nb200_global_average_pooling_f32(const float *x, float *y, int64_t maps, int64_t spatial, void *stream) {
  NB_CHECK(maps >= 0 && spatial > 0 && spatial < (1ll << 31), NB200_EVALUE, "bad extents");
  if (maps == 0)
    return NB200_OK;
  NB_CHECK(x && y, NB200_EVALUE, "null data pointer");
  NB_CUDA(launch_dependent(global_average_pooling_kernel, dim3(grid_for((size_t)maps)), dim3(kThreads), 0,
                           as_stream(stream), x, (size_t)maps, (int)spatial, y));
  return NB200_OK;
}

int nb200_convolution_relu_fxp_codes_nhwc(const float *x, const float *w, const float *bias, int8_t *y_codes,
                                          int batch, int channels, int height, int width, int outmaps, int kernel_h,
                                          int kernel_w, int pad_h, int pad_w, int stride_h, int stride_w, int relu,
                                          int sign, int n, float delta, void *stream) {
  NB_CHECK(batch > 0 && channels > 0 && height > 0 && width > 0 && outmaps > 0 && kernel_h > 0 && kernel_w > 0,
           NB200_EVALUE, "empty convolution operand");
  NB_CHECK(stride_h > 0 && stride_w > 0 && pad_h >= 0 && pad_w >= 0, NB200_EVALUE,
           "stride must be positive, pad non-negative");
  const int eh = height + 2 * pad_h - kernel_h, ew = width + 2 * pad_w - kernel_w;
  NB_CHECK(eh >= 0 && ew >= 0, NB200_EVALUE, "Invalid configuration of convolution.");
  const int Ho = eh / stride_h + 1, Wo = ew / stride_w + 1;
  NB_CHECK(x && w && y_codes, NB200_EVALUE, "null data pointer");
  NB_CHECK((reinterpret_cast<uintptr_t>(y_codes) & 15) == 0, NB200_EVALUE, "the code tensor must be 16-byte aligned");
  // the quantizer's setup (fixed_point_quantize.cpp:31-42); codes are stored as int8
  NB_CHECK(n > 0 && delta > 0.f, NB200_EVALUE, "Both bit width and delta should be positive.");
  const int nn = sign ? n - 1 : n;
  NB_CHECK(nn > 0 && nn <= 7, NB200_ENOTIMPL, "codes need 0 < n - sign <= 7 (they are stored as int8)");
  int ex = 0;
  NB_CHECK(std::frexp(delta, &ex) == 0.5f && ex > -100 && ex < 100, NB200_ENOTIMPL,
           "a power-of-two quantizer step is needed (got %g)", delta);
  NB_CHECK(relu || sign, NB200_ENOTIMPL, "an unsigned quantizer without ReLU is not supported");
  NB_CHECK(narrow_conv_applies(x, channels, height, width, outmaps, kernel_h, kernel_w, pad_w, stride_w, 1, 1, 1, Wo),
           NB200_ENOTIMPL,
           "the fused full-precision convolution is for inputs with few channels (at most 8 / stride_w, stride_w 1 "
           "or 2, kernel_h * ceil(kernel_w / (2 * stride_w)) <= 16, at most 64 maps and 128 output columns)");
  const int kmax = (1 << nn) - 1;
  const int64_t c_pad = (outmaps + 15) / 16 * 16;
  const int slots = (int)(c_pad < 64 ? 64 : c_pad);
  return narrow_conv_tc(x, w, bias, nullptr, batch, channels, height, width, outmaps, kernel_h, kernel_w, pad_h,
                        pad_w, stride_h, stride_w, Ho, Wo, as_stream(stream), y_codes, slots, relu, kmax,
                        sign ? -kmax : 0, delta);
}

int nb200_convolution_f32(const float *x, const float *w, const float *bias, float *y, int batch, int channels,
                          int height, int width, int outmaps, int kernel_h, int kernel_w, int pad_h, int pad_w,
                          int stride_h, int stride_w, int dilation_h, int dilation_w, int group, void *stream) {
  NB_CHECK(batch > 0 && channels > 0 && height > 0 && width > 0 && outmaps > 0 && kernel_h > 0 && kernel_w > 0,
           NB200_EVALUE, "empty convolution operand");
  NB_CHECK(group == 1, NB200_ENOTIMPL, "the full-precision convolution supports group == 1 only (got %d)", group);
  NB_CHECK(stride_h > 0 && stride_w > 0 && dilation_h > 0 && dilation_w > 0 && pad_h >= 0 && pad_w >= 0, NB200_EVALUE,
           "stride and dilation must be positive, pad non-negative");
  const int eh = height + 2 * pad_h - (dilation_h * (kernel_h - 1) + 1);
  const int ew = width + 2 * pad_w - (dilation_w * (kernel_w - 1) + 1);
  NB_CHECK(eh >= 0 && ew >= 0, NB200_EVALUE, "Invalid configuration of convolution.");
  const int Ho = eh / stride_h + 1, Wo = ew / stride_w + 1;
  NB_CHECK(x && w && y, NB200_EVALUE, "null data pointer");
  if (narrow_conv_applies(x, channels, height, width, outmaps, kernel_h, kernel_w, pad_w, stride_w, dilation_h,
                          dilation_w, group, Wo))
    return narrow_conv_tc(x, w, bias, y, batch, channels, height, width, outmaps, kernel_h, kernel_w, pad_h, pad_w,
                          stride_h, stride_w, Ho, Wo, as_stream(stream));
  constexpr int OT = 16, PX = 4;
  const size_t smem = (size_t)OT * channels * kernel_h * kernel_w * sizeof(float);
  NB_CHECK(smem <= 48 * 1024, NB200_ENOTIMPL,
           "the direct full-precision convolution is meant for few input channels (C*kh*kw = %d is too large)",
           channels * kernel_h * kernel_w);
  NB_CHECK(batch <= 65535 && (outmaps + OT - 1) / OT <= 65535, NB200_ENOTIMPL, "grid extent exceeds 65535");
  const int groups = Ho * ((Wo + PX - 1) / PX);
  const dim3 grid((groups + kThreads - 1) / kThreads, (outmaps + OT - 1) / OT, batch);
  if (kernel_w == 7 && stride_w == 2 && dilation_w == 1) {
    // Seven pixels per thread when the output width allows it: fewer shared-memory
    // weight reads per multiply-add (the limiter with four), no idle lanes at Wo = 112.
    // Whole bands of output rows per block with the input staged in shared memory, when
    // the pixel groups of a band fill the block and the staged rows fit.
    if (Wo % 7 == 0 && dilation_h == 1 && Wo / 7 <= kThreads) {
      constexpr int PX7 = 7;
      const int groups_x = Wo / PX7;
      // (128-thread blocks, two per SM, were slower: every block stages all the weights again)
      const int block_threads = kThreads;
      int rows = block_threads / groups_x;
      rows = rows > Ho ? Ho : rows;
      const int in_rows = (rows - 1) * stride_h + kernel_h;
      // shared row: 4 zero columns, the image row, then zeros up to the last column any window reads
      int Wp = 4 + width;
      if (Wp < (Wo - 1) * 2 + 7 + 4 - pad_w)
        Wp = (Wo - 1) * 2 + 7 + 4 - pad_w;
      Wp = (Wp + 3) / 4 * 4;
      const int o_groups = (outmaps + OT - 1) / OT;
      const size_t tile_smem = ((size_t)o_groups * OT * channels * kernel_h * 7 + (size_t)channels * in_rows * Wp) *
                               sizeof(float);
      // (weights take o_groups * OT * C * kh * 7 floats, a multiple of 4: the band stays 16-byte aligned)
      if (tile_smem <= 200 * 1024 && (Ho + rows - 1) / rows <= 65535 && pad_w <= 4 && width % 4 == 0 &&
          (reinterpret_cast<uintptr_t>(x) & 15) == 0) {
        // taps pair up into 64-bit shared loads when the first tap of every pixel sits at an odd column
        const bool pairs = ((4 - pad_w) & 1) == 1;
        auto kernel = pairs ? direct_conv_tile_kernel<OT, PX7, 7, 2, true> : direct_conv_tile_kernel<OT, PX7, 7, 2, false>;
        static bool configured[64][2];
        int dev = 0;
        NB_CUDA(cudaGetDevice(&dev));
        if (!configured[dev & 63][pairs]) {
          NB_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
          configured[dev & 63][pairs] = true;
        }
        const dim3 grid_t((Ho + rows - 1) / rows, 1, batch);
        kernel<<<grid_t, block_threads, tile_smem, as_stream(stream)>>>(x, w, bias, channels, height, width, outmaps,
                                                                  kernel_h, pad_h, pad_w, stride_h, Ho, Wo, rows,
                                                                  in_rows, Wp, y);
        NB_LAUNCH_CHECK();
        return NB200_OK;
      }
    }
    if (Wo % 7 == 0) {
      constexpr int PX7 = 7;
      const int groups7 = Ho * (Wo / PX7);
      const dim3 grid7((groups7 + kThreads - 1) / kThreads, (outmaps + OT - 1) / OT, batch);
      direct_conv_window_kernel<OT, PX7, 7, 2><<<grid7, kThreads, smem, as_stream(stream)>>>(
          x, w, bias, channels, height, width, outmaps, kernel_h, pad_h, pad_w, stride_h, dilation_h, Ho, Wo, y);
    } else {
      direct_conv_window_kernel<OT, PX, 7, 2><<<grid, kThreads, smem, as_stream(stream)>>>(
          x, w, bias, channels, height, width, outmaps, kernel_h, pad_h, pad_w, stride_h, dilation_h, Ho, Wo, y);
    }
    NB_LAUNCH_CHECK();
    return NB200_OK;
  }
  direct_conv_kernel<OT, PX><<<grid, kThreads, smem, as_stream(stream)>>>(x, w, bias, channels, height, width, outmaps,
                                                                      kernel_h, kernel_w, pad_h, pad_w, stride_h,
                                                                      stride_w, dilation_h, dilation_w, Ho, Wo, y);
  NB_LAUNCH_CHECK();
  return NB200_OK;
}
}
