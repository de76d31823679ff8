// The functions a binary-weight ResNet-18 graph needs next to the quantized
// layers, so that the whole graph runs under one context with no CPU
// fallback: BatchNormalization (inference), ReLU, Add2, MaxPooling,
// GlobalAveragePooling and a full-precision Convolution for the network stem.
// All but the convolution are HBM-bound single passes whose arithmetic follows
// the reference's operation order, so their results are bit-identical to its
// CPU code; the convolution accumulates with fused multiply-adds (tolerance
// parity, like the other contractions).
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

// BatchNormalization<T>::forward_impl_global
// (src/nbla/function/generic/batch_normalization.cpp:228-260), channel axis 1:
// y = (x - mean) * gamma / sqrt(var + eps) + beta, each operation rounded.
// x is [N, C, S]; when S % 4 == 0 a thread handles one float4 (one channel).
template <bool kVec>
__global__ void __launch_bounds__(kThreads) bn_inference_kernel(const float *__restrict__ x, const float *beta,
                                                                const float *gamma, const float *mean,
                                                                const float *var, size_t total, int C, int S,
                                                                float eps, float *__restrict__ y) {
  const size_t stride = (size_t)gridDim.x * kThreads;
  if (kVec) {
    const size_t total4 = total / 4;
    const int S4 = S / 4;
    for (size_t i = (size_t)blockIdx.x * kThreads + threadIdx.x; i < total4; i += stride) {
      const int c = (int)((i / S4) % C);
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
    for (size_t i = (size_t)blockIdx.x * kThreads + threadIdx.x; i < total; i += stride) {
      const int c = (int)((i / S) % C);
      const float sd = __fsqrt_rn(__fadd_rn(var[c], eps));
      const float g = gamma ? gamma[c] : 1.0f;
      const float b = beta ? beta[c] : 0.0f;
      y[i] = __fadd_rn(__fdiv_rn(__fmul_rn(__fsub_rn(x[i], mean[c]), g), sd), b);
    }
  }
}

// ReLU (src/nbla/function/generic/relu.cpp): y = max(0, x); Add2 (add2.cpp): y = a + b.
template <int kOp, bool kVec>
__global__ void __launch_bounds__(kThreads) unary_binary_kernel(const float *__restrict__ a,
                                                                const float *__restrict__ b, size_t total,
                                                                float *__restrict__ y) {
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

// GlobalAveragePooling (src/nbla/function/generic/global_average_pooling.cpp):
// std::accumulate in ascending order, then one division; one thread per map
// keeps that order.
__global__ void __launch_bounds__(kThreads) global_average_pooling_kernel(const float *__restrict__ x, size_t maps,
                                                                          int S, float *__restrict__ y) {
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
  if (vec)
    bn_inference_kernel<true><<<grid_for(total / 4, 2), kThreads, 0, as_stream(stream)>>>(
        x, beta, gamma, mean, var, total, (int)channels, (int)inner, eps, y);
  else
    bn_inference_kernel<false><<<grid_for(total, 4), kThreads, 0, as_stream(stream)>>>(
        x, beta, gamma, mean, var, total, (int)channels, (int)inner, eps, y);
  NB_LAUNCH_CHECK();
  return NB200_OK;
}

int nb200_relu_f32(const float *x, float *y, size_t size, void *stream) {
  if (size == 0)
    return NB200_OK;
  NB_CHECK(x && y, NB200_EVALUE, "null data pointer");
  const bool vec = ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y)) & 15) == 0;
  if (vec)
    unary_binary_kernel<0, true><<<grid_for(size / 4 + 1, 2), kThreads, 0, as_stream(stream)>>>(x, nullptr, size, y);
  else
    unary_binary_kernel<0, false><<<grid_for(size, 4), kThreads, 0, as_stream(stream)>>>(x, nullptr, size, y);
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
    unary_binary_kernel<1, true><<<grid_for(size / 4 + 1, 2), kThreads, 0, as_stream(stream)>>>(a, b, size, y);
  else
    unary_binary_kernel<1, false><<<grid_for(size, 4), kThreads, 0, as_stream(stream)>>>(a, b, size, y);
  NB_LAUNCH_CHECK();
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
  max_pooling_kernel<<<grid_for(total, 2), kThreads, 0, as_stream(stream)>>>(
      x, (size_t)maps, height, width, Ho, Wo, kernel_h, kernel_w, stride_h, stride_w, pad_h, pad_w, y);
  NB_LAUNCH_CHECK();
  return NB200_OK;
}

int nb200_global_average_pooling_f32(const float *x, float *y, int64_t maps, int64_t spatial, void *stream) {
  NB_CHECK(maps >= 0 && spatial > 0 && spatial < (1ll << 31), NB200_EVALUE, "bad extents");
  if (maps == 0)
    return NB200_OK;
  NB_CHECK(x && y, NB200_EVALUE, "null data pointer");
  global_average_pooling_kernel<<<grid_for((size_t)maps), kThreads, 0, as_stream(stream)>>>(x, (size_t)maps,
                                                                                          (int)spatial, y);
  NB_LAUNCH_CHECK();
  return NB200_OK;
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
