// Operand preparation for the convolution backward passes. Both passes run on
// the implicit-GEMM contraction kernel of the forward; these kernels only
// bring the gradients and activations into the layouts that kernel reads.
//
//   input gradient:  dx = conv(dy stuffed with the forward stride, flipped
//                    and transposed weights)          -> dy_to_nhwc_stuffed,
//                                                        flip_transpose_weights
//   weight gradient: dW[o, c, ky, kx] = sum over (n, oy, ox) = a convolution of
//                    x^T (batch as the channel axis) with dy^T as the filter,
//                    stride and dilation exchanged     -> batch_to_inner
//   bias gradient:   sums of dy over batch and pixels  -> channel_sums
#include <cuda_bf16.h>

#include "prepare.cuh"

namespace nb200 {
namespace {

__device__ __forceinline__ void split3(float v, __nv_bfloat16 &h, __nv_bfloat16 &m, __nv_bfloat16 &l) {
  h = __float2bfloat16_rn(v);
  const float r1 = __fsub_rn(v, __bfloat162float(h));
  m = __float2bfloat16_rn(r1);
  const float r2 = __fsub_rn(r1, __bfloat162float(m));
  l = __float2bfloat16_rn(r2);
}

// dy [N][Ko][Ho][Wo] fp32 -> three bf16 planes [N][Hs][Ws][ctot]: map o of group g
// lands at slot g * k_pad_g + (o - g * Kog), pixel (oy, ox) at (oy * sh, ox * sw);
// every other position of the (pre-zeroed) output stays zero. chan_scale (per
// map, may be NULL) is multiplied in first with one rounding: dy * alpha.
__global__ void __launch_bounds__(256) dy_to_nhwc_stuffed_kernel(const float *__restrict__ dy, int Ko, int Ho, int Wo,
                                                                 int groups, int Kog, int k_pad_g, int ctot, int Hs,
                                                                 int Ws, int sh, int sw,
                                                                 const float *__restrict__ chan_scale,
                                                                 __nv_bfloat16 *__restrict__ out,
                                                                 int64_t plane_stride) {
  __shared__ float tile[32][33];
  const int n = blockIdx.z;
  const int HW = Ho * Wo;
  const int p0 = blockIdx.x * 32, d0 = blockIdx.y * 32;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  for (int dd = ty; dd < 32; dd += 8) {
    const int d = d0 + dd, p = p0 + tx;
    const int g = d / k_pad_g, oo = d - g * k_pad_g;
    float v = 0.0f;
    if (d < ctot && g < groups && oo < Kog && p < HW) {
      const int o = g * Kog + oo;
      v = dy[((int64_t)n * Ko + o) * HW + p];
      if (chan_scale)
        v = __fmul_rn(v, chan_scale[o]);
    }
    tile[dd][tx] = v;
  }
  __syncthreads();
  for (int pp = ty; pp < 32; pp += 8) {
    const int p = p0 + pp, d = d0 + tx;
    if (p < HW && d < ctot) {
      const int oy = p / Wo, ox = p - oy * Wo;
      const int64_t dst = (((int64_t)n * Hs + (int64_t)oy * sh) * Ws + (int64_t)ox * sw) * ctot + d;
      __nv_bfloat16 h, m, l;
      split3(tile[tx][pp], h, m, l);
      out[dst] = h;
      out[plane_stride + dst] = m;
      out[2 * plane_stride + dst] = l;
    }
  }
}

// wb [Ko][Cg][kh][kw] fp32 -> side [planes][C][kh * kw][k_slots] bf16:
// side[g * Cg + c][ky * kw + kx][o] = wb[g * Kog + o][c][kh - 1 - ky][kw - 1 - kx]; one plane for values
// exact in bf16 (binary weights), three (hi, mid, lo) for full-precision weights.
template <int PLANES>
__global__ void flip_transpose_weights_kernel(const float *__restrict__ wb, int Ko, int Cg, int kh, int kw, int Kog,
                                              int k_slots, __nv_bfloat16 *__restrict__ side, int64_t plane_stride) {
  const int taps = kh * kw;
  const int64_t total = (int64_t)Ko * Cg * taps;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int t = (int)(i % taps);
    const int c = (int)((i / taps) % Cg);
    const int o = (int)(i / ((int64_t)taps * Cg));
    const int g = o / Kog, oo = o - g * Kog;
    const int ky = t / kw, kx = t - ky * kw;
    const int tf = (kh - 1 - ky) * kw + (kw - 1 - kx);
    const int64_t dst = ((int64_t)(g * Cg + c) * taps + tf) * k_slots + oo;
    if (PLANES == 1) {
      side[dst] = __float2bfloat16_rn(wb[i]);
    } else {
      __nv_bfloat16 h, m, l;
      split3(wb[i], h, m, l);
      side[dst] = h;
      side[dst + plane_stride] = m;
      side[dst + 2 * plane_stride] = l;
    }
  }
}

// src: N rows of R values, rows src_row_stride apart -> out [planes][R][Np] bf16
// (the batch index becomes the innermost axis; positions n >= N stay zero in
// the pre-zeroed output). Tile transpose through shared memory.
template <int PLANES>
__global__ void __launch_bounds__(256) batch_to_inner_kernel(const float *__restrict__ src, int N, int64_t R,
                                                             int64_t src_row_stride, int Np,
                                                             __nv_bfloat16 *__restrict__ out, int64_t plane_stride) {
  __shared__ float tile[32][33];
  const int64_t r0 = (int64_t)blockIdx.x * 32;
  const int n0 = blockIdx.y * 32;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  for (int nn = ty; nn < 32; nn += 8) {
    const int n = n0 + nn;
    const int64_t r = r0 + tx;
    tile[nn][tx] = (n < N && r < R) ? src[(int64_t)n * src_row_stride + r] : 0.0f;
  }
  __syncthreads();
  for (int rr = ty; rr < 32; rr += 8) {
    const int64_t r = r0 + rr;
    const int n = n0 + tx;
    if (r < R && n < N) {
      const int64_t dst = r * Np + n;
      __nv_bfloat16 h, m, l;
      split3(tile[tx][rr], h, m, l);
      out[dst] = h;
      if (PLANES > 1)
        out[plane_stride + dst] = m;
      if (PLANES > 2)
        out[2 * plane_stride + dst] = l;
    }
  }
}

// Sums of dy [N][Ko][HW] over n and the pixels, per map (bias gradient,
// convolution.cpp:281-290): block (o, s) adds the images n = s, s + splits, ...;
// a second kernel adds the partials of each map in order.
__global__ void __launch_bounds__(256) channel_partial_sums_kernel(const float *__restrict__ dy, int N, int Ko, int HW,
                                                                   float *__restrict__ partial) {
  const int o = blockIdx.x, s = blockIdx.y, splits = gridDim.y;
  float acc = 0.0f;
  for (int n = s; n < N; n += splits) {
    const float *p = dy + ((int64_t)n * Ko + o) * HW;
    for (int i = threadIdx.x; i < HW; i += 256)
      acc += p[i];
  }
  __shared__ float red[256];
  red[threadIdx.x] = acc;
  __syncthreads();
  for (int d = 128; d > 0; d >>= 1) {
    if ((int)threadIdx.x < d)
      red[threadIdx.x] += red[threadIdx.x + d];
    __syncthreads();
  }
  if (threadIdx.x == 0)
    partial[(int64_t)s * Ko + o] = red[0];
}

__global__ void channel_finish_kernel(const float *__restrict__ partial, int Ko, int splits, float *__restrict__ out,
                                      int accumulate) {
  const int o = blockIdx.x * blockDim.x + threadIdx.x;
  if (o >= Ko)
    return;
  float s = 0.0f;
  for (int k = 0; k < splits; ++k)
    s += partial[(int64_t)k * Ko + o];
  out[o] = accumulate ? __fadd_rn(out[o], s) : s;
}

// staged [splits][Cg][Kog][taps] (the contraction's NCHW-shaped output with the
// input channel as the image axis, one partial result per K split) ->
// dW[o][c][taps]: the splits are added in order, then dW is overwritten or added to.
__global__ void permute_weight_grad_kernel(const float *__restrict__ staged, int splits, int Cg, int Kog, int taps,
                                           float *__restrict__ dw, int accumulate) {
  const int64_t total = (int64_t)Cg * Kog * taps;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int t = (int)(i % taps);
    const int c = (int)((i / taps) % Cg);
    const int o = (int)(i / ((int64_t)taps * Cg));
    float v = 0.0f;
    for (int k = 0; k < splits; ++k)
      v = __fadd_rn(v, staged[k * total + ((int64_t)c * Kog + o) * taps + t]);
    dw[i] = accumulate ? __fadd_rn(dw[i], v) : v;
  }
}

inline unsigned capped(int64_t work, int threads) {
  int64_t b = (work + threads - 1) / threads;
  const int64_t cap = (int64_t)sm_count() * 32;
  b = b > cap ? cap : b;
  return (unsigned)(b < 1 ? 1 : b);
}

} // namespace

int dy_to_nhwc_stuffed(const float *dy, int N, int Ko, int Ho, int Wo, int groups, int Kog, int k_pad_g, int ctot,
                       int Hs, int Ws, int sh, int sw, const float *chan_scale, void *out, cudaStream_t st) {
  NB_CHECK(N <= 65535, NB200_ENOTIMPL, "batch larger than 65535");
  const dim3 grid((Ho * Wo + 31) / 32, (ctot + 31) / 32, N);
  dy_to_nhwc_stuffed_kernel<<<grid, 256, 0, st>>>(dy, Ko, Ho, Wo, groups, Kog, k_pad_g, ctot, Hs, Ws, sh, sw,
                                                  chan_scale, reinterpret_cast<__nv_bfloat16 *>(out),
                                                  (int64_t)N * Hs * Ws * ctot);
  NB_LAUNCH_CHECK();
  return NB200_OK;
}

int flip_transpose_weights(const float *wb, int Ko, int Cg, int kh, int kw, int groups, int k_slots, void *side,
                           cudaStream_t st, int planes) {
  const int64_t plane_stride = (int64_t)groups * Cg * kh * kw * k_slots;
  if (planes == 3)
    flip_transpose_weights_kernel<3><<<capped((int64_t)Ko * Cg * kh * kw, 256), 256, 0, st>>>(
        wb, Ko, Cg, kh, kw, Ko / groups, k_slots, reinterpret_cast<__nv_bfloat16 *>(side), plane_stride);
  else
    flip_transpose_weights_kernel<1><<<capped((int64_t)Ko * Cg * kh * kw, 256), 256, 0, st>>>(
        wb, Ko, Cg, kh, kw, Ko / groups, k_slots, reinterpret_cast<__nv_bfloat16 *>(side), plane_stride);
  NB_LAUNCH_CHECK();
  return NB200_OK;
}

int batch_to_inner(const float *src, int N, int64_t R, int64_t src_row_stride, int Np, int planes, void *out,
                   cudaStream_t st) {
  NB_CHECK((R + 31) / 32 < (1ll << 31) && (N + 31) / 32 <= 65535, NB200_ENOTIMPL, "tensor too large for the batch transpose");
  const dim3 grid((unsigned)((R + 31) / 32), (unsigned)((N + 31) / 32));
  __nv_bfloat16 *o = reinterpret_cast<__nv_bfloat16 *>(out);
  if (planes == 3)
    batch_to_inner_kernel<3><<<grid, 256, 0, st>>>(src, N, R, src_row_stride, Np, o, R * Np);
  else
    batch_to_inner_kernel<1><<<grid, 256, 0, st>>>(src, N, R, src_row_stride, Np, o, R * Np);
  NB_LAUNCH_CHECK();
  return NB200_OK;
}

int channel_sums(const float *dy, int N, int Ko, int HW, float *out, int accumulate, float *partial, int splits,
                 cudaStream_t st) {
  NB_CHECK(splits >= 1 && splits <= 65535, NB200_EVALUE, "bad split count");
  channel_partial_sums_kernel<<<dim3(Ko, splits), 256, 0, st>>>(dy, N, Ko, HW, partial);
  NB_LAUNCH_CHECK();
  channel_finish_kernel<<<(Ko + 255) / 256, 256, 0, st>>>(partial, Ko, splits, out, accumulate);
  NB_LAUNCH_CHECK();
  return NB200_OK;
}

int permute_weight_grad(const float *staged, int splits, int Cg, int Kog, int taps, float *dw, int accumulate,
                        cudaStream_t st) {
  permute_weight_grad_kernel<<<capped((int64_t)Cg * Kog * taps, 256), 256, 0, st>>>(staged, splits, Cg, Kog, taps, dw,
                                                                                      accumulate);
  NB_LAUNCH_CHECK();
  return NB200_OK;
}

} // namespace nb200
