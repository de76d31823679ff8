// Tensor-core path of the full-precision convolution for inputs with few channels (narrow_conv.cu).
#pragma once
#include "common.cuh"

namespace nb200 {

// Whether the geometry fits the kernel: group 1, no dilation, stride_w 1 or 2 with at most
// 8 / stride_w channels, kernel_h <= 8, kernel_h * ceil(kernel_w / (2 * stride_w)) <= 16, at most 64
// output maps and 128 output columns, padded rows of at most 2560 bytes in fp16 channel slots.
// NNABLA_B200_DIRECT_CONV=1 switches the path off (the CUDA-core kernel then runs).
bool narrow_conv_applies(const float *x, int channels, int height, int width, int outmaps, int kernel_h,
                         int kernel_w, int pad_w, int stride_w, int dilation_h, int dilation_w, int group, int Wo);
// y_codes != NULL: the result leaves as int8 channel-last codes [batch][Ho * Wo][slots] of
// FixedPointQuantize(ReLU(conv + bias)) (ReLU optional; delta a power of two, codes in [kmin, kmax])
// instead of fp32 NCHW in y.
int narrow_conv_tc(const float *x, const float *w, const float *bias, float *y, int batch, int channels, int height,
                   int width, int outmaps, int kernel_h, int kernel_w, int pad_h, int pad_w, int stride_h,
                   int stride_w, int Ho, int Wo, cudaStream_t st, int8_t *y_codes = nullptr, int slots = 0,
                   int relu = 0, int kmax = 0, int kmin = 0, float delta = 1.0f);

} // namespace nb200
