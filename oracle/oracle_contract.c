/* CPU restatement of the reference's contraction functions (Affine,
 * Convolution) and of the companion functions a binary-weight ResNet-18
 * graph needs, in plain C.
 *
 * TEST INFRASTRUCTURE ONLY: the checker for the CUDA path; never linked into
 * the product library.
 *
 * Parity status: the reference performs these products with Eigen 3.3.5
 * (include/nbla/utils/eigen.hpp:21, pinned only by download URL in
 * third_party/CMakeLists.txt:52, not vendored and absent here), so bitwise
 * parity of the fp32 summation order is UNPINNED; tolerance parity is pinned
 * by the reference's own tests (python/test/function/test_affine.py,
 * test_convolution.py, refs.py:70-92). Each product here accumulates in fp32
 * in ascending-k order; the *_f64 variants accumulate in double and are used
 * to report how far both the oracle and the GPU are from the true product.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

/* src/nbla/function/generic/affine.cpp:80-96: y[M,N] = x[M,K] * w[K,N] (+ b[N]),
 * all row-major; the bias is added after the product (one extra rounding). */
void oracle_affine(const float *x, const float *w, const float *b, int64_t M,
                   int64_t K, int64_t N, float *y) {
  for (int64_t i = 0; i < M; ++i) {
    float *yr = y + i * N;
    for (int64_t j = 0; j < N; ++j)
      yr[j] = 0.f;
    for (int64_t k = 0; k < K; ++k) {
      const float a = x[i * K + k];
      const float *wr = w + k * N;
      for (int64_t j = 0; j < N; ++j)
        yr[j] += a * wr[j];
    }
    if (b)
      for (int64_t j = 0; j < N; ++j)
        yr[j] += b[j];
  }
}

void oracle_affine_f64(const float *x, const float *w, const float *b,
                       int64_t M, int64_t K, int64_t N, double *y) {
  for (int64_t i = 0; i < M; ++i) {
    double *yr = y + i * N;
    for (int64_t j = 0; j < N; ++j)
      yr[j] = 0.;
    for (int64_t k = 0; k < K; ++k) {
      const double a = x[i * K + k];
      const float *wr = w + k * N;
      for (int64_t j = 0; j < N; ++j)
        yr[j] += a * (double)wr[j];
    }
    if (b)
      for (int64_t j = 0; j < N; ++j)
        yr[j] += (double)b[j];
  }
}

/* 2-D im2col of one sample, the layout of
 * src/nbla/utils/unfold_to_patches.cpp:103-194: col[(c*kh + ky)*kw + kx][oy*Wo + ox]. */
static void im2col(const float *x, float *col, int C, int H, int W, int kh,
                   int kw, int ph, int pw, int sh, int sw, int dh, int dw,
                   int Ho, int Wo) {
  for (int c = 0; c < C; ++c)
    for (int ky = 0; ky < kh; ++ky)
      for (int kx = 0; kx < kw; ++kx) {
        float *row = col + (((int64_t)c * kh + ky) * kw + kx) * Ho * Wo;
        for (int oy = 0; oy < Ho; ++oy) {
          int iy = oy * sh - ph + ky * dh;
          for (int ox = 0; ox < Wo; ++ox) {
            int ix = ox * sw - pw + kx * dw;
            row[oy * Wo + ox] = (iy >= 0 && iy < H && ix >= 0 && ix < W)
                                    ? x[((int64_t)c * H + iy) * W + ix]
                                    : 0.f;
          }
        }
      }
}

/* src/nbla/function/generic/convolution.cpp:160-197, 2-D, NCHW: for each
 * sample, im2col then per group y_g[Ko/g, Ho*Wo] = w_g[Ko/g, Cg*kh*kw] * col_g,
 * then the bias is added per output map. Returns 0 or -1 (bad geometry). */
int oracle_convolution(const float *x, const float *w, const float *b, int N,
                       int C, int H, int W, int Ko, int kh, int kw, int ph,
                       int pw, int sh, int sw, int dh, int dw, int group,
                       float *y, int use_f64, double *y64) {
  int Ho = (H + 2 * ph - (dh * (kh - 1) + 1)) / sh + 1;
  int Wo = (W + 2 * pw - (dw * (kw - 1) + 1)) / sw + 1;
  if (Ho <= 0 || Wo <= 0 || C % group || Ko % group)
    return -1;
  int Cg = C / group, Kg = Ko / group;
  int64_t P = (int64_t)Ho * Wo, Kd = (int64_t)Cg * kh * kw;
  float *col = (float *)malloc(sizeof(float) * (size_t)(Kd * group * P));
  if (!col)
    return -1;
  for (int n = 0; n < N; ++n) {
    im2col(x + (int64_t)n * C * H * W, col, C, H, W, kh, kw, ph, pw, sh, sw, dh,
           dw, Ho, Wo);
    for (int g = 0; g < group; ++g) {
      const float *cg = col + (int64_t)g * Kd * P;
      const float *wg = w + (int64_t)g * Kg * Kd;
      for (int o = 0; o < Kg; ++o) {
        int64_t oo = (int64_t)g * Kg + o;
        if (!use_f64) {
          float *yr = y + ((int64_t)n * Ko + oo) * P;
          for (int64_t p = 0; p < P; ++p)
            yr[p] = 0.f;
          for (int64_t k = 0; k < Kd; ++k) {
            const float a = wg[o * Kd + k];
            const float *cr = cg + k * P;
            for (int64_t p = 0; p < P; ++p)
              yr[p] += a * cr[p];
          }
          if (b)
            for (int64_t p = 0; p < P; ++p)
              yr[p] += b[oo];
        } else {
          double *yr = y64 + ((int64_t)n * Ko + oo) * P;
          for (int64_t p = 0; p < P; ++p)
            yr[p] = 0.;
          for (int64_t k = 0; k < Kd; ++k) {
            const double a = wg[o * Kd + k];
            const float *cr = cg + k * P;
            for (int64_t p = 0; p < P; ++p)
              yr[p] += a * (double)cr[p];
          }
          if (b)
            for (int64_t p = 0; p < P; ++p)
              yr[p] += (double)b[oo];
        }
      }
    }
  }
  free(col);
  return 0;
}

/* src/nbla/function/generic/batch_normalization.cpp:228-260 (inference,
 * channel axis 1): y = (x - mean) * gamma / sqrt(var + eps) + beta, in that
 * operation order. x is [N, C, S]. */
void oracle_batch_norm_inference(const float *x, const float *beta,
                                 const float *gamma, const float *mean,
                                 const float *var, int64_t N, int64_t C,
                                 int64_t S, float eps, float *y) {
  for (int64_t c = 0; c < C; ++c) {
    const float stdvar = sqrtf(var[c] + eps);
    const float scale = gamma ? gamma[c] : 1.f;
    const float bias = beta ? beta[c] : 0.f;
    for (int64_t n = 0; n < N; ++n)
      for (int64_t s = 0; s < S; ++s) {
        int64_t i = (n * C + c) * S + s;
        float t = x[i] - mean[c];
        t = t * scale;
        t = t / stdvar;
        y[i] = t + bias;
      }
  }
}

/* src/nbla/function/generic/relu.cpp: y = max(0, x). */
void oracle_relu(const float *x, float *y, int64_t n) {
  for (int64_t i = 0; i < n; ++i)
    y[i] = x[i] > 0.f ? x[i] : 0.f;
}

/* src/nbla/function/generic/add2.cpp (same-shape case). */
void oracle_add2(const float *a, const float *b, float *y, int64_t n) {
  for (int64_t i = 0; i < n; ++i)
    y[i] = a[i] + b[i];
}

/* Output extent of one pooled axis,
 * src/nbla/function/utils/base_pooling.cpp:59. */
int oracle_pool_out(int w, int k, int s, int p, int ignore_border) {
  return (w + p - (ignore_border ? k - p : 1)) / s + 1;
}

/* src/nbla/function/generic/max_pooling.cpp (2-D forward_map): window clipped
 * to the input, maximum over the valid taps. x is [maps, H, W]. */
void oracle_max_pooling(const float *x, int64_t maps, int H, int W, int kh,
                        int kw, int sh, int sw, int ph, int pw,
                        int ignore_border, float *y) {
  int Ho = oracle_pool_out(H, kh, sh, ph, ignore_border);
  int Wo = oracle_pool_out(W, kw, sw, pw, ignore_border);
  for (int64_t m = 0; m < maps; ++m)
    for (int oy = 0; oy < Ho; ++oy)
      for (int ox = 0; ox < Wo; ++ox) {
        int y0 = oy * sh - ph, x0 = ox * sw - pw;
        int y1 = y0 + kh < H ? y0 + kh : H, x1 = x0 + kw < W ? x0 + kw : W;
        if (y0 < 0)
          y0 = 0;
        if (x0 < 0)
          x0 = 0;
        float best = x[(m * H + y0) * W + x0];
        for (int iy = y0; iy < y1; ++iy)
          for (int ix = x0; ix < x1; ++ix) {
            float v = x[(m * H + iy) * W + ix];
            if (best < v)
              best = v;
          }
        y[(m * Ho + oy) * Wo + ox] = best;
      }
}

/* src/nbla/function/generic/global_average_pooling.cpp: mean over the
 * spatial extent, sum in ascending order then one division. */
void oracle_global_average_pooling(const float *x, int64_t maps, int64_t S,
                                   float *y) {
  for (int64_t m = 0; m < maps; ++m) {
    float s = 0.f;
    for (int64_t i = 0; i < S; ++i)
      s += x[m * S + i];
    y[m] = s / S;
  }
}
