/* CPU restatement of the reference's backward passes on the quantized-layer
 * path (the quantizers' straight-through estimators and the affine backward
 * the binary layers call), in plain C, one function per reference loop.
 *
 * TEST INFRASTRUCTURE ONLY: the checker the CUDA path is compared against.
 * The product library never links or calls it.
 *
 * Parity status: PINNED against the reference's own compiled C++
 * (oracle/_ref/libnnabla_ref.so, Function::backward) by
 * tests/test_oracle_backward_vs_reference.py: bit for bit for the input gradients; the
 * two range gradients of MinMaxQuantize and the affine backward are fp32 sums
 * whose order inside the reference comes from Eigen (absent), so they are
 * pinned to rounding only.
 *
 * Build: gcc -O2 -fno-fast-math -ffp-contract=off, like oracle_quant.c.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>

/* src/nbla/function/generic/fixed_point_quantize.cpp:69-127. With
 * ste_fine_grained the gradient passes where min <= x <= max and is zero in
 * the clipped regions (written only when not accumulating); without it the
 * gradient passes everywhere. */
void oracle_fixed_point_quantize_backward(const float *x, const float *dy,
                                          float *dx, int64_t size, int sign,
                                          int n, float delta,
                                          int ste_fine_grained, int accum) {
  int nn = sign ? n - 1 : n;
  float max_ = (float)((pow(2, nn) - 1) * delta);
  float min_ = sign ? -max_ : 0.0f;
  for (int64_t s = 0; s < size; ++s) {
    if (ste_fine_grained && (x[s] > max_ || x[s] < min_)) {
      if (!accum)
        dx[s] = 0.0f;
    } else if (accum) {
      dx[s] = dx[s] + dy[s];
    } else {
      dx[s] = dy[s];
    }
  }
}

/* src/nbla/function/generic/pow2_quantize.cpp:84-156. The factor c is 0 where
 * the snapped power of two exceeds p_max and, for unsigned quantization, where
 * x is negative; the product c * dy is formed even when c is 0 (so the sign of
 * a zero gradient and NaN/inf in dy behave like the reference). */
void oracle_pow2_quantize_backward(const float *x, const float *dy, float *dx,
                                   int64_t size, int sign, int with_zero,
                                   int n, int m, int ste_fine_grained,
                                   int accum) {
  (void)with_zero;
  (void)n;
  float p_max = (float)pow(2., m);
  for (int64_t s = 0; s < size; ++s) {
    float c = 1.0f;
    if (ste_fine_grained) {
      float x_abs = fabsf(x[s]);
      float q = powf(2.0f, roundf(log2f(x_abs)));
      if (q > p_max)
        c = 0.0f;
      if (!sign && x[s] < 0.0f)
        c = 0.0f;
      float g = c * dy[s];
      dx[s] = accum ? dx[s] + g : g;
    } else {
      dx[s] = accum ? dx[s] + dy[s] : dy[s];
    }
  }
}

/* src/nbla/function/generic/min_max_quantize.cpp:225-350, after a forward
 * that left the nudged qr_min / qr_max in place. Shapes as in
 * oracle_min_max_quantize. propagate / accum hold the flags of x, qr_min,
 * qr_max in that order. The range gradients exist only when neither
 * x_min_max nor ema is set (:300-301). Returns 0, or -1 on a shape error. */
int oracle_min_max_quantize_backward(const float *x, const int64_t *xs, int nd,
                                     const float *qr_min, const float *qr_max,
                                     const float *ql_min, const float *ql_max,
                                     const int64_t *qs, const float *dy,
                                     int x_min_max, int ema,
                                     int ste_fine_grained,
                                     const int32_t *propagate,
                                     const int32_t *accum, float *dx,
                                     float *g_qr_min, float *g_qr_max) {
  int64_t xsize = 1, qsize = 1, xstr[8], qstr[8];
  if (nd > 8)
    return -1;
  for (int d = nd - 1; d >= 0; --d) {
    if (qs[d] != 1 && qs[d] != xs[d])
      return -1;
    xstr[d] = xsize;
    xsize *= xs[d];
    qstr[d] = (qs[d] == 1) ? 0 : qsize;
    qsize *= qs[d];
  }
  size_t qn = (size_t)(qsize ? qsize : 1);
  float *m = (float *)malloc(sizeof(float) * qn);
  float *M = (float *)malloc(sizeof(float) * qn);
  float *smin = (float *)calloc(qn, sizeof(float));
  float *smax = (float *)calloc(qn, sizeof(float));
  if (!m || !M || !smin || !smax)
    return -1;
  for (int64_t q = 0; q < qsize; ++q) {
    /* scale as the forward left it (:184-186), then nudge_qr_min_max (:362-390) */
    float num = qr_max[q] - qr_min[q];
    float den = ql_max[q] - ql_min[q];
    float scale = num / den;
    float t = qr_min[q] / scale;
    float zp_from_min = ql_min[q] - t;
    float zp;
    if (zp_from_min <= ql_min[q])
      zp = ql_min[q];
    else if (zp_from_min >= ql_max[q])
      zp = ql_max[q];
    else
      zp = roundf(zp_from_min);
    float a = ql_min[q] - zp, b = ql_max[q] - zp;
    m[q] = a * scale;
    M[q] = b * scale;
  }
  const int ranges = !(x_min_max || ema);
  for (int64_t i = 0; i < xsize; ++i) {
    int64_t q = 0, r = i;
    for (int d = 0; d < nd; ++d) {
      int64_t c = r / xstr[d];
      r -= c * xstr[d];
      q += c * qstr[d];
    }
    if (propagate[0]) {
      float g = dy[i];
      if (ste_fine_grained) {
        /* greater_equal * less_equal masks (1 or 0), multiplied with dy */
        float mask = ((x[i] >= m[q]) ? 1.0f : 0.0f) * ((x[i] <= M[q]) ? 1.0f : 0.0f);
        g = mask * dy[i];
      }
      dx[i] = accum[0] ? g + dx[i] : g;
    }
    if (ranges) {
      /* less / greater masks times dy, summed over the axes where q is 1 */
      float lo = ((x[i] < m[q]) ? 1.0f : 0.0f) * dy[i];
      float hi = ((x[i] > M[q]) ? 1.0f : 0.0f) * dy[i];
      smin[q] = smin[q] + lo;
      smax[q] = smax[q] + hi;
    }
  }
  if (ranges) {
    for (int64_t q = 0; q < qsize; ++q) {
      if (propagate[1])
        g_qr_min[q] = accum[1] ? g_qr_min[q] + smin[q] : smin[q];
      if (propagate[2])
        g_qr_max[q] = accum[2] ? g_qr_max[q] + smax[q] : smax[q];
    }
  }
  free(m);
  free(M);
  free(smin);
  free(smax);
  return 0;
}

/* src/nbla/function/generic/affine.cpp:98-138 for row-major x [M,K], w [K,N],
 * dy [M,N]: dx (+)= dy . w^T, dw (+)= x^T . dy, db (+)= column sums of dy. A
 * NULL dx / dw / db is skipped. Each product is summed completely (fp32, or
 * double when f64 != 0 — the error yardstick) before it is added to the
 * buffer, like the reference's `mdx += mdy * mw.transpose()`. Summation order
 * inside the reference is Eigen's (absent): pinned to rounding only. */
void oracle_affine_backward(const float *x, const float *w, const float *dy,
                            float *dx, float *dw, float *db, int64_t M,
                            int64_t K, int64_t N, int accum_dx, int accum_dw,
                            int accum_db, int f64) {
  if (dx)
    for (int64_t i = 0; i < M; ++i)
      for (int64_t k = 0; k < K; ++k) {
        float s = 0.f;
        double d = 0.;
        for (int64_t j = 0; j < N; ++j) {
          s += dy[i * N + j] * w[k * N + j];
          d += (double)dy[i * N + j] * (double)w[k * N + j];
        }
        float v = f64 ? (float)d : s;
        dx[i * K + k] = accum_dx ? dx[i * K + k] + v : v;
      }
  if (dw)
    for (int64_t k = 0; k < K; ++k)
      for (int64_t j = 0; j < N; ++j) {
        float s = 0.f;
        double d = 0.;
        for (int64_t i = 0; i < M; ++i) {
          s += x[i * K + k] * dy[i * N + j];
          d += (double)x[i * K + k] * (double)dy[i * N + j];
        }
        float v = f64 ? (float)d : s;
        dw[k * N + j] = accum_dw ? dw[k * N + j] + v : v;
      }
  if (db)
    for (int64_t j = 0; j < N; ++j) {
      float s = 0.f;
      double d = 0.;
      for (int64_t i = 0; i < M; ++i) {
        s += dy[i * N + j];
        d += (double)dy[i * N + j];
      }
      float v = f64 ? (float)d : s;
      db[j] = accum_db ? db[j] + v : v;
    }
}

/* src/nbla/function/generic/convolution.cpp:199-300 (2-D, NCHW), as direct
 * sums instead of the reference's per-sample im2col + GEMM (same terms; the
 * order of the fp32 additions is Eigen's in the reference and not pinned):
 *   dx[n,c,iy,ix] (+)= sum_{o,ky,kx} dy[n,o,oy,ox] * w[o,c,ky,kx], iy = oy*sh - ph + ky*dh
 *   dw[o,c,ky,kx] (+)= sum_{n,oy,ox} dy[n,o,oy,ox] * x[n,c,iy,ix]
 *   db[o]         (+)= sum_{n,oy,ox} dy[n,o,oy,ox]
 * w has shape [Ko][C/group][kh][kw]. f64 != 0 accumulates in double (the error
 * yardstick). A NULL dx / dw / db is skipped. Returns 0, -1 on a bad shape. */
int oracle_convolution_backward(const float *x, const float *w, const float *dy,
                                float *dx, float *dw, float *db, int N, int C,
                                int H, int W, int Ko, int kh, int kw, int ph,
                                int pw, int sh, int sw, int dh, int dw_, int group,
                                int accum_dx, int accum_dw, int accum_db, int f64) {
  if (group <= 0 || C % group || Ko % group)
    return -1;
  const int Cg = C / group, Kog = Ko / group;
  const int Ho = (H + 2 * ph - (dh * (kh - 1) + 1)) / sh + 1;
  const int Wo = (W + 2 * pw - (dw_ * (kw - 1) + 1)) / sw + 1;
  if (Ho <= 0 || Wo <= 0)
    return -1;
  if (dx) {
    double *acc = (double *)calloc((size_t)N * C * H * W, sizeof(double));
    float *accf = (float *)calloc((size_t)N * C * H * W, sizeof(float));
    if (!acc || !accf)
      return -1;
    for (int n = 0; n < N; ++n)
      for (int o = 0; o < Ko; ++o) {
        const int g = o / Kog;
        for (int oy = 0; oy < Ho; ++oy)
          for (int ox = 0; ox < Wo; ++ox) {
            const float gy = dy[(((int64_t)n * Ko + o) * Ho + oy) * Wo + ox];
            for (int c = 0; c < Cg; ++c)
              for (int ky = 0; ky < kh; ++ky) {
                const int iy = oy * sh - ph + ky * dh;
                if (iy < 0 || iy >= H)
                  continue;
                for (int kx = 0; kx < kw; ++kx) {
                  const int ix = ox * sw - pw + kx * dw_;
                  if (ix < 0 || ix >= W)
                    continue;
                  const float wv = w[(((int64_t)o * Cg + c) * kh + ky) * kw + kx];
                  const int64_t i = (((int64_t)n * C + g * Cg + c) * H + iy) * W + ix;
                  acc[i] += (double)gy * (double)wv;
                  accf[i] += gy * wv;
                }
              }
          }
      }
    for (int64_t i = 0; i < (int64_t)N * C * H * W; ++i) {
      const float v = f64 ? (float)acc[i] : accf[i];
      dx[i] = accum_dx ? dx[i] + v : v;
    }
    free(acc);
    free(accf);
  }
  if (dw)
    for (int o = 0; o < Ko; ++o) {
      const int g = o / Kog;
      for (int c = 0; c < Cg; ++c)
        for (int ky = 0; ky < kh; ++ky)
          for (int kx = 0; kx < kw; ++kx) {
            double d = 0.;
            float s = 0.f;
            for (int n = 0; n < N; ++n)
              for (int oy = 0; oy < Ho; ++oy) {
                const int iy = oy * sh - ph + ky * dh;
                if (iy < 0 || iy >= H)
                  continue;
                for (int ox = 0; ox < Wo; ++ox) {
                  const int ix = ox * sw - pw + kx * dw_;
                  if (ix < 0 || ix >= W)
                    continue;
                  const float gy = dy[(((int64_t)n * Ko + o) * Ho + oy) * Wo + ox];
                  const float xv = x[(((int64_t)n * C + g * Cg + c) * H + iy) * W + ix];
                  d += (double)gy * (double)xv;
                  s += gy * xv;
                }
              }
            const int64_t i = (((int64_t)o * Cg + c) * kh + ky) * kw + kx;
            const float v = f64 ? (float)d : s;
            dw[i] = accum_dw ? dw[i] + v : v;
          }
    }
  if (db)
    for (int o = 0; o < Ko; ++o) {
      double d = 0.;
      float s = 0.f;
      for (int n = 0; n < N; ++n)
        for (int p = 0; p < Ho * Wo; ++p) {
          const float gy = dy[((int64_t)n * Ko + o) * Ho * Wo + p];
          d += (double)gy;
          s += gy;
        }
      const float v = f64 ? (float)d : s;
      db[o] = accum_db ? db[o] + v : v;
    }
  return 0;
}
