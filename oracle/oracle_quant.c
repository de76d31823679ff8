/* CPU restatement of the reference's quantizer and weight-binarisation
 * arithmetic, in plain C, one function per reference loop.
 *
 * TEST INFRASTRUCTURE ONLY: this file is the checker the CUDA path is compared
 * against (tests/, the smoke check and the CPU-baseline leg of the benchmark).
 * The product library never links or calls it.
 *
 * Parity status: PINNED. Every function here is compared bit for bit (or, for
 * the floating-point reductions, to rounding) against the reference's own
 * compiled C++ ("cpu:float" context, oracle/_ref/libnnabla_ref.so) by
 * tests/test_oracle_vs_reference.py, and against the fixtures under
 * tests/golden/ that were generated from that library.
 *
 * Build: gcc -O2 -fno-fast-math -ffp-contract=off (see oracle/Makefile); the
 * reference is built for x86-64 SSE2 without FMA, so every fp32 operation
 * below must round separately.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

/* src/nbla/function/generic/fixed_point_quantize.cpp:37-39 (limits) and
 * :53-65 (loop). The 0.5 added before truncation is a double literal. */
void oracle_fixed_point_quantize(const float *x, float *y, int64_t size,
                                 int sign, int n, float delta) {
  int nn = sign ? n - 1 : n;
  float max_ = (float)((pow(2, nn) - 1) * delta);
  float min_ = sign ? -max_ : 0.0f;
  for (int64_t s = 0; s < size; ++s) {
    float y_tmp;
    if (x[s] > max_) {
      y_tmp = max_;
    } else if (x[s] < min_) {
      y_tmp = min_;
    } else {
      int sign_x = (x[s] < 0.0);
      float abs_x = fabsf(x[s]);
      y_tmp = (float)(int)((abs_x / delta) + 0.5) * delta;
      y_tmp = sign_x ? -y_tmp : y_tmp;
    }
    y[s] = y_tmp;
  }
}

/* Constants of src/nbla/function/generic/pow2_quantize.cpp:35-39. */
void oracle_pow2_constants(int sign, int with_zero, int n, int m, float *p_max,
                           float *p_min, float *pruning_threshold) {
  int nn = sign ? n - 1 : n;
  nn = with_zero ? nn - 1 : nn;
  *p_max = (float)pow(2., m);
  *p_min = (float)pow(2., m - ((1 << nn) - 1));
  /* p_min_ is a float member; the product is formed in double. */
  *pruning_threshold = (float)((double)*p_min * pow(2., -0.5));
}

/* src/nbla/function/generic/pow2_quantize.cpp:57-81. log2/round/pow on float
 * arguments resolve to the float overloads of the host libm. */
void oracle_pow2_quantize(const float *x, float *y, int64_t size, int sign,
                          int with_zero, int n, int m) {
  float p_max, p_min, prune;
  oracle_pow2_constants(sign, with_zero, n, m, &p_max, &p_min, &prune);
  for (int64_t s = 0; s < size; ++s) {
    float x_abs = fabsf(x[s]);
    float q = powf(2.f, roundf(log2f(x_abs)));
    if (q > p_max) {
      q = p_max;
    } else if (q < p_min && with_zero) {
      q = x_abs < prune ? 0.f : p_min;
    } else if (q < p_min) {
      q = p_min;
    }
    int sign_x = (x[s] < 0.0);
    if (sign) {
      q = sign_x ? -q : q;
    } else {
      if (with_zero)
        q = sign_x ? 0.f : q;
      else
        q = sign_x ? p_min : q;
    }
    y[s] = q;
  }
}

/* The largest fp32 mantissa field (23 bits) for which
 * roundf(log2f(1.m * 2^e)) is still e, per unbiased exponent e of a normal
 * number: the libm-dependent cut the CUDA kernel snaps against. Found by
 * bisection on the host libm the reference would run with; out[e + 126] for
 * e in [-126, 127]. Returns 0 when log2f is monotone around every cut
 * (checked +-64 ulp), else the number of exponents where it is not. */
int oracle_pow2_thresholds(uint32_t *out) {
  int bad = 0;
  for (int e = -126; e <= 127; ++e) {
    uint32_t lo = 0, hi = 0x7fffff; /* invariant: f(lo) = e, f(hi) = e + 1 */
    uint32_t base = (uint32_t)(e + 127) << 23;
    while (hi - lo > 1) {
      uint32_t mid = (lo + hi) / 2, bits = base | mid;
      float v;
      memcpy(&v, &bits, 4);
      if (roundf(log2f(v)) <= (float)e)
        lo = mid;
      else
        hi = mid;
    }
    for (int d = -64; d <= 64; ++d) {
      int64_t mm = (int64_t)lo + d;
      if (mm < 0 || mm > 0x7fffff)
        continue;
      uint32_t bits = base | (uint32_t)mm;
      float v;
      memcpy(&v, &bits, 4);
      float want = (mm <= (int64_t)lo) ? (float)e : (float)(e + 1);
      if (roundf(log2f(v)) != want) {
        ++bad;
        break;
      }
    }
    out[e + 126] = lo;
  }
  return bad;
}

/* src/nbla/function/generic/min_max_quantize.cpp:129-223 with nudge_range
 * (:352-361) and nudge_qr_min_max (:362-390). x has shape xs[0..nd), the four
 * q tensors share shape qs[0..nd) whose entries are 1 or xs[d]. qr_min and
 * qr_max are updated in place exactly as the reference updates inputs[1] and
 * inputs[2]; scale_out (q-sized, may be NULL) receives the scale kept for
 * backward. Returns 0, or -1 on a shape error / allocation failure. */
int oracle_min_max_quantize(const float *x, const int64_t *xs, int nd,
                            float *qr_min, float *qr_max, const float *ql_min,
                            const float *ql_max, const int64_t *qs,
                            float decay, int x_min_max, int ema, float eps,
                            float *y, float *scale_out) {
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
  float *scale = (float *)malloc(sizeof(float) * (size_t)(qsize ? qsize : 1));
  float *m = (float *)malloc(sizeof(float) * (size_t)(qsize ? qsize : 1));
  float *M = (float *)malloc(sizeof(float) * (size_t)(qsize ? qsize : 1));
  float *mn = NULL, *mx = NULL;
  if (!scale || !m || !M)
    return -1;
#define QIDX(i, q)                                                             \
  do {                                                                         \
    int64_t r_ = (i);                                                          \
    (q) = 0;                                                                   \
    for (int d_ = 0; d_ < nd; ++d_) {                                          \
      int64_t c_ = r_ / xstr[d_];                                              \
      r_ -= c_ * xstr[d_];                                                     \
      (q) += c_ * qstr[d_];                                                    \
    }                                                                          \
  } while (0)
  if (x_min_max) {
    /* Min / Max over the axes where the q shape is 1 (:97-98, :159-178). */
    mn = (float *)malloc(sizeof(float) * (size_t)qsize);
    mx = (float *)malloc(sizeof(float) * (size_t)qsize);
    if (!mn || !mx)
      return -1;
    /* Min / Max scan from +1e8 / -1e8 and replace on a strict comparison
     * (src/nbla/function/generic/max.cpp:49-57, min.cpp): the first of equal
     * values stays (this decides the sign of a zero extremum), a NaN never
     * wins, and values beyond 1e8 in magnitude on the wrong side are ignored. */
    for (int64_t q = 0; q < qsize; ++q) {
      mn[q] = 1e+8;
      mx[q] = -1e+8;
    }
    for (int64_t i = 0; i < xsize; ++i) {
      int64_t q;
      QIDX(i, q);
      if (x[i] < mn[q])
        mn[q] = x[i];
      if (x[i] > mx[q])
        mx[q] = x[i];
    }
    float d1 = (float)decay, d2 = (float)(1.0 - decay); /* :105-106 */
    for (int64_t q = 0; q < qsize; ++q) {
      if (ema) {
        float a = mn[q] * d2, b = qr_min[q] * d1;
        qr_min[q] = b + a;
        a = mx[q] * d2;
        b = qr_max[q] * d1;
        qr_max[q] = b + a;
      } else {
        qr_min[q] = mn[q];
        qr_max[q] = mx[q];
      }
    }
    free(mn);
    free(mx);
  }
  for (int64_t q = 0; q < qsize; ++q) {
    /* nudge_range */
    if (qr_max[q] - qr_min[q] < eps)
      qr_max[q] = qr_min[q] + eps;
    /* scale (:184-186) */
    float num = qr_max[q] - qr_min[q];
    float den = ql_max[q] - ql_min[q];
    scale[q] = num / den;
    /* nudge_qr_min_max */
    float t = qr_min[q] / scale[q];
    float zp_from_min = ql_min[q] - t;
    float zp;
    if (zp_from_min <= ql_min[q])
      zp = ql_min[q];
    else if (zp_from_min >= ql_max[q])
      zp = ql_max[q];
    else
      zp = roundf(zp_from_min);
    float a = ql_min[q] - zp, b = ql_max[q] - zp;
    m[q] = a * scale[q];
    M[q] = b * scale[q];
    if (scale_out)
      scale_out[q] = scale[q];
  }
  for (int64_t i = 0; i < xsize; ++i) {
    int64_t q;
    QIDX(i, q);
    float t = (x[i] > m[q]) ? x[i] : m[q]; /* maximum2.hpp:41 */
    t = (t < M[q]) ? t : M[q];             /* minimum2.hpp:41 */
    t = t - m[q];
    t = t / scale[q];
    t = roundf(t);
    t = t * scale[q];
    y[i] = t + m[q];
  }
#undef QIDX
  free(scale);
  free(m);
  free(M);
  return 0;
}

/* include/nbla/function/sign.hpp:48-50. */
void oracle_sign(const float *x, float *y, int64_t size, float alpha) {
  for (int64_t s = 0; s < size; ++s)
    y[s] = (x[s] > 0.f) ? 1.f : ((x[s] < 0.f) ? -1.f : alpha);
}

/* Weight binarisation of BinaryWeightAffine
 * (src/nbla/function/generic/binary_weight_affine.cpp:83-107): W is
 * [rows, cols] row-major, one alpha per column:
 * alpha[c] = (sum_r |W[r,c]|) * (float)(1/rows). The reference sums with
 * Eigen after a transpose; here the sum runs over r ascending in fp32, so
 * alpha agrees to rounding, wb exactly. scaled (may be NULL) = wb * alpha. */
void oracle_binarize_columns(const float *w, int64_t rows, int64_t cols,
                             float quantize_zero_to, float *wb, float *alpha,
                             float *scaled) {
  float inv = (float)1 / rows; /* binary_weight_affine.cpp:68 */
  for (int64_t c = 0; c < cols; ++c) {
    float s = 0.f;
    for (int64_t r = 0; r < rows; ++r)
      s += fabsf(w[r * cols + c]);
    alpha[c] = s * inv;
  }
  oracle_sign(w, wb, rows * cols, quantize_zero_to);
  if (scaled)
    for (int64_t r = 0; r < rows; ++r)
      for (int64_t c = 0; c < cols; ++c)
        scaled[r * cols + c] = wb[r * cols + c] * alpha[c];
}

/* Weight binarisation of BinaryWeightConvolution
 * (src/nbla/function/generic/binary_weight_convolution.cpp:81-102): W is
 * [outmaps, col_w] row-major, one alpha per row. */
void oracle_binarize_rows(const float *w, int64_t rows, int64_t cols,
                          float quantize_zero_to, float *wb, float *alpha,
                          float *scaled) {
  float inv = (float)1 / cols; /* binary_weight_convolution.cpp:66 */
  for (int64_t r = 0; r < rows; ++r) {
    float s = 0.f;
    for (int64_t c = 0; c < cols; ++c)
      s += fabsf(w[r * cols + c]);
    alpha[r] = s * inv;
  }
  oracle_sign(w, wb, rows * cols, quantize_zero_to);
  if (scaled)
    for (int64_t r = 0; r < rows; ++r)
      for (int64_t c = 0; c < cols; ++c)
        scaled[r * cols + c] = wb[r * cols + c] * alpha[r];
}
