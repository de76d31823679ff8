/* CPU restatement of the sibling quantization functions (BinarySigmoid,
 * BinaryTanh, QuantizeLinear, DequantizeLinear; forward and backward), in
 * plain C, one function per reference loop.
 *
 * TEST INFRASTRUCTURE ONLY: the checker the CUDA path is compared against.
 * The product library never links or calls it.
 *
 * Parity status: PINNED, bit for bit, against the reference's own compiled
 * C++ (oracle/_ref/libnnabla_ref.so) by tests/test_oracle_siblings_vs_reference.py.
 *
 * Build: gcc -O2 -fno-fast-math -ffp-contract=off, like oracle_quant.c.
 */
#include <math.h>
#include <stdint.h>

/* include/nbla/function/binary_sigmoid.hpp:50-52, binary_tanh.hpp:51-52 */
void oracle_binary_act(const float *x, float *y, int64_t n, int tanh_like) {
  for (int64_t i = 0; i < n; ++i)
    y[i] = x[i] > 0.0f ? 1.0f : (tanh_like ? -1.0f : 0.0f);
}

/* gradient of the above through include/nbla/function/utils/base_transform_unary.hpp:104-110 */
void oracle_binary_act_backward(const float *x, const float *dy, float *dx, int64_t n, int tanh_like, int accum) {
  for (int64_t i = 0; i < n; ++i) {
    float g = (fabsf(x[i]) >= 1.0f) ? 0.0f : (tanh_like ? dy[i] : dy[i] * 0.5f);
    dx[i] = (accum ? dx[i] : 0.0f) + g;
  }
}

static int64_t bidx(int64_t i, const int64_t *xs, const int64_t *ps, int nd) {
  /* index into a parameter tensor whose extents are 1 or xs[d] */
  int64_t xstr[8], pstr[8], xsize = 1, psize = 1, q = 0;
  for (int d = nd - 1; d >= 0; --d) {
    xstr[d] = xsize;
    xsize *= xs[d];
    pstr[d] = ps[d] == 1 ? 0 : psize;
    psize *= ps[d];
  }
  for (int d = 0; d < nd; ++d) {
    int64_t c = i / xstr[d];
    i -= c * xstr[d];
    q += c * pstr[d];
  }
  return q;
}

static float ql_round(float v, int half_to_even) {
  float t = roundf(v);
  if (half_to_even && fabsf(v - t) == 0.5f)
    return roundf(v * 0.5f) * 2;
  return t;
}

static float ql_saturate(float v, int lo, int hi) {
  if (v < lo)
    return (float)lo;
  if (v > hi)
    return (float)hi;
  return v;
}

/* src/nbla/function/generic/quantize_linear.cpp:50-61 (range), :63-101
 * (saturate, round), :103-122 (forward). zero_point is rounded and saturated
 * in place. dtype: 1 = BYTE, 2 = UBYTE. Returns -1 for another dtype. */
int oracle_quantize_linear(const float *x, const int64_t *xs, int nd, const float *scale, const int64_t *ss,
                           float *zp, const int64_t *zs, float *y, int half_to_even, int narrow_range, int dtype) {
  int lo, hi;
  if (dtype == 1) {
    lo = narrow_range ? -127 : -128;
    hi = 127;
  } else if (dtype == 2) {
    lo = narrow_range ? 1 : 0;
    hi = 255;
  } else {
    return -1;
  }
  int64_t n = 1, nz = 1;
  for (int d = 0; d < nd; ++d) {
    n *= xs[d];
    nz *= zs[d];
  }
  for (int64_t i = 0; i < nz; ++i)
    zp[i] = ql_saturate(ql_round(zp[i], half_to_even), lo, hi);
  for (int64_t i = 0; i < n; ++i) {
    float t = x[i] / scale[bidx(i, xs, ss, nd)];
    t = ql_round(t, half_to_even);
    t = t + zp[bidx(i, xs, zs, nd)];
    y[i] = ql_saturate(t, lo, hi);
  }
  return 0;
}

/* src/nbla/function/generic/dequantize_linear.cpp:60-71 */
void oracle_dequantize_linear(const float *x, const int64_t *xs, int nd, const float *scale, const int64_t *ss,
                              const float *zp, const int64_t *zs, float *y) {
  int64_t n = 1;
  for (int d = 0; d < nd; ++d)
    n *= xs[d];
  for (int64_t i = 0; i < n; ++i) {
    float t = x[i] - zp[bidx(i, xs, zs, nd)];
    y[i] = t * scale[bidx(i, xs, ss, nd)];
  }
}

/* quantize_linear.cpp:137-147 (divide != 0: dx (+)= dy / scale) and
 * dequantize_linear.cpp:92-102 (dx (+)= dy * scale) */
void oracle_linear_scale_backward(const float *dy, const int64_t *xs, int nd, const float *scale, const int64_t *ss,
                                  float *dx, int divide, int accum) {
  int64_t n = 1;
  for (int d = 0; d < nd; ++d)
    n *= xs[d];
  for (int64_t i = 0; i < n; ++i) {
    float s = scale[bidx(i, xs, ss, nd)];
    float g = divide ? dy[i] / s : dy[i] * s;
    dx[i] = accum ? dx[i] + g : g;
  }
}

/* src/nbla/function/generic/prune.cpp:38-72: the threshold is the
 * (int)((n - 1) * rate)-th smallest magnitude (+ 1 when rate == 1). */
#include <stdlib.h>
#include <string.h>
static int cmp_abs(const void *a, const void *b) {
  float x = fabsf(*(const float *)a), y = fabsf(*(const float *)b);
  return (x > y) - (x < y);
}
int oracle_prune(const float *x, float *y, int64_t n, float rate) {
  if (n == 0)
    return 0;
  float *buf = (float *)malloc(sizeof(float) * (size_t)n);
  if (!buf)
    return -1;
  memcpy(buf, x, sizeof(float) * (size_t)n);
  qsort(buf, (size_t)n, sizeof(float), cmp_abs);
  int idx = (int)(((int)n - 1) * rate);
  float t = fabsf(buf[idx]);
  t += rate == 1.0 ? 1.0 : 0.0;
  free(buf);
  for (int64_t i = 0; i < n; ++i)
    y[i] = (fabsf(x[i]) < t) ? 0.0f : x[i];
  return 0;
}
