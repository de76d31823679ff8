/* CPU restatement of the training side of the companion functions: batch-statistics
 * BatchNormalization forward, and the backward passes of BatchNormalization, ReLU, Add2,
 * MaxPooling and GlobalAveragePooling. TEST INFRASTRUCTURE ONLY (see oracle.py).
 *
 * Every function follows the loop and operation order of the reference file it cites; all
 * arithmetic is float. Sums run in ascending element order as the reference's loops do. */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>

/* src/nbla/function/generic/batch_normalization.cpp:157-226 (forward_impl_batch, channel axis 1).
 * x is [N, C, S]. Writes y, the batch mean / variance, and (update != 0) the running ones. */
void oracle_batch_norm_batch(const float *x, const float *beta, const float *gamma, float *rmean, float *rvar,
                             int64_t N, int64_t C, int64_t S, float eps, float decay, int update, float *y,
                             float *m, float *v) {
  const int64_t n02 = N * S;
  for (int64_t c = 0; c < C; ++c) {
    m[c] = 0.f;
    v[c] = 0.f;
    for (int64_t n = 0; n < N; ++n)
      for (int64_t s = 0; s < S; ++s) {
        const float value = x[(n * C + c) * S + s];
        m[c] += value;
        v[c] += value * value;
      }
    m[c] /= n02;
    v[c] = v[c] / n02 - m[c] * m[c];
    if (update) {
      rmean[c] = decay * rmean[c] + (1 - decay) * m[c];
      rvar[c] = decay * rvar[c] + (1 - decay) * v[c] * n02 / (n02 - 1);
    }
    const float stdvar = sqrtf(v[c] + eps);
    const float scale = gamma ? gamma[c] : 1.f;
    const float bias = beta ? beta[c] : 0.f;
    for (int64_t n = 0; n < N; ++n)
      for (int64_t s = 0; s < S; ++s) {
        const int64_t i = (n * C + c) * S + s;
        y[i] = (x[i] - m[c]) * scale / stdvar + bias;
      }
  }
}

/* batch_normalization.cpp:274-383 (backward_impl_batch). m, v: the batch statistics of the
 * forward pass; dm, dv: gradients arriving at the statistics outputs (may be NULL). dx, dbeta,
 * dgamma may be NULL (not propagated); the accum flags add to what the buffers hold. */
void oracle_batch_norm_batch_backward(const float *x, const float *dy, const float *gamma, const float *m,
                                      const float *v, const float *dm, const float *dv, int64_t N, int64_t C,
                                      int64_t S, float eps, float *dx, int accum_dx, float *dbeta, int accum_dbeta,
                                      float *dgamma, int accum_dgamma) {
  const int64_t n02 = N * S;
  if (dx)
    for (int64_t c = 0; c < C; ++c) {
      float dvar = 0.f, dmean = 0.f, tmp = 0.f;
      const float scale = gamma ? gamma[c] : 1.f;
      for (int64_t n = 0; n < N; ++n)
        for (int64_t s = 0; s < S; ++s) {
          const int64_t i = (n * C + c) * S + s;
          const float dxh = dy[i] * scale;
          const float cx = x[i] - m[c];
          dvar += dxh * cx;
          dmean += dxh;
          tmp += cx;
        }
      dvar = dvar * -0.5f * powf(v[c] + eps, -1.5f) + (dv ? dv[c] : 0.f);
      dmean = dmean * (-1 / sqrtf(v[c] + eps)) + dvar * (-2) * tmp / (n02) + (dm ? dm[c] : 0.f);
      for (int64_t n = 0; n < N; ++n)
        for (int64_t s = 0; s < S; ++s) {
          const int64_t i = (n * C + c) * S + s;
          const float grad = dy[i] * scale / sqrtf(v[c] + eps) + dvar * 2 * (x[i] - m[c]) / (n02) + dmean / (n02);
          if (accum_dx)
            dx[i] += grad;
          else
            dx[i] = grad;
        }
    }
  if (dbeta || dgamma)
    for (int64_t c = 0; c < C; ++c) {
      float dbv = (dbeta && accum_dbeta) ? dbeta[c] : 0.f;
      float dgv = (dgamma && accum_dgamma) ? dgamma[c] : 0.f;
      for (int64_t n = 0; n < N; ++n)
        for (int64_t s = 0; s < S; ++s) {
          const int64_t i = (n * C + c) * S + s;
          if (dbeta)
            dbv += dy[i];
          if (dgamma)
            dgv += dy[i] * (x[i] - m[c]) / sqrtf(v[c] + eps);
        }
      if (dbeta)
        dbeta[c] = dbv;
      if (dgamma)
        dgamma[c] = dgv;
    }
}

/* batch_normalization.cpp:385-486 (backward_impl_global): the composition of PowScalar, Mul2,
 * Sub2, Sum and Add2 that the reference executes, element by element.
 * dx = dy * (gamma * (rvar + eps)^-0.5); dbeta = sum dy; dgamma = sum dy * ((x - rmean) * (rvar + eps)^-0.5). */
void oracle_batch_norm_global_backward(const float *x, const float *dy, const float *gamma, const float *rmean,
                                       const float *rvar, int64_t N, int64_t C, int64_t S, float eps, float *dx,
                                       int accum_dx, float *dbeta, int accum_dbeta, float *dgamma,
                                       int accum_dgamma) {
  for (int64_t c = 0; c < C; ++c) {
    const float rstd_inv = powf(rvar[c] + eps, -0.5f);
    const float iv = gamma ? gamma[c] * rstd_inv : rstd_inv;
    float sb = 0.f, sg = 0.f;
    for (int64_t n = 0; n < N; ++n)
      for (int64_t s = 0; s < S; ++s) {
        const int64_t i = (n * C + c) * S + s;
        if (dx) {
          const float g = dy[i] * iv;
          dx[i] = accum_dx ? dx[i] + g : g;
        }
        sb += dy[i];
        sg += dy[i] * ((x[i] - rmean[c]) * rstd_inv);
      }
    if (dbeta)
      dbeta[c] = accum_dbeta ? dbeta[c] + sb : sb;
    if (dgamma)
      dgamma[c] = accum_dgamma ? dgamma[c] + sg : sg;
  }
}

/* src/nbla/function/generic/relu.cpp:41-49: dx (+)= y > 0 ? dy : 0 with y the forward output. */
void oracle_relu_backward(const float *y, const float *dy, float *dx, int64_t n, int accum) {
  for (int64_t i = 0; i < n; ++i) {
    const float g = y[i] > 0.f ? dy[i] : 0.f;
    dx[i] = accum ? dx[i] + g : g;
  }
}

/* src/nbla/function/generic/add2.cpp (same-shape inputs): each input receives dy. */
void oracle_add2_backward(const float *dy, float *dx, int64_t n, int accum) {
  for (int64_t i = 0; i < n; ++i)
    dx[i] = accum ? dx[i] + dy[i] : dy[i];
}

/* src/nbla/function/generic/global_average_pooling.cpp:75-117: every pixel of a map receives dy / (H W). */
void oracle_global_average_pooling_backward(const float *dy, float *dx, int64_t maps, int64_t S, int accum) {
  for (int64_t m = 0; m < maps; ++m) {
    const float g = dy[m] / (float)S;
    for (int64_t i = 0; i < S; ++i)
      dx[m * S + i] = accum ? dx[m * S + i] + g : g;
  }
}

int oracle_pool_out(int w, int k, int s, int p, int ignore_border);

/* src/nbla/function/generic/max_pooling.cpp:44-77 (the index of the FIRST maximum of every clipped
 * window, strict compare) and :134-139, :194-228 (dx zeroed unless accumulating, then
 * dx[index] += dy in output order). x, dx are [maps, H, W]. */
void oracle_max_pooling_backward(const float *x, const float *dy, float *dx, int64_t maps, int H, int W, int kh,
                                 int kw, int sh, int sw, int ph, int pw, int ignore_border, int accum) {
  const int Ho = oracle_pool_out(H, kh, sh, ph, ignore_border);
  const int Wo = oracle_pool_out(W, kw, sw, pw, ignore_border);
  if (!accum)
    for (int64_t i = 0; i < maps * H * W; ++i)
      dx[i] = 0.f;
  for (int64_t m = 0; m < maps; ++m)
    for (int oy = 0; oy < Ho; ++oy)
      for (int ox = 0; ox < Wo; ++ox) {
        int y0 = oy * sh - ph, x0 = ox * sw - pw;
        int y1 = y0 + kh < H + ph ? y0 + kh : H + ph, x1 = x0 + kw < W + pw ? x0 + kw : W + pw;
        if (y0 < 0)
          y0 = 0;
        if (x0 < 0)
          x0 = 0;
        if (y1 > H)
          y1 = H;
        if (x1 > W)
          x1 = W;
        int64_t best_i = (m * H + y0) * W + x0;
        float best = x[best_i];
        for (int iy = y0; iy < y1; ++iy)
          for (int ix = x0; ix < x1; ++ix) {
            const int64_t i = (m * H + iy) * W + ix;
            if (best < x[i]) {
              best = x[i];
              best_i = i;
            }
          }
        dx[best_i] += dy[(m * Ho + oy) * Wo + ox];
      }
}
