// Backward passes (straight-through estimators) of the three quantizers.
// Included by quantize.cu inside namespace nb200::<anonymous>, after the
// forward code whose limits, tables and shape helpers it shares.
//
// All three are HBM-bound: 4 B of x + 4 B of dy read and 4 B of dx written per
// element (plus 4 B of dx read when accumulating; x is not read at all without
// ste_fine_grained). Same access pattern as the forward kernels: 128-bit
// streaming accesses, four independent groups in flight per thread, many
// short CTAs per SM.
//
// A gradient op provides
//   bool operator()(float x, float dy, size_t i, float &g, const State &) const
// returning whether the element passes a gradient and, if so, the value g.
// The driver combines it with dx exactly like the reference loops:
//   accumulate:  dx = passes ? dx + g : dx        (dx untouched where blocked)
//   overwrite:   dx = passes ? g : 0
#pragma once

template <typename Op, bool kAccum>
__device__ __forceinline__ float grad_combine(const Op &op, const typename Op::State &st, float x, float dy, float dx,
                                              size_t i) {
  float g;
  const bool pass = op(x, dy, i, g, st);
  if (kAccum)
    return pass ? __fadd_rn(dx, g) : dx;
  if (Op::kZeroPlus) // functions defined as (accum ? dx : 0) + g: a negative zero becomes +0
    return pass ? __fadd_rn(0.0f, g) : 0.0f;
  return pass ? g : 0.0f;
}

template <typename Op, bool kAccum>
__global__ void __launch_bounds__(kThreads) grad_vec_kernel(const float *__restrict__ x, const float *__restrict__ dy,
                                                            float *__restrict__ dx, size_t size, size_t n4, Op op) {
  const float4 *x4 = reinterpret_cast<const float4 *>(x);
  const float4 *dy4 = reinterpret_cast<const float4 *>(dy);
  float4 *dx4 = reinterpret_cast<float4 *>(dx);
  const size_t stride = (size_t)gridDim.x * kThreads;
  size_t i = (size_t)blockIdx.x * kThreads + threadIdx.x;
  const typename Op::State st = op.init();
  const float4 zero4 = make_float4(0.f, 0.f, 0.f, 0.f);
  for (; i + (kUnroll - 1) * stride < n4; i += kUnroll * stride) {
    float4 vx[kUnroll], vg[kUnroll], vd[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      vx[u] = Op::kNeedsX ? ld_stream(x4 + i + u * stride) : zero4;
      vg[u] = ld_stream(dy4 + i + u * stride);
      vd[u] = kAccum ? ld_stream(dx4 + i + u * stride) : zero4;
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const size_t e = 4 * (i + u * stride);
      float4 r;
      r.x = grad_combine<Op, kAccum>(op, st, vx[u].x, vg[u].x, vd[u].x, e);
      r.y = grad_combine<Op, kAccum>(op, st, vx[u].y, vg[u].y, vd[u].y, e + 1);
      r.z = grad_combine<Op, kAccum>(op, st, vx[u].z, vg[u].z, vd[u].z, e + 2);
      r.w = grad_combine<Op, kAccum>(op, st, vx[u].w, vg[u].w, vd[u].w, e + 3);
      st_stream(dx4 + i + u * stride, r);
    }
  }
  for (; i < n4; i += stride) {
    const float4 vx = Op::kNeedsX ? ld_stream(x4 + i) : zero4;
    const float4 vg = ld_stream(dy4 + i);
    const float4 vd = kAccum ? ld_stream(dx4 + i) : zero4;
    const size_t e = 4 * i;
    float4 r;
    r.x = grad_combine<Op, kAccum>(op, st, vx.x, vg.x, vd.x, e);
    r.y = grad_combine<Op, kAccum>(op, st, vx.y, vg.y, vd.y, e + 1);
    r.z = grad_combine<Op, kAccum>(op, st, vx.z, vg.z, vd.z, e + 2);
    r.w = grad_combine<Op, kAccum>(op, st, vx.w, vg.w, vd.w, e + 3);
    st_stream(dx4 + i, r);
  }
  if (blockIdx.x == 0) {
    for (size_t e = 4 * n4 + threadIdx.x; e < size; e += kThreads)
      dx[e] = grad_combine<Op, kAccum>(op, st, Op::kNeedsX ? x[e] : 0.0f, dy[e], kAccum ? dx[e] : 0.0f, e);
  }
}

// Pointers that are not all 16-byte aligned: scalar, still coalesced.
template <typename Op, bool kAccum>
__global__ void __launch_bounds__(kThreads) grad_scalar_kernel(const float *__restrict__ x,
                                                               const float *__restrict__ dy, float *__restrict__ dx,
                                                               size_t size, Op op) {
  const size_t stride = (size_t)gridDim.x * kThreads;
  const typename Op::State st = op.init();
  for (size_t i = (size_t)blockIdx.x * kThreads + threadIdx.x; i < size; i += stride)
    dx[i] = grad_combine<Op, kAccum>(op, st, Op::kNeedsX ? x[i] : 0.0f, dy[i], kAccum ? dx[i] : 0.0f, i);
}

template <typename Op, bool kAccum>
int launch_gradient_t(const float *x, const float *dy, float *dx, size_t size, const Op &op, cudaStream_t st) {
  const uintptr_t all = (Op::kNeedsX ? reinterpret_cast<uintptr_t>(x) : 0) | reinterpret_cast<uintptr_t>(dy) |
                        reinterpret_cast<uintptr_t>(dx);
  if (all & 15) {
    grad_scalar_kernel<Op, kAccum><<<grid_for(size), kThreads, 0, st>>>(x, dy, dx, size, op);
  } else {
    const size_t n4 = size / 4;
    grad_vec_kernel<Op, kAccum>
        <<<grid_for((n4 + kUnroll - 1) / kUnroll), kThreads, 0, st>>>(x, dy, dx, size, n4, op);
  }
  NB_LAUNCH_CHECK();
  return NB200_OK;
}

template <typename Op>
int launch_gradient(const float *x, const float *dy, float *dx, size_t size, int accum, const Op &op,
                    cudaStream_t st) {
  if (size == 0)
    return NB200_OK;
  NB_CHECK(dy != nullptr && dx != nullptr && (x != nullptr || !Op::kNeedsX), NB200_EVALUE, "null data pointer");
  NB_CHECK(((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(dy) | reinterpret_cast<uintptr_t>(dx)) & 3) ==
               0,
           NB200_EVALUE, "fp32 pointers must be 4-byte aligned");
  return accum ? launch_gradient_t<Op, true>(x, dy, dx, size, op, st)
               : launch_gradient_t<Op, false>(x, dy, dx, size, op, st);
}

// Gradient passes everywhere (every quantizer without ste_fine_grained):
// fixed_point_quantize.cpp:69-79, pow2_quantize.cpp:85-95,
// min_max_quantize.cpp:288-294.
struct PassAllGrad {
  static constexpr bool kNeedsX = false;
  static constexpr bool kZeroPlus = false;
  struct State {};
  __device__ __forceinline__ State init() const { return State(); }
  __device__ __forceinline__ bool operator()(float, float dy, size_t, float &g, const State &) const {
    g = dy;
    return true;
  }
};

// fixed_point_quantize.cpp:81-101: the gradient passes inside [min, max].
struct FxpGrad {
  static constexpr bool kNeedsX = true;
  static constexpr bool kZeroPlus = false;
  float maxv, minv;
  struct State {};
  __device__ __forceinline__ State init() const { return State(); }
  __device__ __forceinline__ bool operator()(float x, float dy, size_t, float &g, const State &) const {
    g = dy;
    return !(x > maxv) && !(x < minv);
  }
};

// pow2_quantize.cpp:97-125: dx (+)= c * dy with c = 0 where the snapped power
// of two exceeds p_max or (unsigned) x is negative. The snap is monotone in
// |x|, so "exceeds p_max" is one comparison of |x|'s bit pattern with a
// threshold derived on the host from the same libm tables as the forward
// (NaN inputs keep c = 1 like the reference, whose comparison with NaN fails).
struct Pow2Grad {
  static constexpr bool kNeedsX = true;
  static constexpr bool kZeroPlus = false;
  uint32_t threshold_bits; // c = 0 for threshold_bits < bits(|x|) <= bits(inf)
  int sign;
  struct State {};
  __device__ __forceinline__ State init() const { return State(); }
  __device__ __forceinline__ bool operator()(float x, float dy, size_t, float &g, const State &) const {
    const uint32_t bits = __float_as_uint(fabsf(x));
    float c = (bits > threshold_bits && bits <= 0x7f800000u) ? 0.0f : 1.0f;
    if (!sign && x < 0.0f)
      c = 0.0f;
    g = __fmul_rn(c, dy); // the product is formed even for c = 0 (sign of zero, NaN/inf in dy)
    return true;
  }
};

int pow2_gradient_threshold(const Pow2Params &P, uint32_t *threshold_bits) {
  const Pow2Tables *unused = nullptr;
  NB_TRY(pow2_tables_for_current_device(&unused)); // builds and validates the host tables
  const Pow2Tables &T = g_pow2_host;
  for (int k = kMinExp; k < 128; ++k)
    NB_CHECK(T.pw[k - kMinExp] <= T.pw[k + 1 - kMinExp], NB200_ENOTIMPL, "libm: powf(2, k) is not monotone at k=%d", k);
  int kstar = 129; // smallest k with 2^k > p_max
  for (int k = kMinExp; k <= 128; ++k)
    if (T.pw[k - kMinExp] > P.p_max) {
      kstar = k;
      break;
    }
  if (kstar == 129) {
    *threshold_bits = 0x7f800000u; // nothing exceeds p_max
  } else if (kstar == kMinExp) {
    *threshold_bits = 0u; // every non-zero |x| does
  } else {
    const int e = kstar - 1; // binade whose upper part snaps to 2^kstar
    const uint32_t cut = T.cut[e - kMinExp];
    if (e >= -126) {
      *threshold_bits = ((uint32_t)(e + 127) << 23) | cut;
    } else {
      const int p = e + 149;
      *threshold_bits = (1u << p) | (cut >> (23 - p));
    }
  }
  return NB200_OK;
}

// ---- MinMaxQuantize backward (min_max_quantize.cpp:225-350) -------------------
// Nudged range per q, recomputed from the ranges the forward left in place
// (nudge_qr_min_max, :362-390, with the scale of :184-186).
__global__ void minmax_nudged_kernel(size_t Q, const float *qr_min, const float *qr_max, const float *ql_min,
                                     const float *ql_max, float *m_out, float *M_out) {
  const size_t q = blockIdx.x * (size_t)blockDim.x + threadIdx.x;
  if (q >= Q)
    return;
  const float rmin = qr_min[q], rmax = qr_max[q], lmin = ql_min[q], lmax = ql_max[q];
  const float s = __fdiv_rn(__fsub_rn(rmax, rmin), __fsub_rn(lmax, lmin));
  const float z = __fsub_rn(lmin, __fdiv_rn(rmin, s));
  float zp;
  if (z <= lmin)
    zp = lmin;
  else if (z >= lmax)
    zp = lmax;
  else
    zp = roundf(z);
  m_out[q] = __fmul_rn(__fsub_rn(lmin, zp), s);
  M_out[q] = __fmul_rn(__fsub_rn(lmax, zp), s);
}

// Gradient w.r.t. x with ste_fine_grained (:268-287): (x >= m) * (x <= M) * dy.
struct MinMaxGrad {
  static constexpr bool kNeedsX = true;
  static constexpr bool kZeroPlus = false;
  const float *m, *M;
  size_t Q, inner;
  struct State {
    float m, M;
  };
  __device__ __forceinline__ State init() const {
    State st;
    st.m = __ldg(m);
    st.M = __ldg(M);
    return st;
  }
  __device__ __forceinline__ bool operator()(float x, float dy, size_t i, float &g, const State &st) const {
    float lo = st.m, hi = st.M;
    if (Q != 1) {
      const size_t q = ((i | inner | Q) >> 32) ? (i / inner) % Q : ((uint32_t)i / (uint32_t)inner) % (uint32_t)Q;
      lo = __ldg(m + q);
      hi = __ldg(M + q);
    }
    const float mask = __fmul_rn((x >= lo) ? 1.0f : 0.0f, (x <= hi) ? 1.0f : 0.0f);
    g = __fmul_rn(mask, dy);
    return true;
  }
};

// mask * dy as the reference's Mul2 forms it (a NaN or infinite dy stays visible under a zero mask)
__device__ __forceinline__ float masked(bool on, float g) { return __fmul_rn(on ? 1.0f : 0.0f, g); }

// Range gradients (:302-349): g_qr_min[q] = sum over the elements of q of
// (x < m) * dy, g_qr_max[q] = sum of (x > M) * dy. grid = (splits, Q); block
// (s, q) reduces its share to one pair of partial sums, a second kernel adds
// the partials of each q in a fixed order (deterministic).
// kDx: 0 = range sums only; 1 / 2 = per-tensor ranges (Q == 1, 16-byte aligned
// buffers) also write / accumulate the gradient w.r.t. x in the same pass
// (kFine: masked by m <= x <= M), so x and dy are read once.
template <int kDx, bool kFine>
__global__ void __launch_bounds__(kThreads) minmax_range_grad_kernel(const float *__restrict__ x,
                                                                     const float *__restrict__ dy, MinMaxView V,
                                                                     const float *__restrict__ m,
                                                                     const float *__restrict__ M, float *partial,
                                                                     float *__restrict__ dx) {
  const size_t q = blockIdx.y;
  const size_t per_q = V.outer * V.inner;
  const float lo = __ldg(m + q), hi = __ldg(M + q);
  float s_lo = 0.0f, s_hi = 0.0f;
  const size_t stride = (size_t)gridDim.x * kThreads;
  if (kDx != 0 || (V.Q == 1 && ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(dy)) & 15) == 0)) {
    const float4 *x4 = reinterpret_cast<const float4 *>(x);
    const float4 *g4 = reinterpret_cast<const float4 *>(dy);
    float4 *d4 = reinterpret_cast<float4 *>(dx);
    const size_t n4 = per_q / 4;
    // gradient w.r.t. x of one element: (x >= m) * (x <= M) * dy, or dy itself
    auto gx = [&](float a, float g, float d) {
      const float v = __fmul_rn(a >= lo ? 1.0f : 0.0f, a <= hi ? 1.0f : 0.0f);
      const float r = kFine ? __fmul_rn(v, g) : g;
      return kDx == 2 ? __fadd_rn(r, d) : r;
    };
    for (size_t t = (size_t)blockIdx.x * kThreads + threadIdx.x; t < n4; t += stride) {
      const float4 a = ld_stream(x4 + t), g = ld_stream(g4 + t);
      s_lo += masked(a.x < lo, g.x) + masked(a.y < lo, g.y) + masked(a.z < lo, g.z) + masked(a.w < lo, g.w);
      s_hi += masked(a.x > hi, g.x) + masked(a.y > hi, g.y) + masked(a.z > hi, g.z) + masked(a.w > hi, g.w);
      if (kDx != 0) {
        float4 d = make_float4(0.f, 0.f, 0.f, 0.f);
        if (kDx == 2)
          d = ld_stream(d4 + t);
        float4 r;
        r.x = gx(a.x, g.x, d.x);
        r.y = gx(a.y, g.y, d.y);
        r.z = gx(a.z, g.z, d.z);
        r.w = gx(a.w, g.w, d.w);
        st_stream(d4 + t, r);
      }
    }
    if (blockIdx.x == 0)
      for (size_t t = 4 * n4 + threadIdx.x; t < per_q; t += kThreads) {
        s_lo += masked(x[t] < lo, dy[t]);
        s_hi += masked(x[t] > hi, dy[t]);
        if (kDx != 0)
          dx[t] = gx(x[t], dy[t], kDx == 2 ? dx[t] : 0.0f);
      }
  } else {
    for (size_t t = (size_t)blockIdx.x * kThreads + threadIdx.x; t < per_q; t += stride) {
      const size_t o = t / V.inner, j = t - o * V.inner;
      const size_t e = (o * V.Q + q) * V.inner + j;
      const float a = x[e], g = dy[e];
      s_lo += masked(a < lo, g);
      s_hi += masked(a > hi, g);
    }
  }
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) {
    s_lo += __shfl_xor_sync(0xffffffffu, s_lo, d);
    s_hi += __shfl_xor_sync(0xffffffffu, s_hi, d);
  }
  __shared__ float w_lo[kThreads / 32], w_hi[kThreads / 32];
  if ((threadIdx.x & 31) == 0) {
    w_lo[threadIdx.x >> 5] = s_lo;
    w_hi[threadIdx.x >> 5] = s_hi;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < kThreads / 32; ++w) {
      s_lo += w_lo[w];
      s_hi += w_hi[w];
    }
    partial[(q * gridDim.x + blockIdx.x) * 2] = s_lo;
    partial[(q * gridDim.x + blockIdx.x) * 2 + 1] = s_hi;
  }
}

// One block per q: fixed-order sum of the `splits` partial pairs, then the
// accumulate-or-overwrite of :318-322 / :344-348.
__global__ void __launch_bounds__(kThreads) minmax_range_finish_kernel(const float *partial, unsigned splits,
                                                                       float *g_min, float *g_max, int do_min,
                                                                       int do_max, int accum_min, int accum_max) {
  const size_t q = blockIdx.x;
  float s_lo = 0.0f, s_hi = 0.0f;
  for (unsigned s = threadIdx.x; s < splits; s += kThreads) {
    s_lo += partial[(q * splits + s) * 2];
    s_hi += partial[(q * splits + s) * 2 + 1];
  }
  __shared__ float b_lo[kThreads], b_hi[kThreads];
  b_lo[threadIdx.x] = s_lo;
  b_hi[threadIdx.x] = s_hi;
  __syncthreads();
  for (int d = kThreads / 2; d > 0; d >>= 1) {
    if ((int)threadIdx.x < d) {
      b_lo[threadIdx.x] += b_lo[threadIdx.x + d];
      b_hi[threadIdx.x] += b_hi[threadIdx.x + d];
    }
    __syncthreads();
  }
  if (threadIdx.x == 0) {
    if (do_min)
      g_min[q] = accum_min ? __fadd_rn(g_min[q], b_lo[0]) : b_lo[0];
    if (do_max)
      g_max[q] = accum_max ? __fadd_rn(g_max[q], b_hi[0]) : b_hi[0];
  }
}

int minmax_backward(const float *x, const MinMaxView &V, const float *qr_min, const float *qr_max, const float *ql_min,
                    const float *ql_max, const float *dy, int x_min_max, int ema, int fine, const int32_t *prop,
                    const int32_t *accum, float *dx, float *g_min, float *g_max, cudaStream_t st) {
  const bool ranges = !(x_min_max || ema) && (prop[1] || prop[2]);
  const bool need_nudged = (prop[0] && fine) || ranges;
  if (V.size == 0 && !ranges)
    return NB200_OK;
  NB_CHECK(V.Q <= 65535, NB200_ENOTIMPL, "more than 65535 quantization ranges");
  const size_t per_q = V.outer * V.inner;
  size_t splits = (per_q + (size_t)kThreads * 16 - 1) / ((size_t)kThreads * 16);
  const size_t cap = ((size_t)sm_count() * kBlocksPerSm + V.Q - 1) / V.Q;
  splits = splits > cap ? cap : splits;
  splits = splits == 0 ? 1 : splits;
  AsyncScratch scratch(st);
  NB_TRY(scratch.alloc((2 * V.Q + (ranges ? 2 * V.Q * splits : 0)) * sizeof(float)));
  float *m = static_cast<float *>(scratch.p), *M = m + V.Q, *partial = M + V.Q;
  if (need_nudged) {
    NB_CHECK(qr_min && qr_max && ql_min && ql_max, NB200_EVALUE, "null range pointer");
    minmax_nudged_kernel<<<(unsigned)((V.Q + 255) / 256), 256, 0, st>>>(V.Q, qr_min, qr_max, ql_min, ql_max, m, M);
    NB_LAUNCH_CHECK();
  }
  // Per-tensor ranges with aligned buffers: one pass produces dx and the range sums.
  const bool fused = ranges && prop[0] && V.Q == 1 && V.size > 0 &&
                     ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(dy) |
                       reinterpret_cast<uintptr_t>(dx)) & 15) == 0;
  if (prop[0] && !fused) {
    if (fine) {
      MinMaxGrad op{m, M, V.Q, V.inner};
      NB_TRY(launch_gradient(x, dy, dx, V.size, accum[0], op, st));
    } else {
      NB_TRY(launch_gradient(x, dy, dx, V.size, accum[0], PassAllGrad(), st));
    }
  }
  if (ranges) {
    NB_CHECK((!prop[1] || g_min) && (!prop[2] || g_max), NB200_EVALUE, "null range-gradient pointer");
    NB_CHECK(V.size == 0 || (x && dy), NB200_EVALUE, "null data pointer");
    const dim3 grid((unsigned)splits, (unsigned)V.Q);
    if (!fused) {
      minmax_range_grad_kernel<0, false><<<grid, kThreads, 0, st>>>(x, dy, V, m, M, partial, nullptr);
    } else {
      NB_CHECK(dx != nullptr, NB200_EVALUE, "null data pointer");
      if (fine && accum[0])
        minmax_range_grad_kernel<2, true><<<grid, kThreads, 0, st>>>(x, dy, V, m, M, partial, dx);
      else if (fine)
        minmax_range_grad_kernel<1, true><<<grid, kThreads, 0, st>>>(x, dy, V, m, M, partial, dx);
      else if (accum[0])
        minmax_range_grad_kernel<2, false><<<grid, kThreads, 0, st>>>(x, dy, V, m, M, partial, dx);
      else
        minmax_range_grad_kernel<1, false><<<grid, kThreads, 0, st>>>(x, dy, V, m, M, partial, dx);
    }
    NB_LAUNCH_CHECK();
    minmax_range_finish_kernel<<<(unsigned)V.Q, kThreads, 0, st>>>(partial, (unsigned)splits, g_min, g_max, prop[1],
                                                                   prop[2], accum[1], accum[2]);
    NB_LAUNCH_CHECK();
  }
  return NB200_OK;
}
