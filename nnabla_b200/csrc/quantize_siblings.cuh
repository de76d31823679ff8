// Sibling quantization functions of the hot-path quantizers: BinarySigmoid,
// BinaryTanh, QuantizeLinear and DequantizeLinear, forward and backward.
// Included by quantize.cu inside namespace nb200::<anonymous>; they run on
// the same vectorised elementwise drivers (8 B per element forward, 12 B
// backward, HBM-bound).
#pragma once

// include/nbla/function/binary_sigmoid.hpp:50-52 (y = x > 0 ? 1 : 0) and
// binary_tanh.hpp:51-52 (y = x > 0 ? 1 : -1).
template <bool kTanh> struct BinaryActOp {
  static constexpr bool kHasCodes = false;
  bool codes_aligned(size_t) const { return true; }
  __device__ __forceinline__ void store_code(size_t, float) const {}
  __device__ __forceinline__ void store_codes4(size_t, float, float, float, float) const {}
  struct State {};
  __device__ __forceinline__ State init() const { return State(); }
  __device__ __forceinline__ float operator()(float x, size_t, float &, const State &) const {
    return x > 0.0f ? 1.0f : (kTanh ? -1.0f : 0.0f);
  }
};

// Their gradients: |x| >= 1 ? 0 : dy * 0.5 (sigmoid) / dy (tanh), combined as
// (accum ? dx : 0) + g (base_transform_unary.hpp:104-110), so the overwrite
// case still adds to a zero.
template <bool kTanh> struct BinaryActGrad {
  static constexpr bool kNeedsX = true;
  static constexpr bool kZeroPlus = true;
  struct State {};
  __device__ __forceinline__ State init() const { return State(); }
  __device__ __forceinline__ bool operator()(float x, float dy, size_t, float &g, const State &) const {
    g = (fabsf(x) >= 1.0f) ? 0.0f : (kTanh ? dy : __fmul_rn(dy, 0.5f));
    return true;
  }
};

// Index of the broadcast parameter that belongs to flat element i of an
// [outer, Q, inner] view (Q == 1: a single parameter).
struct BroadcastView {
  size_t Q, inner;
  __device__ __forceinline__ size_t at(size_t i) const {
    if (Q == 1)
      return 0;
    if ((i | inner | Q) >> 32)
      return (i / inner) % Q;
    return ((uint32_t)i / (uint32_t)inner) % (uint32_t)Q;
  }
};

// quantize_linear.cpp:86-101: HALF_AWAY_FROM_ZERO is std::round; HALF_TO_EVEN
// re-rounds exact halves as round(x * 0.5) * 2.
__device__ __forceinline__ float ql_round(float v, int half_to_even) {
  const float t = roundf(v);
  if (half_to_even && fabsf(__fsub_rn(v, t)) == 0.5f)
    return __fmul_rn(roundf(__fmul_rn(v, 0.5f)), 2.0f);
  return t;
}
__device__ __forceinline__ float ql_saturate(float v, float lo, float hi) {
  return v < lo ? lo : (v > hi ? hi : v); // NaN passes through, like the reference's comparisons
}

// The zero point is rounded and saturated in place first (quantize_linear.cpp:116-118).
__global__ void ql_zero_point_kernel(float *zp, size_t n, int half_to_even, float lo, float hi) {
  const size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x;
  if (i < n)
    zp[i] = ql_saturate(ql_round(zp[i], half_to_even), lo, hi);
}

// y = saturate(round(x / scale) + zero_point) (quantize_linear.cpp:103-122)
struct QuantizeLinearOp {
  static constexpr bool kHasCodes = false;
  const float *scale, *zp;
  BroadcastView vs, vz;
  int half_to_even;
  float lo, hi;
  bool codes_aligned(size_t) const { return true; }
  __device__ __forceinline__ void store_code(size_t, float) const {}
  __device__ __forceinline__ void store_codes4(size_t, float, float, float, float) const {}
  struct State {
    float s, z;
  };
  __device__ __forceinline__ State init() const {
    State st;
    st.s = __ldg(scale);
    st.z = __ldg(zp);
    return st;
  }
  __device__ __forceinline__ float operator()(float x, size_t i, float &, const State &st) const {
    const float s = vs.Q == 1 ? st.s : __ldg(scale + vs.at(i));
    const float z = vz.Q == 1 ? st.z : __ldg(zp + vz.at(i));
    const float t = ql_round(__fdiv_rn(x, s), half_to_even);
    return ql_saturate(__fadd_rn(t, z), lo, hi);
  }
};

// y = (x - zero_point) * scale (dequantize_linear.cpp:60-71)
struct DequantizeLinearOp {
  static constexpr bool kHasCodes = false;
  const float *scale, *zp;
  BroadcastView vs, vz;
  bool codes_aligned(size_t) const { return true; }
  __device__ __forceinline__ void store_code(size_t, float) const {}
  __device__ __forceinline__ void store_codes4(size_t, float, float, float, float) const {}
  struct State {
    float s, z;
  };
  __device__ __forceinline__ State init() const {
    State st;
    st.s = __ldg(scale);
    st.z = __ldg(zp);
    return st;
  }
  __device__ __forceinline__ float operator()(float x, size_t i, float &, const State &st) const {
    const float s = vs.Q == 1 ? st.s : __ldg(scale + vs.at(i));
    const float z = vz.Q == 1 ? st.z : __ldg(zp + vz.at(i));
    return __fmul_rn(__fsub_rn(x, z), s);
  }
};

// dx (+)= dy / scale (quantize_linear.cpp:137-147) or dy * scale (dequantize_linear.cpp:92-102)
template <bool kDivide> struct LinearScaleGrad {
  static constexpr bool kNeedsX = false;
  static constexpr bool kZeroPlus = false;
  const float *scale;
  BroadcastView vs;
  struct State {
    float s;
  };
  __device__ __forceinline__ State init() const {
    State st;
    st.s = __ldg(scale);
    return st;
  }
  __device__ __forceinline__ bool operator()(float, float dy, size_t i, float &g, const State &st) const {
    const float s = vs.Q == 1 ? st.s : __ldg(scale + vs.at(i));
    g = kDivide ? __fdiv_rn(dy, s) : __fmul_rn(dy, s);
    return true;
  }
};

// View of a broadcast parameter tensor over x (shape rules of
// quantize_linear.cpp:27-48: every extent is 1 or x's).
int broadcast_view(const int64_t *xs, const int64_t *ps, int ndim, BroadcastView *v, size_t *size) {
  MinMaxView V;
  NB_TRY(minmax_view(xs, ps, ndim, &V));
  v->Q = V.Q;
  v->inner = V.inner;
  if (size)
    *size = V.size;
  return NB200_OK;
}

int quantize_linear_range(int narrow_range, int dtype, float *lo, float *hi) {
  // dtypes::BYTE = 1, dtypes::UBYTE = 2 (include/nbla/dtypes.hpp:32-35); the
  // reference leaves the range uninitialised for any other dtype.
  NB_CHECK(dtype == 1 || dtype == 2, NB200_ENOTIMPL, "QuantizeLinear: dtype must be BYTE (1) or UBYTE (2), got %d",
           dtype);
  if (dtype == 1) {
    *lo = narrow_range ? -127.0f : -128.0f;
    *hi = 127.0f;
  } else {
    *lo = narrow_range ? 1.0f : 0.0f;
    *hi = 255.0f;
  }
  return NB200_OK;
}

// ---------------------------------------------------------------------------
// Prune (src/nbla/function/generic/prune.cpp:38-72): y = |x| < t ? 0 : x with
// t = the (int)((n - 1) * rate)-th smallest |x| (+ 1 when rate == 1). The
// reference sorts a copy of x; here the order statistic comes from a radix
// select on the bit pattern of |x| (monotone for non-negative floats): three
// histogram passes over 11 + 11 + 9 bits, each followed by a one-block scan
// that fixes the next bits of the answer, then the elementwise pass. 16 B
// read + 4 B written per element, no sort, no host round trip.
// ---------------------------------------------------------------------------
struct PruneState {
  unsigned int prefix;      // bits of the answer fixed so far (in place)
  unsigned int prefix_mask; // which bits are fixed
  unsigned long long rank;  // rank of the answer among the elements that match the prefix
  float threshold;          // final threshold (after the last scan)
};

__global__ void prune_init_kernel(PruneState *s, unsigned long long rank, unsigned int *hist) {
  if (threadIdx.x == 0 && blockIdx.x == 0) {
    s->prefix = 0u;
    s->prefix_mask = 0u;
    s->rank = rank;
    s->threshold = 0.0f;
  }
  for (int i = threadIdx.x; i < 3 * 2048; i += blockDim.x)
    hist[i] = 0u;
}

// Histogram of bits [shift, shift + nbits) of |x| over the elements whose
// already-fixed bits equal the prefix.
__global__ void __launch_bounds__(kThreads) prune_hist_kernel(const float *__restrict__ x, size_t n, int shift, int nbits,
                                                              const PruneState *__restrict__ s,
                                                              unsigned int *__restrict__ hist) {
  __shared__ unsigned int h[2048];
  for (int i = threadIdx.x; i < 2048; i += kThreads)
    h[i] = 0u;
  __syncthreads();
  const unsigned int prefix = s->prefix, pmask = s->prefix_mask, bmask = (1u << nbits) - 1u;
  const size_t stride = (size_t)gridDim.x * kThreads;
  for (size_t i = (size_t)blockIdx.x * kThreads + threadIdx.x; i < n; i += stride) {
    const unsigned int b = __float_as_uint(x[i]) & 0x7fffffffu;
    if ((b & pmask) == prefix)
      atomicAdd(&h[(b >> shift) & bmask], 1u);
  }
  __syncthreads();
  for (int i = threadIdx.x; i < (1 << nbits); i += kThreads)
    if (h[i] != 0u)
      atomicAdd(&hist[i], h[i]);
}

// One block: finds the bin that holds the wanted rank, fixes its bits.
__global__ void prune_scan_kernel(PruneState *s, const unsigned int *hist, int shift, int nbits, int last,
                                  float add_one) {
  if (threadIdx.x != 0)
    return;
  unsigned long long rank = s->rank, seen = 0;
  int bin = (1 << nbits) - 1;
  for (int i = 0; i < (1 << nbits); ++i) {
    if (seen + hist[i] > rank) {
      bin = i;
      break;
    }
    seen += hist[i];
  }
  s->rank = rank - seen;
  s->prefix |= (unsigned int)bin << shift;
  s->prefix_mask |= ((1u << nbits) - 1u) << shift;
  if (last)
    s->threshold = __fadd_rn(__uint_as_float(s->prefix), add_one);
}

struct PruneOp {
  static constexpr bool kHasCodes = false;
  const PruneState *state;
  bool codes_aligned(size_t) const { return true; }
  __device__ __forceinline__ void store_code(size_t, float) const {}
  __device__ __forceinline__ void store_codes4(size_t, float, float, float, float) const {}
  struct State {
    float t;
  };
  __device__ __forceinline__ State init() const {
    State st;
    st.t = state->threshold;
    return st;
  }
  __device__ __forceinline__ float operator()(float x, size_t, float &, const State &st) const {
    return fabsf(x) < st.t ? 0.0f : x;
  }
};

int prune_forward(const float *x, float *y, size_t size, float rate, cudaStream_t st) {
  NB_CHECK(rate >= 0.0f && rate <= 1.0f, NB200_EVALUE, "Rate %f must be in [0, 1].", rate);
  if (size == 0)
    return NB200_OK;
  NB_CHECK(x && y, NB200_EVALUE, "null data pointer");
  NB_CHECK(size < (1ull << 31), NB200_ENOTIMPL, "Prune: more than 2^31 elements (the reference indexes with int)");
  const unsigned long long rank = (unsigned long long)(int)((float)((int)size - 1) * rate); // prune.cpp:43
  AsyncScratch scratch(st);
  NB_TRY(scratch.alloc(sizeof(PruneState) + 3 * 2048 * sizeof(unsigned int)));
  PruneState *s = static_cast<PruneState *>(scratch.p);
  unsigned int *hist = reinterpret_cast<unsigned int *>(s + 1);
  prune_init_kernel<<<1, 256, 0, st>>>(s, rank, hist);
  NB_LAUNCH_CHECK();
  const int shifts[3] = {20, 9, 0}, bits[3] = {11, 11, 9};
  const float add_one = ((double)rate == 1.0) ? 1.0f : 0.0f; // prune.cpp:62
  const unsigned grid = grid_for((size + 15) / 16);
  for (int p = 0; p < 3; ++p) {
    prune_hist_kernel<<<grid, kThreads, 0, st>>>(x, size, shifts[p], bits[p], s, hist + p * 2048);
    NB_LAUNCH_CHECK();
    prune_scan_kernel<<<1, 32, 0, st>>>(s, hist + p * 2048, shifts[p], bits[p], p == 2, add_one);
    NB_LAUNCH_CHECK();
  }
  PruneOp op{s};
  return launch_elementwise(x, y, size, op, st);
}
