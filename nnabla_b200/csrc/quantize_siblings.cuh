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
