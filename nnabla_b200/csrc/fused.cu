// Inference-time fusion of the elementwise chain that follows every
// convolution of a quantized residual network:
//
//   y = FixedPointQuantize( ReLU( BN_a(a) [+ BN_b(b) | + b] ) )
//
// i.e. BatchNormalization::forward_impl_global
// (src/nbla/function/generic/batch_normalization.cpp:228-260), Add2
// (add2.cpp), ReLU (relu.cpp) and FixedPointQuantize
// (fixed_point_quantize.cpp:45-66) in one pass: 4 B (+4 B for the second
// operand) read and 4 B written per element instead of 8 B per function. The
// reference's own fused form of the first three is FusedBatchNormalization
// (fused_batch_normalization.cpp). Every operation is rounded on its own, in
// the order the separate functions apply them, so the result is bit-identical
// to the unfused chain.
#include <cmath>

#include "common.cuh"

namespace nb200 {
namespace {

constexpr int kThreads = 256;

struct BnTerm {
  const float *x, *beta, *gamma, *mean, *var; // mean == NULL: x is used as it is (plain residual)
};

struct FxpParams {
  float maxv, minv, delta, inv_delta;
  int pow2; // delta is a power of two: the division is an exact multiplication
};

__device__ __forceinline__ float bn_value(float v, float m, float g, float sd, float b) {
  return __fadd_rn(__fdiv_rn(__fmul_rn(__fsub_rn(v, m), g), sd), b);
}

// fixed_point_quantize.cpp:53-65; int(double(q) + 0.5) == floor(q) + (q - floor(q) >= 0.5) for q >= 0
__device__ __forceinline__ float fxp_value(float x, const FxpParams &P) {
  if (x > P.maxv)
    return P.maxv;
  if (x < P.minv)
    return P.minv;
  const float a = fabsf(x);
  const float q = P.pow2 ? __fmul_rn(a, P.inv_delta) : __fdiv_rn(a, P.delta);
  const float t = floorf(q);
  const float k = t + ((__fsub_rn(q, t) >= 0.5f) ? 1.0f : 0.0f);
  const float r = __fmul_rn(k, P.delta);
  return x < 0.0f ? -r : r;
}

struct ChannelConsts {
  float m, g, sd, b;
};
__device__ __forceinline__ ChannelConsts load_consts(const BnTerm &t, int c, float eps) {
  ChannelConsts k;
  k.m = __ldg(t.mean + c);
  k.sd = __fsqrt_rn(__fadd_rn(__ldg(t.var + c), eps));
  k.g = t.gamma ? __ldg(t.gamma + c) : 1.0f;
  k.b = t.beta ? __ldg(t.beta + c) : 0.0f;
  return k;
}

// kSecond: 0 = one term, 1 = plain second operand, 2 = second operand with its own BN.
template <bool kVec, int kSecond>
__global__ void __launch_bounds__(kThreads) bn_add_relu_fxp_kernel(BnTerm A, BnTerm B, size_t total, int C, int S,
                                                                   float eps, int relu, int quantize, FxpParams P,
                                                                   float *__restrict__ y) {
  const size_t stride = (size_t)gridDim.x * kThreads;
  auto finish = [&](float v) {
    if (relu)
      v = v > 0.0f ? v : 0.0f;
    return quantize ? fxp_value(v, P) : v;
  };
  if (kVec) {
    const size_t total4 = total / 4;
    const int S4 = S / 4;
    for (size_t i = (size_t)blockIdx.x * kThreads + threadIdx.x; i < total4; i += stride) {
      const int c = (int)((i / S4) % C);
      const ChannelConsts ka = load_consts(A, c, eps);
      const float4 va = __ldcs(reinterpret_cast<const float4 *>(A.x) + i);
      float4 r;
      r.x = bn_value(va.x, ka.m, ka.g, ka.sd, ka.b);
      r.y = bn_value(va.y, ka.m, ka.g, ka.sd, ka.b);
      r.z = bn_value(va.z, ka.m, ka.g, ka.sd, ka.b);
      r.w = bn_value(va.w, ka.m, ka.g, ka.sd, ka.b);
      if (kSecond != 0) {
        float4 vb = __ldcs(reinterpret_cast<const float4 *>(B.x) + i);
        if (kSecond == 2) {
          const ChannelConsts kb = load_consts(B, c, eps);
          vb.x = bn_value(vb.x, kb.m, kb.g, kb.sd, kb.b);
          vb.y = bn_value(vb.y, kb.m, kb.g, kb.sd, kb.b);
          vb.z = bn_value(vb.z, kb.m, kb.g, kb.sd, kb.b);
          vb.w = bn_value(vb.w, kb.m, kb.g, kb.sd, kb.b);
        }
        r.x = __fadd_rn(r.x, vb.x);
        r.y = __fadd_rn(r.y, vb.y);
        r.z = __fadd_rn(r.z, vb.z);
        r.w = __fadd_rn(r.w, vb.w);
      }
      r.x = finish(r.x);
      r.y = finish(r.y);
      r.z = finish(r.z);
      r.w = finish(r.w);
      __stcs(reinterpret_cast<float4 *>(y) + i, r);
    }
  } else {
    for (size_t i = (size_t)blockIdx.x * kThreads + threadIdx.x; i < total; i += stride) {
      const int c = (int)((i / S) % C);
      const ChannelConsts ka = load_consts(A, c, eps);
      float v = bn_value(A.x[i], ka.m, ka.g, ka.sd, ka.b);
      if (kSecond != 0) {
        float w = B.x[i];
        if (kSecond == 2) {
          const ChannelConsts kb = load_consts(B, c, eps);
          w = bn_value(w, kb.m, kb.g, kb.sd, kb.b);
        }
        v = __fadd_rn(v, w);
      }
      y[i] = finish(v);
    }
  }
}

unsigned grid_for(size_t items, int per_thread) {
  size_t b = (items + (size_t)kThreads * per_thread - 1) / ((size_t)kThreads * per_thread);
  const size_t cap = (size_t)sm_count() * 128;
  if (b > cap)
    b = cap;
  return (unsigned)(b < 1 ? 1 : b);
}

template <int kSecond>
int launch(const BnTerm &A, const BnTerm &B, size_t total, int C, int S, float eps, int relu, int quantize,
           const FxpParams &P, float *y, bool vec, cudaStream_t st) {
  if (vec)
    bn_add_relu_fxp_kernel<true, kSecond><<<grid_for(total / 4, 1), kThreads, 0, st>>>(A, B, total, C, S, eps, relu,
                                                                                        quantize, P, y);
  else
    bn_add_relu_fxp_kernel<false, kSecond><<<grid_for(total, 4), kThreads, 0, st>>>(A, B, total, C, S, eps, relu,
                                                                                     quantize, P, y);
  NB_LAUNCH_CHECK();
  return NB200_OK;
}

} // namespace
} // namespace nb200

using namespace nb200;

extern "C" int nb200_bn_add_relu_fxp_f32(const float *a, const float *beta_a, const float *gamma_a,
                                         const float *mean_a, const float *var_a, const float *b,
                                         const float *beta_b, const float *gamma_b, const float *mean_b,
                                         const float *var_b, float *y, int64_t outer, int64_t channels, int64_t inner,
                                         float eps, int relu, int quantize, int sign, int n, float delta,
                                         void *stream) {
  NB_CHECK(outer >= 0 && channels > 0 && inner > 0, NB200_EVALUE, "bad extents");
  NB_CHECK(channels < (1ll << 31) && inner < (1ll << 31), NB200_EVALUE, "extent exceeds 2^31");
  FxpParams P{0.f, 0.f, 1.f, 1.f, 0};
  if (quantize) {
    // the reference's setup (fixed_point_quantize.cpp:31-42)
    NB_CHECK(n > 0 && delta > 0.f, NB200_EVALUE, "Both bit width and delta should be positive.");
    const int nn = sign ? n - 1 : n;
    NB_CHECK(nn > 0, NB200_EVALUE, "bit width should be positive when considering sign (1bit).");
    P.maxv = (float)((std::pow(2, nn) - 1) * delta);
    P.minv = sign ? -P.maxv : 0.0f;
    P.delta = delta;
    int ex = 0;
    const float mant = std::frexp(delta, &ex);
    P.pow2 = (mant == 0.5f) && ex > -120 && ex < 120;
    P.inv_delta = P.pow2 ? 1.0f / delta : 0.0f;
  }
  const size_t total = (size_t)outer * channels * inner;
  if (total == 0)
    return NB200_OK;
  NB_CHECK(a && y && mean_a && var_a, NB200_EVALUE, "null data pointer");
  NB_CHECK(mean_b == nullptr || (b != nullptr && var_b != nullptr), NB200_EVALUE,
           "statistics of the second operand without the operand");
  const BnTerm A{a, beta_a, gamma_a, mean_a, var_a};
  const BnTerm B{b, beta_b, gamma_b, mean_b, var_b};
  const bool vec = (inner % 4 == 0) &&
                   ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b) | reinterpret_cast<uintptr_t>(y)) &
                    15) == 0;
  cudaStream_t st = as_stream(stream);
  if (b == nullptr)
    return launch<0>(A, B, total, (int)channels, (int)inner, eps, relu, quantize, P, y, vec, st);
  if (mean_b == nullptr)
    return launch<1>(A, B, total, (int)channels, (int)inner, eps, relu, quantize, P, y, vec, st);
  return launch<2>(A, B, total, (int)channels, (int)inner, eps, relu, quantize, P, y, vec, st);
}
