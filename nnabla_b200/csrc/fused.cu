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
#include "prepare.cuh"

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
// (v - mean) * gamma / sqrt(var + eps) + beta, every operation rounded on its own
__device__ __forceinline__ float bn_value(float v, const ChannelConsts &k) {
  return __fadd_rn(__fdiv_rn(__fmul_rn(__fsub_rn(v, k.m), k.g), k.sd), k.b);
}

// kSecond: 0 = one term, 1 = plain second operand, 2 = second operand with its own BN.
// kFast: ReLU on, quantizer on, power-of-two delta: the value is non-negative and the quantizer is
// (floor(v * 2 / delta) + 1) >> 1 capped at the largest code, times delta (same bits, fewer operations).
template <bool kVec, int kSecond, bool kFast = false>
__global__ void __launch_bounds__(kThreads) bn_add_relu_fxp_kernel(BnTerm A, BnTerm B, size_t total, int C, int S,
                                                                   float eps, int relu, int quantize, FxpParams P,
                                                                   int cached, float *__restrict__ y) {
  // the channels' constants (a square root and a reciprocal each) are worked out once per
  // block into shared memory when they fit (cached != 0), else per item
  extern __shared__ __align__(16) uint8_t consts_raw[];
  ChannelConsts *consts = reinterpret_cast<ChannelConsts *>(consts_raw);
  if (cached) {
    for (int c = threadIdx.x; c < C; c += kThreads) {
      consts[c] = load_consts(A, c, eps);
      if (kSecond == 2)
        consts[C + c] = load_consts(B, c, eps);
    }
    __syncthreads();
  }
  auto consts_of = [&](const BnTerm &t, int c, int which) {
    return cached ? consts[which * C + c] : load_consts(t, c, eps);
  };
  const size_t stride = (size_t)gridDim.x * kThreads;
  const float two_inv = __fmul_rn(P.inv_delta, 2.0f), cap = __fmul_rn(__fmul_rn(P.maxv, P.inv_delta), 2.0f) + 0.5f;
  auto finish = [&](float v) {
    if (kFast) {
      v = fmaxf(v, 0.0f); // ReLU; a NaN becomes 0 as below
      const int k = (__float2int_rd(fminf(__fmul_rn(v, two_inv), cap)) + 1) >> 1;
      return __fmul_rn((float)k, P.delta);
    }
    if (relu)
      v = v > 0.0f ? v : 0.0f;
    return quantize ? fxp_value(v, P) : v;
  };
  if (kVec) {
    const size_t total4 = total / 4;
    const int S4 = S / 4;
    const size_t first = (size_t)blockIdx.x * kThreads + threadIdx.x;
    ChannelWalk walk(first, stride, (unsigned)S4, (unsigned)C);
    for (size_t i = first; i < total4; i += stride, walk.next()) {
      const int c = (int)walk.c;
      const ChannelConsts ka = consts_of(A, c, 0);
      const float4 va = __ldcs(reinterpret_cast<const float4 *>(A.x) + i);
      float4 r;
      r.x = bn_value(va.x, ka);
      r.y = bn_value(va.y, ka);
      r.z = bn_value(va.z, ka);
      r.w = bn_value(va.w, ka);
      if (kSecond != 0) {
        float4 vb = __ldcs(reinterpret_cast<const float4 *>(B.x) + i);
        if (kSecond == 2) {
          const ChannelConsts kb = consts_of(B, c, 1);
          vb.x = bn_value(vb.x, kb);
          vb.y = bn_value(vb.y, kb);
          vb.z = bn_value(vb.z, kb);
          vb.w = bn_value(vb.w, kb);
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
    const size_t first = (size_t)blockIdx.x * kThreads + threadIdx.x;
    ChannelWalk walk(first, stride, (unsigned)S, (unsigned)C);
    for (size_t i = first; i < total; i += stride, walk.next()) {
      const int c = (int)walk.c;
      const ChannelConsts ka = consts_of(A, c, 0);
      float v = bn_value(A.x[i], ka);
      if (kSecond != 0) {
        float w = B.x[i];
        if (kSecond == 2) {
          const ChannelConsts kb = consts_of(B, c, 1);
          w = bn_value(w, kb);
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
  const size_t smem = (size_t)C * sizeof(ChannelConsts) * (kSecond == 2 ? 2 : 1);
  const int cached = smem <= 40 * 1024;
  // with the constants in shared memory a block should live long enough to amortise them
  const size_t items = vec ? total / 4 : total;
  unsigned grid = grid_for(items, vec ? 1 : 4);
  if (cached && items >= (size_t)(8 * C) * kThreads) {
    const unsigned few = (unsigned)sm_count() * 16;
    grid = grid > few ? few : grid;
  }
  // the largest code must be exact in fp32 arithmetic for the short form (codes below 2^22: twice the code plus one half is exact)
  const bool fast = vec && relu && quantize && P.pow2 && P.maxv * P.inv_delta < 4194304.0f;
  if (fast)
    bn_add_relu_fxp_kernel<true, kSecond, true><<<grid, kThreads, cached ? smem : 0, st>>>(A, B, total, C, S, eps, relu,
                                                                                            quantize, P, cached, y);
  else if (vec)
    bn_add_relu_fxp_kernel<true, kSecond><<<grid, kThreads, cached ? smem : 0, st>>>(A, B, total, C, S, eps, relu,
                                                                                      quantize, P, cached, y);
  else
    bn_add_relu_fxp_kernel<false, kSecond><<<grid, kThreads, cached ? smem : 0, st>>>(A, B, total, C, S, eps, relu,
                                                                                       quantize, P, cached, y);
  NB_LAUNCH_CHECK();
  return NB200_OK;
}

// ---------------------------------------------------------------------------
// The same chain with its result written as int8 channel-last codes
// [batch][inner][slots] (what the int8 convolution reads): a 64-pixel x 64-slot
// tile per block, normalised values staged in shared memory (fp32, pixel-major)
// and quantized while they are written out four channels per thread. The
// residual, when it is itself a code tensor, is read in the output's own
// layout at that point.
// ---------------------------------------------------------------------------
constexpr int kTilePx = 64, kTileSlots = 64, kTilePitch = kTileSlots + 1;

// fixed_point_quantize.cpp:53-65 as an integer code: y = code * delta. The reference rounds
// with int(|x| / delta + 0.5) = floor(q + 0.5) = (floor(2q) + 1) >> 1 (2q is exact); the two
// range tests of the reference are the clamp of the code, because q grows with |x|. A NaN gives 0.
__device__ __forceinline__ int fxp_code(float x, const FxpParams &P, int kmax, int kmin) {
  const float a = fabsf(x);
  const float q = P.pow2 ? __fmul_rn(a, P.inv_delta) : __fdiv_rn(a, P.delta);
  float q2 = __fmul_rn(q, 2.0f);
  q2 = !(q2 >= 1024.0f) ? q2 : 1024.0f; // keeps the conversion in range; the codes stop at 127 anyway
  int k = (__float2int_rd(q2) + 1) >> 1;
  k = k < kmax ? k : kmax;
  const int nk = -k > kmin ? -k : kmin;
  return x < 0.0f ? nk : k;
}

struct CodesLayout {
  int C, HW, groups, Cg, c_pad_g, slots;
};

// kSecond: 0 = one term, 1 = plain fp32 second operand, 2 = fp32 second operand with its own BN,
// 3 = second operand given as codes (value = code * b_delta).
// kFast: the common case of a residual network (ReLU on, power-of-two delta, every slot holds a
// channel): the value is non-negative, so the code is (floor(v * 2 / delta) + 1) >> 1 capped at
// kmax, six operations instead of the general quantizer's fourteen; same codes.
template <bool kVec, int kSecond, bool kFast = false>
__global__ void __launch_bounds__(256) bn_add_relu_fxp_codes_kernel(BnTerm A, BnTerm B,
                                                                    const int8_t *__restrict__ b_codes, float b_delta,
                                                                    CodesLayout L, float eps, int relu, FxpParams P,
                                                                    int kmax, int kmin, int8_t *__restrict__ out) {
  __shared__ float tile[kTilePx * kTilePitch];
  __shared__ ChannelConsts consts_a[kTileSlots], consts_b[kSecond == 2 ? kTileSlots : 1];
  __shared__ int channel_of[kTileSlots]; // channel held by each slot of the tile, -1 = padding
  const int n = blockIdx.z;
  const int p0 = blockIdx.x * kTilePx, d0 = blockIdx.y * kTileSlots;
  if (threadIdx.x < kTileSlots) {
    // the normalisation constants of the tile's channels, once per block
    const int d = d0 + threadIdx.x;
    const int g = d / L.c_pad_g, cc = d - g * L.c_pad_g;
    const bool live = d < L.slots && g < L.groups && cc < L.Cg;
    const int c = live ? g * L.Cg + cc : -1;
    channel_of[threadIdx.x] = c;
    if (live) {
      consts_a[threadIdx.x] = load_consts(A, c, eps);
      if (kSecond == 2)
        consts_b[threadIdx.x] = load_consts(B, c, eps);
    }
  }
  __syncthreads();
  const int px4 = threadIdx.x & 15, ch = threadIdx.x >> 4; // 16 pixel quads x 16 channel rows
  const int p = p0 + 4 * px4;
  // all loads of the thread's four channel rows are issued before the arithmetic starts
  float av[4][4], bv[4][4];
  int chan[4];
#pragma unroll
  for (int r = 0; r < 4; ++r) {
    const int c = channel_of[ch + 16 * r];
    chan[r] = (c >= 0 && p < L.HW) ? c : -1;
#pragma unroll
    for (int i = 0; i < 4; ++i)
      av[r][i] = bv[r][i] = 0.0f;
    if (chan[r] >= 0) {
      const int64_t base = ((int64_t)n * L.C + c) * L.HW + p;
      if (kVec) {
        const float4 t = __ldcs(reinterpret_cast<const float4 *>(A.x + base));
        av[r][0] = t.x, av[r][1] = t.y, av[r][2] = t.z, av[r][3] = t.w;
        if (kSecond == 1 || kSecond == 2) {
          const float4 u = __ldcs(reinterpret_cast<const float4 *>(B.x + base));
          bv[r][0] = u.x, bv[r][1] = u.y, bv[r][2] = u.z, bv[r][3] = u.w;
        }
      } else {
#pragma unroll
        for (int i = 0; i < 4; ++i)
          if (p + i < L.HW) {
            av[r][i] = A.x[base + i];
            if (kSecond == 1 || kSecond == 2)
              bv[r][i] = B.x[base + i];
          }
      }
    }
  }
#pragma unroll
  for (int r = 0; r < 4; ++r) {
    const int dd = ch + 16 * r;
    float v[4] = {0.f, 0.f, 0.f, 0.f};
    if (chan[r] >= 0) {
      const ChannelConsts ka = consts_a[dd];
      ChannelConsts kb{};
      if (kSecond == 2)
        kb = consts_b[dd];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        v[i] = bn_value(av[r][i], ka);
        if (kSecond == 2)
          v[i] = __fadd_rn(v[i], bn_value(bv[r][i], kb));
        else if (kSecond == 1)
          v[i] = __fadd_rn(v[i], bv[r][i]);
      }
    }
#pragma unroll
    for (int i = 0; i < 4; ++i)
      tile[(4 * px4 + i) * kTilePitch + dd] = v[i];
  }
  __syncthreads();
  const int word = threadIdx.x & 15, prow = threadIdx.x >> 4;
  const int d = d0 + 4 * word;
  if (d >= L.slots)
    return;
  // slots of this word that hold a channel (the others stay 0 whatever the arithmetic gives)
  bool live[4];
#pragma unroll
  for (int k = 0; k < 4; ++k)
    live[k] = channel_of[4 * word + k] >= 0;
#pragma unroll
  for (int pp = prow; pp < kTilePx; pp += 16) {
    const int pix = p0 + pp;
    if (pix >= L.HW)
      break;
    const int64_t o = ((int64_t)n * L.HW + pix) * L.slots + d;
    uint32_t res = 0;
    if (kSecond == 3)
      res = __ldcs(reinterpret_cast<const unsigned int *>(b_codes + o));
    uint32_t packed = 0;
    const float two_inv = __fmul_rn(P.inv_delta, 2.0f), cap = (float)(2 * kmax) + 0.5f;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      float v = tile[pp * kTilePitch + 4 * word + k];
      if (kSecond == 3)
        v = __fadd_rn(v, __fmul_rn((float)(int)(int8_t)((res >> (8 * k)) & 0xffu), b_delta));
      if (kFast) {
        v = fmaxf(v, 0.0f); // ReLU; a NaN becomes 0 as in the general form
        const int code = (__float2int_rd(fminf(__fmul_rn(v, two_inv), cap)) + 1) >> 1;
        packed |= (uint32_t)code << (8 * k);
      } else {
        if (relu)
          v = v > 0.0f ? v : 0.0f;
        const int code = live[k] ? fxp_code(v, P, kmax, kmin) : 0;
        packed |= ((uint32_t)code & 0xffu) << (8 * k);
      }
    }
    *reinterpret_cast<uint32_t *>(out + o) = packed;
  }
}

// codes [batch][HW][slots] -> y [batch][C][HW] = code * delta (64 x 64 tiles through shared memory)
__global__ void __launch_bounds__(256) codes_nhwc_to_f32_kernel(const int8_t *__restrict__ codes, CodesLayout L,
                                                                float delta, float *__restrict__ y) {
  __shared__ int8_t tile[kTilePx][kTileSlots + 4];
  const int n = blockIdx.z;
  const int p0 = blockIdx.x * kTilePx, d0 = blockIdx.y * kTileSlots;
  const int word = threadIdx.x & 15, prow = threadIdx.x >> 4;
  for (int pp = prow; pp < kTilePx; pp += 16) {
    const int pix = p0 + pp, d = d0 + 4 * word;
    uint32_t v = 0;
    if (pix < L.HW && d < L.slots)
      v = *reinterpret_cast<const uint32_t *>(codes + ((int64_t)n * L.HW + pix) * L.slots + d);
    *reinterpret_cast<uint32_t *>(&tile[pp][4 * word]) = v;
  }
  __syncthreads();
  const int px = threadIdx.x & 63, c4 = threadIdx.x >> 6;
  const int pix = p0 + px;
  if (pix >= L.HW)
    return;
  for (int dd = c4; dd < kTileSlots; dd += 4) {
    const int d = d0 + dd;
    const int g = d / L.c_pad_g, cc = d - g * L.c_pad_g;
    if (d < L.slots && g < L.groups && cc < L.Cg)
      y[((int64_t)n * L.C + g * L.Cg + cc) * L.HW + pix] = __fmul_rn((float)tile[px][dd], delta);
  }
}

// ---------------------------------------------------------------------------
// Max-pooling on codes (channel-last): the value code * delta grows with the
// code, so the window maximum of the codes is the code of the window maximum.
// One thread per output pixel and 16 slots: kh * kw 128-bit loads, bytewise maxima.
// ---------------------------------------------------------------------------
struct PoolGeom {
  int H, W, Ho, Wo, kh, kw, sh, sw, ph, pw;
};

__global__ void __launch_bounds__(256) max_pooling_codes_kernel(const int8_t *__restrict__ in, int slots, PoolGeom G,
                                                                int8_t *__restrict__ out) {
  // grid = (chunks of an output row, output rows, samples): no wide divisions per item
  const int vecs = slots / 16; // 16-slot groups per pixel
  const int item = blockIdx.x * 256 + threadIdx.x;
  if (item >= G.Wo * vecs)
    return;
  const int ox = item / vecs, v = item - ox * vecs;
  const int oy = blockIdx.y;
  const size_t n = blockIdx.z;
  // window clipped to the input (max_pooling.cpp:140-191): padding never takes part
  int y0 = oy * G.sh - G.ph, x0 = ox * G.sw - G.pw;
  const int y1 = min(min(y0 + G.kh, G.H + G.ph), G.H), x1 = min(min(x0 + G.kw, G.W + G.pw), G.W);
  y0 = max(y0, 0);
  x0 = max(x0, 0);
  uint4 best = make_uint4(0x80808080u, 0x80808080u, 0x80808080u, 0x80808080u);
  for (int iy = y0; iy < y1; ++iy) {
    const uint4 *row = reinterpret_cast<const uint4 *>(in + ((n * G.H + iy) * (size_t)G.W) * slots) + v;
    for (int ix = x0; ix < x1; ++ix) {
      const uint4 q = __ldg(row + (size_t)ix * vecs);
      best.x = __vmaxs4(best.x, q.x);
      best.y = __vmaxs4(best.y, q.y);
      best.z = __vmaxs4(best.z, q.z);
      best.w = __vmaxs4(best.w, q.w);
    }
  }
  reinterpret_cast<uint4 *>(out)[((n * G.Ho + oy) * (size_t)G.Wo + ox) * vecs + v] = best;
}

int fill_fxp(FxpParams &P, int sign, int n, float delta) {
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
  if (quantize)
    NB_TRY(fill_fxp(P, sign, n, delta));
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

namespace {
int codes_layout(CodesLayout &L, int64_t batch, int64_t channels, int64_t inner, int group) {
  NB_CHECK(batch >= 0 && channels > 0 && inner > 0 && group > 0 && channels % group == 0, NB200_EVALUE, "bad extents");
  NB_CHECK(channels < (1 << 30) && inner < (1 << 30), NB200_EVALUE, "extent exceeds 2^30");
  NB_CHECK(batch <= 65535, NB200_ENOTIMPL, "batch larger than 65535");
  L.C = (int)channels;
  L.HW = (int)inner;
  L.groups = group;
  L.Cg = (int)(channels / group);
  L.c_pad_g = (L.Cg + 15) / 16 * 16;
  L.slots = (int)codes_slots(channels, group);
  return NB200_OK;
}
} // namespace

extern "C" int nb200_bn_add_relu_fxp_codes_nhwc(const float *a, const float *beta_a, const float *gamma_a,
                                                const float *mean_a, const float *var_a, const float *b,
                                                const float *beta_b, const float *gamma_b, const float *mean_b,
                                                const float *var_b, const int8_t *b_codes, float b_delta,
                                                int8_t *y_codes, int64_t batch, int64_t channels, int64_t inner,
                                                int group, float eps, int relu, int sign, int n, float delta,
                                                void *stream) {
  CodesLayout L;
  NB_TRY(codes_layout(L, batch, channels, inner, group));
  FxpParams P{0.f, 0.f, 1.f, 1.f, 0};
  NB_TRY(fill_fxp(P, sign, n, delta));
  const int nn = sign ? n - 1 : n;
  NB_CHECK(nn <= 7, NB200_ENOTIMPL, "codes need n - sign <= 7 (they are stored as int8)");
  const int kmax = (1 << nn) - 1, kmin = sign ? -kmax : 0;
  if (batch == 0)
    return NB200_OK;
  NB_CHECK(a && y_codes && mean_a && var_a, NB200_EVALUE, "null data pointer");
  NB_CHECK(!(b && b_codes), NB200_EVALUE, "the second operand is either fp32 or codes, not both");
  NB_CHECK(mean_b == nullptr || (b != nullptr && var_b != nullptr), NB200_EVALUE,
           "statistics of the second operand without the operand");
  NB_CHECK(b_codes == nullptr || b_delta > 0.f, NB200_EVALUE, "b_delta should be positive");
  NB_CHECK(((reinterpret_cast<uintptr_t>(y_codes) | reinterpret_cast<uintptr_t>(b_codes)) & 3) == 0, NB200_EVALUE,
           "code tensors must be 4-byte aligned");
  const BnTerm A{a, beta_a, gamma_a, mean_a, var_a};
  const BnTerm B{b, beta_b, gamma_b, mean_b, var_b};
  const bool vec = (inner % 4 == 0) && ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b)) & 15) == 0;
  const dim3 grid((L.HW + kTilePx - 1) / kTilePx, (L.slots + kTileSlots - 1) / kTileSlots, (unsigned)batch);
  cudaStream_t st = as_stream(stream);
  const int second = b_codes ? 3 : (b == nullptr ? 0 : (mean_b == nullptr ? 1 : 2));
#define NB_LAUNCH_CODES(V, S)                                                                                          \
  bn_add_relu_fxp_codes_kernel<V, S><<<grid, 256, 0, st>>>(A, B, b_codes, b_delta, L, eps, relu, P, kmax, kmin, y_codes)
#define NB_LAUNCH_CODES_FAST(S)                                                                                        \
  bn_add_relu_fxp_codes_kernel<true, S, true><<<grid, 256, 0, st>>>(A, B, b_codes, b_delta, L, eps, relu, P, kmax,     \
                                                                    kmin, y_codes)
  const bool fast = vec && relu && P.pow2 && group == 1 && L.slots == L.C && kmin <= 0;
  if (fast) {
    switch (second) {
    case 0: NB_LAUNCH_CODES_FAST(0); break;
    case 1: NB_LAUNCH_CODES_FAST(1); break;
    case 2: NB_LAUNCH_CODES_FAST(2); break;
    default: NB_LAUNCH_CODES_FAST(3); break;
    }
  } else
  switch (second * 2 + (vec ? 1 : 0)) {
  case 0: NB_LAUNCH_CODES(false, 0); break;
  case 1: NB_LAUNCH_CODES(true, 0); break;
  case 2: NB_LAUNCH_CODES(false, 1); break;
  case 3: NB_LAUNCH_CODES(true, 1); break;
  case 4: NB_LAUNCH_CODES(false, 2); break;
  case 5: NB_LAUNCH_CODES(true, 2); break;
  case 6: NB_LAUNCH_CODES(false, 3); break;
  default: NB_LAUNCH_CODES(true, 3); break;
  }
#undef NB_LAUNCH_CODES
#undef NB_LAUNCH_CODES_FAST
  NB_LAUNCH_CHECK();
  return NB200_OK;
}

extern "C" int nb200_codes_nhwc_to_f32(const int8_t *codes, float *y, int64_t batch, int64_t channels, int64_t inner,
                                       int group, float delta, void *stream) {
  CodesLayout L;
  NB_TRY(codes_layout(L, batch, channels, inner, group));
  NB_CHECK(delta > 0.f, NB200_EVALUE, "delta should be positive");
  if (batch == 0)
    return NB200_OK;
  NB_CHECK(codes && y, NB200_EVALUE, "null data pointer");
  NB_CHECK((reinterpret_cast<uintptr_t>(codes) & 3) == 0, NB200_EVALUE, "code tensors must be 4-byte aligned");
  const dim3 grid((L.HW + kTilePx - 1) / kTilePx, (L.slots + kTileSlots - 1) / kTileSlots, (unsigned)batch);
  codes_nhwc_to_f32_kernel<<<grid, 256, 0, as_stream(stream)>>>(codes, L, delta, y);
  NB_LAUNCH_CHECK();
  return NB200_OK;
}

extern "C" int nb200_max_pooling_codes_nhwc(const int8_t *codes, int8_t *y_codes, int64_t batch, int64_t channels,
                                            int height, int width, int group, int kernel_h, int kernel_w,
                                            int stride_h, int stride_w, int pad_h, int pad_w, int ignore_border,
                                            void *stream) {
  NB_CHECK(batch >= 0 && channels > 0 && group > 0 && channels % group == 0 && height > 0 && width > 0 &&
               kernel_h > 0 && kernel_w > 0 && stride_h > 0 && stride_w > 0 && pad_h >= 0 && pad_w >= 0,
           NB200_EVALUE, "bad pooling geometry");
  // a window must hold at least one input value (the reference would read outside the input otherwise)
  NB_CHECK(pad_h < kernel_h && pad_w < kernel_w, NB200_EVALUE, "padding must be smaller than the window");
  PoolGeom G;
  G.H = height, G.W = width, G.kh = kernel_h, G.kw = kernel_w, G.sh = stride_h, G.sw = stride_w, G.ph = pad_h,
  G.pw = pad_w;
  // Output extent: src/nbla/function/utils/base_pooling.cpp:59.
  G.Ho = (height + pad_h - (ignore_border ? kernel_h - pad_h : 1)) / stride_h + 1;
  G.Wo = (width + pad_w - (ignore_border ? kernel_w - pad_w : 1)) / stride_w + 1;
  NB_CHECK(G.Ho > 0 && G.Wo > 0, NB200_EVALUE, "pooling output would be empty");
  if (batch == 0)
    return NB200_OK;
  NB_CHECK(codes && y_codes, NB200_EVALUE, "null data pointer");
  NB_CHECK(((reinterpret_cast<uintptr_t>(codes) | reinterpret_cast<uintptr_t>(y_codes)) & 15) == 0, NB200_EVALUE,
           "code tensors must be 16-byte aligned");
  const int slots = (int)codes_slots(channels, group);
  NB_CHECK(batch <= 65535 && G.Ho <= 65535, NB200_ENOTIMPL, "more than 65535 samples or output rows");
  const dim3 grid((unsigned)((G.Wo * (slots / 16) + 255) / 256), (unsigned)G.Ho, (unsigned)batch);
  max_pooling_codes_kernel<<<grid, 256, 0, as_stream(stream)>>>(codes, slots, G, y_codes);
  NB_LAUNCH_CHECK();
  return NB200_OK;
}
