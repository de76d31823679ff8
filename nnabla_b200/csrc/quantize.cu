// Elementwise quantizers for sm_100a: FixedPointQuantize, Pow2Quantize and
// MinMaxQuantize forward. All three are HBM-bound (4 B read + 4 B written per
// element): 128-bit coalesced streaming accesses, grid-stride loops with four
// independent loads in flight per thread, grid sized in multiples of the SM
// count. Arithmetic is arranged to be bit-identical to the reference's scalar
// CPU loops; each kernel names the loop it replaces.
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>

#include "common.cuh"
#include "pdl.cuh"

namespace nb200 {
namespace {

constexpr int kThreads = 256;
constexpr int kBlocksPerSm = 128; // measured: 8 -> 87 %, 32 -> 94 %, 128 -> 99 % of the copy bandwidth at 2^30 elements
constexpr int kUnroll = 4;

// ---------------------------------------------------------------------------
// Generic vectorised elementwise driver. Op provides
//   float operator()(float x, size_t i, float &k) const   (i = flat element index,
//   k = integer code for ops with an int8 side-band).
// The body handles n4 float4 groups starting at element `head`; the first
// `head` and the last `tail` elements are done by the first threads of block 0.
// ---------------------------------------------------------------------------
// Applies op to one float4 group starting at flat element e and stores it;
// ops with an int8 side-band store their four codes as one 32-bit word.
template <typename Op>
__device__ __forceinline__ void apply4(const Op &op, const typename Op::State &st, const float4 v, const size_t e,
                                       float4 *dst) {
  float4 r;
  float k0, k1, k2, k3;
  r.x = op(v.x, e, k0, st);
  r.y = op(v.y, e + 1, k1, st);
  r.z = op(v.z, e + 2, k2, st);
  r.w = op(v.w, e + 3, k3, st);
  st_stream(dst, r);
  if (Op::kHasCodes)
    op.store_codes4(e, k0, k1, k2, k3);
}

template <typename Op>
__global__ void __launch_bounds__(kThreads) ew_vec_kernel(const float *__restrict__ x, float *__restrict__ y,
                                                          size_t size, size_t head, size_t n4, Op op) {
  pdl_wait();
  pdl_trigger();
  const float4 *x4 = reinterpret_cast<const float4 *>(x + head);
  float4 *y4 = reinterpret_cast<float4 *>(y + head);
  const size_t stride = (size_t)gridDim.x * kThreads;
  size_t i = (size_t)blockIdx.x * kThreads + threadIdx.x;
  const typename Op::State st = op.init(); // per-thread constants, loaded once
  for (; i + (kUnroll - 1) * stride < n4; i += kUnroll * stride) {
    float4 v[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u)
      v[u] = ld_stream(x4 + i + u * stride);
#pragma unroll
    for (int u = 0; u < kUnroll; ++u)
      apply4(op, st, v[u], head + 4 * (i + u * stride), y4 + i + u * stride);
  }
  for (; i < n4; i += stride)
    apply4(op, st, ld_stream(x4 + i), head + 4 * i, y4 + i);
  if (blockIdx.x == 0) {
    const size_t tail_begin = head + 4 * n4;
    const size_t n_edge = head + (size - tail_begin);
    for (size_t t = threadIdx.x; t < n_edge; t += kThreads) {
      const size_t e = (t < head) ? t : tail_begin + (t - head);
      float k;
      y[e] = op(x[e], e, k, st);
      if (Op::kHasCodes)
        op.store_code(e, k);
    }
  }
}

// Fallback for x and y with different 16-byte phases: scalar, still coalesced.
template <typename Op>
__global__ void __launch_bounds__(kThreads) ew_scalar_kernel(const float *__restrict__ x, float *__restrict__ y,
                                                             size_t size, Op op) {
  pdl_wait();
  pdl_trigger();
  const size_t stride = (size_t)gridDim.x * kThreads;
  const typename Op::State st = op.init();
  for (size_t i = (size_t)blockIdx.x * kThreads + threadIdx.x; i < size; i += stride) {
    float k;
    y[i] = op(x[i], i, k, st);
    if (Op::kHasCodes)
      op.store_code(i, k);
  }
}

inline unsigned grid_for(size_t work_items) {
  size_t blocks = (work_items + kThreads - 1) / kThreads;
  // NNABLA_B200_EW_BLOCKS_PER_SM overrides the grid size per SM (tuning aid).
  static const int per_sm = []() {
    const char *e = std::getenv("NNABLA_B200_EW_BLOCKS_PER_SM");
    const int v = e ? std::atoi(e) : 0;
    return v > 0 ? v : kBlocksPerSm;
  }();
  const size_t cap = (size_t)sm_count() * per_sm;
  if (blocks > cap)
    blocks = cap;
  if (blocks == 0)
    blocks = 1;
  return (unsigned)blocks;
}

template <typename Op> int launch_elementwise(const float *x, float *y, size_t size, Op op, cudaStream_t st) {
  if (size == 0)
    return NB200_OK;
  NB_CHECK(x != nullptr && y != nullptr, NB200_EVALUE, "null data pointer");
  NB_CHECK((reinterpret_cast<uintptr_t>(x) & 3) == 0 && (reinterpret_cast<uintptr_t>(y) & 3) == 0, NB200_EVALUE,
           "fp32 pointers must be 4-byte aligned");
  const size_t phase_x = (reinterpret_cast<uintptr_t>(x) & 15) / 4;
  const size_t phase_y = (reinterpret_cast<uintptr_t>(y) & 15) / 4;
  size_t head = (4 - phase_x) & 3;
  if (head > size)
    head = size;
  if (phase_x != phase_y || !op.codes_aligned(head)) {
    NB_CUDA(launch_dependent(ew_scalar_kernel<Op>, dim3(grid_for(size)), dim3(kThreads), 0, st, x, y, size, op));
    return NB200_OK;
  }
  const size_t n4 = (size - head) / 4;
  NB_CUDA(launch_dependent(ew_vec_kernel<Op>, dim3(grid_for((n4 + kUnroll - 1) / kUnroll)), dim3(kThreads), 0, st, x, y,
                           size, head, n4, op));
  return NB200_OK;
}

// ---------------------------------------------------------------------------
// FixedPointQuantize — replaces the loop of
// src/nbla/function/generic/fixed_point_quantize.cpp:53-65.
// The reference rounds with int(double(|x|/delta) + 0.5): the quotient is a
// single fp32 division, the +0.5 is exact in double, the conversion truncates.
// That equals floor(q) + (q - floor(q) >= 0.5) with q - floor(q) exact in
// fp32. When delta is a power of two the division is an exact scaling and is
// done as a multiplication.
// ---------------------------------------------------------------------------
template <bool kPow2Delta, bool kCodes> struct FxpOp {
  static constexpr bool kHasCodes = kCodes;
  float maxv, minv, delta, inv_delta;
  float code_max, code_min; // integer codes of the clip values
  int8_t *codes;
  bool codes_aligned(size_t head) const { return !kCodes || ((reinterpret_cast<uintptr_t>(codes) + head) & 3) == 0; }
  __device__ __forceinline__ void store_code(size_t i, float k) const { codes[i] = (int8_t)(int)k; }
  __device__ __forceinline__ void store_codes4(size_t e, float k0, float k1, float k2, float k3) const {
    const uint32_t w = ((uint32_t)(int)k0 & 0xffu) | (((uint32_t)(int)k1 & 0xffu) << 8) |
                       (((uint32_t)(int)k2 & 0xffu) << 16) | (((uint32_t)(int)k3 & 0xffu) << 24);
    *reinterpret_cast<uint32_t *>(codes + e) = w;
  }
  struct State {};
  __device__ __forceinline__ State init() const { return State(); }
  __device__ __forceinline__ float operator()(float x, size_t, float &k, const State &) const {
    float r;
    if (x > maxv) {
      r = maxv;
      k = code_max;
    } else if (x < minv) {
      r = minv;
      k = code_min;
    } else {
      const float a = fabsf(x);
      const float q = kPow2Delta ? __fmul_rn(a, inv_delta) : __fdiv_rn(a, delta);
      const float t = floorf(q);
      k = t + ((__fsub_rn(q, t) >= 0.5f) ? 1.0f : 0.0f);
      r = __fmul_rn(k, delta);
      if (x < 0.0f) {
        r = -r;
        k = -k;
      }
    }
    return r;
  }
};

struct FxpLimits {
  float maxv, minv, code_max, code_min;
  bool pow2;
  float inv;
};

int fxp_limits(int sign, int n, float delta, FxpLimits *L) {
  // The reference's setup checks (fixed_point_quantize.cpp:31-42).
  NB_CHECK(n > 0 && delta > 0.f, NB200_EVALUE, "Both bit width and delta should be positive.");
  const int nn = sign ? n - 1 : n;
  NB_CHECK(nn > 0, NB200_EVALUE, "bit width should be positive when considering sign (1bit).");
  L->maxv = (float)((std::pow(2, nn) - 1) * delta); // double product narrowed, as the reference
  L->minv = sign ? -L->maxv : 0.0f;
  L->code_max = (float)(std::pow(2, nn) - 1);
  L->code_min = sign ? -L->code_max : 0.0f;
  int ex = 0;
  const float mant = std::frexp(delta, &ex);
  // A power of two whose reciprocal is a normal float.
  L->pow2 = (mant == 0.5f) && ex > -120 && ex < 120;
  L->inv = L->pow2 ? 1.0f / delta : 0.0f;
  return NB200_OK;
}

template <bool kCodes>
int fxp_launch(const float *x, float *y, int8_t *codes, size_t size, int sign, int n, float delta, cudaStream_t st) {
  FxpLimits L;
  NB_TRY(fxp_limits(sign, n, delta, &L));
  if (kCodes) {
    NB_CHECK((sign ? n - 1 : n) <= 7, NB200_EVALUE, "int8 codes need n - sign <= 7 (got n=%d, sign=%d)", n, sign);
    NB_CHECK(codes != nullptr || size == 0, NB200_EVALUE, "codes is NULL");
  }
  if (L.pow2) {
    FxpOp<true, kCodes> op{L.maxv, L.minv, delta, L.inv, L.code_max, L.code_min, codes};
    return launch_elementwise(x, y, size, op, st);
  }
  FxpOp<false, kCodes> op{L.maxv, L.minv, delta, L.inv, L.code_max, L.code_min, codes};
  return launch_elementwise(x, y, size, op, st);
}

// FixedPointQuantize of an [N, C, S] tensor that also leaves the result as int8 channel-last codes
// [N][S][slots] (the layout the int8 convolutions read): the quantizer of a layer and the re-layout pass of
// the convolution behind it in one pass over the activations (4 B read, 4 + 1 B written per value instead of
// 4 + 4 and then 4 + 1). Blocks of 64 pixels x 64 channel slots; a thread quantizes four neighbouring
// channels of four pixels, stores the fp32 results where they came from and hands the four codes of each
// pixel to shared memory as one word; the codes leave as 64-byte runs per pixel. S % 4 == 0, 16-byte aligned.
template <bool kPow2Delta>
__global__ void __launch_bounds__(256)
    fxp_nhwc_codes_kernel(const float *__restrict__ x, float *__restrict__ y, int8_t *__restrict__ codes, int C, int HW,
                          int slots, FxpOp<kPow2Delta, false> op) {
  pdl_wait();
  pdl_trigger();
  __shared__ uint32_t tile[64][17];
  const int n = blockIdx.z;
  const int p0 = blockIdx.x * 64, d0 = blockIdx.y * 64;
  const int px4 = threadIdx.x & 15, chq = threadIdx.x >> 4;
  const int p = p0 + 4 * px4;
  const int c0 = d0 + 4 * chq;
  const typename FxpOp<kPow2Delta, false>::State st = op.init();
  uint32_t f[4][4];
#pragma unroll
  for (int r = 0; r < 4; ++r) {
    float k0 = 0.f, k1 = 0.f, k2 = 0.f, k3 = 0.f;
    if (c0 + r < C && p < HW) {
      const size_t off = ((size_t)n * C + (c0 + r)) * HW + p;
      const float4 v = ld_stream(reinterpret_cast<const float4 *>(x + off));
      float4 q;
      q.x = op(v.x, 0, k0, st);
      q.y = op(v.y, 0, k1, st);
      q.z = op(v.z, 0, k2, st);
      q.w = op(v.w, 0, k3, st);
      st_stream(reinterpret_cast<float4 *>(y + off), q);
    }
    // the codes are small integers: 1.5 * 2^23 + k has k's two's complement in its low mantissa bits
    f[r][0] = __float_as_uint(__fadd_rn(k0, 12582912.0f));
    f[r][1] = __float_as_uint(__fadd_rn(k1, 12582912.0f));
    f[r][2] = __float_as_uint(__fadd_rn(k2, 12582912.0f));
    f[r][3] = __float_as_uint(__fadd_rn(k3, 12582912.0f));
  }
#pragma unroll
  for (int k = 0; k < 4; ++k)
    tile[4 * px4 + k][chq] = __byte_perm(__byte_perm(f[0][k], f[1][k], 0x0040), __byte_perm(f[2][k], f[3][k], 0x0040),
                                         0x5410);
  __syncthreads();
  const int word = threadIdx.x & 15, prow = threadIdx.x >> 4;
#pragma unroll
  for (int pp = prow; pp < 64; pp += 16) {
    const int pix = p0 + pp, d = d0 + 4 * word;
    if (pix < HW && d < slots)
      *reinterpret_cast<uint32_t *>(codes + ((size_t)n * HW + pix) * slots + d) = tile[pp][word];
  }
}

int fxp_nhwc_codes(const float *x, float *y, int8_t *codes, int64_t batch, int64_t channels, int64_t inner, int slots,
                   int sign, int n, float delta, cudaStream_t st) {
  FxpLimits L;
  NB_TRY(fxp_limits(sign, n, delta, &L));
  NB_CHECK((sign ? n - 1 : n) <= 7, NB200_EVALUE, "int8 codes need n - sign <= 7 (got n=%d, sign=%d)", n, sign);
  NB_CHECK(batch >= 0 && channels > 0 && inner > 0 && batch <= 65535 && channels < (1 << 30) && inner < (1 << 30),
           NB200_EVALUE, "bad extents");
  if (batch == 0)
    return NB200_OK;
  NB_CHECK(x && y && codes, NB200_EVALUE, "null data pointer");
  NB_CHECK(inner % 4 == 0 && ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y)) & 15) == 0 &&
               (reinterpret_cast<uintptr_t>(codes) & 3) == 0,
           NB200_ENOTIMPL, "the quantizer with channel-last codes needs planes of a multiple of 4 values and aligned tensors");
  NB_CHECK(slots >= channels && slots % 16 == 0, NB200_EVALUE, "bad slot count");
  const dim3 grid((unsigned)((inner + 63) / 64), (unsigned)((slots + 63) / 64), (unsigned)batch);
  if (L.pow2) {
    FxpOp<true, false> op{L.maxv, L.minv, delta, L.inv, L.code_max, L.code_min, nullptr};
    NB_CUDA(launch_dependent(fxp_nhwc_codes_kernel<true>, grid, dim3(256), 0, st, x, y, codes, (int)channels, (int)inner,
                             slots, op));
  } else {
    FxpOp<false, false> op{L.maxv, L.minv, delta, L.inv, L.code_max, L.code_min, nullptr};
    NB_CUDA(launch_dependent(fxp_nhwc_codes_kernel<false>, grid, dim3(256), 0, st, x, y, codes, (int)channels, (int)inner,
                             slots, op));
  }
  NB_LAUNCH_CHECK();
  return NB200_OK;
}

// ---------------------------------------------------------------------------
// Pow2Quantize — replaces the loop of
// src/nbla/function/generic/pow2_quantize.cpp:57-81.
//
// q = powf(2, roundf(log2f(a))) takes, within one binade [2^e, 2^(e+1)), the
// value 2^e up to some mantissa and 2^(e+1) above it. Where that step sits
// depends on the host libm's log2f rounding (it is not the exact sqrt(2) cut
// for most exponents), so the table is derived on the host with the same libm
// the reference would call: for each binade e = -149..127 (denormal binades
// included) cut[e] = the largest 23-bit left-aligned mantissa fraction for
// which the expression still gives 2^e, and pw[k] = powf(2, k) for
// k = -149..128. The kernel then needs integer compares only.
// ---------------------------------------------------------------------------
constexpr int kMinExp = -149;
constexpr int kNumBinades = 127 - kMinExp + 1; // 277
constexpr int kNumPow = kNumBinades + 1;       // k up to 128

struct Pow2Tables {
  uint32_t cut[kNumBinades];
  float pw[kNumPow];
};

// Value of mantissa fraction f (p significant bits, 0 <= f < 2^p) in binade e.
inline float binade_value(int e, int p, uint32_t f) {
  uint32_t bits;
  if (e >= -126)
    bits = ((uint32_t)(e + 127) << 23) | f; // p == 23
  else
    bits = (1u << p) | f; // denormal: leading bit at position p = e + 149
  float v;
  std::memcpy(&v, &bits, 4);
  return v;
}

inline float host_snap_exponent(float a) { return roundf(log2f(a)); }

// Builds the tables; returns false (with a reason) when the host libm does not
// behave as a single monotone step per binade, in which case the kernel
// cannot reproduce it and the entry point refuses to run.
bool build_pow2_tables(Pow2Tables *T, char *why, size_t why_len) {
  for (int k = kMinExp; k <= 128; ++k)
    T->pw[k - kMinExp] = powf(2.0f, (float)k);
  for (int e = kMinExp; e <= 127; ++e) {
    const int p = (e >= -126) ? 23 : e + 149;
    const uint32_t fmax = (p == 0) ? 0u : ((1u << p) - 1u);
    if (host_snap_exponent(binade_value(e, p, 0)) != (float)e) {
      snprintf(why, why_len, "libm: roundf(log2f(2^%d)) != %d", e, e);
      return false;
    }
    uint32_t lo = 0, hi = fmax;
    if (host_snap_exponent(binade_value(e, p, fmax)) == (float)e) {
      lo = fmax; // no step inside this binade
    } else {
      if (host_snap_exponent(binade_value(e, p, fmax)) != (float)(e + 1)) {
        snprintf(why, why_len, "libm: unexpected snap at the top of binade %d", e);
        return false;
      }
      while (hi - lo > 1) {
        const uint32_t mid = lo + (hi - lo) / 2;
        if (host_snap_exponent(binade_value(e, p, mid)) == (float)e)
          lo = mid;
        else
          hi = mid;
      }
      // Monotonicity around the cut.
      for (int d = -64; d <= 64; ++d) {
        const int64_t f = (int64_t)lo + d;
        if (f < 0 || f > (int64_t)fmax)
          continue;
        const float want = (f <= (int64_t)lo) ? (float)e : (float)(e + 1);
        if (host_snap_exponent(binade_value(e, p, (uint32_t)f)) != want) {
          snprintf(why, why_len, "libm: log2f is not monotone around the cut of binade %d", e);
          return false;
        }
      }
    }
    T->cut[e - kMinExp] = lo << (23 - p); // left-align to 23 bits
  }
  return true;
}

struct Pow2Device {
  bool ready = false;
  Pow2Tables *tables = nullptr; // device copy
};
std::mutex g_pow2_mutex;
Pow2Device g_pow2_dev[64];
Pow2Tables g_pow2_host;
int g_pow2_host_state = 0; // 0 = not built, 1 = ok, -1 = unusable
char g_pow2_why[160];
// Facts about the tables that allow a lookup-free common case: every pw[k] is
// exactly 2^k (so it can be assembled from the exponent), and for normal
// binades every cut lies within g_pow2_margin of kCutCentre.
constexpr uint32_t kCutCentre = 0x3504f3u; // mantissa field of sqrt(2)
bool g_pow2_exact_powers = false;
uint32_t g_pow2_margin = 0;

void analyse_pow2_tables(const Pow2Tables &T) {
  g_pow2_exact_powers = true;
  for (int k = kMinExp; k <= 128; ++k) {
    const float want = (k == 128) ? INFINITY : ldexpf(1.0f, k);
    if (T.pw[k - kMinExp] != want)
      g_pow2_exact_powers = false;
  }
  uint32_t margin = 0;
  for (int e = -126; e <= 127; ++e) {
    const uint32_t c = T.cut[e - kMinExp];
    const uint32_t d = c > kCutCentre ? c - kCutCentre : kCutCentre - c;
    if (d > margin)
      margin = d;
  }
  g_pow2_margin = margin + 1;
}

int pow2_tables_for_current_device(const Pow2Tables **out) {
  int dev = 0;
  NB_CUDA(cudaGetDevice(&dev));
  NB_CHECK(dev >= 0 && dev < 64, NB200_EVALUE, "device index %d out of range", dev);
  std::lock_guard<std::mutex> lock(g_pow2_mutex);
  if (g_pow2_host_state == 0) {
    g_pow2_host_state = build_pow2_tables(&g_pow2_host, g_pow2_why, sizeof(g_pow2_why)) ? 1 : -1;
    if (g_pow2_host_state == 1)
      analyse_pow2_tables(g_pow2_host);
  }
  NB_CHECK(g_pow2_host_state == 1, NB200_ENOTIMPL, "Pow2Quantize: cannot reproduce the host libm (%s)", g_pow2_why);
  Pow2Device &d = g_pow2_dev[dev];
  if (!d.ready) {
    NB_CUDA(cudaMalloc(&d.tables, sizeof(Pow2Tables)));
    NB_CUDA(cudaMemcpy(d.tables, &g_pow2_host, sizeof(Pow2Tables), cudaMemcpyHostToDevice));
    d.ready = true;
  }
  *out = d.tables;
  return NB200_OK;
}

struct Pow2Params {
  float p_max, p_min, prune;
  int sign, with_zero;
};

__device__ __forceinline__ float pow2_snap(float x, const Pow2Params &P, const uint32_t *cut, const float *pw) {
  const float a = fabsf(x);
  const uint32_t bits = __float_as_uint(a);
  float q;
  if (bits == 0u) {
    q = 0.0f; // log2f(0) = -inf, powf(2, -inf) = 0
  } else if (bits >= 0x7f800000u) {
    q = a; // +inf stays +inf (clipped to p_max below); NaN propagates
  } else {
    const uint32_t E = bits >> 23;
    uint32_t frac = bits & 0x7fffffu;
    int e;
    if (E == 0u) {
      const int p = 31 - __clz(frac);
      e = p - 149;
      frac = (frac << (23 - p)) & 0x7fffffu;
    } else {
      e = (int)E - 127;
    }
    const int k = e + (frac > cut[e - kMinExp] ? 1 : 0);
    q = pw[k - kMinExp];
  }
  if (q > P.p_max) {
    q = P.p_max;
  } else if (q < P.p_min) {
    q = P.with_zero ? (a < P.prune ? 0.0f : P.p_min) : P.p_min;
  }
  const bool neg = x < 0.0f;
  if (P.sign)
    q = neg ? -q : q;
  else if (P.with_zero)
    q = neg ? 0.0f : q;
  else
    q = neg ? P.p_min : q;
  return q;
}

// The tables (2.2 KB) are staged in shared memory: the lookup index varies per
// lane, which constant memory would serialise.
__global__ void __launch_bounds__(kThreads) pow2_kernel(const float *__restrict__ x, float *__restrict__ y, size_t size,
                                                        size_t head, size_t n4, int vectorised, Pow2Params P,
                                                        const Pow2Tables *__restrict__ tables) {
  __shared__ uint32_t s_cut[kNumBinades];
  __shared__ float s_pw[kNumPow];
  for (int t = threadIdx.x; t < kNumBinades; t += kThreads)
    s_cut[t] = tables->cut[t];
  for (int t = threadIdx.x; t < kNumPow; t += kThreads)
    s_pw[t] = tables->pw[t];
  __syncthreads();
  const size_t stride = (size_t)gridDim.x * kThreads;
  size_t i = (size_t)blockIdx.x * kThreads + threadIdx.x;
  if (!vectorised) {
    for (; i < size; i += stride)
      y[i] = pow2_snap(x[i], P, s_cut, s_pw);
    return;
  }
  const float4 *x4 = reinterpret_cast<const float4 *>(x + head);
  float4 *y4 = reinterpret_cast<float4 *>(y + head);
  for (; i + (kUnroll - 1) * stride < n4; i += kUnroll * stride) {
    float4 v[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u)
      v[u] = ld_stream(x4 + i + u * stride);
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      float4 r;
      r.x = pow2_snap(v[u].x, P, s_cut, s_pw);
      r.y = pow2_snap(v[u].y, P, s_cut, s_pw);
      r.z = pow2_snap(v[u].z, P, s_cut, s_pw);
      r.w = pow2_snap(v[u].w, P, s_cut, s_pw);
      st_stream(y4 + i + u * stride, r);
    }
  }
  for (; i < n4; i += stride) {
    const float4 v = ld_stream(x4 + i);
    float4 r;
    r.x = pow2_snap(v.x, P, s_cut, s_pw);
    r.y = pow2_snap(v.y, P, s_cut, s_pw);
    r.z = pow2_snap(v.z, P, s_cut, s_pw);
    r.w = pow2_snap(v.w, P, s_cut, s_pw);
    st_stream(y4 + i, r);
  }
  if (blockIdx.x == 0) {
    const size_t tail_begin = head + 4 * n4;
    const size_t n_edge = head + (size - tail_begin);
    for (size_t t = threadIdx.x; t < n_edge; t += kThreads) {
      const size_t e = (t < head) ? t : tail_begin + (t - head);
      y[e] = pow2_snap(x[e], P, s_cut, s_pw);
    }
  }
}

// Lookup-free common case (used when the host libm's powers of two are exact
// and its cuts sit close to sqrt(2), which analyse_pow2_tables verified): the
// snapped exponent of a normal number is decided by comparing its mantissa
// with kCutCentre -/+ margin, the power of two is assembled from the exponent
// bits, and only mantissas inside the +-margin window (a few in 10^5) or
// denormal inputs read the per-binade table from global memory.
struct Pow2FastOp {
  static constexpr bool kHasCodes = false;
  Pow2Params P;
  uint32_t margin;
  const Pow2Tables *tables;
  bool codes_aligned(size_t) const { return true; }
  __device__ __forceinline__ void store_code(size_t, float) const {}
  __device__ __forceinline__ void store_codes4(size_t, float, float, float, float) const {}
  struct State {};
  __device__ __forceinline__ State init() const { return State(); }
  __device__ __forceinline__ float operator()(float x, size_t, float &, const State &) const {
    const float a = fabsf(x);
    const uint32_t bits = __float_as_uint(a);
    const uint32_t E = bits >> 23;
    float q;
    if (E - 1u < 254u) { // normal number
      const uint32_t frac = bits & 0x7fffffu;
      int k = (int)E - 127;
      if (frac >= kCutCentre + margin) {
        k += 1;
      } else if (frac + margin > kCutCentre) {
        k += (frac > __ldg(&tables->cut[k - kMinExp])) ? 1 : 0;
      }
      // 2^k for k in [-126, 128]; k = 128 assembles +inf like powf(2, 128); k = -126 - 1 cannot occur here
      q = __uint_as_float((uint32_t)(k + 127) << 23);
    } else if (bits == 0u) {
      q = 0.0f;
    } else if (E == 255u) {
      q = a;
    } else { // denormal input
      const int p = 31 - __clz(bits);
      const int e = p - 149;
      const uint32_t frac = (bits << (23 - p)) & 0x7fffffu;
      const int k = e + ((frac > __ldg(&tables->cut[e - kMinExp])) ? 1 : 0);
      q = __ldg(&tables->pw[k - kMinExp]);
    }
    if (q > P.p_max) {
      q = P.p_max;
    } else if (q < P.p_min) {
      q = P.with_zero ? (a < P.prune ? 0.0f : P.p_min) : P.p_min;
    }
    const bool neg = x < 0.0f;
    if (P.sign)
      q = neg ? -q : q;
    else if (P.with_zero)
      q = neg ? 0.0f : q;
    else
      q = neg ? P.p_min : q;
    return q;
  }
};

int pow2_params(int sign, int with_zero, int n, int m, Pow2Params *P) {
  // The reference's setup (pow2_quantize.cpp:31-44).
  NB_CHECK(n > 0, NB200_EVALUE, "bit width should be positive.");
  int nn = sign ? n - 1 : n;
  nn = with_zero ? nn - 1 : nn;
  NB_CHECK(nn > 0, NB200_EVALUE, "bit width should be positive when considering zero (1bit) and sign (1bit).");
  NB_CHECK(nn < 31, NB200_EVALUE, "bit width too large (1 << %d overflows int in the reference)", nn);
  P->p_max = (float)std::pow(2., m);
  P->p_min = (float)std::pow(2., m - ((1 << nn) - 1));
  P->prune = (float)((double)P->p_min * std::pow(2., -0.5));
  P->sign = sign ? 1 : 0;
  P->with_zero = with_zero ? 1 : 0;
  return NB200_OK;
}

int pow2_launch(const float *x, float *y, size_t size, int sign, int with_zero, int n, int m, cudaStream_t st) {
  Pow2Params P;
  NB_TRY(pow2_params(sign, with_zero, n, m, &P));
  if (size == 0)
    return NB200_OK;
  NB_CHECK(x != nullptr && y != nullptr, NB200_EVALUE, "null data pointer");
  NB_CHECK((reinterpret_cast<uintptr_t>(x) & 3) == 0 && (reinterpret_cast<uintptr_t>(y) & 3) == 0, NB200_EVALUE,
           "fp32 pointers must be 4-byte aligned");
  const Pow2Tables *tables = nullptr;
  NB_TRY(pow2_tables_for_current_device(&tables));
  if (g_pow2_exact_powers && g_pow2_margin < 4096u) {
    Pow2FastOp op{P, g_pow2_margin, tables};
    return launch_elementwise(x, y, size, op, st);
  }
  const size_t phase_x = (reinterpret_cast<uintptr_t>(x) & 15) / 4;
  const size_t phase_y = (reinterpret_cast<uintptr_t>(y) & 15) / 4;
  if (phase_x != phase_y) {
    pow2_kernel<<<grid_for(size), kThreads, 0, st>>>(x, y, size, 0, 0, 0, P, tables);
  } else {
    size_t head = (4 - phase_x) & 3;
    if (head > size)
      head = size;
    const size_t n4 = (size - head) / 4;
    pow2_kernel<<<grid_for((n4 + kUnroll - 1) / kUnroll), kThreads, 0, st>>>(x, y, size, head, n4, 1, P, tables);
  }
  NB_LAUNCH_CHECK();
  return NB200_OK;
}

// ---------------------------------------------------------------------------
// MinMaxQuantize — replaces src/nbla/function/generic/min_max_quantize.cpp
// :129-223. The reference runs ~14 sub-functions, 11 of them full passes over
// x; here one optional reduction pass, one tiny parameter kernel and one
// apply pass. The q tensors broadcast over x; the supported (and fast) case
// is a q shape whose non-1 extents form one contiguous run of axes, so that
// x is viewed as [outer, Q, inner] and the q index of flat element i is
// (i / inner) % Q. Scratch per call: 7*Q words (min and max keys, m, M, scale).
// ---------------------------------------------------------------------------
struct MinMaxView {
  size_t outer, Q, inner, size;
};
constexpr size_t kMinMaxScratchWords = 7; // per range: two 64-bit keys (min, max), m, M, scale

// Min / Max of the reference (src/nbla/function/generic/max.cpp:44-61, min.cpp): a serial scan that
// starts from -1e8 (Max) / +1e8 (Min) and replaces the running value only on a strict comparison,
// so among equal values the FIRST one in scan order wins. That matters for zeros: -0.0 == +0.0
// compares equal, the first one's sign ends up in qr_min / qr_max (which are written back), and a
// NaN never wins. Each candidate is packed into a 64-bit key whose unsigned order is that rule:
//   high word: the value as an order-preserving integer, both zeros mapped to the same code
//              (complemented for Min, so that one atomicMax serves both);
//   low word:  (2^31 - 1 - t) << 1 | sign bit, t = position in the reference's scan order: for
//              equal values the earlier one has the larger key, and the zero's sign survives.
// The starting value has the largest low word: an element equal to it never replaces it.
__device__ __forceinline__ uint32_t ordered_bits(float v) {
  const uint32_t u = (v == 0.0f) ? 0u : __float_as_uint(v);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ unsigned long long extremum_key(float v, uint32_t t, bool is_min) {
  const uint32_t hi = is_min ? ~ordered_bits(v) : ordered_bits(v);
  const uint32_t lo = ((0x7fffffffu - t) << 1) | (__float_as_uint(v) >> 31);
  return ((unsigned long long)hi << 32) | lo;
}
__device__ __forceinline__ unsigned long long extremum_start(bool is_min) {
  const float v = is_min ? 1e8f : -1e8f;
  const uint32_t hi = is_min ? ~ordered_bits(v) : ordered_bits(v);
  return ((unsigned long long)hi << 32) | 0xfffffffeu | (__float_as_uint(v) >> 31);
}
__device__ __forceinline__ float extremum_value(unsigned long long key, bool is_min) {
  uint32_t o = (uint32_t)(key >> 32);
  if (is_min)
    o = ~o;
  const uint32_t u = (o & 0x80000000u) ? (o & 0x7fffffffu) : ~o;
  return __uint_as_float(u == 0u ? ((uint32_t)key & 1u) << 31 : u);
}

__global__ void minmax_init_kernel(unsigned long long *mn, unsigned long long *mx, size_t Q) {
  const size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x;
  if (i < Q) {
    mn[i] = extremum_start(true);
    mx[i] = extremum_start(false);
  }
}

// grid = (splits, Q). Block (s, q) reduces its share of the outer*inner
// elements that belong to q, then one atomic pair per block. t = o * inner + j
// is the element's position in the reference's scan over the reduced axes.
__global__ void __launch_bounds__(kThreads) minmax_reduce_kernel(const float *__restrict__ x, MinMaxView V,
                                                                 unsigned long long *mn, unsigned long long *mx) {
  const size_t q = blockIdx.y;
  const size_t per_q = V.outer * V.inner;
  float lo = 1e8f, hi = -1e8f;
  uint32_t t_lo = 0xffffffffu, t_hi = 0xffffffffu; // position of the thread's extremum; none yet
  const size_t stride = (size_t)gridDim.x * kThreads;
  for (size_t t = (size_t)blockIdx.x * kThreads + threadIdx.x; t < per_q; t += stride) {
    const size_t o = t / V.inner, j = t - o * V.inner;
    const float v = x[(o * V.Q + q) * V.inner + j];
    if (v < lo)
      lo = v, t_lo = (uint32_t)t;
    if (v > hi)
      hi = v, t_hi = (uint32_t)t;
  }
  unsigned long long klo = t_lo == 0xffffffffu ? extremum_start(true) : extremum_key(lo, t_lo, true);
  unsigned long long khi = t_hi == 0xffffffffu ? extremum_start(false) : extremum_key(hi, t_hi, false);
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) {
    const unsigned long long lo2 = __shfl_xor_sync(0xffffffffu, klo, d), hi2 = __shfl_xor_sync(0xffffffffu, khi, d);
    klo = lo2 > klo ? lo2 : klo;
    khi = hi2 > khi ? hi2 : khi;
  }
  __shared__ unsigned long long s_lo[kThreads / 32], s_hi[kThreads / 32];
  if ((threadIdx.x & 31) == 0) {
    s_lo[threadIdx.x >> 5] = klo;
    s_hi[threadIdx.x >> 5] = khi;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < kThreads / 32; ++w) {
      klo = s_lo[w] > klo ? s_lo[w] : klo;
      khi = s_hi[w] > khi ? s_hi[w] : khi;
    }
    if (per_q > 0) {
      atomicMax(mn + q, klo);
      atomicMax(mx + q, khi);
    }
  }
}

// Parameter step, one thread per q: the moving average (:159-178), nudge_range
// (:352-361), the scale (:184-186) and nudge_qr_min_max (:362-390), with every
// fp32 operation rounded on its own.
__global__ void minmax_params_kernel(size_t Q, float *qr_min, float *qr_max, const float *ql_min, const float *ql_max,
                                     const unsigned long long *mn_key, const unsigned long long *mx_key,
                                     int x_min_max, int ema, float decay_f,
                                     float one_minus_decay_f, float eps, float *m_out, float *M_out, float *s_out,
                                     float *scale_user) {
  const size_t q = blockIdx.x * (size_t)blockDim.x + threadIdx.x;
  if (q >= Q)
    return;
  float rmin = qr_min[q], rmax = qr_max[q];
  if (x_min_max) {
    const float mn = extremum_value(mn_key[q], true), mx = extremum_value(mx_key[q], false);
    if (ema) {
      rmin = __fadd_rn(__fmul_rn(rmin, decay_f), __fmul_rn(mn, one_minus_decay_f));
      rmax = __fadd_rn(__fmul_rn(rmax, decay_f), __fmul_rn(mx, one_minus_decay_f));
    } else {
      rmin = mn;
      rmax = mx;
    }
    qr_min[q] = rmin;
  }
  if (__fsub_rn(rmax, rmin) < eps)
    rmax = __fadd_rn(rmin, eps);
  qr_max[q] = rmax;
  const float lmin = ql_min[q], lmax = ql_max[q];
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
  s_out[q] = s;
  if (scale_user)
    scale_user[q] = s;
}

__device__ __forceinline__ float minmax_apply_one(float x, float m, float M, float s) {
  float t = (x > m) ? x : m; // maximum2.hpp:41 (NaN takes m)
  t = (t < M) ? t : M;       // minimum2.hpp:41
  t = __fsub_rn(t, m);
  t = __fdiv_rn(t, s);
  t = roundf(t); // half away from zero, like std::round
  t = __fmul_rn(t, s);
  return __fadd_rn(t, m);
}

// Elementwise op over the [outer, Q, inner] view; parameters are read from the
// scratch written by minmax_params_kernel (L1/L2 resident).
struct MinMaxOp {
  static constexpr bool kHasCodes = false;
  const float *m, *M, *s;
  size_t Q, inner;
  bool codes_aligned(size_t) const { return true; }
  __device__ __forceinline__ void store_code(size_t, float) const {}
  __device__ __forceinline__ void store_codes4(size_t, float, float, float, float) const {}
  // Per-tensor ranges (Q == 1): the three parameters are read once per thread.
  struct State {
    float m, M, s;
  };
  __device__ __forceinline__ State init() const {
    State st;
    st.m = __ldg(m);
    st.M = __ldg(M);
    st.s = __ldg(s);
    return st;
  }
  __device__ __forceinline__ float operator()(float x, size_t i, float &, const State &st) const {
    if (Q == 1)
      return minmax_apply_one(x, st.m, st.M, st.s);
    size_t q;
    if ((i | inner | Q) >> 32) {
      q = (i / inner) % Q;
    } else {
      q = ((uint32_t)i / (uint32_t)inner) % (uint32_t)Q;
    }
    return minmax_apply_one(x, __ldg(m + q), __ldg(M + q), __ldg(s + q));
  }
};

int minmax_view(const int64_t *xs, const int64_t *qs, int ndim, MinMaxView *V) {
  NB_CHECK(ndim >= 1 && ndim <= 8, NB200_EVALUE, "ndim must be in 1..8 (got %d)", ndim);
  size_t size = 1, Q = 1;
  int first = -1, last = -1;
  for (int d = 0; d < ndim; ++d) {
    NB_CHECK(xs[d] >= 0 && qs[d] >= 1, NB200_EVALUE, "bad extent at axis %d", d);
    // min_max_quantize.cpp:69-83
    NB_CHECK(qs[d] == 1 || qs[d] == xs[d], NB200_EVALUE,
             "x.shape and ql_min.shape must be same except for i-th dimension where ql_min.shape[i] == 1.");
    size *= (size_t)xs[d];
    if (qs[d] != 1) {
      if (first < 0)
        first = d;
      last = d;
      Q *= (size_t)qs[d];
    }
  }
  size_t outer = 1, inner = 1;
  if (first >= 0) {
    for (int d = first; d <= last; ++d)
      NB_CHECK(qs[d] != 1 || xs[d] == 1, NB200_ENOTIMPL,
               "q shapes whose non-1 axes are separated by a broadcast axis are not supported");
    for (int d = 0; d < first; ++d)
      outer *= (size_t)xs[d];
    for (int d = last + 1; d < ndim; ++d)
      inner *= (size_t)xs[d];
  } else {
    inner = size;
  }
  V->outer = outer;
  V->Q = Q;
  V->inner = inner;
  V->size = size;
  return NB200_OK;
}

// Runs the three steps on device buffers. `scratch` (8-byte aligned) holds kMinMaxScratchWords
// 32-bit words per range: two 64-bit extremum keys, then m, M and the scale.
int minmax_run(const float *x, const MinMaxView &V, float *qr_min, float *qr_max, const float *ql_min,
               const float *ql_max, float decay, int x_min_max, int ema, float eps, float *y, float *scale,
               float *scratch, cudaStream_t st) {
  unsigned long long *mn = reinterpret_cast<unsigned long long *>(scratch), *mx = mn + V.Q;
  float *m = scratch + 4 * V.Q, *M = scratch + 5 * V.Q, *s = scratch + 6 * V.Q;
  const unsigned qblocks = (unsigned)((V.Q + 255) / 256);
  if (x_min_max) {
    NB_CHECK(V.size > 0, NB200_EVALUE, "min/max of an empty tensor");
    minmax_init_kernel<<<qblocks, 256, 0, st>>>(mn, mx, V.Q);
    NB_LAUNCH_CHECK();
    NB_CHECK(V.Q <= 65535, NB200_ENOTIMPL, "more than 65535 quantization ranges");
    const size_t per_q = V.outer * V.inner;
    // the reference scans with an int index (max.cpp:51); positions are kept in 31 bits here
    NB_CHECK(per_q < (1ull << 31), NB200_ENOTIMPL, "min/max over 2^31 or more elements per range");
    size_t splits = (per_q + (size_t)kThreads * 16 - 1) / ((size_t)kThreads * 16);
    const size_t cap = ((size_t)sm_count() * kBlocksPerSm + V.Q - 1) / V.Q;
    if (splits > cap)
      splits = cap;
    if (splits == 0)
      splits = 1;
    minmax_reduce_kernel<<<dim3((unsigned)splits, (unsigned)V.Q), kThreads, 0, st>>>(x, V, mn, mx);
    NB_LAUNCH_CHECK();
  }
  // (T)decay_ and (T)(1.0 - decay_) as in min_max_quantize.cpp:105-106.
  const float d1 = decay, d2 = (float)(1.0 - (double)decay);
  minmax_params_kernel<<<qblocks, 256, 0, st>>>(V.Q, qr_min, qr_max, ql_min, ql_max, mn, mx, x_min_max, ema, d1, d2,
                                                 eps, m, M, s, scale);
  NB_LAUNCH_CHECK();
  MinMaxOp op{m, M, s, V.Q, V.inner};
  return launch_elementwise(x, y, V.size, op, st);
}

// ---------------------------------------------------------------------------
// Allocation-free variant of MinMaxQuantize: the 7*Q words of scratch live in
// a fixed array in device global memory that belongs to the library image
// (every GPU that loads the library carries it until the process exits).
// Host code must not pass the array's name to a kernel: on the host that name
// is only a handle. The device address is looked up once per device with
// cudaGetSymbolAddress while that device is current, and the kernels receive
// that address.
// ---------------------------------------------------------------------------
constexpr size_t kNoAllocMaxRanges = 4096; // quantization ranges (elements of qr_min) per call
static __device__ __align__(256) float g_minmax_static_scratch[kMinMaxScratchWords * kNoAllocMaxRanges];

std::mutex g_static_scratch_mutex;
float *g_static_scratch_addr[64];

int static_scratch_for_current_device(float **out) {
  int dev = 0;
  NB_CUDA(cudaGetDevice(&dev));
  NB_CHECK(dev >= 0 && dev < 64, NB200_EVALUE, "device index %d out of range", dev);
  std::lock_guard<std::mutex> lock(g_static_scratch_mutex);
  if (g_static_scratch_addr[dev] == nullptr) {
    void *p = nullptr;
    NB_CUDA(cudaGetSymbolAddress(&p, g_minmax_static_scratch));
    NB_CHECK(p != nullptr, NB200_ECUDA, "cudaGetSymbolAddress returned a null address");
    g_static_scratch_addr[dev] = static_cast<float *>(p);
  }
  *out = g_static_scratch_addr[dev];
  return NB200_OK;
}

#include "quantize_backward.cuh"
#include "quantize_siblings.cuh"

// ---- chunk callbacks of the _host variants ---------------------------------
struct FxpHostArgs {
  int sign, n;
  float delta;
};
int fxp_chunk(const float *dx, float *dy, size_t count, size_t, cudaStream_t st, void *user) {
  const FxpHostArgs *a = static_cast<const FxpHostArgs *>(user);
  return fxp_launch<false>(dx, dy, nullptr, count, a->sign, a->n, a->delta, st);
}
struct Pow2HostArgs {
  int sign, with_zero, n, m;
};
int pow2_chunk(const float *dx, float *dy, size_t count, size_t, cudaStream_t st, void *user) {
  const Pow2HostArgs *a = static_cast<const Pow2HostArgs *>(user);
  return pow2_launch(dx, dy, count, a->sign, a->with_zero, a->n, a->m, st);
}
struct MinMaxHostArgs {
  const float *params; // device: m, M, s
};
int minmax_chunk(const float *dx, float *dy, size_t count, size_t, cudaStream_t st, void *user) {
  const MinMaxHostArgs *a = static_cast<const MinMaxHostArgs *>(user);
  MinMaxOp op{a->params, a->params + 1, a->params + 2, 1, count};
  return launch_elementwise(dx, dy, count, op, st);
}

} // namespace
} // namespace nb200

using namespace nb200;

extern "C" {

int nb200_fixed_point_quantize_f32(const float *x, float *y, size_t size, int sign, int n, float delta, void *stream) {
  return fxp_launch<false>(x, y, nullptr, size, sign, n, delta, as_stream(stream));
}

int nb200_fixed_point_quantize_f32_codes(const float *x, float *y, int8_t *codes, size_t size, int sign, int n,
                                         float delta, void *stream) {
  return fxp_launch<true>(x, y, codes, size, sign, n, delta, as_stream(stream));
}

int nb200_fixed_point_quantize_nhwc_codes_f32(const float *x, float *y, int8_t *codes, int64_t batch, int64_t channels,
                                              int64_t inner, int sign, int n, float delta, void *stream) {
  // slots of a one-group code tensor (nb200_codes_nhwc_slots): channels padded to 16, at least 64
  const int64_t padded = (channels + 15) / 16 * 16;
  const int64_t block = padded <= 64 ? 64 : 128;
  const int slots = (int)(padded < block ? block : padded);
  return fxp_nhwc_codes(x, y, codes, batch, channels, inner, slots, sign, n, delta, as_stream(stream));
}

int nb200_fixed_point_quantize_f32_host(const float *x, float *y, size_t size, int sign, int n, float delta) {
  FxpLimits L;
  NB_TRY(fxp_limits(sign, n, delta, &L));
  NB_CHECK(size == 0 || (x && y), NB200_EVALUE, "null data pointer");
  FxpHostArgs a{sign, n, delta};
  return host_pipeline(x, y, size, fxp_chunk, &a);
}

int nb200_pow2_quantize_f32(const float *x, float *y, size_t size, int sign, int with_zero, int n, int m,
                            void *stream) {
  return pow2_launch(x, y, size, sign, with_zero, n, m, as_stream(stream));
}

int nb200_pow2_quantize_f32_host(const float *x, float *y, size_t size, int sign, int with_zero, int n, int m) {
  Pow2Params P;
  NB_TRY(pow2_params(sign, with_zero, n, m, &P));
  NB_CHECK(size == 0 || (x && y), NB200_EVALUE, "null data pointer");
  Pow2HostArgs a{sign, with_zero, n, m};
  return host_pipeline(x, y, size, pow2_chunk, &a);
}

int nb200_min_max_quantize_f32(const float *x, const int64_t *x_shape, int ndim, float *qr_min, float *qr_max,
                               const float *ql_min, const float *ql_max, const int64_t *q_shape, float decay,
                               int x_min_max, int ema, float eps, float *y, float *scale, void *stream) {
  NB_CHECK(x_shape && q_shape, NB200_EVALUE, "null shape pointer");
  MinMaxView V;
  NB_TRY(minmax_view(x_shape, q_shape, ndim, &V));
  NB_CHECK(qr_min && qr_max && ql_min && ql_max, NB200_EVALUE, "null range pointer");
  NB_CHECK(V.size == 0 || (x && y), NB200_EVALUE, "null data pointer");
  cudaStream_t st = as_stream(stream);
  AsyncScratch scratch(st);
  NB_TRY(scratch.alloc(kMinMaxScratchWords * V.Q * sizeof(float)));
  return minmax_run(x, V, qr_min, qr_max, ql_min, ql_max, decay, x_min_max, ema, eps, y, scale,
                    static_cast<float *>(scratch.p), st);
}

int nb200_min_max_quantize_f32_noalloc(const float *x, const int64_t *x_shape, int ndim, float *qr_min,
                                       float *qr_max, const float *ql_min, const float *ql_max,
                                       const int64_t *q_shape, float decay, int x_min_max, int ema, float eps,
                                       float *y, float *scale, void *stream) {
  NB_CHECK(x_shape && q_shape, NB200_EVALUE, "null shape pointer");
  MinMaxView V;
  NB_TRY(minmax_view(x_shape, q_shape, ndim, &V));
  NB_CHECK(V.Q <= kNoAllocMaxRanges, NB200_EVALUE,
           "nb200_min_max_quantize_f32_noalloc handles at most %zu quantization ranges per call (got %zu); "
           "use nb200_min_max_quantize_f32 for more",
           kNoAllocMaxRanges, V.Q);
  NB_CHECK(qr_min && qr_max && ql_min && ql_max, NB200_EVALUE, "null range pointer");
  NB_CHECK(V.size == 0 || (x && y), NB200_EVALUE, "null data pointer");
  float *scratch = nullptr;
  NB_TRY(static_scratch_for_current_device(&scratch));
  // The min/max slots are re-initialised by minmax_run when they are used and
  // the parameter slots are fully overwritten, so nothing of the previous
  // call's contents is read.
  return minmax_run(x, V, qr_min, qr_max, ql_min, ql_max, decay, x_min_max, ema, eps, y, scale, scratch,
                    as_stream(stream));
}

int nb200_min_max_quantize_f32_host(const float *x, size_t size, float *qr_min, float *qr_max, const float *ql_min,
                                    const float *ql_max, float eps, float *y) {
  NB_CHECK(qr_min && qr_max && ql_min && ql_max, NB200_EVALUE, "null range pointer");
  NB_CHECK(size == 0 || (x && y), NB200_EVALUE, "null data pointer");
  // Ranges: 4 floats in, (qr_max, m, M, s) out, through a small device buffer.
  float *d = nullptr;
  NB_CUDA(cudaMalloc(&d, 16 * sizeof(float)));
  float h[4] = {*qr_min, *qr_max, *ql_min, *ql_max};
  int rc = NB200_OK;
  do {
    if (cudaMemcpy(d, h, sizeof(h), cudaMemcpyHostToDevice) != cudaSuccess) {
      rc = fail(NB200_ECUDA, "copy of the quantization range failed");
      break;
    }
    minmax_params_kernel<<<1, 32>>>(1, d, d + 1, d + 2, d + 3, nullptr, nullptr, 0, 0, 0.f, 0.f, eps, d + 8, d + 9,
                                    d + 10, nullptr);
    if (cudaMemcpy(h, d, 2 * sizeof(float), cudaMemcpyDeviceToHost) != cudaSuccess) {
      rc = fail(NB200_ECUDA, "parameter kernel failed: %s", cudaGetErrorString(cudaGetLastError()));
      break;
    }
    *qr_max = h[1];
    MinMaxHostArgs a{d + 8};
    rc = host_pipeline(x, y, size, minmax_chunk, &a);
  } while (0);
  cudaFree(d);
  return rc;
}

int nb200_fixed_point_quantize_backward_f32(const float *x, const float *dy, float *dx, size_t size, int sign, int n,
                                            float delta, int ste_fine_grained, int accum, void *stream) {
  FxpLimits L;
  NB_TRY(fxp_limits(sign, n, delta, &L));
  if (ste_fine_grained)
    return launch_gradient(x, dy, dx, size, accum, FxpGrad{L.maxv, L.minv}, as_stream(stream));
  return launch_gradient(x, dy, dx, size, accum, PassAllGrad(), as_stream(stream));
}

int nb200_pow2_quantize_backward_f32(const float *x, const float *dy, float *dx, size_t size, int sign, int with_zero,
                                     int n, int m, int ste_fine_grained, int accum, void *stream) {
  Pow2Params P;
  NB_TRY(pow2_params(sign, with_zero, n, m, &P));
  if (!ste_fine_grained)
    return launch_gradient(x, dy, dx, size, accum, PassAllGrad(), as_stream(stream));
  Pow2Grad op{0u, P.sign};
  NB_TRY(pow2_gradient_threshold(P, &op.threshold_bits));
  return launch_gradient(x, dy, dx, size, accum, op, as_stream(stream));
}

int nb200_min_max_quantize_backward_f32(const float *x, const int64_t *x_shape, int ndim, const float *qr_min,
                                        const float *qr_max, const float *ql_min, const float *ql_max,
                                        const int64_t *q_shape, const float *dy, int x_min_max, int ema,
                                        int ste_fine_grained, const int32_t *propagate_down, const int32_t *accum,
                                        float *dx, float *g_qr_min, float *g_qr_max, void *stream) {
  NB_CHECK(x_shape && q_shape && propagate_down && accum, NB200_EVALUE, "null shape or flag pointer");
  MinMaxView V;
  NB_TRY(minmax_view(x_shape, q_shape, ndim, &V));
  return minmax_backward(x, V, qr_min, qr_max, ql_min, ql_max, dy, x_min_max, ema, ste_fine_grained, propagate_down,
                         accum, dx, g_qr_min, g_qr_max, as_stream(stream));
}

int nb200_binary_sigmoid_f32(const float *x, float *y, size_t size, void *stream) {
  return launch_elementwise(x, y, size, BinaryActOp<false>(), as_stream(stream));
}
int nb200_binary_tanh_f32(const float *x, float *y, size_t size, void *stream) {
  return launch_elementwise(x, y, size, BinaryActOp<true>(), as_stream(stream));
}
int nb200_binary_sigmoid_backward_f32(const float *x, const float *dy, float *dx, size_t size, int accum,
                                      void *stream) {
  return launch_gradient(x, dy, dx, size, accum, BinaryActGrad<false>(), as_stream(stream));
}
int nb200_binary_tanh_backward_f32(const float *x, const float *dy, float *dx, size_t size, int accum, void *stream) {
  return launch_gradient(x, dy, dx, size, accum, BinaryActGrad<true>(), as_stream(stream));
}

int nb200_quantize_linear_f32(const float *x, const int64_t *x_shape, int ndim, const float *scale,
                              const int64_t *scale_shape, float *zero_point, const int64_t *zero_point_shape, float *y,
                              int round_mode, int narrow_range, int dtype, void *stream) {
  NB_CHECK(x_shape && scale_shape && zero_point_shape, NB200_EVALUE, "null shape pointer");
  NB_CHECK(round_mode == 0 || round_mode == 1, NB200_EVALUE,
           "round_mode must be 0 (HALF_AWAY_FROM_ZERO) or 1 (HALF_TO_EVEN)");
  QuantizeLinearOp op{};
  size_t size = 0;
  NB_TRY(broadcast_view(x_shape, scale_shape, ndim, &op.vs, &size));
  NB_TRY(broadcast_view(x_shape, zero_point_shape, ndim, &op.vz, nullptr));
  NB_TRY(quantize_linear_range(narrow_range, dtype, &op.lo, &op.hi));
  NB_CHECK(scale && zero_point, NB200_EVALUE, "null parameter pointer");
  op.scale = scale;
  op.zp = zero_point;
  op.half_to_even = round_mode;
  cudaStream_t st = as_stream(stream);
  ql_zero_point_kernel<<<(unsigned)((op.vz.Q + 255) / 256), 256, 0, st>>>(zero_point, op.vz.Q, round_mode, op.lo,
                                                                           op.hi);
  NB_LAUNCH_CHECK();
  return launch_elementwise(x, y, size, op, st);
}

int nb200_dequantize_linear_f32(const float *x, const int64_t *x_shape, int ndim, const float *scale,
                                const int64_t *scale_shape, const float *zero_point, const int64_t *zero_point_shape,
                                float *y, void *stream) {
  NB_CHECK(x_shape && scale_shape && zero_point_shape, NB200_EVALUE, "null shape pointer");
  DequantizeLinearOp op{};
  size_t size = 0;
  NB_TRY(broadcast_view(x_shape, scale_shape, ndim, &op.vs, &size));
  NB_TRY(broadcast_view(x_shape, zero_point_shape, ndim, &op.vz, nullptr));
  NB_CHECK(scale && zero_point, NB200_EVALUE, "null parameter pointer");
  op.scale = scale;
  op.zp = zero_point;
  return launch_elementwise(x, y, size, op, as_stream(stream));
}

int nb200_quantize_linear_backward_f32(const float *dy, const int64_t *x_shape, int ndim, const float *scale,
                                       const int64_t *scale_shape, float *dx, int accum, void *stream) {
  NB_CHECK(x_shape && scale_shape && scale, NB200_EVALUE, "null pointer");
  LinearScaleGrad<true> op{scale, {}};
  size_t size = 0;
  NB_TRY(broadcast_view(x_shape, scale_shape, ndim, &op.vs, &size));
  return launch_gradient(nullptr, dy, dx, size, accum, op, as_stream(stream));
}

int nb200_dequantize_linear_backward_f32(const float *dy, const int64_t *x_shape, int ndim, const float *scale,
                                         const int64_t *scale_shape, float *dx, int accum, void *stream) {
  NB_CHECK(x_shape && scale_shape && scale, NB200_EVALUE, "null pointer");
  LinearScaleGrad<false> op{scale, {}};
  size_t size = 0;
  NB_TRY(broadcast_view(x_shape, scale_shape, ndim, &op.vs, &size));
  return launch_gradient(nullptr, dy, dx, size, accum, op, as_stream(stream));
}

int nb200_prune_f32(const float *x, float *y, size_t size, float rate, void *stream) {
  return prune_forward(x, y, size, rate, as_stream(stream));
}

int nb200_prune_backward_f32(const float *dy, float *dx, size_t size, int accum, void *stream) {
  return launch_gradient(nullptr, dy, dx, size, accum, PassAllGrad(), as_stream(stream));
}
}
