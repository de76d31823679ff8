// Operand preparation for the tensor-core contractions (all HBM-bound passes):
//  * weight binarisation fused with the per-output alpha = mean|W| reduction
//    and with the emission of the K-major +-1 side-band the MMA reads,
//  * fp32 -> three bf16 planes (hi, mid, lo with hi + mid + lo == x exactly
//    for normal-range values), optionally with NCHW -> NHWC re-layout,
//  * int8 code transposition.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "prepare.cuh"
#include "pdl.cuh"

namespace nb200 {
namespace {

__device__ __forceinline__ float sign_of(float w, float zero_to) {
  // include/nbla/function/sign.hpp:48-50 (+0, -0 and NaN take zero_to)
  return (w > 0.0f) ? 1.0f : ((w < 0.0f) ? -1.0f : zero_to);
}

// ---------------------------------------------------------------------------
// BinaryWeightAffine / BinaryConnectAffine weights: W is [R, C] row-major, one
// alpha per COLUMN (binary_weight_affine.cpp:83-107). Grid (C/64, R/64);
// each block handles a 64 x 64 tile: reads W coalesced along c, writes Wb
// coalesced, transposes the signs through shared memory and writes the
// side-band [C][Kp] (K = R contiguous) coalesced along r, and stores the
// tile's column sums of |W| to partial[row_block][c]. A second tiny kernel
// sums the partials in a fixed order (deterministic) and scales by 1/R.
// ---------------------------------------------------------------------------
constexpr int kBT = 64;

template <bool kInt8>
__global__ void __launch_bounds__(256) binarize_columns_kernel(const float *__restrict__ w, int R, int C,
                                                               float zero_to, float *__restrict__ wb,
                                                               void *__restrict__ side, int64_t side_pitch,
                                                               float *__restrict__ partial) {
  __shared__ float s_sign[kBT][kBT + 1];
  __shared__ float s_sum[4][kBT];
  const int c0 = blockIdx.x * kBT, r0 = blockIdx.y * kBT;
  const int tx = threadIdx.x & 63, ty = threadIdx.x >> 6; // 64 x 4
  const int c = c0 + tx;
  float acc = 0.0f;
  for (int rr = ty; rr < kBT; rr += 4) {
    const int r = r0 + rr;
    float s = 0.0f;
    if (r < R && c < C) {
      const float v = w[(int64_t)r * C + c];
      s = sign_of(v, zero_to);
      wb[(int64_t)r * C + c] = s;
      acc += fabsf(v);
    }
    s_sign[rr][tx] = s;
  }
  s_sum[ty][tx] = acc;
  __syncthreads();
  if (partial != nullptr && ty == 0 && c < C)
    partial[(int64_t)blockIdx.y * C + c] = (s_sum[0][tx] + s_sum[1][tx]) + (s_sum[2][tx] + s_sum[3][tx]);
  // side-band: row = output column c, contiguous index = input row r
  for (int cc = ty; cc < kBT; cc += 4) {
    const int oc = c0 + cc, r = r0 + tx;
    if (oc < C && r < R) {
      const float s = s_sign[tx][cc];
      if (kInt8)
        reinterpret_cast<int8_t *>(side)[(int64_t)oc * side_pitch + r] = (int8_t)(int)s;
      else
        reinterpret_cast<__nv_bfloat16 *>(side)[(int64_t)oc * side_pitch + r] = __float2bfloat16_rn(s);
    }
  }
}

// The same with 128-bit accesses (C a multiple of 4, 16-byte aligned W / Wb, side-band rows
// aligned to 8 bytes): a thread handles four columns of a row, and four rows of a side-band row.
template <bool kInt8>
__global__ void __launch_bounds__(256) binarize_columns_vec_kernel(const float *__restrict__ w, int R, int C,
                                                                   float zero_to, float *__restrict__ wb,
                                                                   void *__restrict__ side, int64_t side_pitch,
                                                                   float *__restrict__ partial) {
  __shared__ float s_sign[kBT][kBT + 1];
  __shared__ float s_sum[16][kBT];
  const int c0 = blockIdx.x * kBT, r0 = blockIdx.y * kBT;
  const int tx4 = threadIdx.x & 15, ty = threadIdx.x >> 4; // 16 column quads x 16 rows
  const int c = c0 + 4 * tx4;
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
  for (int it = 0; it < 4; ++it) {
    const int rr = ty + 16 * it, r = r0 + rr;
    float4 sg = make_float4(0.f, 0.f, 0.f, 0.f);
    if (r < R && c < C) { // C % 4 == 0: the quad is inside or outside as a whole
      const float4 v = __ldg(reinterpret_cast<const float4 *>(w + (int64_t)r * C + c));
      sg = make_float4(sign_of(v.x, zero_to), sign_of(v.y, zero_to), sign_of(v.z, zero_to), sign_of(v.w, zero_to));
      *reinterpret_cast<float4 *>(wb + (int64_t)r * C + c) = sg;
      acc[0] += fabsf(v.x), acc[1] += fabsf(v.y), acc[2] += fabsf(v.z), acc[3] += fabsf(v.w);
    }
    s_sign[rr][4 * tx4 + 0] = sg.x;
    s_sign[rr][4 * tx4 + 1] = sg.y;
    s_sign[rr][4 * tx4 + 2] = sg.z;
    s_sign[rr][4 * tx4 + 3] = sg.w;
  }
#pragma unroll
  for (int i = 0; i < 4; ++i)
    s_sum[ty][4 * tx4 + i] = acc[i];
  __syncthreads();
  if (partial != nullptr && threadIdx.x < kBT && c0 + threadIdx.x < C) {
    float t = 0.0f; // fixed order: deterministic
#pragma unroll
    for (int k = 0; k < 16; ++k)
      t += s_sum[k][threadIdx.x];
    partial[(int64_t)blockIdx.y * C + c0 + threadIdx.x] = t;
  }
  // side-band: row = output column, contiguous index = input row; four input rows per thread
  const int r = r0 + 4 * tx4;
#pragma unroll
  for (int it = 0; it < 4; ++it) {
    const int cc = ty + 16 * it, oc = c0 + cc;
    if (oc >= C || r >= R)
      continue;
    float sv[4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
      sv[i] = (r + i < R) ? s_sign[4 * tx4 + i][cc] : 0.0f;
    if (kInt8) {
      const uint32_t packed = ((uint32_t)(uint8_t)(int8_t)(int)sv[0]) | ((uint32_t)(uint8_t)(int8_t)(int)sv[1] << 8) |
                              ((uint32_t)(uint8_t)(int8_t)(int)sv[2] << 16) | ((uint32_t)(uint8_t)(int8_t)(int)sv[3] << 24);
      *reinterpret_cast<uint32_t *>(reinterpret_cast<int8_t *>(side) + (int64_t)oc * side_pitch + r) = packed;
    } else {
      const __nv_bfloat162 lo = __floats2bfloat162_rn(sv[0], sv[1]), hi = __floats2bfloat162_rn(sv[2], sv[3]);
      uint2 out;
      out.x = *reinterpret_cast<const uint32_t *>(&lo);
      out.y = *reinterpret_cast<const uint32_t *>(&hi);
      *reinterpret_cast<uint2 *>(reinterpret_cast<__nv_bfloat16 *>(side) + (int64_t)oc * side_pitch + r) = out;
    }
  }
}

__global__ void finalize_alpha_kernel(const float *__restrict__ partial, int blocks, int C, float inv,
                                      float *__restrict__ alpha) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C)
    return;
  float s = 0.0f;
  for (int b = 0; b < blocks; ++b)
    s += partial[(int64_t)b * C + c];
  alpha[c] = __fmul_rn(s, inv);
}

// ---------------------------------------------------------------------------
// BinaryWeightConvolution / BinaryConnectConvolution weights: W is
// [Ko, Cg, kh, kw]; one alpha per output map = mean over its Cg*kh*kw taps
// (binary_weight_convolution.cpp:81-102). One block per output map; the
// side-band is [Ko][Kp] with K ordered (ky, kx, c) so that one 128-byte K
// block is one filter tap over consecutive channels, matching the NHWC
// activation planes.
// ---------------------------------------------------------------------------
// kMode: 0 = bf16 signs, 1 = int8 signs, 2 = fp16 signs.
template <int kMode>
__device__ __forceinline__ void binarize_row(int o, const float *__restrict__ w, int Cg, int kh, int kw,
                                             float zero_to, float inv, float *__restrict__ wb,
                                             float *__restrict__ alpha, void *__restrict__ side, int64_t side_pitch,
                                             int c_pad) {
  const int taps = kh * kw, Kd = Cg * taps;
  const float *wr = w + (int64_t)o * Kd;
  float acc = 0.0f;
  for (int k = threadIdx.x; k < Kd; k += 256) {
    const float v = wr[k];
    const float s = sign_of(v, zero_to);
    wb[(int64_t)o * Kd + k] = s;
    acc += fabsf(v);
    const int c = k / taps, t = k - c * taps;
    const int64_t dst = (int64_t)o * side_pitch + (int64_t)t * c_pad + c;
    if (kMode == 1) {
      reinterpret_cast<int8_t *>(side)[dst] = (int8_t)(int)s;
    } else if (kMode == 2) {
      reinterpret_cast<__half *>(side)[dst] = __float2half_rn(s);
    } else {
      reinterpret_cast<__nv_bfloat16 *>(side)[dst] = __float2bfloat16_rn(s);
    }
  }
  if (alpha == nullptr)
    return;
#pragma unroll
  for (int d = 16; d > 0; d >>= 1)
    acc += __shfl_xor_sync(0xffffffffu, acc, d);
  __shared__ float s_part[8];
  if ((threadIdx.x & 31) == 0)
    s_part[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    float s = 0.0f;
    for (int i = 0; i < 8; ++i)
      s += s_part[i];
    alpha[o] = __fmul_rn(s, inv);
  }
}

template <int kMode>
__global__ void __launch_bounds__(256) binarize_rows_kernel(const float *__restrict__ w, int Cg, int kh, int kw,
                                                            float zero_to, float inv, float *__restrict__ wb,
                                                            float *__restrict__ alpha, void *__restrict__ side,
                                                            int64_t side_pitch, int c_pad) {
  pdl_wait();
  pdl_trigger();
  binarize_row<kMode>(blockIdx.x, w, Cg, kh, kw, zero_to, inv, wb, alpha, side, side_pitch, c_pad);
}

// Fixed-point convolution weights: wq [Ko, Cg, kh, kw] holds multiples of delta
// (|code| <= 127); the int8 codes go to the same tap-major side-band layout.
__global__ void __launch_bounds__(256) codes_conv_weights_kernel(const float *__restrict__ wq, int Cg, int kh, int kw,
                                                                 float inv_delta, int8_t *__restrict__ side,
                                                                 int64_t side_pitch, int c_pad) {
  const int o = blockIdx.x;
  const int taps = kh * kw, Kd = Cg * taps;
  const float *wr = wq + (int64_t)o * Kd;
  for (int k = threadIdx.x; k < Kd; k += 256) {
    const int c = k / taps, t = k - c * taps;
    side[(int64_t)o * side_pitch + (int64_t)t * c_pad + c] = (int8_t)__float2int_rn(__fmul_rn(wr[k], inv_delta));
  }
}

// ---------------------------------------------------------------------------
// fp32 [rows, K] -> bf16 planes [3][rows][Kp]: hi = bf16(x), mid = bf16(x - hi),
// lo = bf16(x - hi - mid); the two subtractions are exact in fp32.
// ---------------------------------------------------------------------------
__device__ __forceinline__ void split3(float x, __nv_bfloat16 &h, __nv_bfloat16 &m, __nv_bfloat16 &l) {
  h = __float2bfloat16_rn(x);
  const float r1 = __fsub_rn(x, __bfloat162float(h));
  m = __float2bfloat16_rn(r1);
  const float r2 = __fsub_rn(r1, __bfloat162float(m));
  l = __float2bfloat16_rn(r2);
}

// Block = 64 columns x 4 rows (Kp is a multiple of 64): coalesced along K, no
// 64-bit divisions.
__global__ void __launch_bounds__(256) split_rows_kernel(const float *__restrict__ x, int64_t rows, int K, int64_t Kp,
                                                         int planes, const float *__restrict__ col_scale,
                                                         __nv_bfloat16 *__restrict__ out) {
  const int k = blockIdx.x * 64 + threadIdx.x;
  const int64_t plane_stride = rows * Kp;
  const float cs = (col_scale != nullptr && k < K) ? col_scale[k] : 1.0f;
  for (int64_t r = (int64_t)blockIdx.y * 4 + threadIdx.y; r < rows; r += (int64_t)gridDim.y * 4) {
    float v = (k < K) ? x[r * K + k] : 0.0f;
    if (col_scale != nullptr)
      v = __fmul_rn(v, cs);
    __nv_bfloat16 h, m, l;
    split3(v, h, m, l);
    const int64_t i = r * Kp + k;
    out[i] = h;
    if (planes > 1)
      out[plane_stride + i] = m;
    if (planes > 2)
      out[2 * plane_stride + i] = l;
  }
}

// Column sums of a row-major [rows, C] matrix (bias gradient, affine.cpp:130-137):
// block (cx, s) adds its share of the rows for 256 columns (coalesced along the
// columns), a second kernel adds the `splits` partials of each column in order.
__global__ void __launch_bounds__(256) column_partial_sums_kernel(const float *__restrict__ a, int64_t rows, int C,
                                                                  float *__restrict__ partial) {
  const int c = blockIdx.x * 256 + threadIdx.x;
  if (c >= C)
    return;
  const int64_t per = (rows + gridDim.y - 1) / gridDim.y;
  const int64_t r0 = blockIdx.y * per, r1 = (r0 + per < rows) ? r0 + per : rows;
  float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
  int64_t r = r0;
  for (; r + 3 < r1; r += 4) {
    s0 += a[r * C + c];
    s1 += a[(r + 1) * C + c];
    s2 += a[(r + 2) * C + c];
    s3 += a[(r + 3) * C + c];
  }
  for (; r < r1; ++r)
    s0 += a[r * C + c];
  partial[(int64_t)blockIdx.y * C + c] = (s0 + s1) + (s2 + s3);
}

__global__ void __launch_bounds__(256) column_finish_kernel(const float *__restrict__ partial, int C, int splits,
                                                            float *__restrict__ out, int accumulate) {
  const int c = blockIdx.x * 256 + threadIdx.x;
  if (c >= C)
    return;
  float s = 0.f;
  for (int k = 0; k < splits; ++k)
    s += partial[(int64_t)k * C + c];
  out[c] = accumulate ? __fadd_rn(out[c], s) : s;
}

// fp32 NCHW -> planes of NHWC: out[plane][n][hw][ctot], where channel c of
// group g lands at g * c_pad_g + (c - g * Cg) and every other slot is zero.
// Tile transpose through shared memory: reads coalesced along hw, writes
// coalesced along the channel slots. OutT = bf16 (PLANES pieces) or int8
// (codes of values that are multiples of delta).
template <typename OutT, int PLANES>
__global__ void __launch_bounds__(256) nchw_to_nhwc_kernel(const float *__restrict__ x, int C, int HW, int groups,
                                                           int Cg, int c_pad_g, int ctot, OutT *__restrict__ out,
                                                           int64_t plane_stride, float inv_delta) {
  __shared__ float tile[32][33];
  const int n = blockIdx.z;
  const int p0 = blockIdx.x * 32, d0 = blockIdx.y * 32; // d = destination channel slot
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5; // 32 x 8
  for (int dd = ty; dd < 32; dd += 8) {
    const int d = d0 + dd, p = p0 + tx;
    const int g = d / c_pad_g, cc = d - g * c_pad_g;
    const bool live = d < ctot && g < groups && cc < Cg && p < HW;
    tile[dd][tx] = live ? x[((int64_t)n * C + (g * Cg + cc)) * HW + p] : 0.0f;
  }
  __syncthreads();
  for (int pp = ty; pp < 32; pp += 8) {
    const int p = p0 + pp, d = d0 + tx;
    if (p < HW && d < ctot) {
      const float v = tile[tx][pp];
      const int64_t dst = ((int64_t)n * HW + p) * ctot + d;
      if constexpr (sizeof(OutT) == 1) {
        out[dst] = (OutT)__float2int_rn(__fmul_rn(v, inv_delta)); // v is k * delta
      } else {
        __nv_bfloat16 h, m, l;
        split3(v, h, m, l);
        out[dst] = h;
        if (PLANES > 1)
          out[plane_stride + dst] = m;
        if (PLANES > 2)
          out[2 * plane_stride + dst] = l;
      }
    }
  }
}

// fp32 NCHW (multiples of delta) -> int8 NHWC codes, 64 pixels x 64 channel
// slots per block. Reads are coalesced along the pixels of one channel plane;
// the codes are transposed through shared memory (row pitch 17 words, so both
// the byte writes and the word reads are bank-conflict free) and written as
// 64-byte runs per pixel.
__device__ __forceinline__ void nchw_to_nhwc_i8_tile(int bx, int by, int n, const float *__restrict__ x, int C, int HW,
                                                     int groups, int Cg, int c_pad_g, int ctot,
                                                     int8_t *__restrict__ out, float inv_delta) {
  __shared__ uint32_t tile[64][17]; // [pixel][16 words of 4 codes + 1 pad]
  int8_t *tile8 = reinterpret_cast<int8_t *>(&tile[0][0]);
  const int p0 = bx * 64, d0 = by * 64;
  const int tx = threadIdx.x & 63, ty = threadIdx.x >> 6;
  const int p = p0 + tx;
  for (int dd = ty; dd < 64; dd += 4) {
    const int d = d0 + dd;
    const int g = d / c_pad_g, cc = d - g * c_pad_g;
    float v = 0.0f;
    if (d < ctot && g < groups && cc < Cg && p < HW)
      v = __ldcs(x + ((int64_t)n * C + (g * Cg + cc)) * HW + p);
    tile8[tx * 68 + dd] = (int8_t)__float2int_rn(__fmul_rn(v, inv_delta));
  }
  __syncthreads();
  const int word = threadIdx.x & 15, prow = threadIdx.x >> 4; // 16 pixels per pass
  for (int pp = prow; pp < 64; pp += 16) {
    const int pix = p0 + pp, d = d0 + 4 * word;
    if (pix < HW && d < ctot)
      *reinterpret_cast<uint32_t *>(out + ((int64_t)n * HW + pix) * ctot + d) = tile[pp][word];
  }
}

__global__ void __launch_bounds__(256) nchw_to_nhwc_i8_kernel(const float *__restrict__ x, int C, int HW, int groups,
                                                              int Cg, int c_pad_g, int ctot,
                                                              int8_t *__restrict__ out, float inv_delta) {
  nchw_to_nhwc_i8_tile(blockIdx.x, blockIdx.y, blockIdx.z, x, C, HW, groups, Cg, c_pad_g, ctot, out, inv_delta);
}

// Same conversion with 128-bit loads (HW a multiple of 4): every thread has
// four independent float4 loads in flight (4 pixels x 4 channel rows).
__device__ __forceinline__ void nchw_to_nhwc_i8_vec_tile(int bx, int by, int n, const float *__restrict__ x, int C,
                                                         int HW, int groups, int Cg, int c_pad_g, int ctot,
                                                         int8_t *__restrict__ out, float inv_delta) {
  __shared__ uint32_t tile[64][17];
  const int p0 = bx * 64, d0 = by * 64;
  // 16 pixel quads x 16 channel quads: a thread converts four neighbouring channel slots of four pixels, so
  // that the four codes of a pixel leave as one word
  const int px4 = threadIdx.x & 15, chq = threadIdx.x >> 4;
  const int p = p0 + 4 * px4;
  const int dq = d0 + 4 * chq;
  const int g = dq / c_pad_g, cc0 = dq - g * c_pad_g; // c_pad_g is a multiple of 16: one group for the four slots
  const bool ok = dq < ctot && g < groups && p < HW;
  const float *base = x + ((int64_t)n * C + (g * Cg + cc0)) * HW + p;
  // round(v / delta) on the add pipe: for |t| < 2^22 the low mantissa bits of 1.5 * 2^23 + t, rounded to
  // nearest even by the addition itself, are the two's complement integer (its low byte is the code)
  uint32_t f[4][4];
#pragma unroll
  for (int r = 0; r < 4; ++r) {
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (ok && cc0 + r < Cg)
      v = __ldcs(reinterpret_cast<const float4 *>(base + (int64_t)r * HW));
    f[r][0] = __float_as_uint(__fadd_rn(__fmul_rn(v.x, inv_delta), 12582912.0f));
    f[r][1] = __float_as_uint(__fadd_rn(__fmul_rn(v.y, inv_delta), 12582912.0f));
    f[r][2] = __float_as_uint(__fadd_rn(__fmul_rn(v.z, inv_delta), 12582912.0f));
    f[r][3] = __float_as_uint(__fadd_rn(__fmul_rn(v.w, inv_delta), 12582912.0f));
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
    if (pix < HW && d < ctot)
      *reinterpret_cast<uint32_t *>(out + ((int64_t)n * HW + pix) * ctot + d) = tile[pp][word];
  }
}

__global__ void __launch_bounds__(256) nchw_to_nhwc_i8_vec_kernel(const float *__restrict__ x, int C, int HW,
                                                                  int groups, int Cg, int c_pad_g, int ctot,
                                                                  int8_t *__restrict__ out, float inv_delta) {
  pdl_wait();
  pdl_trigger();
  nchw_to_nhwc_i8_vec_tile(blockIdx.x, blockIdx.y, blockIdx.z, x, C, HW, groups, Cg, c_pad_g, ctot, out, inv_delta);
}

// Both operands of a binary-weight convolution over fixed-point activations in one launch: blocks
// [0, Ko) binarise one filter each (sign, scale, int8 side-band), the others convert one 64 x 64 tile of
// the activations to channel-last codes. The two jobs are independent, and at a few dozen images the
// weights' pass costs as much as the activations': side by side it disappears behind them.
template <bool kVec>
__global__ void __launch_bounds__(256)
    binary_conv_operands_i8_kernel(const float *__restrict__ w, int Ko, int Cg_w, int kh, int kw, float zero_to, float inv,
                                   float *__restrict__ wb, float *__restrict__ alpha, void *__restrict__ side,
                                   int64_t side_pitch, int c_pad, const float *__restrict__ x, int C, int HW,
                                   int groups, int Cg, int c_pad_g, int ctot, int8_t *__restrict__ out,
                                   float inv_delta, int gx, int gy) {
  pdl_wait();
  pdl_trigger();
  if ((int)blockIdx.x < Ko) {
    binarize_row<1>(blockIdx.x, w, Cg_w, kh, kw, zero_to, inv, wb, alpha, side, side_pitch, c_pad);
    return;
  }
  const int lin = (int)blockIdx.x - Ko;
  const int bx = lin % gx, r = lin / gx;
  if (kVec)
    nchw_to_nhwc_i8_vec_tile(bx, r % gy, r / gy, x, C, HW, groups, Cg, c_pad_g, ctot, out, inv_delta);
  else
    nchw_to_nhwc_i8_tile(bx, r % gy, r / gy, x, C, HW, groups, Cg, c_pad_g, ctot, out, inv_delta);
}

// int8 [R, C] -> [C][pitch] (transpose), tile 64 x 64 through shared memory.
__global__ void __launch_bounds__(256) transpose_i8_kernel(const int8_t *__restrict__ src, int R, int C,
                                                           int8_t *__restrict__ dst, int64_t pitch) {
  __shared__ int8_t tile[64][65];
  const int c0 = blockIdx.x * 64, r0 = blockIdx.y * 64;
  const int tx = threadIdx.x & 63, ty = threadIdx.x >> 6;
  for (int rr = ty; rr < 64; rr += 4) {
    const int r = r0 + rr, c = c0 + tx;
    tile[rr][tx] = (r < R && c < C) ? src[(int64_t)r * C + c] : (int8_t)0;
  }
  __syncthreads();
  for (int cc = ty; cc < 64; cc += 4) {
    const int c = c0 + cc, r = r0 + tx;
    if (c < C && r < R)
      dst[(int64_t)c * pitch + r] = tile[tx][cc];
  }
}

// fp32 [R, C] -> [C][R] (transpose), tile 32 x 32 through shared memory.
__global__ void __launch_bounds__(256) transpose_f32_kernel(const float *__restrict__ src, int R, int C,
                                                            float *__restrict__ dst) {
  __shared__ float tile[32][33];
  const int c0 = blockIdx.x * 32, r0 = blockIdx.y * 32;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  for (int rr = ty; rr < 32; rr += 8) {
    const int r = r0 + rr, c = c0 + tx;
    tile[rr][tx] = (r < R && c < C) ? src[(int64_t)r * C + c] : 0.0f;
  }
  __syncthreads();
  for (int cc = ty; cc < 32; cc += 8) {
    const int c = c0 + cc, r = r0 + tx;
    if (c < C && r < R)
      dst[(int64_t)c * R + r] = tile[tx][cc];
  }
}

// fp32 values that are integer multiples of delta -> int8 codes, [rows, K] -> [rows][pitch].
__global__ void __launch_bounds__(256) codes_rows_kernel(const float *__restrict__ x, int64_t rows, int K,
                                                         int64_t pitch, float inv_delta, int8_t *__restrict__ out) {
  const int64_t total = rows * pitch;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = i / pitch;
    const int k = (int)(i - r * pitch);
    out[i] = (k < K) ? (int8_t)__float2int_rn(__fmul_rn(x[r * K + k], inv_delta)) : (int8_t)0;
  }
}

inline unsigned capped_grid(int64_t items, int threads) {
  int64_t b = (items + threads - 1) / threads;
  const int64_t cap = (int64_t)sm_count() * 64;
  if (b > cap)
    b = cap;
  return (unsigned)(b < 1 ? 1 : b);
}

} // namespace

int binarize_columns(const float *w, int R, int C, float zero_to, float *wb, float *alpha, void *side,
                     int64_t side_pitch, bool int8, float *partial_scratch, cudaStream_t st) {
  const dim3 grid((C + kBT - 1) / kBT, (R + kBT - 1) / kBT);
  float *partial = alpha ? partial_scratch : nullptr;
  // the side-band rows hold K padded to a multiple of 64 values: four rows past R stay inside a row
  const bool vec = C % 4 == 0 && side_pitch % 4 == 0 && side_pitch >= (int64_t)(R + 3) / 4 * 4 &&
                   ((reinterpret_cast<uintptr_t>(w) | reinterpret_cast<uintptr_t>(wb)) & 15) == 0 &&
                   (reinterpret_cast<uintptr_t>(side) & 7) == 0;
  if (vec && int8)
    binarize_columns_vec_kernel<true><<<grid, 256, 0, st>>>(w, R, C, zero_to, wb, side, side_pitch, partial);
  else if (vec)
    binarize_columns_vec_kernel<false><<<grid, 256, 0, st>>>(w, R, C, zero_to, wb, side, side_pitch, partial);
  else if (int8)
    binarize_columns_kernel<true><<<grid, 256, 0, st>>>(w, R, C, zero_to, wb, side, side_pitch, partial);
  else
    binarize_columns_kernel<false><<<grid, 256, 0, st>>>(w, R, C, zero_to, wb, side, side_pitch, partial);
  NB_LAUNCH_CHECK();
  if (alpha) {
    const float inv = (float)1 / R; // binary_weight_affine.cpp:68
    finalize_alpha_kernel<<<(C + 255) / 256, 256, 0, st>>>(partial, (int)grid.y, C, inv, alpha);
    NB_LAUNCH_CHECK();
  }
  return NB200_OK;
}

int binarize_rows(const float *w, int Ko, int Cg, int kh, int kw, float zero_to, float *wb, float *alpha, void *side,
                  int64_t side_pitch, int c_pad, bool int8, cudaStream_t st, bool half) {
  const float inv = (float)1 / (Cg * kh * kw); // binary_weight_convolution.cpp:66
  if (int8)
    NB_CUDA(launch_dependent(binarize_rows_kernel<1>, dim3(Ko), dim3(256), 0, st, w, Cg, kh, kw, zero_to, inv, wb, alpha,
                             side, side_pitch, c_pad));
  else if (half)
    binarize_rows_kernel<2><<<Ko, 256, 0, st>>>(w, Cg, kh, kw, zero_to, inv, wb, alpha, side, side_pitch, c_pad);
  else
    binarize_rows_kernel<0><<<Ko, 256, 0, st>>>(w, Cg, kh, kw, zero_to, inv, wb, alpha, side, side_pitch, c_pad);
  NB_LAUNCH_CHECK();
  return NB200_OK;
}

bool binary_conv_operands_i8_applies(const float *x, int N, int HW, int ctot, int Ko) {
  const int64_t blocks = (int64_t)Ko + (int64_t)((HW + 63) / 64) * ((ctot + 63) / 64) * N;
  return x != nullptr && blocks < (1ll << 31);
}

int binary_conv_operands_i8(const float *w, int Ko, int Cg, int kh, int kw, float zero_to, float *wb, float *alpha,
                            void *side, int64_t side_pitch, int c_pad, const float *x, int N, int C, int HW, int groups,
                            int c_pad_g, int ctot, float delta, void *out, cudaStream_t st) {
  const float inv = (float)1 / (Cg * kh * kw); // binary_weight_convolution.cpp:66
  const int gx = (HW + 63) / 64, gy = (ctot + 63) / 64;
  const int64_t blocks = (int64_t)Ko + (int64_t)gx * gy * N;
  NB_CHECK(binary_conv_operands_i8_applies(x, N, HW, ctot, Ko), NB200_EVALUE, "operand preparation does not apply");
  // 128-bit loads when the planes allow it (nchw_to_nhwc_planes has the same rule)
  if (HW % 4 == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0)
    NB_CUDA(launch_dependent(binary_conv_operands_i8_kernel<true>, dim3((unsigned)blocks), dim3(256), 0, st, w, Ko, Cg,
                             kh, kw, zero_to, inv, wb, alpha, side, side_pitch, c_pad, x, C, HW, groups, Cg, c_pad_g,
                             ctot, reinterpret_cast<int8_t *>(out), 1.0f / delta, gx, gy));
  else
    NB_CUDA(launch_dependent(binary_conv_operands_i8_kernel<false>, dim3((unsigned)blocks), dim3(256), 0, st, w, Ko, Cg,
                             kh, kw, zero_to, inv, wb, alpha, side, side_pitch, c_pad, x, C, HW, groups, Cg, c_pad_g,
                             ctot, reinterpret_cast<int8_t *>(out), 1.0f / delta, gx, gy));
  NB_LAUNCH_CHECK();
  return NB200_OK;
}

int codes_conv_weights(const float *wq, int Ko, int Cg, int kh, int kw, float delta, void *side, int64_t side_pitch,
                       int c_pad, cudaStream_t st) {
  codes_conv_weights_kernel<<<Ko, 256, 0, st>>>(wq, Cg, kh, kw, 1.0f / delta, reinterpret_cast<int8_t *>(side),
                                                side_pitch, c_pad);
  NB_LAUNCH_CHECK();
  return NB200_OK;
}

int split_rows_bf16(const float *x, int64_t rows, int K, int64_t Kp, int planes, void *out, cudaStream_t st,
                    const float *col_scale) {
  NB_CHECK(Kp % 64 == 0 && Kp / 64 < (1ll << 31), NB200_EVALUE, "the padded K extent must be a multiple of 64");
  int64_t gy = (rows + 3) / 4;
  const int64_t cap = (int64_t)sm_count() * 64;
  gy = gy > cap ? cap : (gy < 1 ? 1 : gy);
  gy = gy > 65535 ? 65535 : gy;
  split_rows_kernel<<<dim3((unsigned)(Kp / 64), (unsigned)gy), dim3(64, 4), 0, st>>>(
      x, rows, K, Kp, planes, col_scale, reinterpret_cast<__nv_bfloat16 *>(out));
  NB_LAUNCH_CHECK();
  return NB200_OK;
}

// ---------------------------------------------------------------------------
// Two fp16 pieces of an fp32 tensor: with s = 2^-e chosen from the tensor's largest magnitude so that
// max |x| * s lies in [2^14, 2^15), x * s = p0 + p1 with p0 = fp16(x * s), p1 = fp16(x * s - p0): 22
// significant bits for every element within 2^-18 of the maximum, an absolute error of at most 2^-40
// of the maximum below that (p1 is then subnormal), which no fp32 sum over a filter window resolves.
// ---------------------------------------------------------------------------
__device__ __forceinline__ int half_pair_exponent(uint32_t maxbits) {
  const int E = (int)(maxbits >> 23);
  if (E == 0 || E >= 255)
    return 0; // zero, denormal or non-finite maximum: no scaling
  const int e = E - 127 - 14;
  return e < -100 ? -100 : e;
}

__global__ void __launch_bounds__(256) absmax_bits_kernel(const float *__restrict__ x, size_t n,
                                                          uint32_t *__restrict__ maxbits) {
  uint32_t m = 0;
  const size_t stride = (size_t)gridDim.x * 256;
  const size_t n4 = ((reinterpret_cast<uintptr_t>(x) & 15) == 0) ? n / 4 : 0;
  for (size_t i = (size_t)blockIdx.x * 256 + threadIdx.x; i < n4; i += stride) {
    const float4 v = __ldg(reinterpret_cast<const float4 *>(x) + i);
    m = max(max(m, __float_as_uint(fabsf(v.x))), max(__float_as_uint(fabsf(v.y)), __float_as_uint(fabsf(v.z))));
    m = max(m, __float_as_uint(fabsf(v.w)));
  }
  for (size_t i = n4 * 4 + (size_t)blockIdx.x * 256 + threadIdx.x; i < n; i += stride)
    m = max(m, __float_as_uint(fabsf(__ldg(x + i))));
  m = __reduce_max_sync(0xffffffffu, m);
  if ((threadIdx.x & 31) == 0 && m != 0)
    atomicMax(maxbits, m);
}

// out[i] = (in ? in[i] : 1) * 2^e: the per-row factor that undoes the activation scaling
__global__ void half_pair_row_scale_kernel(const float *__restrict__ in, int n, const uint32_t *__restrict__ maxbits,
                                           float *__restrict__ out) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) {
    const float up = __int_as_float((127 + half_pair_exponent(*maxbits)) << 23);
    out[i] = in ? __fmul_rn(in[i], up) : up;
  }
}

// nchw_to_nhwc_kernel for the two fp16 pieces; plane 1 lies plane_stride elements behind plane 0.
// Tiles of 32 pixels x 64 channel slots: loads run along the pixels, every thread stores two
// neighbouring slots of a pixel as one 32-bit word per plane (ctot is even: slots come in sixteens).
__global__ void __launch_bounds__(256) nchw_to_nhwc_half_pair_kernel(const float *__restrict__ x, int C, int HW,
                                                                     int groups, int Cg, int c_pad_g, int ctot,
                                                                     const uint32_t *__restrict__ maxbits,
                                                                     __half *__restrict__ out, int64_t plane_stride) {
  __shared__ float tile[64][33];
  const float down = __int_as_float((127 - half_pair_exponent(*maxbits)) << 23);
  const int n = blockIdx.z;
  const int p0 = blockIdx.x * 32, d0 = blockIdx.y * 64;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
#pragma unroll
  for (int dd = ty; dd < 64; dd += 8) {
    const int d = d0 + dd, p = p0 + tx;
    const int g = d / c_pad_g, cc = d - g * c_pad_g;
    const bool live = d < ctot && g < groups && cc < Cg && p < HW;
    tile[dd][tx] = live ? __ldcs(x + ((int64_t)n * C + (g * Cg + cc)) * HW + p) : 0.0f;
  }
  __syncthreads();
#pragma unroll
  for (int pp = ty; pp < 32; pp += 8) {
    const int p = p0 + pp, d = d0 + 2 * tx;
    if (p < HW && d < ctot) {
      const float v0 = __fmul_rn(tile[2 * tx][pp], down), v1 = __fmul_rn(tile[2 * tx + 1][pp], down);
      const __half a0 = __float2half_rn(v0), a1 = __float2half_rn(v1);
      const __half b0 = __float2half_rn(__fsub_rn(v0, __half2float(a0)));
      const __half b1 = __float2half_rn(__fsub_rn(v1, __half2float(a1)));
      const int64_t dst = ((int64_t)n * HW + p) * ctot + d;
      *reinterpret_cast<__half2 *>(out + dst) = __halves2half2(a0, a1);
      *reinterpret_cast<__half2 *>(out + plane_stride + dst) = __halves2half2(b0, b1);
    }
  }
}

int nchw_to_nhwc_half_pair(const float *x, int N, int C, int HW, int groups, int Cg, int c_pad_g, int ctot, void *out,
                           uint32_t *maxbits, const float *row_scale_in, int rows, float *row_scale_out,
                           cudaStream_t st) {
  NB_CHECK(N <= 65535, NB200_ENOTIMPL, "batch larger than 65535");
  NB_CUDA(cudaMemsetAsync(maxbits, 0, 4, st));
  const size_t n = (size_t)N * C * HW;
  size_t blocks = (n / 4 + 255) / 256;
  const size_t cap = (size_t)sm_count() * 16;
  blocks = blocks < 1 ? 1 : (blocks > cap ? cap : blocks);
  absmax_bits_kernel<<<(unsigned)blocks, 256, 0, st>>>(x, n, maxbits);
  NB_LAUNCH_CHECK();
  half_pair_row_scale_kernel<<<(rows + 255) / 256, 256, 0, st>>>(row_scale_in, rows, maxbits, row_scale_out);
  NB_LAUNCH_CHECK();
  NB_CHECK(ctot % 2 == 0, NB200_EVALUE, "channel slots must come in pairs");
  const dim3 grid((HW + 31) / 32, (ctot + 63) / 64, N);
  nchw_to_nhwc_half_pair_kernel<<<grid, 256, 0, st>>>(x, C, HW, groups, Cg, c_pad_g, ctot, maxbits,
                                                      reinterpret_cast<__half *>(out), (int64_t)N * HW * ctot);
  NB_LAUNCH_CHECK();
  return NB200_OK;
}

int nchw_to_nhwc_planes(const float *x, int N, int C, int HW, int groups, int Cg, int c_pad_g, int ctot, int planes,
                        float delta, void *out, cudaStream_t st) {
  const dim3 grid((HW + 31) / 32, (ctot + 31) / 32, N);
  NB_CHECK(N <= 65535, NB200_ENOTIMPL, "batch larger than 65535");
  const int64_t ps = (int64_t)N * HW * ctot;
  if (planes == 0) {
    // ctot is a multiple of 16 (channel slots are padded to 16 per group), so word stores are aligned.
    const dim3 grid8((HW + 63) / 64, (ctot + 63) / 64, N);
    if (HW % 4 == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0)
      NB_CUDA(launch_dependent(nchw_to_nhwc_i8_vec_kernel, grid8, dim3(256), 0, st, x, C, HW, groups, Cg, c_pad_g, ctot,
                               reinterpret_cast<int8_t *>(out), 1.0f / delta));
    else
      nchw_to_nhwc_i8_kernel<<<grid8, 256, 0, st>>>(x, C, HW, groups, Cg, c_pad_g, ctot,
                                                    reinterpret_cast<int8_t *>(out), 1.0f / delta);
  } else if (planes == 3) {
    nchw_to_nhwc_kernel<__nv_bfloat16, 3><<<grid, 256, 0, st>>>(x, C, HW, groups, Cg, c_pad_g, ctot,
                                                                reinterpret_cast<__nv_bfloat16 *>(out), ps, 0.f);
  } else {
    nchw_to_nhwc_kernel<__nv_bfloat16, 1><<<grid, 256, 0, st>>>(x, C, HW, groups, Cg, c_pad_g, ctot,
                                                                reinterpret_cast<__nv_bfloat16 *>(out), ps, 0.f);
  }
  NB_LAUNCH_CHECK();
  return NB200_OK;
}

int column_sums(const float *a, int64_t rows, int C, float *out, int accumulate, float *partial, int splits,
                cudaStream_t st) {
  const dim3 grid((C + 255) / 256, splits);
  column_partial_sums_kernel<<<grid, 256, 0, st>>>(a, rows, C, partial);
  NB_LAUNCH_CHECK();
  column_finish_kernel<<<(C + 255) / 256, 256, 0, st>>>(partial, C, splits, out, accumulate);
  NB_LAUNCH_CHECK();
  return NB200_OK;
}

int transpose_i8(const int8_t *src, int R, int C, int8_t *dst, int64_t pitch, cudaStream_t st) {
  const dim3 grid((C + 63) / 64, (R + 63) / 64);
  transpose_i8_kernel<<<grid, 256, 0, st>>>(src, R, C, dst, pitch);
  NB_LAUNCH_CHECK();
  return NB200_OK;
}

int transpose_f32(const float *src, int R, int C, float *dst, cudaStream_t st) {
  const dim3 grid((C + 31) / 32, (R + 31) / 32);
  transpose_f32_kernel<<<grid, 256, 0, st>>>(src, R, C, dst);
  NB_LAUNCH_CHECK();
  return NB200_OK;
}

int codes_rows_i8(const float *x, int64_t rows, int K, int64_t pitch, float delta, int8_t *out, cudaStream_t st) {
  codes_rows_kernel<<<capped_grid(rows * pitch, 256), 256, 0, st>>>(x, rows, K, pitch, 1.0f / delta, out);
  NB_LAUNCH_CHECK();
  return NB200_OK;
}

} // namespace nb200
