// Implicit-GEMM convolution on the tcgen05 contraction kernel: host-side
// planning (pixel boxes, tensor maps) and the C-ABI entry points for
// BinaryWeightConvolution / BinaryConnectConvolution.
//
// Data layout in HBM for one call (scratch, stream-ordered allocation):
//   activations  [planes][N][H][W][Ctot]  bf16 (3 planes: hi, mid, lo) or int8 codes,
//                channels of group g at [g * c_pad_g, g * c_pad_g + Cg), zero padded
//   weights      [Ko][taps][c_slots]      +-1 (or quantize_zero_to) as bf16 / int8,
//                K ordered tap-major, channel-minor, zero padded per tap
// D = weights x activations^T with rows = output maps, columns = a box of
// output pixels; y is written NCHW directly from the epilogue.
#include <cmath>
#include <cstring>

#include "conv_codes.cuh"
#include "gemm.cuh"
#include "prepare.cuh"

namespace nb200 {
namespace {

inline int64_t round_up(int64_t v, int64_t m) { return (v + m - 1) / m * m; }

bool bf16_exact(float v) {
  uint32_t b;
  std::memcpy(&b, &v, 4);
  return (b & 0xffffu) == 0;
}

struct ConvGeometry {
  int N, C, H, W, Ko, kh, kw, ph, pw, sh, sw, dh, dw, group;
  int Cg, Kog, Ho, Wo;
};

// Pixel-major kernel (conv_codes.cuh), defined further down.
bool pixel_major_applies(const ConvGeometry &g);
int convolution_codes_folded(const int8_t *x_codes, const int8_t *side, const float *scale, const float *bias,
                             const int8_t *res_codes, float res_delta, const float *res_f32, int8_t *y_codes,
                             float *y_f32, ConvGeometry g, int relu, int sign, int n, float delta, cudaStream_t st,
                             float *y_nchw = nullptr, float nchw_scale = 1.0f);

// The reference's checks (src/nbla/function/generic/convolution.cpp:40-158).
int check_geometry(ConvGeometry &g) {
  NB_CHECK(g.N > 0 && g.C > 0 && g.H > 0 && g.W > 0 && g.Ko > 0 && g.kh > 0 && g.kw > 0, NB200_EVALUE,
           "empty convolution operand");
  NB_CHECK(g.group > 0 && g.C % g.group == 0, NB200_EVALUE,
           "Number of input channel needs to be divisible by group. Input channel: %d, group: %d.", g.C, g.group);
  NB_CHECK(g.Ko % g.group == 0, NB200_EVALUE,
           "Number of output channel needs to be divisible by group. Output channel: %d, group: %d.", g.Ko, g.group);
  NB_CHECK(g.sh > 0 && g.sw > 0 && g.dh > 0 && g.dw > 0 && g.ph >= 0 && g.pw >= 0, NB200_EVALUE,
           "stride and dilation must be positive, pad non-negative");
  g.Cg = g.C / g.group;
  g.Kog = g.Ko / g.group;
  g.Ho = (g.H + 2 * g.ph - (g.dh * (g.kh - 1) + 1)) / g.sh + 1;
  g.Wo = (g.W + 2 * g.pw - (g.dw * (g.kw - 1) + 1)) / g.sw + 1;
  NB_CHECK((g.H + 2 * g.ph - (g.dh * (g.kh - 1) + 1)) >= 0 && (g.W + 2 * g.pw - (g.dw * (g.kw - 1) + 1)) >= 0 &&
               g.Ho > 0 && g.Wo > 0,
           NB200_EVALUE, "Invalid configuration of convolution: {input:%dx%d, kernel:%dx%d, pad:%dx%d, stride:%dx%d, "
                         "dilation:%dx%d}.",
           g.H, g.W, g.kh, g.kw, g.ph, g.pw, g.sh, g.sw, g.dh, g.dw);
  return NB200_OK;
}

// Picks the pixel box: whole output rows, h_box rows of n_box images, at most
// `bn_max` pixels. Several images share a box only when a whole image fits.
void plan_box(const ConvGeometry &g, int bn_max, int &h_box, int &n_box) {
  const int per_img = g.Ho * g.Wo;
  if (per_img <= bn_max) {
    h_box = g.Ho;
    n_box = bn_max / per_img;
    if (n_box > g.N)
      n_box = g.N;
    return;
  }
  n_box = 1;
  int best = bn_max / g.Wo;
  if (best < 1)
    best = 1;
  // Prefer a divisor of Ho (no ragged last box) unless it wastes over a third of the box.
  for (int h = best; h >= 1; --h)
    if (g.Ho % h == 0) {
      if (3 * h >= 2 * best)
        best = h;
      break;
    }
  h_box = best;
}

template <bool kInt8, int PA, int PB, int BN, int STAGES, int RB = kRowBytes, int kSkip = 0,
          bool kResidentA = false>
int launch_conv(const ConvGeometry &g, const void *act, int planes_b, int64_t ctot, const void *wside, int64_t wpitch,
                int c_pad_g, int cblocks, int h_box, int n_box, const GemmEpilogue &ep, cudaStream_t st,
                int k_splits = 1, int64_t split_stride = 0) {
  const int es = kInt8 ? 1 : 2;
  const int E = RB / es;
  CUtensorMap ma, mb;
  // weights: (K, Ko, planes)
  NB_TRY(make_operand_map(&ma, wside, kInt8, wpitch, wpitch, g.Ko, PA, kTileM, RB));
  // activations: (C, W, H, N, planes); the box walks W and H with the convolution stride
  const uint64_t dims[5] = {(uint64_t)ctot, (uint64_t)g.W, (uint64_t)g.H, (uint64_t)g.N, (uint64_t)planes_b};
  const uint64_t strides[4] = {(uint64_t)ctot * es, (uint64_t)ctot * es * g.W, (uint64_t)ctot * es * g.W * g.H,
                               (uint64_t)ctot * es * g.W * g.H * g.N};
  const uint32_t box[5] = {(uint32_t)E, (uint32_t)(g.Wo * g.sw), (uint32_t)(h_box * g.sh), (uint32_t)n_box, 1};
  const uint32_t estr[5] = {1, (uint32_t)g.sw, (uint32_t)g.sh, 1, 1};
  NB_TRY(encode_tiled(&mb, kInt8 ? 1 : 0, 5, act, dims, strides, box, estr, RB));
  ConvProblem p;
  p.row_bytes = RB;
  p.chunk_blocks = kInt8 ? 0 : k_chunk_blocks((kSkip == 1 ? 6 : PA * PB) * (RB / 32));
  p.Nimg = g.N;
  p.Ko = g.Ko;
  p.Kog = g.Kog;
  p.groups = g.group;
  p.Ho = g.Ho;
  p.Wo = g.Wo;
  p.h_box = h_box;
  p.n_box = n_box;
  p.tiles_h = (g.Ho + h_box - 1) / h_box;
  p.tiles_n = (g.N + n_box - 1) / n_box;
  p.m_tiles_g = (g.Kog + kTileM - 1) / kTileM;
  p.kw = g.kw;
  p.taps = g.kh * g.kw;
  p.cblocks = cblocks;
  p.sh = g.sh;
  p.sw = g.sw;
  p.ph = g.ph;
  p.pw = g.pw;
  p.dh = g.dh;
  p.dw = g.dw;
  p.c_group_stride = c_pad_g;
  p.pixels = n_box * h_box * g.Wo;
  p.n_run = (int)round_up(p.pixels, 16);
  p.k_splits = k_splits;
  p.split_stride = split_stride;
  const int tiles = k_splits * p.groups * p.m_tiles_g * p.tiles_h * p.tiles_n;
  return launch_contraction<kInt8, PA, PB, BN, STAGES, kSkip, ConvProblem, RB, kResidentA>(ma, mb, p, tiles, ep, st,
                                                                                            p.taps * p.cblocks);
}

// Shared body of BinaryWeightConvolution / BinaryConnectConvolution forward.
// weight_delta > 0: w itself holds multiples of weight_delta (a fixed-point convolution of two
// 8-bit operands: no binarisation, wb / alpha unused, int8 path only).
// x_codes != NULL: the activations arrive as int8 channel-last codes in the layout below
// (x unused, act_delta > 0 required) and the re-layout pass is skipped.
int binary_convolution(const float *x, const float *w, float *wb, float *alpha, const float *bias, float *y,
                       ConvGeometry g, float zero_to, float act_delta, cudaStream_t st, float weight_delta = 0.0f,
                       const int8_t *x_codes = nullptr, const int8_t *prepared_side = nullptr) {
  // prepared_side != NULL: the weights' int8 side-band (and alpha) were made once by
  // nb200_binary_weights_prepare_i8; w / wb are unused and nothing is binarised here.
  NB_TRY(check_geometry(g));
  const bool fxp_weights = weight_delta > 0.0f;
  NB_CHECK((x || x_codes) && (w || prepared_side) && (wb || fxp_weights || prepared_side) && y, NB200_EVALUE,
           "null data pointer");
  NB_CHECK(!prepared_side || (act_delta > 0.0f && !fxp_weights), NB200_EVALUE,
           "prepared weights are for the int8 path (activation_delta > 0)");
  const bool int8 = act_delta > 0.0f;
  NB_CHECK(int8 || !x_codes, NB200_EVALUE, "activation codes need their step (activation_delta > 0)");
  NB_CHECK(int8 || !fxp_weights, NB200_EVALUE, "fixed-point weights need fixed-point activations");
  if (fxp_weights) {
    // |acc| <= taps * Cg * 127 * 127 must fit int32
    NB_CHECK((int64_t)g.Cg * g.kh * g.kw <= 133000, NB200_ENOTIMPL, "the int32 accumulator could overflow");
  } else if (int8)
    NB_CHECK(zero_to == 1.0f || zero_to == -1.0f || zero_to == 0.0f, NB200_ENOTIMPL,
             "the int8 path needs quantize_zero_to in {-1, 0, 1} (got %g)", zero_to);
  else
    NB_CHECK(bf16_exact(zero_to), NB200_ENOTIMPL,
             "quantize_zero_to = %g is not representable in bf16; the exact tensor-core path needs it to be", zero_to);
  NB_CHECK(g.Wo * g.sw <= 256 && g.Wo <= 256, NB200_ENOTIMPL,
           "output rows wider than 256 pixels (Wo=%d, stride %d) are not supported", g.Wo, g.sw);
  const int es = int8 ? 1 : 2;
  const int c_pad_g = (int)round_up(g.Cg, 16);
  // One K block is one filter tap over E channel slots. With few channels per
  // group a 128-byte row would be half zero padding: use 64-byte rows then.
  const bool narrow_rows = c_pad_g * es <= 64;
  const int E = (narrow_rows ? 64 : kRowBytes) / es;
  const int cblocks = (c_pad_g + E - 1) / E;
  const int c_slots = cblocks * E;
  int64_t ctot = (int64_t)g.group * c_pad_g;
  if (ctot < E)
    ctot = E;
  NB_CHECK(!int8 || ctot == codes_slots(g.C, g.group), NB200_EVALUE, "activation code layout mismatch");
  const int taps = g.kh * g.kw;
  const int64_t wpitch = (int64_t)taps * c_slots;
  // fp32 activations against +-1 weights: two fp16 pieces of the activations scaled by a power of two
  // (x * 2^-e = p0 + p1), two thirds of the operand rows and MMAs of the exact three-piece bf16 split;
  // the bf16 form stays for a quantize_zero_to other than -1, 0, 1
  const bool half_pair = !int8 && (zero_to == 1.0f || zero_to == -1.0f || zero_to == 0.0f);
  const int planes = int8 ? 1 : (half_pair ? 2 : 3);
  const size_t act_bytes = x_codes ? 0 : (size_t)planes * g.N * g.H * g.W * ctot * es;
  const size_t side_bytes = prepared_side ? 0 : (size_t)g.Ko * wpitch * es;
  const size_t extra_bytes = half_pair ? round_up((size_t)g.Ko * 4 + 16, 1024) : 0;
  AsyncScratch scratch(st);
  NB_TRY(scratch.alloc(round_up(act_bytes, 1024) + round_up(side_bytes, 1024) + extra_bytes));
  const uint8_t *act = x_codes ? reinterpret_cast<const uint8_t *>(x_codes) : static_cast<uint8_t *>(scratch.p);
  uint8_t *side = prepared_side ? const_cast<uint8_t *>(reinterpret_cast<const uint8_t *>(prepared_side))
                                : static_cast<uint8_t *>(scratch.p) + round_up(act_bytes, 1024);
  NB_CHECK(((reinterpret_cast<uintptr_t>(act) | reinterpret_cast<uintptr_t>(side)) & 15) == 0, NB200_EVALUE,
           "activation codes and prepared weights must be 16-byte aligned");
  bool operands_done = false;
  if (!prepared_side) {
    if (c_slots != g.Cg)
      NB_CUDA(cudaMemsetAsync(side, 0, side_bytes, st));
    if (fxp_weights)
      NB_TRY(codes_conv_weights(w, g.Ko, g.Cg, g.kh, g.kw, weight_delta, side, wpitch, c_slots, st));
    else if (int8 && !x_codes && binary_conv_operands_i8_applies(x, g.N, g.H * g.W, (int)ctot, g.Ko)) {
      // weights and activations in one launch
      NB_TRY(binary_conv_operands_i8(w, g.Ko, g.Cg, g.kh, g.kw, zero_to, wb, alpha, side, wpitch, c_slots, x, g.N, g.C,
                                     g.H * g.W, g.group, c_pad_g, (int)ctot, act_delta, scratch.p, st));
      operands_done = true;
    } else
      NB_TRY(binarize_rows(w, g.Ko, g.Cg, g.kh, g.kw, zero_to, wb, alpha, side, wpitch, c_slots, int8, st, half_pair));
  }
  float *row_scale_half = nullptr;
  if (half_pair) {
    uint8_t *extra = static_cast<uint8_t *>(scratch.p) + round_up(act_bytes, 1024) + round_up(side_bytes, 1024);
    row_scale_half = reinterpret_cast<float *>(extra + 16);
    NB_TRY(nchw_to_nhwc_half_pair(x, g.N, g.C, g.H * g.W, g.group, g.Cg, c_pad_g, (int)ctot, scratch.p,
                                  reinterpret_cast<uint32_t *>(extra), alpha, g.Ko, row_scale_half, st));
  } else if (!x_codes && !operands_done)
    NB_TRY(nchw_to_nhwc_planes(x, g.N, g.C, g.H * g.W, g.group, g.Cg, c_pad_g, (int)ctot, int8 ? 0 : 3, act_delta,
                               static_cast<uint8_t *>(scratch.p), st));
  GemmEpilogue ep{};
  ep.y = y;
  ep.scale = fxp_weights ? act_delta * weight_delta : (int8 ? act_delta : 1.0f);
  ep.row_scale = fxp_weights ? nullptr : (half_pair ? row_scale_half : alpha);
  ep.row_bias = bias;
  // Box selection: prefer the 128-column kernel (deeper pipeline) unless the
  // 256-column box is better filled.
  int h128, n128, h256, n256;
  plan_box(g, 128, h128, n128);
  plan_box(g, 256, h256, n256);
  const int px128 = h128 * n128 * g.Wo, px256 = h256 * n256 * g.Wo;
  const double fill128 = (double)px128 / (double)round_up(px128, 16) * px128 / 128.0;
  const double fill256 = (double)px256 / (double)round_up(px256, 16) * px256 / 256.0;
  const bool can128 = px128 <= 128;
  const bool use256 = !can128 || (int8 && fill256 > fill128 + 0.05);
  if (int8 && pixel_major_applies(g)) {
    // pixels on the MMA rows: same accumulators, same rounded operations in the epilogue, faster loads and stores
    return convolution_codes_folded(reinterpret_cast<const int8_t *>(act), reinterpret_cast<const int8_t *>(side),
                                    fxp_weights ? nullptr : alpha, bias, nullptr, 0.0f, nullptr, nullptr, nullptr, g, 0,
                                    1, 8, 1.0f, st, y, ep.scale);
  }
  if (int8) {
    // All tiles share the weights when the output maps fit one M tile: keep them in shared
    // memory for the whole launch if their K blocks fit beside the ring (64-byte rows only:
    // there the copy engine's request rate, one request per row, bounds the kernel).
    const bool resident = narrow_rows && g.group == 1 && g.Ko <= kTileM &&
                          (size_t)taps * cblocks * kTileM * 64 <= 72 * 1024;
    if (resident) {
      if (use256)
        return launch_conv<true, 1, 1, 256, 6, 64, false, true>(g, act, 1, ctot, side, wpitch, c_pad_g, cblocks, h256,
                                                                n256, ep, st);
      return launch_conv<true, 1, 1, 128, 10, 64, false, true>(g, act, 1, ctot, side, wpitch, c_pad_g, cblocks, h128,
                                                               n128, ep, st);
    }
    if (narrow_rows) {
      if (use256)
        return launch_conv<true, 1, 1, 256, 8, 64>(g, act, 1, ctot, side, wpitch, c_pad_g, cblocks, h256, n256, ep,
                                                   st);
      return launch_conv<true, 1, 1, 128, 10, 64>(g, act, 1, ctot, side, wpitch, c_pad_g, cblocks, h128, n128, ep, st);
    }
    if (use256)
      return launch_conv<true, 1, 1, 256, 4>(g, act, 1, ctot, side, wpitch, c_pad_g, cblocks, h256, n256, ep, st);
    return launch_conv<true, 1, 1, 128, 6>(g, act, 1, ctot, side, wpitch, c_pad_g, cblocks, h128, n128, ep, st);
  }
  NB_CHECK(can128, NB200_ENOTIMPL,
           "fp32-activation convolution with output rows wider than 128 pixels (Wo=%d) is not supported", g.Wo);
  if (half_pair) {
    if (narrow_rows)
      return launch_conv<false, 1, 2, 128, 8, 64, 2>(g, act, 2, ctot, side, wpitch, c_pad_g, cblocks, h128, n128, ep,
                                                     st);
    return launch_conv<false, 1, 2, 128, 4, kRowBytes, 2>(g, act, 2, ctot, side, wpitch, c_pad_g, cblocks, h128, n128,
                                                          ep, st);
  }
  if (narrow_rows)
    return launch_conv<false, 1, 3, 128, 6, 64>(g, act, 3, ctot, side, wpitch, c_pad_g, cblocks, h128, n128, ep, st);
  return launch_conv<false, 1, 3, 128, 3>(g, act, 3, ctot, side, wpitch, c_pad_g, cblocks, h128, n128, ep, st);
}

// ---------------------------------------------------------------------------
// Backward (Convolution::backward_impl, src/nbla/function/generic/convolution.cpp:199-300,
// called by the binary convolutions with their binarised weights,
// binary_weight_convolution.cpp:119-146, binary_connect_convolution.cpp:82-104).
// Both gradients run on the forward's implicit-GEMM kernel:
//
//  dx = convolution of dy (each map scaled by alpha, pixels spread by the
//       forward stride over a zeroed grid) with the flipped, transposed +-1
//       weights: stride 1, same dilation, padding d * (k - 1) - p.
//  dW[o, c, ky, kx] = sum over (n, oy, ox) of dy[n, o, oy, ox] * x[n, c, oy*s - p + ky*d, ox*s - p + kx*d]
//       = a convolution whose "images" are the input channels, whose channel
//       axis is the batch, whose filter is dy^T (kernel size Ho x Wo) and whose
//       stride / dilation are the forward's dilation / stride; its Ho' x Wo'
//       output is the kh x kw filter window. One launch per group.
//  db = sums of dy over batch and pixels.
// ---------------------------------------------------------------------------
// full_precision: the weights are arbitrary fp32 values (three bf16 pieces, the products that matter at fp32
// resolution) instead of values exact in one bf16 piece
int conv_input_grad(const float *wb, const float *alpha, const float *dy, float *dx, const ConvGeometry &g,
                    int accum, cudaStream_t st, bool full_precision = false) {
  // geometry of the equivalent forward convolution
  ConvGeometry b = g;
  b.C = g.Ko;
  b.Ko = g.C;
  b.Cg = g.Kog;
  b.Kog = g.Cg;
  b.H = g.H + 2 * g.ph - g.dh * (g.kh - 1); // stuffed dy grid, padded so that the output is exactly H x W
  b.W = g.W + 2 * g.pw - g.dw * (g.kw - 1);
  b.sh = b.sw = 1;
  b.ph = g.dh * (g.kh - 1) - g.ph;
  b.pw = g.dw * (g.kw - 1) - g.pw;
  b.Ho = g.H;
  b.Wo = g.W;
  NB_CHECK(b.Wo <= 128, NB200_ENOTIMPL, "input gradient for images wider than 128 pixels (W=%d) is not supported",
           b.Wo);
  const int k_pad_g = (int)round_up(b.Cg, 16);
  const bool narrow_rows = !full_precision && k_pad_g * 2 <= 64; // the three-piece kernel has 128-byte rows only
  const int E = (narrow_rows ? 64 : kRowBytes) / 2;
  const int cblocks = (k_pad_g + E - 1) / E;
  const int k_slots = cblocks * E;
  int64_t ctot = (int64_t)g.group * k_pad_g;
  if (ctot < E)
    ctot = E;
  const int taps = g.kh * g.kw;
  const int64_t wpitch = (int64_t)taps * k_slots;
  const size_t act_bytes = (size_t)3 * g.N * b.H * b.W * ctot * 2;
  const size_t side_bytes = (size_t)(full_precision ? 3 : 1) * g.C * wpitch * 2;
  AsyncScratch scratch(st);
  NB_TRY(scratch.alloc(round_up(act_bytes, 1024) + round_up(side_bytes, 1024)));
  uint8_t *act = static_cast<uint8_t *>(scratch.p);
  uint8_t *side = act + round_up(act_bytes, 1024);
  NB_CUDA(cudaMemsetAsync(act, 0, round_up(act_bytes, 1024) + side_bytes, st));
  NB_TRY(dy_to_nhwc_stuffed(dy, g.N, g.Ko, g.Ho, g.Wo, g.group, g.Kog, k_pad_g, (int)ctot, b.H, b.W, g.sh, g.sw, alpha,
                            act, st));
  NB_TRY(flip_transpose_weights(wb, g.Ko, g.Cg, g.kh, g.kw, g.group, k_slots, side, st, full_precision ? 3 : 1));
  GemmEpilogue ep{};
  ep.y = dx;
  ep.scale = 1.0f;
  ep.accumulate = accum;
  int h_box, n_box;
  if (full_precision) {
    plan_box(b, 64, h_box, n_box);
    return launch_conv<false, 3, 3, 64, 2, kRowBytes, 1>(b, act, 3, ctot, side, wpitch, k_pad_g, cblocks, h_box, n_box,
                                                         ep, st);
  }
  plan_box(b, 128, h_box, n_box);
  if (narrow_rows)
    return launch_conv<false, 1, 3, 128, 6, 64>(b, act, 3, ctot, side, wpitch, k_pad_g, cblocks, h_box, n_box, ep, st);
  return launch_conv<false, 1, 3, 128, 3>(b, act, 3, ctot, side, wpitch, k_pad_g, cblocks, h_box, n_box, ep, st);
}

int conv_weight_grad(const float *x, const float *dy, float *dw, const ConvGeometry &g, int accum, float act_delta,
                     cudaStream_t st) {
  NB_CHECK(g.kw * g.dw <= 256 && g.kh * g.kw <= 64, NB200_ENOTIMPL,
           "weight gradient for a %d x %d filter (dilation %d) is not supported", g.kh, g.kw, g.dw);
  NB_CHECK((int64_t)g.Ho * g.Wo <= (1 << 20), NB200_ENOTIMPL, "output maps larger than 2^20 pixels");
  // activations that are multiples of act_delta with |code| <= 127 are exact in one bf16 piece
  const int planes_x = act_delta > 0.0f ? 1 : 3;
  const int E = kRowBytes / 2;
  const int Np = (int)round_up(g.N, E);
  const int cblocks = Np / E;
  const int taps_f = g.Ho * g.Wo;          // filter taps of the equivalent convolution
  const int taps_w = g.kh * g.kw;          // its output pixels per image
  const int64_t wpitch = (int64_t)taps_f * Np;
  const int64_t Rx = (int64_t)g.Cg * g.H * g.W, Rdy = (int64_t)g.Kog * taps_f;
  const size_t x_bytes = round_up((size_t)planes_x * Rx * Np * 2, 1024);
  const size_t dy_bytes = round_up((size_t)3 * Rdy * Np * 2, 1024);
  ConvGeometry b = g;
  b.N = g.Cg;   // images = input channels of the group
  b.C = g.N;    // channel axis = batch
  b.Cg = g.N;
  b.Ko = g.Kog; // output maps = maps of the group
  b.Kog = g.Kog;
  b.group = 1;
  b.kh = g.Ho;
  b.kw = g.Wo;
  b.sh = g.dh;
  b.sw = g.dw;
  b.dh = g.sh;
  b.dw = g.sw;
  b.Ho = g.kh;
  b.Wo = g.kw;
  int h_box, n_box;
  plan_box(b, 64, h_box, n_box);
  // The output is small and K (batch x output pixels) is long: cut K over the SMs that the
  // output tiles alone would leave idle; each split writes its own staged result.
  const int base_tiles = ((g.Kog + kTileM - 1) / kTileM) * ((g.Cg + n_box - 1) / n_box) * ((b.Ho + h_box - 1) / h_box);
  const int kb_all = taps_f * cblocks;
  int k_splits = sm_count() / base_tiles;
  k_splits = k_splits > 32 ? 32 : k_splits;
  k_splits = k_splits > kb_all / 8 ? kb_all / 8 : k_splits;
  k_splits = k_splits < 1 ? 1 : k_splits;
  {
    const int per = (kb_all + k_splits - 1) / k_splits;
    k_splits = (kb_all + per - 1) / per; // no empty split
  }
  const int64_t split_stride = (int64_t)g.Cg * g.Kog * taps_w;
  const size_t out_bytes = round_up((size_t)k_splits * split_stride * 4, 1024);
  AsyncScratch scratch(st);
  NB_TRY(scratch.alloc(x_bytes + dy_bytes + out_bytes));
  uint8_t *xt = static_cast<uint8_t *>(scratch.p);
  uint8_t *dyt = xt + x_bytes;
  float *staged = reinterpret_cast<float *>(dyt + dy_bytes);
  for (int grp = 0; grp < g.group; ++grp) {
    if (g.N != Np)
      NB_CUDA(cudaMemsetAsync(xt, 0, x_bytes + dy_bytes, st));
    NB_TRY(batch_to_inner(x + (int64_t)grp * Rx, g.N, Rx, (int64_t)g.C * g.H * g.W, Np, planes_x, xt, st));
    NB_TRY(batch_to_inner(dy + (int64_t)grp * Rdy, g.N, Rdy, (int64_t)g.Ko * taps_f, Np, 3, dyt, st));
    GemmEpilogue ep{};
    ep.y = staged;
    ep.scale = 1.0f;
    if (planes_x == 3)
      NB_TRY((launch_conv<false, 3, 3, 64, 2, kRowBytes, true>(b, xt, 3, Np, dyt, wpitch, Np, cblocks, h_box, n_box, ep,
                                                               st, k_splits, split_stride)));
    else
      NB_TRY((launch_conv<false, 3, 1, 64, 3>(b, xt, 1, Np, dyt, wpitch, Np, cblocks, h_box, n_box, ep, st, k_splits,
                                              split_stride)));
    NB_TRY(permute_weight_grad(staged, k_splits, g.Cg, g.Kog, taps_w, dw + (int64_t)grp * g.Kog * g.Cg * taps_w, accum,
                               st));
  }
  return NB200_OK;
}

int convolution_backward(const float *x, const float *w_exact, const float *alpha, const float *dy, float *dx,
                         float *dw, float *db, ConvGeometry g, int accum_dx, int accum_dw, int accum_db,
                         float act_delta, cudaStream_t st, bool full_precision_weights = false) {
  NB_TRY(check_geometry(g));
  NB_CHECK(dy != nullptr, NB200_EVALUE, "dy is NULL");
  if (dx) {
    NB_CHECK(w_exact != nullptr, NB200_EVALUE, "the gradient w.r.t. x needs the weights");
    NB_TRY(conv_input_grad(w_exact, alpha, dy, dx, g, accum_dx, st, full_precision_weights));
  }
  if (dw) {
    NB_CHECK(x != nullptr, NB200_EVALUE, "the gradient w.r.t. the weights needs x");
    NB_TRY(conv_weight_grad(x, dy, dw, g, accum_dw, act_delta, st));
  }
  if (db) {
    int splits = g.N < 32 ? g.N : 32;
    AsyncScratch scratch(st);
    NB_TRY(scratch.alloc((size_t)splits * g.Ko * 4));
    NB_TRY(channel_sums(dy, g.N, g.Ko, g.Ho * g.Wo, db, accum_db, static_cast<float *>(scratch.p), splits, st));
  }
  return NB200_OK;
}

} // namespace
} // namespace nb200

using namespace nb200;

extern "C" {

int nb200_binary_weight_convolution_f32(const float *x, const float *w, float *wb, float *alpha, const float *bias,
                                        float *y, int batch, int channels, int height, int width, int outmaps,
                                        int kernel_h, int kernel_w, int pad_h, int pad_w, int stride_h, int stride_w,
                                        int dilation_h, int dilation_w, int group, float quantize_zero_to,
                                        float activation_delta, void *stream) {
  NB_CHECK(alpha != nullptr, NB200_EVALUE, "alpha is NULL");
  ConvGeometry g{batch, channels, height, width, outmaps, kernel_h, kernel_w, pad_h, pad_w, stride_h, stride_w,
                 dilation_h, dilation_w, group, 0, 0, 0, 0};
  return binary_convolution(x, w, wb, alpha, bias, y, g, quantize_zero_to, activation_delta, as_stream(stream));
}

int nb200_binary_connect_convolution_f32(const float *x, const float *w, float *wb, const float *bias, float *y,
                                         int batch, int channels, int height, int width, int outmaps, int kernel_h,
                                         int kernel_w, int pad_h, int pad_w, int stride_h, int stride_w,
                                         int dilation_h, int dilation_w, int group, float quantize_zero_to,
                                         float activation_delta, void *stream) {
  ConvGeometry g{batch, channels, height, width, outmaps, kernel_h, kernel_w, pad_h, pad_w, stride_h, stride_w,
                 dilation_h, dilation_w, group, 0, 0, 0, 0};
  return binary_convolution(x, w, wb, nullptr, bias, y, g, quantize_zero_to, activation_delta, as_stream(stream));
}

int64_t nb200_codes_nhwc_slots(int64_t channels, int group) {
  if (channels <= 0 || group <= 0 || channels % group != 0)
    return 0;
  return codes_slots(channels, group);
}

int nb200_fixed_point_codes_nhwc(const float *xq, int8_t *codes, int64_t batch, int64_t channels, int64_t inner,
                                 int group, float delta, void *stream) {
  NB_CHECK(batch >= 0 && channels > 0 && inner > 0 && group > 0 && channels % group == 0, NB200_EVALUE, "bad extents");
  NB_CHECK(delta > 0.f, NB200_EVALUE, "delta should be positive");
  NB_CHECK(channels < (1 << 30) && inner < (1 << 30), NB200_EVALUE, "extent exceeds 2^30");
  if (batch == 0)
    return NB200_OK;
  NB_CHECK(xq && codes, NB200_EVALUE, "null data pointer");
  const int Cg = (int)(channels / group);
  return nchw_to_nhwc_planes(xq, (int)batch, (int)channels, (int)inner, group, Cg, (Cg + 15) / 16 * 16,
                             (int)codes_slots(channels, group), 0, delta, codes, as_stream(stream));
}

int nb200_binary_convolution_codes_f32(const int8_t *x_codes, const float *w, float *wb, float *alpha,
                                       const float *bias, float *y, int batch, int channels, int height, int width,
                                       int outmaps, int kernel_h, int kernel_w, int pad_h, int pad_w, int stride_h,
                                       int stride_w, int dilation_h, int dilation_w, int group,
                                       float quantize_zero_to, float activation_delta, void *stream) {
  NB_CHECK(x_codes != nullptr, NB200_EVALUE, "x_codes is NULL");
  NB_CHECK(activation_delta > 0.f, NB200_EVALUE, "activation_delta should be positive");
  ConvGeometry g{batch, channels, height, width, outmaps, kernel_h, kernel_w, pad_h, pad_w, stride_h, stride_w,
                 dilation_h, dilation_w, group, 0, 0, 0, 0};
  return binary_convolution(nullptr, w, wb, alpha, bias, y, g, quantize_zero_to, activation_delta, as_stream(stream),
                            0.0f, x_codes);
}

} // extern "C" (reopened below)
namespace nb200 {
namespace {
// slots per filter tap and row pitch of the int8 weight side-band [outmaps][taps * c_slots]
void int8_side_layout(int Cg, int taps, int &c_slots, int64_t &wpitch) {
  const int c_pad_g = (int)round_up(Cg, 16);
  const int E = c_pad_g <= 64 ? 64 : kRowBytes;
  c_slots = (c_pad_g + E - 1) / E * E;
  wpitch = (int64_t)taps * c_slots;
}

// ---------------------------------------------------------------------------
// Convolution of activation codes with the layer's inference tail in the
// epilogue (conv_codes.cuh): pixels on the MMA rows, channel-last codes out.
// ---------------------------------------------------------------------------
#ifdef NB200_CC_TRACE
long long *g_cc_trace = nullptr;
#endif

template <int BN, int STAGES, int RB, bool kResidentB = false, bool kHalo = false>
int launch_conv_codes(const ConvGeometry &g, const int8_t *x_codes, int64_t ctot, const int8_t *side, int64_t wpitch,
                      int cblocks, int h_box, int n_box, int slots_out, const ConvCodesEpilogue &ep, cudaStream_t st) {
  CUtensorMap mx, mw;
  // activations: (C, W, H, N, 1); the box walks W and H with the convolution stride
  const uint64_t dims[5] = {(uint64_t)ctot, (uint64_t)g.W, (uint64_t)g.H, (uint64_t)g.N, 1};
  const uint64_t strides[4] = {(uint64_t)ctot, (uint64_t)ctot * g.W, (uint64_t)ctot * g.W * g.H,
                               (uint64_t)ctot * g.W * g.H * g.N};
  const int wp = g.Wo + (g.kw - 1) * g.dw, hp = h_box + (g.kh - 1) * g.dh;
  if (kHalo) {
    // one box of hp x wp input pixels per tile and channel block
    const uint32_t hbox[5] = {(uint32_t)RB, (uint32_t)wp, (uint32_t)hp, 1, 1};
    NB_TRY(encode_tiled(&mx, 1, 5, x_codes, dims, strides, hbox, nullptr, RB));
  } else {
    const uint32_t box[5] = {(uint32_t)RB, (uint32_t)(g.Wo * g.sw), (uint32_t)(h_box * g.sh), (uint32_t)n_box, 1};
    const uint32_t estr[5] = {1, (uint32_t)g.sw, (uint32_t)g.sh, 1, 1};
    NB_TRY(encode_tiled(&mx, 1, 5, x_codes, dims, strides, box, estr, RB));
  }
  // weights: (K, Ko, 1), BN maps per box
  NB_TRY(make_operand_map(&mw, side, true, wpitch, wpitch, g.Ko, 1, BN, RB));
  ConvCodesProblem p;
  p.Nimg = g.N;
  p.Ko = g.Ko;
  p.Ho = g.Ho;
  p.Wo = g.Wo;
  p.h_box = h_box;
  p.n_box = n_box;
  p.tiles_h = (g.Ho + h_box - 1) / h_box;
  p.tiles_n = (g.N + n_box - 1) / n_box;
  p.n_tiles = (g.Ko + BN - 1) / BN;
  p.bn = BN;
  p.kw = g.kw;
  p.taps = g.kh * g.kw;
  p.cblocks = cblocks;
  p.sh = g.sh;
  p.sw = g.sw;
  p.ph = g.ph;
  p.pw = g.pw;
  p.dh = g.dh;
  p.dw = g.dw;
  p.pixels = n_box * h_box * g.Wo;
  p.slots_out = slots_out;
  p.wp = wp;
  p.hp = hp;
  // rows a shifted descriptor may read: the largest tap shift plus the 128 rows of the MMA, in whole
  // swizzle patterns of 8 rows (rows the box does not write hold stale data that no stored pixel uses)
  const int rows_alloc = (((g.kh - 1) * g.dh * wp + (g.kw - 1) * g.dw + kTileM) + 7) / 8 * 8;
  p.a_tile_bytes = (rows_alloc > hp * wp ? rows_alloc : (hp * wp + 7) / 8 * 8) * RB;
  auto kernel = conv_codes_tcgen05_kernel<BN, STAGES, RB, kResidentB, kHalo>;
  constexpr size_t smem_fixed = conv_codes_smem_bytes<BN, STAGES, RB, kResidentB, kHalo>();
  static_assert(smem_fixed <= 227 * 1024, "shared memory budget");
  const size_t smem = smem_fixed + (kResidentB ? (size_t)p.taps * p.cblocks * BN * RB : 0) +
                      (kHalo ? (size_t)2 * p.cblocks * p.a_tile_bytes : 0);
  NB_CHECK(smem <= 227 * 1024, NB200_EVALUE, "resident weights do not fit in shared memory");
  static bool configured[64];
  int dev = 0;
  NB_CUDA(cudaGetDevice(&dev));
  if (!configured[dev & 63]) {
    NB_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 kResidentB ? 227 * 1024 : (int)smem));
    configured[dev & 63] = true;
  }
  int *status = nullptr;
  NB_TRY(device_status_word(&status));
  const int tiles = p.n_tiles * p.tiles_h * p.tiles_n;
  const int grid = tiles < sm_count() ? tiles : sm_count();
  kernel<<<grid, kGemmThreads, smem, st>>>(mx, mw, p, ep, status);
  NB_LAUNCH_CHECK();
  return NB200_OK;
}

// Whether a convolution can run on the pixel-major kernel (group 1, at most kCodesMaxMaps maps, output rows
// of at most 128 pixels).
bool pixel_major_applies(const ConvGeometry &g) {
  return g.group == 1 && g.Ko <= kCodesMaxMaps && g.Wo * g.sw <= 256 && g.Wo <= 128;
}

// y_nchw != NULL: plain fp32 [batch][maps][pixels] result, acc * scale[o] (+ bias[o]) with each operation
// rounded on its own (what the unfused functions return); no residual, ReLU or quantizer then.
int convolution_codes_folded(const int8_t *x_codes, const int8_t *side, const float *scale, const float *bias,
                             const int8_t *res_codes, float res_delta, const float *res_f32, int8_t *y_codes,
                             float *y_f32, ConvGeometry g, int relu, int sign, int n, float delta, cudaStream_t st,
                             float *y_nchw, float nchw_scale) {
  NB_TRY(check_geometry(g));
  NB_CHECK(g.group == 1, NB200_ENOTIMPL, "grouped convolutions are not supported by the folded code path");
  NB_CHECK(x_codes && side && (scale || y_nchw) && (y_codes || y_f32 || y_nchw), NB200_EVALUE, "null data pointer");
  NB_CHECK(!(y_codes && y_f32), NB200_EVALUE, "the result is either codes or fp32, not both");
  NB_CHECK(!y_nchw || !(y_codes || y_f32 || res_codes || res_f32), NB200_EVALUE,
           "the plain fp32 result takes no residual and no second result");
  NB_CHECK(!(res_codes && res_f32), NB200_EVALUE, "the residual is either codes or fp32, not both");
  NB_CHECK(res_codes == nullptr || res_delta > 0.f, NB200_EVALUE, "res_delta should be positive");
  NB_CHECK(g.Ko <= kCodesMaxMaps, NB200_ENOTIMPL, "more than %d output maps", kCodesMaxMaps);
  NB_CHECK(g.Wo * g.sw <= 256 && g.Wo <= 128, NB200_ENOTIMPL,
           "output rows wider than 128 pixels (Wo=%d, stride %d) are not supported", g.Wo, g.sw);
  ConvCodesEpilogue ep{};
  ep.scale = scale;
  ep.bias = bias;
  ep.res_codes = res_codes;
  ep.res_f32 = res_f32;
  ep.y_codes = y_codes;
  ep.y_f32 = y_codes ? nullptr : y_f32;
  ep.y_nchw = y_nchw;
  ep.has_bias = bias != nullptr;
  ep.relu = relu;
  ep.out_scale = 1.0f;
  ep.kmax = ep.kmin = 0;
  if (y_codes) {
    // the quantizer's setup (fixed_point_quantize.cpp:31-42); the step must be a power of two
    NB_CHECK(n > 0 && delta > 0.f, NB200_EVALUE, "Both bit width and delta should be positive.");
    const int nn = sign ? n - 1 : n;
    NB_CHECK(nn > 0 && nn <= 7, NB200_ENOTIMPL, "codes need 0 < n - sign <= 7 (they are stored as int8)");
    int ex = 0;
    NB_CHECK(std::frexp(delta, &ex) == 0.5f && ex > -100 && ex < 100, NB200_ENOTIMPL,
             "the folded code path needs a power-of-two quantizer step (got %g)", delta);
    NB_CHECK(relu || sign, NB200_ENOTIMPL, "an unsigned quantizer without ReLU is not supported");
    ep.out_scale = 2.0f / delta;
    ep.kmax = (1 << nn) - 1;
    ep.kmin = sign ? -ep.kmax : 0;
  }
  ep.bias_scale = ep.out_scale;
  ep.res_scale = (res_codes ? res_delta : 1.0f) * ep.out_scale;
  if (y_nchw) {
    ep.out_scale = nchw_scale; // the step of the activation codes (times the weights' step for fixed-point weights)
    ep.bias_scale = 1.0f;
  }
#ifdef NB200_CC_TRACE
  ep.trace = g_cc_trace;
#endif
  const int64_t slots_out = codes_slots(g.Ko, 1);
  NB_CHECK((((reinterpret_cast<uintptr_t>(x_codes) | reinterpret_cast<uintptr_t>(side) |
              reinterpret_cast<uintptr_t>(res_codes) | reinterpret_cast<uintptr_t>(res_f32) |
              reinterpret_cast<uintptr_t>(y_codes) | reinterpret_cast<uintptr_t>(y_f32)) &
             15) == 0) && (reinterpret_cast<uintptr_t>(y_nchw) & 3) == 0,
           NB200_EVALUE, "code and result tensors must be 16-byte aligned");
  const int c_pad = (int)round_up(g.C, 16);
  const bool narrow_rows = c_pad <= 64;
  const int E = narrow_rows ? 64 : kRowBytes;
  const int cblocks = (c_pad + E - 1) / E;
  const int64_t ctot = codes_slots(g.C, 1);
  int c_slots;
  int64_t wpitch;
  int8_side_layout(g.C, g.kh * g.kw, c_slots, wpitch);
  int h_box, n_box;
  plan_box(g, 128, h_box, n_box);
  NB_CHECK(h_box * n_box * g.Wo <= 128, NB200_ENOTIMPL, "no pixel box of at most 128 pixels");
#define NB_CC(BN_, ST_, RB_)                                                                                          \
  return launch_conv_codes<BN_, ST_, RB_>(g, x_codes, ctot, side, wpitch, cblocks, h_box, n_box, (int)slots_out, ep, st)
#define NB_CC_RES(BN_, ST_, RB_)                                                                                      \
  return launch_conv_codes<BN_, ST_, RB_, true>(g, x_codes, ctot, side, wpitch, cblocks, h_box, n_box, (int)slots_out, \
                                                ep, st)
#define NB_CC_HALO(BN_, RB_)                                                                                          \
  return launch_conv_codes<BN_, 1, RB_, true, true>(g, x_codes, ctot, side, wpitch, cblocks, hh, 1, (int)slots_out,   \
                                                    ep, st)
  // weights resident in shared memory when one column tile covers the maps and they fit beside the ring
  const size_t w_bytes = (size_t)g.kh * g.kw * cblocks * (narrow_rows ? 64 : 128);
  if (g.sh == 1 && g.sw == 1 && g.kh * g.kw > 1 && g.Ko <= 128) {
    // halo form: the tile's rows are h rows of the padded width wp; one input box per tile
    const int RBh = narrow_rows ? 64 : 128, BNh = g.Ko <= 64 ? 64 : 128;
    const int wp = g.Wo + (g.kw - 1) * g.dw;
    int hh = wp <= 128 ? (128 - g.Wo) / wp + 1 : 0; // (hh - 1) * wp + Wo <= 128
    if (hh > g.Ho)
      hh = g.Ho;
    if (hh >= 1) {
      for (int h = hh; h >= 1; --h) // prefer a divisor of Ho unless it wastes over a third of the rows
        if (g.Ho % h == 0) {
          if (3 * h >= 2 * hh)
            hh = h;
          break;
        }
      const int hp = hh + (g.kh - 1) * g.dh;
      const int rows_alloc = (((g.kh - 1) * g.dh * wp + (g.kw - 1) * g.dw + kTileM) + 7) / 8 * 8;
      const size_t a_bytes = (size_t)(rows_alloc > hp * wp ? rows_alloc : (hp * wp + 7) / 8 * 8) * RBh;
      const size_t need = 2 * cblocks * a_bytes + w_bytes * BNh + 8 * 1024;
      if (need <= 220 * 1024 && wp <= 256 && hp <= 256) {
        if (narrow_rows) {
          if (g.Ko <= 64)
            NB_CC_HALO(64, 64);
          NB_CC_HALO(128, 64);
        }
        if (g.Ko <= 64)
          NB_CC_HALO(64, 128);
        NB_CC_HALO(128, 128);
      }
    }
  }
  if (narrow_rows && g.Ko <= 64 && w_bytes * 64 <= 96 * 1024)
    NB_CC_RES(64, 12, 64);
  if (narrow_rows && g.Ko <= 128 && w_bytes * 128 <= 96 * 1024)
    NB_CC_RES(128, 12, 64);
  if (!narrow_rows && g.Ko <= 64 && w_bytes * 64 <= 128 * 1024)
    NB_CC_RES(64, 5, 128);
  if (!narrow_rows && g.Ko <= 128 && w_bytes * 128 <= 150 * 1024)
    NB_CC_RES(128, 4, 128);
  if (narrow_rows) {
    if (g.Ko <= 64)
      NB_CC(64, 10, 64);
    if (g.Ko <= 128)
      NB_CC(128, 8, 64);
    NB_CC(256, 6, 64);
  }
  if (g.Ko <= 64)
    NB_CC(64, 8, 128);
  if (g.Ko <= 128)
    NB_CC(128, 6, 128);
  {
    // Few pixels (late stages, small batches): 256-map tiles would leave most SMs idle. Narrower tiles give
    // more blocks; an MMA of N columns costs about 55 + 0.6 N cycles, so a narrower tile pays only while it
    // does not add a second round of tiles per SM.
    const int64_t ptiles = ((int64_t)g.N * g.Ho * g.Wo + kTileM - 1) / kTileM;
    const int sms = sm_count();
    if (ptiles * ((g.Ko + 255) / 256) < sms) {
      auto cost = [&](int bn) {
        const int64_t blocks = ptiles * ((g.Ko + bn - 1) / bn);
        return (double)((blocks + sms - 1) / sms) * (55.0 + 0.6 * bn);
      };
      if (cost(64) < cost(128) && cost(64) < cost(256))
        NB_CC(64, 8, 128);
      if (cost(128) < cost(256))
        NB_CC(128, 6, 128);
    }
  }
  NB_CC(256, 4, 128);
#undef NB_CC
#undef NB_CC_RES
#undef NB_CC_HALO
}
} // namespace
} // namespace nb200
extern "C" {

int64_t nb200_binary_weights_side_bytes(int outmaps, int channels, int kernel_h, int kernel_w, int group) {
  if (outmaps <= 0 || channels <= 0 || kernel_h <= 0 || kernel_w <= 0 || group <= 0 || channels % group != 0)
    return 0;
  int c_slots;
  int64_t wpitch;
  int8_side_layout(channels / group, kernel_h * kernel_w, c_slots, wpitch);
  return (int64_t)outmaps * wpitch;
}

int nb200_binary_weights_prepare_i8(const float *w, float *wb, float *alpha, int8_t *side, int outmaps, int channels,
                                    int kernel_h, int kernel_w, int group, float quantize_zero_to, void *stream) {
  NB_CHECK(outmaps > 0 && channels > 0 && kernel_h > 0 && kernel_w > 0 && group > 0 && channels % group == 0 &&
               outmaps % group == 0,
           NB200_EVALUE, "bad weight shape");
  NB_CHECK(w && wb && side, NB200_EVALUE, "null data pointer");
  NB_CHECK(quantize_zero_to == 1.0f || quantize_zero_to == -1.0f || quantize_zero_to == 0.0f, NB200_ENOTIMPL,
           "the int8 path needs quantize_zero_to in {-1, 0, 1} (got %g)", quantize_zero_to);
  NB_CHECK((reinterpret_cast<uintptr_t>(side) & 15) == 0, NB200_EVALUE, "the side-band must be 16-byte aligned");
  const int Cg = channels / group;
  int c_slots;
  int64_t wpitch;
  int8_side_layout(Cg, kernel_h * kernel_w, c_slots, wpitch);
  cudaStream_t st = as_stream(stream);
  if (c_slots != Cg)
    NB_CUDA(cudaMemsetAsync(side, 0, (size_t)outmaps * wpitch, st));
  return binarize_rows(w, outmaps, Cg, kernel_h, kernel_w, quantize_zero_to, wb, alpha, side, wpitch, c_slots, true, st);
}

int nb200_binary_convolution_codes_prepared_f32(const int8_t *x_codes, const int8_t *side, const float *alpha,
                                                const float *bias, float *y, int batch, int channels, int height,
                                                int width, int outmaps, int kernel_h, int kernel_w, int pad_h,
                                                int pad_w, int stride_h, int stride_w, int dilation_h,
                                                int dilation_w, int group, float activation_delta, void *stream) {
  NB_CHECK(x_codes != nullptr && side != nullptr, NB200_EVALUE, "null data pointer");
  NB_CHECK(activation_delta > 0.f, NB200_EVALUE, "activation_delta should be positive");
  ConvGeometry g{batch, channels, height, width, outmaps, kernel_h, kernel_w, pad_h, pad_w, stride_h, stride_w,
                 dilation_h, dilation_w, group, 0, 0, 0, 0};
  return binary_convolution(nullptr, nullptr, nullptr, const_cast<float *>(alpha), bias, y, g, 1.0f, activation_delta,
                            as_stream(stream), 0.0f, x_codes, side);
}

int nb200_binary_weight_convolution_backward_f32(const float *x, const float *wb, const float *alpha, const float *dy,
                                                 float *dx, float *dw, float *db, int batch, int channels, int height,
                                                 int width, int outmaps, int kernel_h, int kernel_w, int pad_h,
                                                 int pad_w, int stride_h, int stride_w, int dilation_h,
                                                 int dilation_w, int group, int accum_dx, int accum_dw, int accum_db,
                                                 float activation_delta, void *stream) {
  NB_CHECK(alpha != nullptr || dx == nullptr, NB200_EVALUE, "alpha is NULL");
  ConvGeometry g{batch, channels, height, width, outmaps, kernel_h, kernel_w, pad_h, pad_w, stride_h, stride_w,
                 dilation_h, dilation_w, group, 0, 0, 0, 0};
  return convolution_backward(x, wb, alpha, dy, dx, dw, db, g, accum_dx, accum_dw, accum_db, activation_delta,
                              as_stream(stream));
}

int nb200_binary_connect_convolution_backward_f32(const float *x, const float *wb, const float *dy, float *dx,
                                                  float *dw, float *db, int batch, int channels, int height,
                                                  int width, int outmaps, int kernel_h, int kernel_w, int pad_h,
                                                  int pad_w, int stride_h, int stride_w, int dilation_h,
                                                  int dilation_w, int group, int accum_dx, int accum_dw,
                                                  int accum_db, float activation_delta, void *stream) {
  ConvGeometry g{batch, channels, height, width, outmaps, kernel_h, kernel_w, pad_h, pad_w, stride_h, stride_w,
                 dilation_h, dilation_w, group, 0, 0, 0, 0};
  return convolution_backward(x, wb, nullptr, dy, dx, dw, db, g, accum_dx, accum_dw, accum_db, activation_delta,
                              as_stream(stream));
}

int nb200_convolution_backward_f32(const float *x, const float *dy, float *dw, float *db, int batch, int channels,
                                   int height, int width, int outmaps, int kernel_h, int kernel_w, int pad_h,
                                   int pad_w, int stride_h, int stride_w, int dilation_h, int dilation_w, int group,
                                   int accum_dw, int accum_db, void *stream) {
  ConvGeometry g{batch, channels, height, width, outmaps, kernel_h, kernel_w, pad_h, pad_w, stride_h, stride_w,
                 dilation_h, dilation_w, group, 0, 0, 0, 0};
  return convolution_backward(x, nullptr, nullptr, dy, nullptr, dw, db, g, 0, accum_dw, accum_db, 0.0f,
                              as_stream(stream));
}

int nb200_convolution_input_backward_f32(const float *w, const float *dy, float *dx, int batch, int channels, int height,
                                         int width, int outmaps, int kernel_h, int kernel_w, int pad_h, int pad_w,
                                         int stride_h, int stride_w, int dilation_h, int dilation_w, int group,
                                         int accum_dx, void *stream) {
  NB_CHECK(w && dx, NB200_EVALUE, "null data pointer");
  ConvGeometry g{batch, channels, height, width, outmaps, kernel_h, kernel_w, pad_h, pad_w, stride_h, stride_w,
                 dilation_h, dilation_w, group, 0, 0, 0, 0};
  return convolution_backward(nullptr, w, nullptr, dy, dx, nullptr, nullptr, g, accum_dx, 0, 0, 0.0f,
                              as_stream(stream), true);
}

int nb200_convolution_fxp8_f32(const float *xq, const float *wq, float delta_x, float delta_w, const float *bias,
                               float *y, int batch, int channels, int height, int width, int outmaps, int kernel_h,
                               int kernel_w, int pad_h, int pad_w, int stride_h, int stride_w, int dilation_h,
                               int dilation_w, int group, void *stream) {
  NB_CHECK(delta_x > 0.f && delta_w > 0.f, NB200_EVALUE, "step sizes must be positive");
  ConvGeometry g{batch, channels, height, width, outmaps, kernel_h, kernel_w, pad_h, pad_w, stride_h, stride_w,
                 dilation_h, dilation_w, group, 0, 0, 0, 0};
  return binary_convolution(xq, wq, nullptr, nullptr, bias, y, g, 1.0f, delta_x, as_stream(stream), delta_w);
}

int nb200_convolution_codes_folded_nhwc(const int8_t *x_codes, const int8_t *side, const float *scale,
                                        const float *bias, const int8_t *res_codes, float res_delta,
                                        const float *res_f32, int8_t *y_codes, float *y_f32, int batch, int channels,
                                        int height, int width, int outmaps, int kernel_h, int kernel_w, int pad_h,
                                        int pad_w, int stride_h, int stride_w, int dilation_h, int dilation_w,
                                        int relu, int sign, int n, float delta, void *stream) {
  ConvGeometry g{batch, channels, height, width, outmaps, kernel_h, kernel_w, pad_h, pad_w, stride_h, stride_w,
                 dilation_h, dilation_w, 1, 0, 0, 0, 0};
  return convolution_codes_folded(x_codes, side, scale, bias, res_codes, res_delta, res_f32, y_codes, y_f32, g, relu,
                                  sign, n, delta, as_stream(stream));
}
#ifdef NB200_CC_TRACE
void nb200_debug_conv_trace(long long *buffer) { g_cc_trace = buffer; }
#endif
}
