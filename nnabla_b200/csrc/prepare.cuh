// Host-callable operand preparation passes (prepare.cu).
#pragma once
#include "common.cuh"

namespace nb200 {

// W [R, C] -> wb (signs, fp32, same layout), alpha[C] = mean_r |W| (NULL to
// skip, BinaryConnect), side-band [C][side_pitch] (bf16 or int8 signs with
// K = R contiguous). partial_scratch: ceil(R/64) * C floats (only with alpha).
int binarize_columns(const float *w, int R, int C, float zero_to, float *wb, float *alpha, void *side,
                     int64_t side_pitch, bool int8, float *partial_scratch, cudaStream_t st);
// W [Ko, Cg, kh, kw] -> wb, alpha[Ko] (NULL to skip), side-band [Ko][side_pitch]
// with K ordered (ky, kx, c) and c padded to c_pad.
// half: the signs of the side-band are fp16 instead of bf16.
int binarize_rows(const float *w, int Ko, int Cg, int kh, int kw, float zero_to, float *wb, float *alpha, void *side,
                  int64_t side_pitch, int c_pad, bool int8, cudaStream_t st, bool half = false);
// wq [Ko, Cg, kh, kw] multiples of delta -> int8 codes in the side-band layout of binarize_rows.
int codes_conv_weights(const float *wq, int Ko, int Cg, int kh, int kw, float delta, void *side, int64_t side_pitch,
                       int c_pad, cudaStream_t st);
// Channel slots per pixel of the int8 channel-last activation layout: every group padded to a
// multiple of 16, the whole row at least one K block (64 slots when a group fits 64, else 128).
inline int64_t codes_slots(int64_t channels, int group) {
  const int64_t c_pad_g = (channels / group + 15) / 16 * 16;
  const int64_t E = c_pad_g <= 64 ? 64 : 128;
  const int64_t ctot = (int64_t)group * c_pad_g;
  return ctot < E ? E : ctot;
}
// fp32 [rows, K] -> bf16 [planes][rows][Kp] (planes = 1 or 3; hi, mid, lo).
// col_scale (K floats or NULL): x[r, k] is multiplied by col_scale[k] first.
int split_rows_bf16(const float *x, int64_t rows, int K, int64_t Kp, int planes, void *out, cudaStream_t st,
                    const float *col_scale = nullptr);
// out[c] (+)= sum over rows of a[rows, C]; partial: splits * C floats of scratch.
int column_sums(const float *a, int64_t rows, int C, float *out, int accumulate, float *partial, int splits,
                cudaStream_t st);
// fp32 NCHW -> NHWC planes [planes][N][HW][ctot] (planes = 3 or 1: bf16 pieces;
// planes = 0: int8 codes of multiples of delta). Channel c of group g is stored
// at slot g * c_pad_g + (c - g * Cg); all other slots are zero.
int nchw_to_nhwc_planes(const float *x, int N, int C, int HW, int groups, int Cg, int c_pad_g, int ctot, int planes,
                        float delta, void *out, cudaStream_t st);
// fp32 NCHW -> two fp16 NHWC planes [2][N][HW][ctot] of x * 2^-e (e from the tensor's largest magnitude,
// left in *maxbits as the bits of that magnitude): p0 + p1 = x * 2^-e. row_scale_out[r] =
// (row_scale_in ? row_scale_in[r] : 1) * 2^e for r < rows: the factor that undoes the scaling.
int nchw_to_nhwc_half_pair(const float *x, int N, int C, int HW, int groups, int Cg, int c_pad_g, int ctot, void *out,
                           uint32_t *maxbits, const float *row_scale_in, int rows, float *row_scale_out,
                           cudaStream_t st);
// int8 [R, C] -> [C][pitch].
int transpose_i8(const int8_t *src, int R, int C, int8_t *dst, int64_t pitch, cudaStream_t st);
// fp32 [R, C] -> [C][R].
int transpose_f32(const float *src, int R, int C, float *dst, cudaStream_t st);
// fp32 multiples of delta [rows, K] -> int8 [rows][pitch].
int codes_rows_i8(const float *x, int64_t rows, int K, int64_t pitch, float delta, int8_t *out, cudaStream_t st);

// ---- convolution backward (prepare_backward.cu) ------------------------------
// dy [N][Ko][Ho][Wo] -> 3 bf16 planes [N][Hs][Ws][ctot] (pre-zeroed by the caller):
// pixel (oy, ox) at (oy * sh, ox * sw), map o of group g at slot g * k_pad_g + o - g * Kog,
// multiplied by chan_scale[o] first when given.
int dy_to_nhwc_stuffed(const float *dy, int N, int Ko, int Ho, int Wo, int groups, int Kog, int k_pad_g, int ctot,
                       int Hs, int Ws, int sh, int sw, const float *chan_scale, void *out, cudaStream_t st);
// binarize_rows (int8 side-band) and the activations' conversion to channel-last int8 codes (nchw_to_nhwc_planes
// with planes = 0) as ONE launch.
bool binary_conv_operands_i8_applies(const float *x, int N, int HW, int ctot, int Ko);
int binary_conv_operands_i8(const float *w, int Ko, int Cg, int kh, int kw, float zero_to, float *wb, float *alpha,
                            void *side, int64_t side_pitch, int c_pad, const float *x, int N, int C, int HW, int groups,
                            int c_pad_g, int ctot, float delta, void *out, cudaStream_t st);
// wb [Ko][Cg][kh][kw] -> side [planes][C][kh * kw][k_slots] bf16 (pre-zeroed), taps flipped, maps innermost;
// planes = 1 for weights exact in bf16, 3 for full-precision weights (hi, mid, lo pieces).
int flip_transpose_weights(const float *wb, int Ko, int Cg, int kh, int kw, int groups, int k_slots, void *side,
                           cudaStream_t st, int planes = 1);
// N rows of R fp32 values (rows src_row_stride apart) -> bf16 [planes][R][Np] (pre-zeroed), batch innermost.
int batch_to_inner(const float *src, int N, int64_t R, int64_t src_row_stride, int Np, int planes, void *out,
                   cudaStream_t st);
// out[o] (+)= sum over n and pixels of dy [N][Ko][HW]; partial: splits * Ko floats.
int channel_sums(const float *dy, int N, int Ko, int HW, float *out, int accumulate, float *partial, int splits,
                 cudaStream_t st);
// staged [splits][Cg][Kog][taps] -> dw [Kog][Cg][taps] = sum over the splits (overwrite or add).
int permute_weight_grad(const float *staged, int splits, int Cg, int Kog, int taps, float *dw, int accumulate,
                        cudaStream_t st);

} // namespace nb200
