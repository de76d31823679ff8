/* nnabla_b200 — C ABI of the B200 (sm_100a) implementation of nnabla's
 * quantized-layer forward path.
 *
 * nnabla has no C plugin ABI: a backend plugs in by registering C++ Function
 * classes (include/nbla/function_registry.hpp:165-197) whose forward_impl is
 * called by Function::forward (src/nbla/function.cpp:107-123). Each entry point
 * below is the body of one such forward_impl with plain pointers and sizes, so
 * that the nnabla extension classes (ext/ in this repository), the Python
 * mirror (nnabla_b200/functions.py) and any other host can bind it without
 * sharing C++ types. The comment on each entry names the reference code it
 * replaces.
 *
 * Conventions
 *  - Every function returns 0 on success; otherwise a non-zero NB200_E* code,
 *    and nb200_last_error() returns a message for the calling thread. This is
 *    the C form of the reference's NBLA_CHECK / NBLA_ERROR exceptions
 *    (include/nbla/exception.hpp:42-82).
 *  - Unless the name ends in _host, data pointers are DEVICE pointers on the
 *    current CUDA device, fp32, densely packed, row-major. `stream` is a
 *    cudaStream_t passed as void* (NULL = the legacy default stream). Calls are
 *    asynchronous with respect to the host unless stated otherwise.
 *  - _host variants take HOST pointers (pinned memory from nb200_malloc_host
 *    runs fastest; pageable memory works), copy in, compute and copy out in
 *    overlapped chunks, and return after the result is in the host buffer.
 *  - Sizes are element counts (size_t / int64_t), never bytes, unless named
 *    `bytes`.
 */
#ifndef NNABLA_B200_H_
#define NNABLA_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define NB200_OK 0
#define NB200_EVALUE 1   /* bad argument (reference: error_code::value) */
#define NB200_ECUDA 2    /* CUDA runtime/driver failure (error_code::target_specific) */
#define NB200_EMEMORY 3  /* allocation failure (error_code::memory) */
#define NB200_ENOTIMPL 4 /* configuration not supported (error_code::not_implemented) */
#define NB200_EDEVICE 5  /* a bounded device-side wait gave up; the context stays usable */

/* ---- runtime: what nnabla's backend layer needs from a device ------------- */

/* Message of the last failure on this thread ("" if none). */
const char *nb200_last_error(void);
/* ABI version of this library (bumped on incompatible changes). */
int nb200_abi_version(void);
/* Replaces Cpu::get_device_count-style queries of an extension
 * (python/src/nnabla_ext/cpu/__init__.py:17-45): number of CUDA devices. */
int nb200_device_count(int *count);
int nb200_set_device(int device);
int nb200_get_device(int *device);
/* Fails with NB200_ENOTIMPL unless the current device is compute capability
 * 10.x: the kernels are built for sm_100a only and there is no fallback. */
int nb200_check_device(void);
/* Memory::alloc_impl / ~Memory of a device Memory class
 * (include/nbla/memory/memory.hpp:285-312; CPU counterpart
 * src/nbla/memory/cpu_memory.cpp:31-80). */
int nb200_malloc(void **dev_ptr, size_t bytes);
int nb200_free(void *dev_ptr);
/* Pinned host memory for the _host entry points and for synchronizers. */
int nb200_malloc_host(void **host_ptr, size_t bytes);
int nb200_free_host(void *host_ptr);
/* ArraySynchronizer bodies (include/nbla/array_registry.hpp:136-137): raw
 * copies between a host array and a device array, asynchronous on `stream`. */
int nb200_memcpy_h2d(void *dev_dst, const void *host_src, size_t bytes, void *stream);
int nb200_memcpy_d2h(void *host_dst, const void *dev_src, size_t bytes, void *stream);
int nb200_memcpy_d2d(void *dev_dst, const void *dev_src, size_t bytes, void *stream);
/* Array::zero / Array::fill (include/nbla/array.hpp:128-140): zero for any
 * dtype (byte-wise), fill for fp32 arrays. */
int nb200_memset_zero(void *dev_ptr, size_t bytes, void *stream);
int nb200_fill_f32(float *dev_ptr, size_t n, float value, void *stream);
/* Sharing one GPU's array with the other ranks of the box (one process per
 * GPU). The reference moves data between devices only through
 * Communicator::all_gather and friends (include/nbla/communicator.hpp:232-241);
 * here a rank exports an array it allocated with nb200_malloc as a 64-byte
 * handle, the other ranks map it with nb200_ipc_open, and the *_gather_f32
 * contractions below store their results straight into those mappings.
 * `handle` points at NB200_IPC_HANDLE_BYTES bytes; a mapping is released with
 * nb200_ipc_close before the owner frees the array. */
#define NB200_IPC_HANDLE_BYTES 64
int nb200_ipc_export(const void *dev_ptr, void *handle);
int nb200_ipc_open(const void *handle, void **peer_ptr);
int nb200_ipc_close(void *peer_ptr);
int nb200_stream_create(void **stream);
int nb200_stream_destroy(void *stream);
/* BackendBase::device_synchronize (include/nbla/backend_base.hpp:32-91). */
int nb200_stream_synchronize(void *stream);
int nb200_device_synchronize(void);
/* Bytes of the current device's stream-ordered scratch pool (the pool every
 * entry point's temporary side-band tensors come from) in use now, and the
 * high-water mark since it was last reset (reset_high != 0 resets it first).
 * Either pointer may be NULL. The counterpart of the caching allocator's
 * usage queries (include/nbla/memory/allocator.hpp:209-251). */
int nb200_scratch_pool_stats(int64_t *used_now, int64_t *used_high, int reset_high);

/* ---- elementwise quantizers ------------------------------------------------ */

/* FixedPointQuantize<float>::forward_impl
 * (src/nbla/function/generic/fixed_point_quantize.cpp:45-66; limits :37-39).
 * y[i] = max if x>max; min if x<min; else sgn(x)*float(int(|x|/delta + 0.5))*delta,
 * bit-identical to the reference for every non-NaN input. Requires n > 0,
 * delta > 0 and n - sign > 0 (the reference's setup checks). x == y allowed. */
int nb200_fixed_point_quantize_f32(const float *x, float *y, size_t size, int sign, int n, float delta,
                                   void *stream);
/* Same, and additionally writes the integer code k (y = k*delta, |k| <= 127)
 * as int8 to `codes` (size elements): the operand format of the int8
 * tensor-core contraction. Requires n - sign <= 7. */
int nb200_fixed_point_quantize_f32_codes(const float *x, float *y, int8_t *codes, size_t size, int sign, int n,
                                         float delta, void *stream);
/* FixedPointQuantize of x [batch, channels, inner] that also leaves the result as int8 channel-last codes
 * [batch][inner][nb200_codes_nhwc_slots(channels, 1)] (zero in the padding slots): the activation operand of
 * nb200_binary_convolution_codes_f32 and the other *_codes_* entry points, written by the quantizer itself so
 * that the convolution behind it does not read the fp32 tensor again. inner % 4 == 0, 16-byte aligned tensors,
 * n - sign <= 7, batch <= 65535. y is bit-identical to nb200_fixed_point_quantize_f32's. */
int nb200_fixed_point_quantize_nhwc_codes_f32(const float *x, float *y, int8_t *codes, int64_t batch, int64_t channels,
                                              int64_t inner, int sign, int n, float delta, void *stream);
int nb200_fixed_point_quantize_f32_host(const float *x, float *y, size_t size, int sign, int n, float delta);

/* Pow2Quantize<float>::forward_impl
 * (src/nbla/function/generic/pow2_quantize.cpp:47-82; constants :35-39).
 * The reference evaluates powf(2, roundf(log2f(|x|))) with the host libm; this
 * library derives, once per process and with the host libm, the mantissa cut
 * per exponent at which that expression steps, and the kernel snaps with
 * integer compares against that table — bit-identical for every non-NaN
 * input, denormals included. */
int nb200_pow2_quantize_f32(const float *x, float *y, size_t size, int sign, int with_zero, int n, int m,
                            void *stream);
int nb200_pow2_quantize_f32_host(const float *x, float *y, size_t size, int sign, int with_zero, int n, int m);

/* MinMaxQuantize<float>::forward_impl
 * (src/nbla/function/generic/min_max_quantize.cpp:129-223, nudge_range
 * :352-361, nudge_qr_min_max :362-390). x has shape x_shape[0..ndim); qr_min,
 * qr_max, ql_min, ql_max share q_shape[0..ndim) whose extents are 1 or equal
 * to x's. Like the reference, the call UPDATES qr_min and qr_max in place
 * (min/max of x or their moving average when x_min_max, then the eps nudge of
 * qr_max). `scale` (q-sized, may be NULL) receives the scale the reference
 * keeps for backward. Every fp32 operation rounds separately (no FMA), so y,
 * qr_min and qr_max are bit-identical to the reference for non-NaN input. */
int nb200_min_max_quantize_f32(const float *x, const int64_t *x_shape, int ndim, float *qr_min, float *qr_max,
                               const float *ql_min, const float *ql_max, const int64_t *q_shape, float decay,
                               int x_min_max, int ema, float eps, float *y, float *scale, void *stream);
/* Same computation and arguments as nb200_min_max_quantize_f32, for callers
 * that must not allocate. It has no counterpart in the reference. Two kinds of
 * host need it: frameworks that own every byte of device memory through their
 * own allocator (nnabla's caching allocator is one: a function that goes to the
 * driver for memory behind its back breaks its accounting and can fail when
 * the pool has taken the whole device), and serving loops that cannot afford
 * the locks and device synchronisation an allocation call may bring. This
 * entry point never calls cudaMalloc, cudaMallocAsync, cudaFree or any other
 * allocating routine: its scratch (28 bytes per quantization range) is a
 * fixed 112 KiB array inside the library image, so every GPU that loads the
 * library holds that array until the process exits.
 *  - Limit: at most 4096 quantization ranges (elements of qr_min) per call;
 *    more is refused with NB200_EVALUE.
 *  - The first call on each device looks up the array's device address (the
 *    device must be current); make that first call before any stream capture.
 *    The address is kept for the life of the process: a host that tears the
 *    device's primary context down (cudaDeviceReset) and goes on must not
 *    call this entry point again afterwards.
 *  - All calls on a device share the one array. Calls that may overlap on the
 *    GPU (different streams, no ordering between them) race on it; serialise
 *    them or use nb200_min_max_quantize_f32. */
int nb200_min_max_quantize_f32_noalloc(const float *x, const int64_t *x_shape, int ndim, float *qr_min,
                                       float *qr_max, const float *ql_min, const float *ql_max,
                                       const int64_t *q_shape, float decay, int x_min_max, int ema, float eps,
                                       float *y, float *scale, void *stream);
/* Host variant for per-tensor ranges with x_min_max == 0 (q tensors of one
 * element each, host pointers; qr_max is updated by the eps nudge). */
int nb200_min_max_quantize_f32_host(const float *x, size_t size, float *qr_min, float *qr_max, const float *ql_min,
                                    const float *ql_max, float eps, float *y);

/* ---- sibling quantization functions (forward and backward) ----------------------- */
/* BinarySigmoid / BinaryTanh (include/nbla/function/binary_sigmoid.hpp:50-52,
 * binary_tanh.hpp:51-52): y = x > 0 ? 1 : 0 (or -1); gradient |x| >= 1 ? 0 :
 * dy * 0.5 (or dy), combined as (accum ? dx : 0) + g
 * (include/nbla/function/utils/base_transform_unary.hpp:104-110). */
int nb200_binary_sigmoid_f32(const float *x, float *y, size_t size, void *stream);
int nb200_binary_tanh_f32(const float *x, float *y, size_t size, void *stream);
int nb200_binary_sigmoid_backward_f32(const float *x, const float *dy, float *dx, size_t size, int accum,
                                      void *stream);
int nb200_binary_tanh_backward_f32(const float *x, const float *dy, float *dx, size_t size, int accum, void *stream);
/* QuantizeLinear<float>::forward_impl (src/nbla/function/generic/quantize_linear.cpp:103-122):
 * y = saturate(round(x / scale) + zero_point). scale and zero_point broadcast
 * over x (every extent 1 or x's); zero_point is ROUNDED AND SATURATED IN PLACE
 * first, as the reference does. round_mode 0 = HALF_AWAY_FROM_ZERO, 1 =
 * HALF_TO_EVEN; dtype 1 = BYTE, 2 = UBYTE (include/nbla/dtypes.hpp:32-35). */
int nb200_quantize_linear_f32(const float *x, const int64_t *x_shape, int ndim, const float *scale,
                              const int64_t *scale_shape, float *zero_point, const int64_t *zero_point_shape, float *y,
                              int round_mode, int narrow_range, int dtype, void *stream);
/* DequantizeLinear<float>::forward_impl (dequantize_linear.cpp:60-71): y = (x - zero_point) * scale. */
int nb200_dequantize_linear_f32(const float *x, const int64_t *x_shape, int ndim, const float *scale,
                                const int64_t *scale_shape, const float *zero_point, const int64_t *zero_point_shape,
                                float *y, void *stream);
/* Their gradients w.r.t. x: dx (+)= dy / scale (quantize_linear.cpp:137-147),
 * dx (+)= dy * scale (dequantize_linear.cpp:92-102). The reference has no
 * gradient w.r.t. scale or zero point. */
int nb200_quantize_linear_backward_f32(const float *dy, const int64_t *x_shape, int ndim, const float *scale,
                                       const int64_t *scale_shape, float *dx, int accum, void *stream);
int nb200_dequantize_linear_backward_f32(const float *dy, const int64_t *x_shape, int ndim, const float *scale,
                                         const int64_t *scale_shape, float *dx, int accum, void *stream);

/* Prune<float>::forward_impl (src/nbla/function/generic/prune.cpp:38-72): y = |x| < t ? 0 : x
 * with t the (int)((size - 1) * rate)-th smallest |x| (+ 1 when rate == 1),
 * found by a radix select on the device instead of the reference's sort.
 * backward (prune.cpp:74-88): the gradient passes unchanged. */
int nb200_prune_f32(const float *x, float *y, size_t size, float rate, void *stream);
int nb200_prune_backward_f32(const float *dy, float *dx, size_t size, int accum, void *stream);

/* ---- inference-time fusion ---------------------------------------------------------
 * y = FixedPointQuantize(ReLU(BN_a(a) [+ BN_b(b) | + b])) over [outer, channels, inner]
 * tensors in one pass: BatchNormalization::forward_impl_global
 * (src/nbla/function/generic/batch_normalization.cpp:228-260), Add2 (add2.cpp),
 * ReLU (relu.cpp) and FixedPointQuantize (fixed_point_quantize.cpp:45-66),
 * bit-identical to calling them one after the other (the reference's own fused
 * form of the first three is FusedBatchNormalization,
 * fused_batch_normalization.cpp). b == NULL: no second operand; mean_b == NULL:
 * b is added as it is (a residual); beta / gamma may be NULL (0 / 1).
 * relu / quantize switch those two stages on. */
int nb200_bn_add_relu_fxp_f32(const float *a, const float *beta_a, const float *gamma_a, const float *mean_a,
                              const float *var_a, const float *b, const float *beta_b, const float *gamma_b,
                              const float *mean_b, const float *var_b, float *y, int64_t outer, int64_t channels,
                              int64_t inner, float eps, int relu, int quantize, int sign, int n, float delta,
                              void *stream);

/* ---- binary weights prepared once per weight update -----------------------------------
 * The binary convolutions re-derive sign(w), alpha and the tensor core's int8 side-band
 * from w on every call, as the reference's forward_impl does
 * (binary_weight_convolution.cpp:72-117). For inference, where w does not change between
 * calls, they can be made once (what a cache keyed on SyncedArray::modification_count,
 * include/nbla/synced_array.hpp:183, would hold) and passed to
 * nb200_binary_convolution_codes_prepared_f32. side: int8, nb200_binary_weights_side_bytes
 * bytes, 16-byte aligned; wb and alpha (NULL for BinaryConnect) are written as by the
 * convolution itself. */
int64_t nb200_binary_weights_side_bytes(int outmaps, int channels, int kernel_h, int kernel_w, int group);
int nb200_binary_weights_prepare_i8(const float *w, float *wb, float *alpha, int8_t *side, int outmaps, int channels,
                                    int kernel_h, int kernel_w, int group, float quantize_zero_to, void *stream);

/* ---- activations kept as 8-bit codes between the layers -----------------------------
 * An output of FixedPointQuantize with n - sign <= 7 is k * delta with an integer
 * |k| <= 127 (fixed_point_quantize.cpp:53-65): the int8 code k carries the whole
 * value. Between the layers of a quantized network the codes can replace the
 * fp32 tensor: 1 byte per activation instead of 4, already in the channel-last
 * layout that the int8 convolution reads, and the residual of a block is
 * code * delta exactly. A "codes_nhwc" tensor is int8 [batch, inner, slots]
 * (inner = height * width); channel c of group g = c / (channels / group) sits in
 * slot g * pad16(channels / group) + c % (channels / group), the other slots
 * hold 0. Results are bit-identical to the fp32 chain (a -0.0 of the chain is a
 * +0.0 here; with the ReLU in front of the quantizer none occurs). */

/* Slots per pixel of a codes_nhwc tensor (>= channels, a multiple of 16). */
int64_t nb200_codes_nhwc_slots(int64_t channels, int group);
/* xq [batch, channels, inner] fp32 multiples of delta, |multiple| <= 127 -> codes_nhwc. */
int nb200_fixed_point_codes_nhwc(const float *xq, int8_t *codes, int64_t batch, int64_t channels, int64_t inner,
                                 int group, float delta, void *stream);
/* codes_nhwc -> y [batch, channels, inner] fp32 = code * delta. */
int nb200_codes_nhwc_to_f32(const int8_t *codes, float *y, int64_t batch, int64_t channels, int64_t inner, int group,
                            float delta, void *stream);
/* nb200_bn_add_relu_fxp_f32 whose result is written as codes_nhwc (the
 * quantizer is always applied; n - sign <= 7). The second operand is either
 * b (fp32 [batch, channels, inner], with or without its own normalisation) or
 * b_codes (codes_nhwc of the same shape and group, value code * b_delta), not both. */
int nb200_bn_add_relu_fxp_codes_nhwc(const float *a, const float *beta_a, const float *gamma_a, const float *mean_a,
                                     const float *var_a, const float *b, const float *beta_b, const float *gamma_b,
                                     const float *mean_b, const float *var_b, const int8_t *b_codes, float b_delta,
                                     int8_t *y_codes, int64_t batch, int64_t channels, int64_t inner, int group,
                                     float eps, int relu, int sign, int n, float delta, void *stream);
/* MaxPooling<float>::forward_impl (src/nbla/function/generic/max_pooling.cpp:140-191,
 * output extent base_pooling.cpp:59) on a codes_nhwc tensor [batch, height * width,
 * slots] -> [batch, Ho * Wo, slots]: the maximum of the codes is the code of the maximum. */
int nb200_max_pooling_codes_nhwc(const int8_t *codes, int8_t *y_codes, int64_t batch, int64_t channels, int height,
                                 int width, int group, int kernel_h, int kernel_w, int stride_h, int stride_w,
                                 int pad_h, int pad_w, int ignore_border, void *stream);
/* nb200_binary_weight_convolution_f32 / nb200_binary_connect_convolution_f32
 * (alpha == NULL) on x given as codes_nhwc [batch, height * width, slots] with
 * step activation_delta > 0; y is fp32 NCHW as usual. */
int nb200_binary_convolution_codes_f32(const int8_t *x_codes, const float *w, float *wb, float *alpha,
                                       const float *bias, float *y, int batch, int channels, int height, int width,
                                       int outmaps, int kernel_h, int kernel_w, int pad_h, int pad_w, int stride_h,
                                       int stride_w, int dilation_h, int dilation_w, int group,
                                       float quantize_zero_to, float activation_delta, void *stream);
/* The same with weights prepared by nb200_binary_weights_prepare_i8 (alpha == NULL: BinaryConnect). */
int nb200_binary_convolution_codes_prepared_f32(const int8_t *x_codes, const int8_t *side, const float *alpha,
                                                const float *bias, float *y, int batch, int channels, int height,
                                                int width, int outmaps, int kernel_h, int kernel_w, int pad_h,
                                                int pad_w, int stride_h, int stride_w, int dilation_h,
                                                int dilation_w, int group, float activation_delta, void *stream);

/* ---- batch normalization folded into the convolutions (inference) -------------------
 * nnabla's BatchNormalizationFolding converter
 * (python/src/nnabla/experimental/graph_converters/batch_normalization_folding.py:92-200)
 * rewrites Convolution -> BatchNormalization into one Convolution with
 * w' = c0 * w, b' = c1 (c0 = gamma / sqrt(var + eps), c1 = beta - gamma * mean /
 * sqrt(var + eps)). For a binary-weight layer w = Wb * alpha, so the fold lands in
 * the per-map factor: y = conv(x, Wb) * (alpha * c0) + c1. The two entries below
 * run such a folded layer with the rest of its inference tail, Add2 of the
 * residual, ReLU and FixedPointQuantize (relu.cpp, add2.cpp,
 * fixed_point_quantize.cpp:45-66), inside the convolution's epilogue, and emit the
 * int8 channel-last codes the next layer reads: nothing but codes travels between
 * the layers. Results follow the folded graph (Convolution with the folded
 * weights, then the separate functions) within the contraction tolerance before the
 * quantizer; they are not bit-identical to the unfolded graph, as the reference's
 * own folded graphs are not.
 *
 * nb200_convolution_codes_folded_nhwc: x_codes [batch][H * W][slots(channels)] int8
 * (value = code * the step already folded into scale), side = weights prepared by
 * nb200_binary_weights_prepare_i8 (group 1), scale / bias per output map:
 *   v = fma(acc, scale[o], bias[o])                       (bias may be NULL)
 *   v = fma(res_codes, res_delta, v)  |  v = v + res_f32  (residual in the result's own
 *                                                          channel-last layout; at most one)
 *   either y_f32 (channel-last [batch][Ho * Wo][slots(outmaps)]) = v
 *   or y_codes = code of FixedPointQuantize(sign, n, delta)(relu ? max(v, 0) : v)
 * (exactly one of y_f32 / y_codes; one rounding per fused multiply-add). delta must be a
 * power of two, n - sign <= 7, all tensors 16-byte aligned. */
int nb200_convolution_codes_folded_nhwc(const int8_t *x_codes, const int8_t *side, const float *scale,
                                        const float *bias, const int8_t *res_codes, float res_delta,
                                        const float *res_f32, int8_t *y_codes, float *y_f32, int batch, int channels,
                                        int height, int width, int outmaps, int kernel_h, int kernel_w, int pad_h,
                                        int pad_w, int stride_h, int stride_w, int dilation_h, int dilation_w,
                                        int relu, int sign, int n, float delta, void *stream);
/* The network stem in the same form: full-precision Convolution (few input channels,
 * convolution.cpp:160-197) with folded weights and bias, then ReLU (optional) and
 * FixedPointQuantize in the epilogue; y_codes [batch][Ho * Wo][slots(outmaps)] int8. Geometries
 * outside the tensor-core stem kernel (kernel_w * channels <= 24, kernel_h <= 7, at most 64 maps
 * and 112 output columns, no dilation, group 1) return NB200_ENOTIMPL. */
int nb200_convolution_relu_fxp_codes_nhwc(const float *x, const float *w, const float *bias, int8_t *y_codes,
                                          int batch, int channels, int height, int width, int outmaps, int kernel_h,
                                          int kernel_w, int pad_h, int pad_w, int stride_h, int stride_w, int relu,
                                          int sign, int n, float delta, void *stream);

/* Convolution<float>::forward_impl (src/nbla/function/generic/convolution.cpp:160-197)
 * for operands that are outputs of FixedPointQuantize with at most 8 bits (what
 * fixed_point_quantized_convolution builds, python/src/nnabla/parametric_functions.py:2411-):
 * xq multiples of delta_x, wq [outmaps, channels / group, kh, kw] multiples of
 * delta_w, |code| <= 127. int8 tensor-core path with int32 accumulation:
 * y = float(acc) * (delta_x * delta_w) + bias, exact whenever the reference's
 * fp32 result is. */
int nb200_convolution_fxp8_f32(const float *xq, const float *wq, float delta_x, float delta_w, const float *bias,
                               float *y, int batch, int channels, int height, int width, int outmaps, int kernel_h,
                               int kernel_w, int pad_h, int pad_w, int stride_h, int stride_w, int dilation_h,
                               int dilation_w, int group, void *stream);

/* ---- binary convolution backward passes ------------------------------------------
 * Convolution<float>::backward_impl
 * (src/nbla/function/generic/convolution.cpp:199-300) as the binary layers
 * call it (binary_weight_convolution.cpp:119-146 with wb * alpha,
 * binary_connect_convolution.cpp:82-104 with wb), geometry as in the forward:
 *   dx (+)= transposed convolution of dy with the weights,
 *   dw (+)= correlation of x with dy (the gradient of the FLOAT weights: it
 *           passes straight through Sign),
 *   db (+)= sums of dy over batch and pixels.
 * NULL dx / dw / db is not computed. wb / alpha are what the forward wrote.
 * activation_delta > 0 declares x to hold multiples of that step with codes
 * in [-127, 127] (then x is exact in one bf16 piece). Both gradients run on
 * the forward's implicit-GEMM tensor-core kernel. */
int nb200_binary_weight_convolution_backward_f32(const float *x, const float *wb, const float *alpha, const float *dy,
                                                 float *dx, float *dw, float *db, int batch, int channels, int height,
                                                 int width, int outmaps, int kernel_h, int kernel_w, int pad_h,
                                                 int pad_w, int stride_h, int stride_w, int dilation_h,
                                                 int dilation_w, int group, int accum_dx, int accum_dw, int accum_db,
                                                 float activation_delta, void *stream);
int nb200_binary_connect_convolution_backward_f32(const float *x, const float *wb, const float *dy, float *dx,
                                                  float *dw, float *db, int batch, int channels, int height,
                                                  int width, int outmaps, int kernel_h, int kernel_w, int pad_h,
                                                  int pad_w, int stride_h, int stride_w, int dilation_h,
                                                  int dilation_w, int group, int accum_dx, int accum_dw,
                                                  int accum_db, float activation_delta, void *stream);

/* Weight and bias gradients of the full-precision Convolution (the network
 * stem; convolution.cpp:199-300): dw (+)= correlation of x with dy, db (+)=
 * sums of dy. The gradient w.r.t. x of a full-precision convolution is not
 * provided (a first layer does not need it). */
int nb200_convolution_backward_f32(const float *x, const float *dy, float *dw, float *db, int batch, int channels,
                                   int height, int width, int outmaps, int kernel_h, int kernel_w, int pad_h,
                                   int pad_w, int stride_h, int stride_w, int dilation_h, int dilation_w, int group,
                                   int accum_dw, int accum_db, void *stream);
/* Its gradient w.r.t. x (convolution.cpp:236-262): dx (+)= transposed convolution of dy with w, both operands in
 * three bf16 pieces on the tensor cores (the products that matter at fp32 resolution). Images up to 128 pixels
 * wide. */
int nb200_convolution_input_backward_f32(const float *w, const float *dy, float *dx, int batch, int channels, int height,
                                         int width, int outmaps, int kernel_h, int kernel_w, int pad_h, int pad_w,
                                         int stride_h, int stride_w, int dilation_h, int dilation_w, int group,
                                         int accum_dx, void *stream);

/* ---- quantizer backward passes (straight-through estimators) -------------------
 * dx (+)= gradient for n elements; accum != 0 adds to dx (elements that pass no
 * gradient are left untouched), accum == 0 overwrites (zero where blocked),
 * exactly like the reference loops. x is not read when ste_fine_grained == 0. */
/* FixedPointQuantize<float>::backward_impl
 * (src/nbla/function/generic/fixed_point_quantize.cpp:69-127). */
int nb200_fixed_point_quantize_backward_f32(const float *x, const float *dy, float *dx, size_t size, int sign, int n,
                                            float delta, int ste_fine_grained, int accum, void *stream);
/* Pow2Quantize<float>::backward_impl
 * (src/nbla/function/generic/pow2_quantize.cpp:84-156). */
int nb200_pow2_quantize_backward_f32(const float *x, const float *dy, float *dx, size_t size, int sign, int with_zero,
                                     int n, int m, int ste_fine_grained, int accum, void *stream);
/* MinMaxQuantize<float>::backward_impl
 * (src/nbla/function/generic/min_max_quantize.cpp:225-350), called after the
 * forward: qr_min / qr_max hold the ranges the forward left in place. Shapes
 * as in nb200_min_max_quantize_f32. propagate_down[3] / accum[3] are the
 * flags of x, qr_min, qr_max. g_qr_min / g_qr_max (q-shaped) are written only
 * when neither x_min_max nor ema is set (the reference returns before them,
 * :300-301). */
int nb200_min_max_quantize_backward_f32(const float *x, const int64_t *x_shape, int ndim, const float *qr_min,
                                        const float *qr_max, const float *ql_min, const float *ql_max,
                                        const int64_t *q_shape, const float *dy, int x_min_max, int ema,
                                        int ste_fine_grained, const int32_t *propagate_down, const int32_t *accum,
                                        float *dx, float *g_qr_min, float *g_qr_max, void *stream);

/* ---- binary-weight and fixed-point affine layers ----------------------------- */

/* Device-side waits in the contraction kernels are time-bounded. A wait that
 * gives up stores a non-zero code in a per-device status word and the kernel
 * returns (its output is then incomplete). This call synchronises `stream`,
 * returns the word in *code (0 = no wait ever gave up) and clears it. */
int nb200_take_device_status(int *code, void *stream);
/* Runs the give-up path of those waits on purpose, harmlessly: a one-block
 * kernel waits on a barrier nobody arrives at, with a limit of limit_us
 * microseconds (1..100000). The kernel returns by itself, the status word
 * holds the producer-timeout code afterwards (read it with
 * nb200_take_device_status) and the context stays usable. *waited_us (may be
 * NULL) receives how long a second role waited before the abort flag
 * released it. No counterpart in the reference (it has no device code). */
int nb200_selftest_wait_timeout(int limit_us, int *waited_us, void *stream);

/* BinaryWeightAffine<float>::forward_impl
 * (src/nbla/function/generic/binary_weight_affine.cpp:74-122).
 * x [rows, w_row], w [w_row, w_col] (the reference's 2-D view of N-D weights,
 * :57-59), bias [w_col] or NULL. WRITES wb = sign(w; quantize_zero_to)
 * [w_row, w_col] and alpha[c] = (sum_r |w[r,c]|) * float(1/w_row) [w_col],
 * like the reference writes inputs[2] and inputs[3]; y [rows, w_col] =
 * (x . wb) * alpha + bias. x is split into three bf16 pieces whose products
 * with the +-1 weights are exact; accumulation is fp32 in tensor memory. */
int nb200_binary_weight_affine_f32(const float *x, const float *w, float *wb, float *alpha, const float *bias,
                                   float *y, int64_t rows, int64_t w_row, int64_t w_col, float quantize_zero_to,
                                   void *stream);
/* BinaryConnectAffine<float>::forward_impl
 * (src/nbla/function/generic/binary_connect_affine.cpp:59-71): as above
 * without alpha. */
int nb200_binary_connect_affine_f32(const float *x, const float *w, float *wb, const float *bias, float *y,
                                    int64_t rows, int64_t w_row, int64_t w_col, float quantize_zero_to,
                                    void *stream);
/* Affine<float>::forward_impl (src/nbla/function/generic/affine.cpp:80-96)
 * for operands that are outputs of FixedPointQuantize with at most 8 bits:
 * xq [rows, w_row] holds multiples of delta_x, wq [w_row, w_col] multiples of
 * delta_w (|code| <= 127). The product runs on the int8 tensor-core path with
 * int32 accumulation; y = float(acc) * (delta_x * delta_w) + bias, which
 * equals the reference's fp32 result whenever that is itself exact. */
int nb200_affine_fxp8_f32(const float *xq, const float *wq, float delta_x, float delta_w, const float *bias, float *y,
                          int64_t rows, int64_t w_row, int64_t w_col, void *stream);
/* Same contraction from the int8 codes that
 * nb200_fixed_point_quantize_f32_codes wrote (x_codes [rows, w_row],
 * w_codes [w_row, w_col]). */
int nb200_affine_codes_i8_f32(const int8_t *x_codes, const int8_t *w_codes, float delta_x, float delta_w,
                              const float *bias, float *y, int64_t rows, int64_t w_row, int64_t w_col, void *stream);
/* The same with the weight codes already in the layout the tensor core reads
 * (K-major: [w_col][w_pitch], w_pitch >= w_row a multiple of 16, padding zero),
 * which nb200_transpose_codes_i8 produces: weights are parameters, so this
 * re-layout is done once per weight update instead of once per call. */
int nb200_transpose_codes_i8(const int8_t *w_codes, int8_t *w_codes_kmajor, int64_t w_row, int64_t w_col,
                             int64_t pitch, void *stream);
int nb200_affine_codes_i8_kmajor_f32(const int8_t *x_codes, const int8_t *w_codes_kmajor, int64_t w_pitch,
                                     float delta_x, float delta_w, const float *bias, float *y, int64_t rows,
                                     int64_t w_row, int64_t w_col, void *stream);
/* Output-column shards of the two contractions above, with the gather of the
 * shards fused into the kernel: this rank owns columns [col_begin, col_begin +
 * w_col) of a [w_row, w_col_total] weight (wq / w_codes and bias are its slab)
 * and stores its [rows, w_col] result into the row-major [rows, w_col_total]
 * matrix of EVERY rank: y_ranks[rank] is this GPU's own, the other entries are
 * mappings of the peers' matrices (nb200_ipc_open). When all ranks' calls have
 * completed, every rank holds the full product; no rank waits on another
 * inside the kernel, so the caller orders the ranks afterwards (a barrier).
 * Replaces Affine::forward_impl (affine.cpp:80-96) on a column shard followed
 * by Communicator::all_gather (include/nbla/communicator.hpp:232-241).
 * n_ranks <= 8; n_ranks == 1 is the unsharded call. */
int nb200_affine_fxp8_gather_f32(const float *xq, const float *wq, float delta_x, float delta_w, const float *bias,
                                 float *const *y_ranks, int n_ranks, int rank, int64_t rows, int64_t w_row,
                                 int64_t w_col, int64_t w_col_total, int64_t col_begin, void *stream);
int nb200_affine_codes_i8_gather_f32(const int8_t *x_codes, const int8_t *w_codes, float delta_x, float delta_w,
                                     const float *bias, float *const *y_ranks, int n_ranks, int rank, int64_t rows,
                                     int64_t w_row, int64_t w_col, int64_t w_col_total, int64_t col_begin,
                                     void *stream);
/* Affine<float>::forward_impl (affine.cpp:80-96) for arbitrary fp32 operands:
 * both are split into bf16 pieces and the six leading piece products are
 * accumulated in fp32 (error of the order of fp32 rounding). */
int nb200_affine_f32(const float *x, const float *w, const float *bias, float *y, int64_t rows, int64_t w_row,
                     int64_t w_col, void *stream);

/* ---- affine backward passes ------------------------------------------------------
 * Affine<float>::backward_impl (src/nbla/function/generic/affine.cpp:98-138)
 * for row-major x [rows, w_row], w [w_row, w_col], dy [rows, w_col]:
 *   dx (+)= dy . w^T,   dw (+)= x^T . dy,   db (+)= column sums of dy.
 * A NULL dx / dw / db is not computed (propagate_down false); accum_* != 0
 * adds to the buffer. Operands are split into bf16 pieces and accumulated in
 * fp32 in tensor memory (error of the order of fp32 rounding). */
int nb200_affine_backward_f32(const float *x, const float *w, const float *dy, float *dx, float *dw, float *db,
                              int64_t rows, int64_t w_row, int64_t w_col, int accum_dx, int accum_dw, int accum_db,
                              void *stream);
/* BinaryWeightAffine<float>::backward_impl
 * (src/nbla/function/generic/binary_weight_affine.cpp:124-146): the affine
 * backward against the scaled binary weights wb * alpha, with the gradient of
 * those weights passed straight through Sign to the float weights
 * (include/nbla/function/sign.hpp:48-50), so dw is the gradient of inputs[1].
 * wb / alpha are what the forward wrote. The products dy * alpha * (+-1) are
 * the reference's own, rounding for rounding. */
int nb200_binary_weight_affine_backward_f32(const float *x, const float *wb, const float *alpha, const float *dy,
                                            float *dx, float *dw, float *db, int64_t rows, int64_t w_row,
                                            int64_t w_col, int accum_dx, int accum_dw, int accum_db, void *stream);
/* BinaryConnectAffine<float>::backward_impl
 * (src/nbla/function/generic/binary_connect_affine.cpp:73-93). */
int nb200_binary_connect_affine_backward_f32(const float *x, const float *wb, const float *dy, float *dx, float *dw,
                                             float *db, int64_t rows, int64_t w_row, int64_t w_col, int accum_dx,
                                             int accum_dw, int accum_db, void *stream);

/* ---- binary-weight convolutions ------------------------------------------------ */

/* BinaryWeightConvolution<float>::forward_impl
 * (src/nbla/function/generic/binary_weight_convolution.cpp:72-117, which calls
 * Convolution<float>::forward_impl, convolution.cpp:160-197). 2-D, NCHW:
 * x [batch, channels, height, width], w [outmaps, channels/group, kernel_h,
 * kernel_w], bias [outmaps] or NULL. WRITES wb = sign(w; quantize_zero_to) and
 * alpha[o] = (sum |w[o,...]|) * float(1/(channels/group*kernel_h*kernel_w))
 * like the reference writes inputs[2] and inputs[3]; y [batch, outmaps, Ho, Wo]
 * = conv(x, wb) * alpha[o] + bias[o] with the reference's output-size rule.
 * The reference unfolds each sample to patches and multiplies per sample;
 * here the convolution is an implicit GEMM fed by TMA boxes of an NHWC copy
 * of x (zero padding = out-of-range fill).
 * activation_delta == 0: x is arbitrary fp32 and is split into three bf16
 * pieces (exact products with the +-1 weights, fp32 accumulation).
 * activation_delta > 0: the caller asserts that x holds integer multiples of
 * activation_delta with |multiple| <= 127 (the output of FixedPointQuantize
 * with n <= 8); the contraction then runs on the int8 path, exactly. */
int nb200_binary_weight_convolution_f32(const float *x, const float *w, float *wb, float *alpha, const float *bias,
                                        float *y, int batch, int channels, int height, int width, int outmaps,
                                        int kernel_h, int kernel_w, int pad_h, int pad_w, int stride_h, int stride_w,
                                        int dilation_h, int dilation_w, int group, float quantize_zero_to,
                                        float activation_delta, void *stream);
/* BinaryConnectConvolution<float>::forward_impl
 * (src/nbla/function/generic/binary_connect_convolution.cpp:67-80): as above
 * without alpha. */
int nb200_binary_connect_convolution_f32(const float *x, const float *w, float *wb, const float *bias, float *y,
                                         int batch, int channels, int height, int width, int outmaps, int kernel_h,
                                         int kernel_w, int pad_h, int pad_w, int stride_h, int stride_w,
                                         int dilation_h, int dilation_w, int group, float quantize_zero_to,
                                         float activation_delta, void *stream);

/* ---- companions: the other functions of a binary-weight ResNet-18 graph ---- */
/* Needed so the whole graph runs under one context with no CPU fallback
 * (nnabla's NNP loader also probes a context with ReLU before using it,
 * python/src/nnabla/utils/load.py:95-103). Bit-identical to the reference's
 * CPU code for non-NaN input, except the convolution (fp32 rounding). */

/* BatchNormalization<float>::forward_impl_global
 * (src/nbla/function/generic/batch_normalization.cpp:228-260), batch_stat =
 * false, one normalised axis: x viewed as [outer, channels, inner];
 * y = (x - mean) * gamma / sqrt(var + eps) + beta in that operation order.
 * beta / gamma may be NULL (no_bias / no_scale). */
int nb200_batch_normalization_inference_f32(const float *x, const float *beta, const float *gamma, const float *mean,
                                            const float *var, float *y, int64_t outer, int64_t channels,
                                            int64_t inner, float eps, void *stream);
/* ReLU<float>::forward_impl (src/nbla/function/generic/relu.cpp). x == y allowed. */
int nb200_relu_f32(const float *x, float *y, size_t size, void *stream);
/* Add2<float>::forward_impl (src/nbla/function/generic/add2.cpp), equal shapes. */
int nb200_add2_f32(const float *a, const float *b, float *y, size_t size, void *stream);
/* x[i] *= factor in place: the division by the number of workers after a summing collective
 * (Communicator::all_reduce with division, include/nbla/communicator.hpp:157-170). */
int nb200_scale_f32(float *x, size_t size, float factor, void *stream);
/* MaxPooling<float>::forward_impl (src/nbla/function/generic/max_pooling.cpp:140-191),
 * 2-D, x [maps, height, width]; output extent by base_pooling.cpp:59. */
int nb200_max_pooling_f32(const float *x, float *y, int64_t maps, int height, int width, int kernel_h, int kernel_w,
                          int stride_h, int stride_w, int pad_h, int pad_w, int ignore_border, void *stream);
/* GlobalAveragePooling<float>::forward_impl
 * (src/nbla/function/generic/global_average_pooling.cpp): x [maps, spatial] -> y [maps]. */
int nb200_global_average_pooling_f32(const float *x, float *y, int64_t maps, int64_t spatial, void *stream);
/* ---- incremental network quantization (INQAffine / INQConvolution) ---- */
/* The weight update of INQAffine<float, int>::forward_impl (src/nbla/function/generic/inq_affine.cpp:82-203)
 * in two calls, around the selection step that the caller performs a few times per training run (:108-148:
 * a sort by magnitude or a Bernoulli draw per learnable weight, then indicator = 1 for the chosen ones):
 *   nb200_inq_restore_f32   :101-105  weights[i] = old_weights[i] where old_indicators[i] == 1
 *   nb200_inq_quantize_f32  :150-203  n1 from max |w|, n2 = n1 + 1 - 2^(num_bits - 2); every weight whose
 *       indicator is 1 (all of them when fix_all != 0, the last INQ iteration, which also sets the
 *       indicators) becomes 0 below 2^(n2 - 1), else sign * 2^e with e = floor(log2 |w|) +
 *       (log2 |w| - floor >= log2 1.5) clipped to [n2, n1]; then weights and indicators are copied to
 *       old_weights / old_indicators. The exponent rule reproduces the host libm's log2f binade by binade
 *       (the step near a mantissa of 1.5 is located with it at first use); NB200_ENOTIMPL if that libm does
 *       not behave as one step per binade. Indicators are int32 (the reference's T1 = int). */
int nb200_inq_restore_f32(float *weights, const float *old_weights, const int32_t *old_indicators, size_t size,
                          void *stream);
int nb200_inq_quantize_f32(float *weights, int32_t *indicators, float *old_weights, int32_t *old_indicators,
                           size_t size, int num_bits, int fix_all, void *stream);

/* ---- training side of the companions ---- */
/* BatchNormalization<float>::forward_impl_batch
 * (src/nbla/function/generic/batch_normalization.cpp:157-226), batch_stat = true, one normalised
 * axis: batch_mean / batch_var [channels] receive the statistics of x (variance = E[x^2] - mean^2),
 * y = (x - mean) * gamma / sqrt(var + eps) + beta in that operation order, and (update_running != 0)
 * running = decay * running + (1 - decay) * batch (the variance unbiased by n / (n - 1)) as :201-205.
 * The per-channel sums are block partials added in a fixed order (deterministic; they agree with the
 * reference's sequential fp32 sums to rounding). beta / gamma may be NULL. */
int nb200_batch_normalization_batch_f32(const float *x, const float *beta, const float *gamma, float *running_mean,
                                        float *running_var, float *y, float *batch_mean, float *batch_var,
                                        int64_t outer, int64_t channels, int64_t inner, float eps, float decay_rate,
                                        int update_running, void *stream);
/* BatchNormalization<float>::backward_impl (batch_normalization.cpp:262-486). batch_stat != 0
 * (backward_impl_batch): mean / var are the batch statistics of the forward pass, dmean / dvar the
 * gradients arriving at the statistics outputs (NULL: none). batch_stat == 0 (backward_impl_global):
 * mean / var are the running statistics, dx = dy * gamma * (var + eps)^-0.5. dx, dbeta, dgamma may
 * each be NULL (not propagated); the accum flags add to what the buffers hold. */
int nb200_batch_normalization_backward_f32(const float *x, const float *dy, const float *gamma, const float *mean,
                                           const float *var, const float *dmean, const float *dvar, float *dx,
                                           float *dbeta, float *dgamma, int64_t outer, int64_t channels,
                                           int64_t inner, float eps, int batch_stat, int accum_dx, int accum_dbeta,
                                           int accum_dgamma, void *stream);
/* ReLU<float>::backward_impl (src/nbla/function/generic/relu.cpp:41-66): dx (+)= y > 0 ? dy : 0 with
 * y the forward OUTPUT. */
int nb200_relu_backward_f32(const float *y, const float *dy, float *dx, size_t size, int accum, void *stream);
/* Add2<float>::backward_impl (src/nbla/function/generic/add2.cpp), equal shapes: one call per input,
 * dx (+)= dy. */
int nb200_add2_backward_f32(const float *dy, float *dx, size_t size, int accum, void *stream);
/* GlobalAveragePooling<float>::backward_impl (global_average_pooling.cpp:75-117):
 * dx[m][.] (+)= dy[m] / spatial. */
int nb200_global_average_pooling_backward_f32(const float *dy, float *dx, int64_t maps, int64_t spatial, int accum,
                                              void *stream);
/* MaxPooling<float>::backward_impl (src/nbla/function/generic/max_pooling.cpp:194-228): dy of every
 * output goes to the FIRST maximum of its clipped window (:63-73), summed in output order, which is
 * how the reference's index map and its `dx[index] += dy` loop behave; x is the forward input. */
int nb200_max_pooling_backward_f32(const float *x, const float *dy, float *dx, int64_t maps, int height, int width,
                                   int kernel_h, int kernel_w, int stride_h, int stride_w, int pad_h, int pad_w,
                                   int ignore_border, int accum, void *stream);
/* Convolution<float>::forward_impl (src/nbla/function/generic/convolution.cpp:160-197)
 * in full precision for layers with few input channels (the network stem):
 * direct convolution, products accumulated with fused multiply-adds in the
 * order of the reference's im2col rows (channel, kernel row, kernel column).
 * group == 1. */
int nb200_convolution_f32(const float *x, const float *w, const float *bias, float *y, int batch, int channels,
                          int height, int width, int outmaps, int kernel_h, int kernel_w, int pad_h, int pad_w,
                          int stride_h, int stride_w, int dilation_h, int dilation_w, int group, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* NNABLA_B200_H_ */
