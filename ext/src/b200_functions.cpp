// Function implementations of the "b200" nnabla extension and init_b200().
//
// Each class derives from the reference's own function class, so name(),
// copy(), in/out types, argument storage and the gradient-dependency
// predicates the graph engine reads (src/nbla/computation_graph/variable.cpp:203-273)
// are the reference's by construction. Overridden: the allowed array classes
// (device arrays), forward_impl (one call into libnnabla_b200.so) and, for the
// composites, setup_impl — the reference's setup creates CPU sub-functions
// through the registry (binary_weight_affine.cpp:35,65-70;
// min_max_quantize.cpp:97-119; batch_normalization.cpp:119-131), which would
// look up "b200:float" for each of them and throw, so only the shape checks and
// the output reshape are repeated here. backward_impl is implemented for the
// quantizers, their siblings, the affine family and the binary convolutions.
#include <nbla_b200/b200.hpp>

#include <nbla/array/cpu_array.hpp>
#include <nbla/array_registry.hpp>
#include <nbla/backend_registry.hpp>
#include <nbla/function/add2.hpp>
#include <nbla/function/affine.hpp>
#include <nbla/function/batch_normalization.hpp>
#include <nbla/function/binary_connect_affine.hpp>
#include <nbla/function/binary_connect_convolution.hpp>
#include <nbla/function/binary_weight_affine.hpp>
#include <nbla/function/binary_weight_convolution.hpp>
#include <nbla/function/convolution.hpp>
#include <nbla/function/fixed_point_quantize.hpp>
#include <nbla/function/global_average_pooling.hpp>
#include <nbla/function/inq_affine.hpp>
#include <nbla/function/inq_convolution.hpp>
#include <nbla/random_manager.hpp>
#include <nbla/function/max_pooling.hpp>
#include <nbla/function/binary_sigmoid.hpp>
#include <nbla/function/binary_tanh.hpp>
#include <nbla/function/dequantize_linear.hpp>
#include <nbla/function/min_max_quantize.hpp>
#include <nbla/function/prune.hpp>
#include <nbla/function/quantize_linear.hpp>
#include <nbla/function/pow2_quantize.hpp>
#include <nbla/function/relu.hpp>
#include <nbla/function_registry.hpp>
#include <nbla/nd_array.hpp>
#include <nbla/utils/axis_utils.hpp>

#include <nnabla_b200.h>
#include <nvtx3/nvToolsExt.h>

#include <algorithm>
#include <mutex>
#include <numeric>
#include <random>

namespace nbla {

void install_write_tracking(); // b200_backend.cpp
void register_b200_communicator(); // b200_communicator.cpp
void synchronizer_cpu_to_b200(Array *src, Array *dst, const int async_flags);
void synchronizer_b200_to_cpu(Array *src, Array *dst, const int async_flags);

namespace {

vector<string> device_array_classes() { return SingletonManager::get<B200>()->array_classes(); }

// Makes the context's device current; returns the stream the function enqueues its work on.
void *enter(const Context &ctx) { return b200_stream(ctx.device_id); }

// NVTX range "<Function>::forward_impl" / "::backward_impl" around every function of the backend, so that a
// timeline shows nnabla's functions over the kernels they launch (header-only NVTX: a few nanoseconds
// when no tool is attached).
struct NvtxRange {
  NvtxRange(const string &function, const char *method) { nvtxRangePushA((function + "::" + method).c_str()); }
  ~NvtxRange() { nvtxRangePop(); }
  NvtxRange(const NvtxRange &) = delete;
  NvtxRange &operator=(const NvtxRange &) = delete;
};
#define B200_ENTER(ST)                                                                                            \
  NvtxRange nvtx_range_(this->name(), __func__);                                                                  \
  void *ST = enter(this->ctx_)

const float *rd(Variable *v, const Context &ctx) { return v->get_data_pointer<float>(ctx); }
// Gradient buffer of an input for backward: NULL when nothing propagates to it.
float *grad_wr(Variable *v, const Context &ctx, bool propagate, bool accum) {
  return propagate ? v->cast_grad_and_get_pointer<float>(ctx, !accum) : nullptr;
}
float *wr(Variable *v, const Context &ctx, bool write_only = true) {
  return v->cast_data_and_get_pointer<float>(ctx, write_only);
}

// Affine::setup_impl's shape rules (src/nbla/function/generic/affine.cpp:29-78).
struct AffineDims {
  Size_t rows, w_row, w_col;
};
AffineDims setup_affine_shapes(int &base_axis, Variable *x, Variable *w, Variable *bias, Variable *y) {
  const Shape_t sx = x->shape(), sw = w->shape();
  NBLA_CHECK(sw.size() >= 2, error_code::value, "Weights(inputs[1]) must be matrix or tensor.");
  refine_axis(base_axis, x->ndim());
  NBLA_CHECK(static_cast<Shape_t::size_type>(base_axis) < sx.size(), error_code::value,
             "Base_axis must be less than ndim of input data(inputs[0]). base_axis: %d >= ndim of input: %d.",
             base_axis, (int)sx.size());
  NBLA_CHECK(x->size(base_axis) == sw[0], error_code::value,
             "Size of input data(inputs[0]) and weights(inputs[1]) mismatch. size of input: %d != size of weights: %d.",
             (int)x->size(base_axis), (int)sw[0]);
  AffineDims d;
  d.w_row = sw[0];
  d.w_col = w->size() / d.w_row;
  d.rows = x->size() / x->size(base_axis);
  Shape_t so(sx.begin(), sx.begin() + base_axis);
  so.insert(so.end(), sw.begin() + 1, sw.end());
  y->reshape(so, true);
  if (bias) {
    const Shape_t sb = bias->shape();
    NBLA_CHECK(sb.size() == sw.size() - 1, error_code::value,
               "Length of bias(inputs[2]) and weights(inputs[1]) mismatch. bias length: %d != weights length-1: %d.",
               (int)sb.size(), (int)sw.size() - 1);
    for (Shape_t::size_type i = 0; i < sb.size(); ++i)
      NBLA_CHECK(sb[i] == sw[i + 1], error_code::value, "Shape of bias(inputs[2]) and weights(inputs[1]) mismatch.");
  }
  return d;
}

void check_same_shape(Variable *w, Variable *wb) {
  NBLA_CHECK(w->shape() == wb->shape(), error_code::value, "Binary and float weights must have same size.");
}

// Convolution::setup_impl's shape rules (src/nbla/function/generic/convolution.cpp:40-158), 2-D NCHW.
struct ConvDims {
  int batch, C, H, W, Ko, kh, kw;
};
ConvDims setup_conv_shapes(int &base_axis, const vector<int> &pad, const vector<int> &stride,
                           const vector<int> &dilation, int group, Variable *x, Variable *w, Variable *bias,
                           Variable *y) {
  const Shape_t sx = x->shape(), sw = w->shape();
  refine_axis(base_axis, x->ndim());
  NBLA_CHECK(static_cast<Shape_t::size_type>(base_axis) < sx.size() - 1, error_code::unclassified,
             "base_axis must be less than ndim - 1 of inputs[0]. base_axis: %d >= ndim of inputs[0] - 1: %d.",
             base_axis, (int)sx.size() - 1);
  const size_t spatial = sx.size() - base_axis - 1;
  NBLA_CHECK(sw.size() == 2 + spatial, error_code::value, "Weights must be a tensor more than 3D.");
  NBLA_CHECK(spatial == 2, error_code::not_implemented, "the b200 backend implements 2-D convolution only");
  NBLA_CHECK(pad.size() == spatial, error_code::value, "pad size mismatch.");
  NBLA_CHECK(stride.size() == spatial, error_code::value, "stride size mismatch.");
  NBLA_CHECK(dilation.size() == spatial, error_code::value, "dilation size mismatch.");
  ConvDims d;
  d.C = sx[base_axis];
  d.H = sx[base_axis + 1];
  d.W = sx[base_axis + 2];
  d.Ko = sw[0];
  d.kh = sw[2];
  d.kw = sw[3];
  NBLA_CHECK(d.C % group == 0, error_code::value,
             "Number of input channel needs to be divisible by group. Input channel: %d, group: %d.", d.C, group);
  NBLA_CHECK(d.Ko % group == 0, error_code::value,
             "Number of output channel needs to be divisible by group. Output channel: %d, group: %d.", d.Ko, group);
  NBLA_CHECK(d.C / group == sw[1], error_code::value, "Number of grouped channel mismatch.");
  Shape_t so(sx.begin(), sx.begin() + base_axis);
  d.batch = 1;
  for (int i = 0; i < base_axis; ++i)
    d.batch *= sx[i];
  so.push_back(d.Ko);
  const int in[2] = {d.H, d.W}, k[2] = {d.kh, d.kw};
  for (int i = 0; i < 2; ++i) {
    const int kk = dilation[i] * (k[i] - 1) + 1;
    const int o = (in[i] + 2 * pad[i] - kk) / stride[i] + 1;
    NBLA_CHECK(in[i] + 2 * pad[i] - kk >= 0 && o > 0, error_code::value,
               "Invalid configuration of convolution at %d-th spatial dimension.  {input:%d, kernel:%d, pad:%d, "
               "stride:%d, dilation:%d}.",
               i, in[i], k[i], pad[i], stride[i], dilation[i]);
    so.push_back(o);
  }
  y->reshape(so, true);
  if (bias) {
    NBLA_CHECK(bias->shape().size() == 1, error_code::value, "Bias(inputs[2]) must be a 1d tensor.");
    NBLA_CHECK(bias->shape()[0] == d.Ko, error_code::value, "Shape of bias(inputs[2]) and weights(inputs[1]) mismatch.");
  }
  return d;
}

// ------------------------------------------------------------- quantizers
template <typename T> class FixedPointQuantizeB200 : public FixedPointQuantize<T> {
public:
  using FixedPointQuantize<T>::FixedPointQuantize;
  virtual vector<string> allowed_array_classes() { return device_array_classes(); }

protected:
  virtual void forward_impl(const Variables &in, const Variables &out) {
    B200_ENTER(st);
    const float *x = rd(in[0], this->ctx_);
    float *y = wr(out[0], this->ctx_);
    const bool small_codes = (this->sign_ ? this->n_ - 1 : this->n_) <= 7;
    const Shape_t shape = in[0]->shape();
    // [N, C, H, W] with planes of a multiple of 4 values: the same pass leaves the int8 channel-last codes that the
    // convolution behind this quantizer reads (its weights are kept prepared, so the codes always save it a pass)
    if (small_codes && shape.size() == 4 && (shape[2] * shape[3]) % 4 == 0 && shape[0] > 0 && shape[0] <= 65535 &&
        in[0]->size() >= (1 << 12) && ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y)) & 15) == 0) {
      const int64_t slots = nb200_codes_nhwc_slots(shape[1], 1);
      NdArrayPtr codes = make_shared<NdArray>(Shape_t{shape[0] * shape[2] * shape[3] * slots});
      int8_t *c = codes->cast(dtypes::BYTE, this->ctx_, true)->template pointer<int8_t>();
      nb200_check(nb200_fixed_point_quantize_nhwc_codes_f32(x, y, c, shape[0], shape[1], shape[2] * shape[3], this->sign_,
                                                            this->n_, this->delta_, st),
                  "FixedPointQuantize (with codes)");
      fxp_tag_set(out[0], this->delta_, codes);
      return;
    }
    nb200_check(nb200_fixed_point_quantize_f32(x, y, in[0]->size(), this->sign_, this->n_, this->delta_, st),
                "FixedPointQuantize");
    if (small_codes)
      fxp_tag_set(out[0], this->delta_);
  }
  // fixed_point_quantize.cpp:103-127
  virtual void backward_impl(const Variables &in, const Variables &out, const vector<bool> &propagate_down,
                             const vector<bool> &accum) {
    if (!propagate_down[0])
      return;
    B200_ENTER(st);
    const float *x = rd(in[0], this->ctx_);
    float *dx = in[0]->cast_grad_and_get_pointer<float>(this->ctx_, !accum[0]);
    const float *dy = out[0]->get_grad_pointer<float>(this->ctx_);
    nb200_check(nb200_fixed_point_quantize_backward_f32(x, dy, dx, in[0]->size(), this->sign_, this->n_, this->delta_,
                                                        this->ste_fine_grained_, accum[0], st),
                "FixedPointQuantize backward");
  }
};

template <typename T> class Pow2QuantizeB200 : public Pow2Quantize<T> {
public:
  using Pow2Quantize<T>::Pow2Quantize;
  virtual vector<string> allowed_array_classes() { return device_array_classes(); }

protected:
  virtual void forward_impl(const Variables &in, const Variables &out) {
    B200_ENTER(st);
    const float *x = rd(in[0], this->ctx_);
    float *y = wr(out[0], this->ctx_);
    nb200_check(nb200_pow2_quantize_f32(x, y, in[0]->size(), this->sign_, this->with_zero_, this->n_, this->m_,
                                        st),
                "Pow2Quantize");
  }
  // pow2_quantize.cpp:127-156
  virtual void backward_impl(const Variables &in, const Variables &out, const vector<bool> &propagate_down,
                             const vector<bool> &accum) {
    if (!propagate_down[0])
      return;
    B200_ENTER(st);
    const float *x = rd(in[0], this->ctx_);
    float *dx = in[0]->cast_grad_and_get_pointer<float>(this->ctx_, !accum[0]);
    const float *dy = out[0]->get_grad_pointer<float>(this->ctx_);
    nb200_check(nb200_pow2_quantize_backward_f32(x, dy, dx, in[0]->size(), this->sign_, this->with_zero_, this->n_,
                                                 this->m_, this->ste_fine_grained_, accum[0], st),
                "Pow2Quantize backward");
  }
};

template <typename T> class MinMaxQuantizeB200 : public MinMaxQuantize<T> {
public:
  using MinMaxQuantize<T>::MinMaxQuantize;
  virtual vector<string> allowed_array_classes() { return device_array_classes(); }

protected:
  virtual void setup_impl(const Variables &in, const Variables &out) {
    // Shape rules of min_max_quantize.cpp:54-83.
    Variable *x = in[0], *q = in[1];
    for (int i = 2; i <= 4; ++i) {
      NBLA_CHECK(in[i]->ndim() == q->ndim(), error_code::value, "All input dimensions must be same.");
      NBLA_CHECK(in[i]->shape() == q->shape(), error_code::value,
                 "All shapes among ql_min, ql_max, qr_min, and qr_max must be same.");
    }
    NBLA_CHECK(q->ndim() == x->ndim(), error_code::value, "x and the quantization ranges must have the same ndim.");
    for (int a = 0; a < q->ndim(); ++a)
      NBLA_CHECK(q->shape()[a] == 1 || q->shape()[a] == x->shape()[a], error_code::value,
                 "x.shape and ql_min.shape must be same except for i-th dimension where ql_min.shape[i] == 1.");
    out[0]->reshape(x->shape(), true);
    this->scale_sptr_ = make_shared<Variable>(q->shape());
  }
  virtual void forward_impl(const Variables &in, const Variables &out) {
    B200_ENTER(st);
    const Shape_t sx = in[0]->shape(), sq = in[1]->shape();
    const float *x = rd(in[0], this->ctx_);
    float *qr_min = wr(in[1], this->ctx_, false), *qr_max = wr(in[2], this->ctx_, false);
    const float *ql_min = rd(in[3], this->ctx_), *ql_max = rd(in[4], this->ctx_);
    float *scale = wr(this->scale_sptr_.get(), this->ctx_);
    float *y = wr(out[0], this->ctx_);
    nb200_check(nb200_min_max_quantize_f32(x, sx.data(), (int)sx.size(), qr_min, qr_max, ql_min, ql_max, sq.data(),
                                           this->decay_, this->x_min_max_, this->ema_, this->eps_, y, scale, st),
                "MinMaxQuantize");
  }
  // min_max_quantize.cpp:225-350
  virtual void backward_impl(const Variables &in, const Variables &out, const vector<bool> &propagate_down,
                             const vector<bool> &accum) {
    NBLA_CHECK(!(propagate_down[3] || propagate_down[4]), error_code::value,
               "Backward to x(inputs[0]), qr_min(inputs[1]), and/or qr_max(inputs[2])"
               "are only allowed.");
    B200_ENTER(st);
    const bool ranges = !(this->x_min_max_ || this->ema_);
    const int32_t pd[3] = {propagate_down[0], ranges && propagate_down[1], ranges && propagate_down[2]};
    const int32_t ac[3] = {accum[0], accum[1], accum[2]};
    if (!(pd[0] || pd[1] || pd[2]))
      return;
    const Shape_t sx = in[0]->shape(), sq = in[1]->shape();
    const float *x = rd(in[0], this->ctx_);
    const float *qr_min = rd(in[1], this->ctx_), *qr_max = rd(in[2], this->ctx_);
    const float *ql_min = rd(in[3], this->ctx_), *ql_max = rd(in[4], this->ctx_);
    const float *dy = out[0]->get_grad_pointer<float>(this->ctx_);
    float *dx = pd[0] ? in[0]->cast_grad_and_get_pointer<float>(this->ctx_, !accum[0]) : nullptr;
    float *g_min = pd[1] ? in[1]->cast_grad_and_get_pointer<float>(this->ctx_, !accum[1]) : nullptr;
    float *g_max = pd[2] ? in[2]->cast_grad_and_get_pointer<float>(this->ctx_, !accum[2]) : nullptr;
    nb200_check(nb200_min_max_quantize_backward_f32(x, sx.data(), (int)sx.size(), qr_min, qr_max, ql_min, ql_max,
                                                    sq.data(), dy, this->x_min_max_, this->ema_,
                                                    this->ste_fine_grained_, pd, ac, dx, g_min, g_max, st),
                "MinMaxQuantize backward");
  }
};

// ------------------------------------------- sibling quantization functions
template <typename T> class BinarySigmoidB200 : public BinarySigmoid<T> {
public:
  using BinarySigmoid<T>::BinarySigmoid;
  virtual vector<string> allowed_array_classes() { return device_array_classes(); }

protected:
  virtual void forward_impl(const Variables &in, const Variables &out) {
    B200_ENTER(st);
    nb200_check(nb200_binary_sigmoid_f32(rd(in[0], this->ctx_), wr(out[0], this->ctx_), in[0]->size(), st),
                "BinarySigmoid");
  }
  virtual void backward_impl(const Variables &in, const Variables &out, const vector<bool> &pd,
                             const vector<bool> &accum) {
    if (!pd[0])
      return;
    B200_ENTER(st);
    const float *x = rd(in[0], this->ctx_), *dy = out[0]->get_grad_pointer<float>(this->ctx_);
    nb200_check(nb200_binary_sigmoid_backward_f32(x, dy, grad_wr(in[0], this->ctx_, true, accum[0]), in[0]->size(),
                                                  accum[0], st),
                "BinarySigmoid backward");
  }
};

template <typename T> class BinaryTanhB200 : public BinaryTanh<T> {
public:
  using BinaryTanh<T>::BinaryTanh;
  virtual vector<string> allowed_array_classes() { return device_array_classes(); }

protected:
  virtual void forward_impl(const Variables &in, const Variables &out) {
    B200_ENTER(st);
    nb200_check(nb200_binary_tanh_f32(rd(in[0], this->ctx_), wr(out[0], this->ctx_), in[0]->size(), st),
                "BinaryTanh");
  }
  virtual void backward_impl(const Variables &in, const Variables &out, const vector<bool> &pd,
                             const vector<bool> &accum) {
    if (!pd[0])
      return;
    B200_ENTER(st);
    const float *x = rd(in[0], this->ctx_), *dy = out[0]->get_grad_pointer<float>(this->ctx_);
    nb200_check(nb200_binary_tanh_backward_f32(x, dy, grad_wr(in[0], this->ctx_, true, accum[0]), in[0]->size(),
                                               accum[0], st),
                "BinaryTanh backward");
  }
};

template <typename T> class PruneB200 : public Prune<T> {
public:
  using Prune<T>::Prune;
  virtual vector<string> allowed_array_classes() { return device_array_classes(); }

protected:
  virtual void forward_impl(const Variables &in, const Variables &out) {
    B200_ENTER(st);
    nb200_check(nb200_prune_f32(rd(in[0], this->ctx_), wr(out[0], this->ctx_), in[0]->size(), this->rate_, st),
                "Prune");
  }
  virtual void backward_impl(const Variables &in, const Variables &out, const vector<bool> &pd,
                             const vector<bool> &accum) {
    if (!pd[0])
      return;
    B200_ENTER(st);
    nb200_check(nb200_prune_backward_f32(out[0]->get_grad_pointer<float>(this->ctx_),
                                         grad_wr(in[0], this->ctx_, true, accum[0]), in[0]->size(), accum[0], st),
                "Prune backward");
  }
};

// Shape rules shared by QuantizeLinear / DequantizeLinear (quantize_linear.cpp:27-48).
void setup_linear_shapes(const Variables &in, const Variables &out) {
  NBLA_CHECK(in[0]->ndim() == in[1]->ndim() && in[0]->ndim() == in[2]->ndim(), error_code::value,
             "Dimensions of inputs must be same (%d, %d, %d).", in[0]->ndim(), in[1]->ndim(), in[2]->ndim());
  for (int i = 0; i < in[0]->ndim(); ++i)
    for (int k = 1; k <= 2; ++k)
      NBLA_CHECK(in[k]->shape()[i] == 1 || in[k]->shape()[i] == in[0]->shape()[i], error_code::value,
                 "Size at %d-th dimension of inputs[%d] (%d) should be 1 or match the size at %d-th dimension of "
                 "inputs[0] (%d).",
                 i, k, (int)in[k]->shape()[i], i, (int)in[0]->shape()[i]);
  out[0]->reshape(in[0]->shape(), true);
}

template <typename T> class QuantizeLinearB200 : public QuantizeLinear<T> {
public:
  using QuantizeLinear<T>::QuantizeLinear;
  virtual vector<string> allowed_array_classes() { return device_array_classes(); }

protected:
  virtual void setup_impl(const Variables &in, const Variables &out) { setup_linear_shapes(in, out); }
  virtual void forward_impl(const Variables &in, const Variables &out) {
    B200_ENTER(st);
    NBLA_CHECK(this->round_mode_ == "HALF_AWAY_FROM_ZERO" || this->round_mode_ == "HALF_TO_EVEN", error_code::value,
               "unknown round_mode %s", this->round_mode_.c_str());
    const Shape_t sx = in[0]->shape(), ss = in[1]->shape(), sz = in[2]->shape();
    const float *x = rd(in[0], this->ctx_), *scale = rd(in[1], this->ctx_);
    float *zp = wr(in[2], this->ctx_, false);
    nb200_check(nb200_quantize_linear_f32(x, sx.data(), (int)sx.size(), scale, ss.data(), zp, sz.data(),
                                          wr(out[0], this->ctx_), this->round_mode_ == "HALF_TO_EVEN",
                                          this->narrow_range_, this->dtype_, st),
                "QuantizeLinear");
  }
  virtual void backward_impl(const Variables &in, const Variables &out, const vector<bool> &pd,
                             const vector<bool> &accum) {
    if (!(pd[0] || pd[1] || pd[2]))
      return;
    NBLA_CHECK(!pd[1], error_code::not_implemented, "Backward w.r.t. the scale is not supported now.");
    NBLA_CHECK(!pd[2], error_code::not_implemented, "Backward w.r.t. the zero point is not supported now.");
    B200_ENTER(st);
    const Shape_t sx = in[0]->shape(), ss = in[1]->shape();
    const float *dy = out[0]->get_grad_pointer<float>(this->ctx_), *scale = rd(in[1], this->ctx_);
    nb200_check(nb200_quantize_linear_backward_f32(dy, sx.data(), (int)sx.size(), scale, ss.data(),
                                                   grad_wr(in[0], this->ctx_, true, accum[0]), accum[0], st),
                "QuantizeLinear backward");
  }
};

template <typename T> class DequantizeLinearB200 : public DequantizeLinear<T> {
public:
  using DequantizeLinear<T>::DequantizeLinear;
  virtual vector<string> allowed_array_classes() { return device_array_classes(); }

protected:
  virtual void setup_impl(const Variables &in, const Variables &out) { setup_linear_shapes(in, out); }
  virtual void forward_impl(const Variables &in, const Variables &out) {
    B200_ENTER(st);
    const Shape_t sx = in[0]->shape(), ss = in[1]->shape(), sz = in[2]->shape();
    nb200_check(nb200_dequantize_linear_f32(rd(in[0], this->ctx_), sx.data(), (int)sx.size(), rd(in[1], this->ctx_),
                                            ss.data(), rd(in[2], this->ctx_), sz.data(), wr(out[0], this->ctx_),
                                            st),
                "DequantizeLinear");
  }
  virtual void backward_impl(const Variables &in, const Variables &out, const vector<bool> &pd,
                             const vector<bool> &accum) {
    if (!(pd[0] || pd[1] || pd[2]))
      return;
    NBLA_CHECK(!pd[1], error_code::not_implemented, "Backward w.r.t. the scale is not supported now.");
    NBLA_CHECK(!pd[2], error_code::not_implemented, "Backward w.r.t. the zero point is not supported now.");
    B200_ENTER(st);
    const Shape_t sx = in[0]->shape(), ss = in[1]->shape();
    const float *dy = out[0]->get_grad_pointer<float>(this->ctx_), *scale = rd(in[1], this->ctx_);
    nb200_check(nb200_dequantize_linear_backward_f32(dy, sx.data(), (int)sx.size(), scale, ss.data(),
                                                     grad_wr(in[0], this->ctx_, true, accum[0]), accum[0], st),
                "DequantizeLinear backward");
  }
};

// --------------------------------------------------------- binary affines
template <typename T> class BinaryWeightAffineB200 : public BinaryWeightAffine<T> {
  Size_t rows_;

public:
  using BinaryWeightAffine<T>::BinaryWeightAffine;
  virtual vector<string> allowed_array_classes() { return device_array_classes(); }

protected:
  virtual void setup_impl(const Variables &in, const Variables &out) {
    const AffineDims d = setup_affine_shapes(this->base_axis_, in[0], in[1], in.size() == 5 ? in[4] : nullptr, out[0]);
    check_same_shape(in[1], in[2]);
    rows_ = d.rows;
    this->w_row_ = d.w_row;
    this->w_col_ = d.w_col;
    NBLA_CHECK(in[3]->size() == this->w_col_, error_code::value, "Size of alpha must be equal to output size.");
  }
  virtual void forward_impl(const Variables &in, const Variables &out) {
    B200_ENTER(st);
    const float *x = rd(in[0], this->ctx_), *w = rd(in[1], this->ctx_);
    float *wb = wr(in[2], this->ctx_), *alpha = wr(in[3], this->ctx_);
    const float *b = in.size() == 5 ? rd(in[4], this->ctx_) : nullptr;
    float *y = wr(out[0], this->ctx_);
    nb200_check(nb200_binary_weight_affine_f32(x, w, wb, alpha, b, y, rows_, this->w_row_, this->w_col_,
                                               this->quantize_zero_to_, st),
                "BinaryWeightAffine");
  }
  // binary_weight_affine.cpp:124-146; inputs [x, w, wb, alpha, b?]
  virtual void backward_impl(const Variables &in, const Variables &out, const vector<bool> &pd,
                             const vector<bool> &accum) {
    const bool has_b = in.size() == 5;
    if (!(pd[0] || pd[1] || (has_b && pd[4])))
      return;
    B200_ENTER(st);
    const float *x = rd(in[0], this->ctx_), *wb = rd(in[2], this->ctx_), *alpha = rd(in[3], this->ctx_);
    const float *dy = out[0]->get_grad_pointer<float>(this->ctx_);
    float *dx = grad_wr(in[0], this->ctx_, pd[0], accum[0]), *dw = grad_wr(in[1], this->ctx_, pd[1], accum[1]);
    float *db = has_b ? grad_wr(in[4], this->ctx_, pd[4], accum[4]) : nullptr;
    nb200_check(nb200_binary_weight_affine_backward_f32(x, wb, alpha, dy, dx, dw, db, rows_, this->w_row_,
                                                        this->w_col_, accum[0], accum[1], has_b && accum[4], st),
                "BinaryWeightAffine backward");
  }
};

template <typename T> class BinaryConnectAffineB200 : public BinaryConnectAffine<T> {
  AffineDims d_;

public:
  using BinaryConnectAffine<T>::BinaryConnectAffine;
  virtual vector<string> allowed_array_classes() { return device_array_classes(); }

protected:
  virtual void setup_impl(const Variables &in, const Variables &out) {
    d_ = setup_affine_shapes(this->base_axis_, in[0], in[1], in.size() == 4 ? in[3] : nullptr, out[0]);
    check_same_shape(in[1], in[2]);
  }
  virtual void forward_impl(const Variables &in, const Variables &out) {
    B200_ENTER(st);
    const float *x = rd(in[0], this->ctx_), *w = rd(in[1], this->ctx_);
    float *wb = wr(in[2], this->ctx_);
    const float *b = in.size() == 4 ? rd(in[3], this->ctx_) : nullptr;
    float *y = wr(out[0], this->ctx_);
    nb200_check(nb200_binary_connect_affine_f32(x, w, wb, b, y, d_.rows, d_.w_row, d_.w_col, this->quantize_zero_to_,
                                                st),
                "BinaryConnectAffine");
  }
  // binary_connect_affine.cpp:73-93; inputs [x, w, wb, b?]
  virtual void backward_impl(const Variables &in, const Variables &out, const vector<bool> &pd,
                             const vector<bool> &accum) {
    const bool has_b = in.size() == 4;
    if (!(pd[0] || pd[1] || (has_b && pd[3])))
      return;
    B200_ENTER(st);
    const float *x = rd(in[0], this->ctx_), *wb = rd(in[2], this->ctx_);
    const float *dy = out[0]->get_grad_pointer<float>(this->ctx_);
    float *dx = grad_wr(in[0], this->ctx_, pd[0], accum[0]);
    // Like the reference, the weight gradient is first written to the gradient of the BINARY weights
    // (inputs[2], overwritten) and from there passed through Sign to the float weights' gradient.
    float *dwb = grad_wr(in[2], this->ctx_, pd[1], false);
    float *db = has_b ? grad_wr(in[3], this->ctx_, pd[3], accum[3]) : nullptr;
    nb200_check(nb200_binary_connect_affine_backward_f32(x, wb, dy, dx, dwb, db, d_.rows, d_.w_row, d_.w_col, accum[0],
                                                         0, has_b && accum[3], st),
                "BinaryConnectAffine backward");
    if (pd[1]) {
      float *dw = grad_wr(in[1], this->ctx_, true, accum[1]);
      const size_t n = in[1]->size();
      if (accum[1])
        nb200_check(nb200_add2_f32(dw, dwb, dw, n, st), "BinaryConnectAffine backward (accumulate)");
      else
        nb200_check(nb200_memcpy_d2d(dw, dwb, n * sizeof(float), st), "BinaryConnectAffine backward (copy)");
    }
  }
};

// ---------------------------------------------------- binary convolutions
template <typename T> class BinaryWeightConvolutionB200 : public BinaryWeightConvolution<T> {
  ConvDims d_;
  // The weights' int8 side-band for the tensor cores, kept across calls while the float weights
  // (and the Wb / alpha this function wrote) are unchanged: their data stamps are the key.
  NdArrayPtr side_;
  DataStamp w_stamp_, wb_stamp_, alpha_stamp_;

public:
  using BinaryWeightConvolution<T>::BinaryWeightConvolution;
  virtual vector<string> allowed_array_classes() { return device_array_classes(); }

protected:
  virtual void setup_impl(const Variables &in, const Variables &out) {
    d_ = setup_conv_shapes(this->base_axis_, this->pad_, this->stride_, this->dilation_, this->group_, in[0], in[1],
                           in.size() == 5 ? in[4] : nullptr, out[0]);
    check_same_shape(in[1], in[2]);
    NBLA_CHECK(in[3]->size() == d_.Ko, error_code::value, "Size of alpha must be equal to the number of output maps.");
  }
  virtual void forward_impl(const Variables &in, const Variables &out) {
    B200_ENTER(st);
    const float delta = fxp_tag_get(in[0]);
    const bool sign_ok = this->quantize_zero_to_ == 1.f || this->quantize_zero_to_ == -1.f ||
                         this->quantize_zero_to_ == 0.f;
    const float *x = rd(in[0], this->ctx_);
    const float *b = in.size() == 5 ? rd(in[4], this->ctx_) : nullptr;
    if (sign_ok && delta > 0.f) {
      // 8-bit fixed-point activations: exact int8 contraction. The weights are binarised (Wb, alpha
      // and the side-band written) only when they changed since the last call.
      b200_count("int8_convolutions");
      const bool hit = side_ && data_stamp(in[1]) == w_stamp_ && data_stamp(in[2]) == wb_stamp_ &&
                       data_stamp(in[3]) == alpha_stamp_;
      if (!hit) {
        b200_count("weight_cache_misses");
        const float *w = rd(in[1], this->ctx_);
        float *wb = wr(in[2], this->ctx_), *alpha = wr(in[3], this->ctx_);
        const int64_t bytes = nb200_binary_weights_side_bytes(d_.Ko, d_.C, d_.kh, d_.kw, this->group_);
        side_ = make_shared<NdArray>(Shape_t{bytes});
        int8_t *side = side_->cast(dtypes::BYTE, this->ctx_, true)->template pointer<int8_t>();
        nb200_check(nb200_binary_weights_prepare_i8(w, wb, alpha, side, d_.Ko, d_.C, d_.kh, d_.kw, this->group_,
                                                    this->quantize_zero_to_, st),
                    "BinaryWeightConvolution (weights)");
        w_stamp_ = data_stamp(in[1]);
        wb_stamp_ = data_stamp(in[2]);
        alpha_stamp_ = data_stamp(in[3]);
      } else {
        b200_count("weight_cache_hits");
      }
      const int8_t *side = side_->get(dtypes::BYTE, this->ctx_)->template const_pointer<int8_t>();
      const float *alpha = rd(in[3], this->ctx_);
      const int64_t slots = nb200_codes_nhwc_slots(d_.C, this->group_);
      const int64_t n_codes = (int64_t)d_.batch * d_.H * d_.W * slots;
      // the quantizer that made the input may have left its codes (one group, this very layout)
      NdArrayPtr left = this->group_ == 1 ? fxp_tag_codes(in[0]) : nullptr;
      if (left && left->size() != n_codes)
        left = nullptr;
      NdArray codes(Shape_t{left ? 1 : n_codes});
      const int8_t *xc;
      if (left) {
        b200_count("activation_codes_from_quantizer");
        xc = left->get(dtypes::BYTE, this->ctx_)->template const_pointer<int8_t>();
      } else {
        int8_t *fresh = codes.cast(dtypes::BYTE, this->ctx_, true)->template pointer<int8_t>();
        nb200_check(nb200_fixed_point_codes_nhwc(x, fresh, d_.batch, d_.C, (int64_t)d_.H * d_.W, this->group_, delta, st),
                    "BinaryWeightConvolution (activation codes)");
        xc = fresh;
      }
      float *y = wr(out[0], this->ctx_);
      nb200_check(nb200_binary_convolution_codes_prepared_f32(
                      xc, side, alpha, b, y, d_.batch, d_.C, d_.H, d_.W, d_.Ko, d_.kh, d_.kw, this->pad_[0],
                      this->pad_[1], this->stride_[0], this->stride_[1], this->dilation_[0], this->dilation_[1],
                      this->group_, delta, st),
                  "BinaryWeightConvolution");
      return;
    }
    b200_count("bf16_convolutions");
    const float *w = rd(in[1], this->ctx_);
    float *wb = wr(in[2], this->ctx_), *alpha = wr(in[3], this->ctx_);
    float *y = wr(out[0], this->ctx_);
    nb200_check(nb200_binary_weight_convolution_f32(
                    x, w, wb, alpha, b, y, d_.batch, d_.C, d_.H, d_.W, d_.Ko, d_.kh, d_.kw, this->pad_[0],
                    this->pad_[1], this->stride_[0], this->stride_[1], this->dilation_[0], this->dilation_[1],
                    this->group_, this->quantize_zero_to_, sign_ok ? delta : 0.0f, st),
                "BinaryWeightConvolution");
  }
  // binary_weight_convolution.cpp:119-146; inputs [x, w, wb, alpha, b?]
  virtual void backward_impl(const Variables &in, const Variables &out, const vector<bool> &pd,
                             const vector<bool> &accum) {
    const bool has_b = in.size() == 5;
    if (!(pd[0] || pd[1] || (has_b && pd[4])))
      return;
    B200_ENTER(st);
    const float delta = fxp_tag_get(in[0]);
    const float *x = rd(in[0], this->ctx_), *wb = rd(in[2], this->ctx_), *alpha = rd(in[3], this->ctx_);
    const float *dy = out[0]->get_grad_pointer<float>(this->ctx_);
    float *dx = grad_wr(in[0], this->ctx_, pd[0], accum[0]), *dw = grad_wr(in[1], this->ctx_, pd[1], accum[1]);
    float *db = has_b ? grad_wr(in[4], this->ctx_, pd[4], accum[4]) : nullptr;
    nb200_check(nb200_binary_weight_convolution_backward_f32(
                    x, wb, alpha, dy, dx, dw, db, d_.batch, d_.C, d_.H, d_.W, d_.Ko, d_.kh, d_.kw, this->pad_[0],
                    this->pad_[1], this->stride_[0], this->stride_[1], this->dilation_[0], this->dilation_[1],
                    this->group_, accum[0], accum[1], has_b && accum[4], delta, st),
                "BinaryWeightConvolution backward");
  }
};

template <typename T> class BinaryConnectConvolutionB200 : public BinaryConnectConvolution<T> {
  ConvDims d_;

public:
  using BinaryConnectConvolution<T>::BinaryConnectConvolution;
  virtual vector<string> allowed_array_classes() { return device_array_classes(); }

protected:
  virtual void setup_impl(const Variables &in, const Variables &out) {
    d_ = setup_conv_shapes(this->base_axis_, this->pad_, this->stride_, this->dilation_, this->group_, in[0], in[1],
                           in.size() == 4 ? in[3] : nullptr, out[0]);
    check_same_shape(in[1], in[2]);
  }
  virtual void forward_impl(const Variables &in, const Variables &out) {
    B200_ENTER(st);
    const float delta = fxp_tag_get(in[0]);
    const bool sign_ok = this->quantize_zero_to_ == 1.f || this->quantize_zero_to_ == -1.f ||
                         this->quantize_zero_to_ == 0.f;
    const float *x = rd(in[0], this->ctx_), *w = rd(in[1], this->ctx_);
    float *wb = wr(in[2], this->ctx_);
    const float *b = in.size() == 4 ? rd(in[3], this->ctx_) : nullptr;
    float *y = wr(out[0], this->ctx_);
    nb200_check(nb200_binary_connect_convolution_f32(
                    x, w, wb, b, y, d_.batch, d_.C, d_.H, d_.W, d_.Ko, d_.kh, d_.kw, this->pad_[0], this->pad_[1],
                    this->stride_[0], this->stride_[1], this->dilation_[0], this->dilation_[1], this->group_,
                    this->quantize_zero_to_, sign_ok ? delta : 0.0f, st),
                "BinaryConnectConvolution");
  }
  // binary_connect_convolution.cpp:82-104; inputs [x, w, wb, b?]. Like the reference, the weight gradient
  // is first written to the gradient of the binary weights (inputs[2]) and passed through Sign from there.
  virtual void backward_impl(const Variables &in, const Variables &out, const vector<bool> &pd,
                             const vector<bool> &accum) {
    const bool has_b = in.size() == 4;
    if (!(pd[0] || pd[1] || (has_b && pd[3])))
      return;
    B200_ENTER(st);
    const float delta = fxp_tag_get(in[0]);
    const float *x = rd(in[0], this->ctx_), *wb = rd(in[2], this->ctx_);
    const float *dy = out[0]->get_grad_pointer<float>(this->ctx_);
    float *dx = grad_wr(in[0], this->ctx_, pd[0], accum[0]);
    float *dwb = grad_wr(in[2], this->ctx_, pd[1], false);
    float *db = has_b ? grad_wr(in[3], this->ctx_, pd[3], accum[3]) : nullptr;
    nb200_check(nb200_binary_connect_convolution_backward_f32(
                    x, wb, dy, dx, dwb, db, d_.batch, d_.C, d_.H, d_.W, d_.Ko, d_.kh, d_.kw, this->pad_[0],
                    this->pad_[1], this->stride_[0], this->stride_[1], this->dilation_[0], this->dilation_[1],
                    this->group_, accum[0], 0, has_b && accum[3], delta, st),
                "BinaryConnectConvolution backward");
    if (pd[1]) {
      float *dw = grad_wr(in[1], this->ctx_, true, accum[1]);
      const size_t n = in[1]->size();
      if (accum[1])
        nb200_check(nb200_add2_f32(dw, dwb, dw, n, st), "BinaryConnectConvolution backward (accumulate)");
      else
        nb200_check(nb200_memcpy_d2d(dw, dwb, n * sizeof(float), st), "BinaryConnectConvolution backward (copy)");
    }
  }
};

// ------------------------------------------------------------- companions
template <typename T> class AffineB200 : public Affine<T> {
  AffineDims d_;

public:
  using Affine<T>::Affine;
  virtual vector<string> allowed_array_classes() { return device_array_classes(); }

protected:
  virtual void setup_impl(const Variables &in, const Variables &out) {
    d_ = setup_affine_shapes(this->base_axis_, in[0], in[1], in.size() == 3 ? in[2] : nullptr, out[0]);
  }
  virtual void forward_impl(const Variables &in, const Variables &out) {
    B200_ENTER(st);
    const float dx = fxp_tag_get(in[0]), dw = fxp_tag_get(in[1]);
    const float *x = rd(in[0], this->ctx_), *w = rd(in[1], this->ctx_);
    const float *b = in.size() == 3 ? rd(in[2], this->ctx_) : nullptr;
    float *y = wr(out[0], this->ctx_);
    if (dx > 0.f && dw > 0.f && d_.w_row <= 133000)
      b200_count("int8_affines");
    if (dx > 0.f && dw > 0.f && d_.w_row <= 133000)
      nb200_check(nb200_affine_fxp8_f32(x, w, dx, dw, b, y, d_.rows, d_.w_row, d_.w_col, st),
                  "Affine (fixed-point operands)");
    else
      nb200_check(nb200_affine_f32(x, w, b, y, d_.rows, d_.w_row, d_.w_col, st), "Affine");
  }
  // affine.cpp:98-138; inputs [x, w, b?]
  virtual void backward_impl(const Variables &in, const Variables &out, const vector<bool> &pd,
                             const vector<bool> &accum) {
    const bool has_b = in.size() == 3;
    if (!(pd[0] || pd[1] || (has_b && pd[2])))
      return;
    B200_ENTER(st);
    const float *x = rd(in[0], this->ctx_), *w = rd(in[1], this->ctx_);
    const float *dy = out[0]->get_grad_pointer<float>(this->ctx_);
    float *dx = grad_wr(in[0], this->ctx_, pd[0], accum[0]), *dw = grad_wr(in[1], this->ctx_, pd[1], accum[1]);
    float *db = has_b ? grad_wr(in[2], this->ctx_, pd[2], accum[2]) : nullptr;
    nb200_check(nb200_affine_backward_f32(x, w, dy, dx, dw, db, d_.rows, d_.w_row, d_.w_col, accum[0], accum[1],
                                          has_b && accum[2], st),
                "Affine backward");
  }
};

template <typename T> class ConvolutionB200 : public Convolution<T> {
  ConvDims d_;

public:
  using Convolution<T>::Convolution;
  virtual vector<string> allowed_array_classes() { return device_array_classes(); }

protected:
  virtual void setup_impl(const Variables &in, const Variables &out) {
    NBLA_CHECK(!this->channel_last_, error_code::not_implemented, "channel_last is not supported");
    d_ = setup_conv_shapes(this->base_axis_, this->pad_, this->stride_, this->dilation_, this->group_, in[0], in[1],
                           in.size() == 3 ? in[2] : nullptr, out[0]);
  }
  virtual void forward_impl(const Variables &in, const Variables &out) {
    B200_ENTER(st);
    const float *x = rd(in[0], this->ctx_), *w = rd(in[1], this->ctx_);
    const float *b = in.size() == 3 ? rd(in[2], this->ctx_) : nullptr;
    float *y = wr(out[0], this->ctx_);
    nb200_check(nb200_convolution_f32(x, w, b, y, d_.batch, d_.C, d_.H, d_.W, d_.Ko, d_.kh, d_.kw, this->pad_[0],
                                      this->pad_[1], this->stride_[0], this->stride_[1], this->dilation_[0],
                                      this->dilation_[1], this->group_, st),
                "Convolution");
  }
  // convolution.cpp:199-300: weight and bias gradients; the input gradient of a full-precision
  // convolution (a network's first layer) is not provided by the b200 library.
  virtual void backward_impl(const Variables &in, const Variables &out, const vector<bool> &pd,
                             const vector<bool> &accum) {
    const bool has_b = in.size() == 3;
    if (!(pd[0] || pd[1] || (has_b && pd[2])))
      return;
    B200_ENTER(st);
    const float *x = rd(in[0], this->ctx_);
    const float *dy = out[0]->get_grad_pointer<float>(this->ctx_);
    if (pd[0]) {
      const float *w = rd(in[1], this->ctx_);
      float *dx = grad_wr(in[0], this->ctx_, true, accum[0]);
      nb200_check(nb200_convolution_input_backward_f32(w, dy, dx, d_.batch, d_.C, d_.H, d_.W, d_.Ko, d_.kh, d_.kw,
                                                       this->pad_[0], this->pad_[1], this->stride_[0], this->stride_[1],
                                                       this->dilation_[0], this->dilation_[1], this->group_, accum[0],
                                                       st),
                  "Convolution backward (input)");
    }
    if (!(pd[1] || (has_b && pd[2])))
      return;
    float *dw = grad_wr(in[1], this->ctx_, pd[1], accum[1]);
    float *db = has_b ? grad_wr(in[2], this->ctx_, pd[2], accum[2]) : nullptr;
    nb200_check(nb200_convolution_backward_f32(x, dy, dw, db, d_.batch, d_.C, d_.H, d_.W, d_.Ko, d_.kh, d_.kw,
                                               this->pad_[0], this->pad_[1], this->stride_[0], this->stride_[1],
                                               this->dilation_[0], this->dilation_[1], this->group_,
                                               pd[1] && accum[1], has_b && pd[2] && accum[2], st),
                "Convolution backward");
  }
};

template <typename T> class BatchNormalizationB200 : public BatchNormalization<T> {
public:
  using BatchNormalization<T>::BatchNormalization;
  virtual vector<string> allowed_array_classes() { return device_array_classes(); }

protected:
  virtual void setup_impl(const Variables &in, const Variables &out) {
    // Index and size rules of batch_normalization.cpp:31-115.
    NBLA_CHECK(this->axes_.size() == 1, error_code::not_implemented, "Specifying axis more than one is not supported");
    NBLA_CHECK(out.size() == 1 || out.size() == 3, error_code::value, "1 or 3 outputs are expected.");
    NBLA_CHECK(this->batch_stat_ || out.size() == 1, error_code::value,
               "If batch_stat_ is false, it cannot output batch mean and variance.");
    const int n = (int)in.size();
    this->b_idx_ = this->no_bias_ ? -1 : 1;
    this->g_idx_ = this->no_scale_ ? -1 : (this->no_bias_ ? 1 : 2);
    this->m_idx_ = n - 2;
    this->v_idx_ = n - 1;
    NBLA_CHECK(n == 3 + (this->no_bias_ ? 0 : 1) + (this->no_scale_ ? 0 : 1), error_code::value,
               "Number of inputs does not match no_scale / no_bias.");
    const Shape_t sx = in[0]->shape();
    refine_axis(this->axes_[0], in[0]->ndim());
    const Size_t size = in[0]->size();
    const Size_t size_axis = in[0]->size(this->axes_[0]);
    this->size0_ = size / size_axis;
    this->size1_ = sx[this->axes_[0]];
    this->size2_ = size / this->size0_ / this->size1_;
    this->size12_ = this->size1_ * this->size2_;
    this->size02_ = this->size0_ * this->size2_;
    for (int i = 1; i < n; ++i)
      NBLA_CHECK(in[i]->size() == this->size1_, error_code::value,
                 "Shape of inputs[%d] does not match the normalised axis (%d elements expected).", i,
                 (int)this->size1_);
    out[0]->reshape(sx, true);
    const Shape_t sm = in[this->m_idx_]->shape();
    if (out.size() == 3) {
      out[1]->reshape(sm, true);
      out[2]->reshape(sm, true);
    } else {
      this->mean_.reshape(sm, true);
      this->var_.reshape(sm, true);
    }
  }
  Variable *batch_mean(const Variables &out) { return out.size() == 3 ? out[1] : &this->mean_; }
  Variable *batch_var(const Variables &out) { return out.size() == 3 ? out[2] : &this->var_; }
  void run_forward(const Variables &in, const Variables &out, bool update_running) {
    B200_ENTER(st);
    const float *x = rd(in[0], this->ctx_);
    const float *beta = this->no_bias_ ? nullptr : rd(in[this->b_idx_], this->ctx_);
    const float *gamma = this->no_scale_ ? nullptr : rd(in[this->g_idx_], this->ctx_);
    float *y = wr(out[0], this->ctx_);
    if (!this->batch_stat_) {
      const float *mean = rd(in[this->m_idx_], this->ctx_), *var = rd(in[this->v_idx_], this->ctx_);
      nb200_check(nb200_batch_normalization_inference_f32(x, beta, gamma, mean, var, y, this->size0_, this->size1_,
                                                          this->size2_, this->eps_, st),
                  "BatchNormalization");
      return;
    }
    // forward_impl_batch (batch_normalization.cpp:157-226): the running statistics are inputs written in place
    float *m = wr(batch_mean(out), this->ctx_), *v = wr(batch_var(out), this->ctx_);
    float *rm = update_running ? wr(in[this->m_idx_], this->ctx_, false) : nullptr;
    float *rv = update_running ? wr(in[this->v_idx_], this->ctx_, false) : nullptr;
    nb200_check(nb200_batch_normalization_batch_f32(x, beta, gamma, rm, rv, y, m, v, this->size0_, this->size1_,
                                                    this->size2_, this->eps_, this->decay_rate_, update_running, st),
                "BatchNormalization");
  }
  virtual void forward_impl(const Variables &in, const Variables &out) { run_forward(in, out, true); }
  virtual void recompute_impl(const Variables &in, const Variables &out) { run_forward(in, out, false); }
  // batch_normalization.cpp:262-486 (both modes)
  virtual void backward_impl(const Variables &in, const Variables &out, const vector<bool> &pd,
                             const vector<bool> &accum) {
    const bool pd_beta = !this->no_bias_ && pd[this->b_idx_];
    const bool pd_gamma = !this->no_scale_ && pd[this->g_idx_];
    if (!(pd[0] || pd_beta || pd_gamma))
      return;
    B200_ENTER(st);
    const float *x = rd(in[0], this->ctx_);
    const float *dy = out[0]->get_grad_pointer<float>(this->ctx_);
    const float *gamma = this->no_scale_ ? nullptr : rd(in[this->g_idx_], this->ctx_);
    const float *mean, *var, *dm = nullptr, *dv = nullptr;
    if (this->batch_stat_) {
      mean = rd(batch_mean(out), this->ctx_);
      var = rd(batch_var(out), this->ctx_);
      if (out.size() == 3) {
        dm = out[1]->get_grad_pointer<float>(this->ctx_);
        dv = out[2]->get_grad_pointer<float>(this->ctx_);
      }
    } else {
      mean = rd(in[this->m_idx_], this->ctx_);
      var = rd(in[this->v_idx_], this->ctx_);
    }
    float *dx = grad_wr(in[0], this->ctx_, pd[0], accum[0]);
    float *db = pd_beta ? grad_wr(in[this->b_idx_], this->ctx_, true, accum[this->b_idx_]) : nullptr;
    float *dg = pd_gamma ? grad_wr(in[this->g_idx_], this->ctx_, true, accum[this->g_idx_]) : nullptr;
    nb200_check(nb200_batch_normalization_backward_f32(
                    x, dy, gamma, mean, var, dm, dv, dx, db, dg, this->size0_, this->size1_, this->size2_, this->eps_,
                    this->batch_stat_, pd[0] && accum[0], pd_beta && accum[this->b_idx_],
                    pd_gamma && accum[this->g_idx_], st),
                "BatchNormalization backward");
  }
};

template <typename T> class ReLUB200 : public ReLU<T> {
public:
  using ReLU<T>::ReLU;
  virtual vector<string> allowed_array_classes() { return device_array_classes(); }

protected:
  virtual void forward_impl(const Variables &in, const Variables &out) {
    B200_ENTER(st);
    const float tag = fxp_tag_get(in[0]);
    const float *x = rd(in[0], this->ctx_);
    float *y = wr(out[0], this->ctx_);
    nb200_check(nb200_relu_f32(x, y, in[0]->size(), st), "ReLU");
    if (tag > 0.f)
      fxp_tag_set(out[0], tag); // max(0, k * delta) is still a multiple of delta
  }
  // relu.cpp:52-66
  virtual void backward_impl(const Variables &in, const Variables &out, const vector<bool> &pd,
                             const vector<bool> &accum) {
    if (!pd[0])
      return;
    B200_ENTER(st);
    const float *y = rd(out[0], this->ctx_);
    const float *dy = out[0]->get_grad_pointer<float>(this->ctx_);
    float *dx = grad_wr(in[0], this->ctx_, true, accum[0]);
    nb200_check(nb200_relu_backward_f32(y, dy, dx, in[0]->size(), accum[0], st), "ReLU backward");
  }
};

template <typename T> class Add2B200 : public Add2<T> {
public:
  using Add2<T>::Add2;
  virtual vector<string> allowed_array_classes() { return device_array_classes(); }

protected:
  virtual void setup_impl(const Variables &in, const Variables &out) {
    NBLA_CHECK(in[0]->shape() == in[1]->shape(), error_code::not_implemented,
               "broadcasting Add2 is not implemented in the b200 backend");
    out[0]->reshape(in[0]->shape(), true);
  }
  virtual void forward_impl(const Variables &in, const Variables &out) {
    B200_ENTER(st);
    const float *a = rd(in[0], this->ctx_), *b = rd(in[1], this->ctx_);
    float *y = wr(out[0], this->ctx_);
    nb200_check(nb200_add2_f32(a, b, y, in[0]->size(), st), "Add2");
  }
  virtual void backward_impl(const Variables &in, const Variables &out, const vector<bool> &pd,
                             const vector<bool> &accum) {
    if (!(pd[0] || pd[1]))
      return;
    B200_ENTER(st);
    const float *dy = out[0]->get_grad_pointer<float>(this->ctx_);
    for (int i = 0; i < 2; ++i)
      if (pd[i]) {
        float *dx = grad_wr(in[i], this->ctx_, true, accum[i]);
        nb200_check(nb200_add2_backward_f32(dy, dx, in[i]->size(), accum[i], st), "Add2 backward");
      }
  }
};

template <typename T> class MaxPoolingB200 : public MaxPooling<T> {
public:
  using MaxPooling<T>::MaxPooling;
  virtual vector<string> allowed_array_classes() { return device_array_classes(); }

protected:
  virtual void forward_impl(const Variables &in, const Variables &out) {
    NBLA_CHECK(!this->channel_last_, error_code::not_implemented, "channel_last is not supported");
    NBLA_CHECK(this->kernel_.size() == 2, error_code::not_implemented, "the b200 backend implements 2-D pooling only");
    B200_ENTER(st);
    const float tag = fxp_tag_get(in[0]);
    const Shape_t sx = in[0]->shape();
    const int H = sx[sx.size() - 2], W = sx[sx.size() - 1];
    const float *x = rd(in[0], this->ctx_);
    float *y = wr(out[0], this->ctx_);
    nb200_check(nb200_max_pooling_f32(x, y, in[0]->size() / (H * W), H, W, this->kernel_[0], this->kernel_[1],
                                      this->stride_[0], this->stride_[1], this->pad_[0], this->pad_[1],
                                      this->ignore_border_, st),
                "MaxPooling");
    if (tag > 0.f)
      fxp_tag_set(out[0], tag); // a maximum of multiples of delta is one of them
  }
  // max_pooling.cpp:194-228. No index map is kept: the backward pass finds the windows' first maxima
  // again from the input, which therefore has to stay alive until then.
  virtual bool grad_depends_input_data_impl(int i, int j) const { return true; }
  virtual void backward_impl(const Variables &in, const Variables &out, const vector<bool> &pd,
                             const vector<bool> &accum) {
    if (!pd[0])
      return;
    B200_ENTER(st);
    const Shape_t sx = in[0]->shape();
    const int H = sx[sx.size() - 2], W = sx[sx.size() - 1];
    const float *x = rd(in[0], this->ctx_);
    const float *dy = out[0]->get_grad_pointer<float>(this->ctx_);
    float *dx = grad_wr(in[0], this->ctx_, true, accum[0]);
    nb200_check(nb200_max_pooling_backward_f32(x, dy, dx, in[0]->size() / (H * W), H, W, this->kernel_[0],
                                               this->kernel_[1], this->stride_[0], this->stride_[1], this->pad_[0],
                                               this->pad_[1], this->ignore_border_, accum[0], st),
                "MaxPooling backward");
  }
};

template <typename T> class GlobalAveragePoolingB200 : public GlobalAveragePooling<T> {
public:
  using GlobalAveragePooling<T>::GlobalAveragePooling;
  virtual vector<string> allowed_array_classes() { return device_array_classes(); }

protected:
  virtual void forward_impl(const Variables &in, const Variables &out) {
    B200_ENTER(st);
    const Shape_t sx = in[0]->shape();
    const Size_t maps = sx[0] * sx[1];
    const float *x = rd(in[0], this->ctx_);
    float *y = wr(out[0], this->ctx_);
    nb200_check(nb200_global_average_pooling_f32(x, y, maps, in[0]->size() / maps, st), "GlobalAveragePooling");
  }
  // global_average_pooling.cpp:75-117
  virtual void backward_impl(const Variables &in, const Variables &out, const vector<bool> &pd,
                             const vector<bool> &accum) {
    if (!pd[0])
      return;
    B200_ENTER(st);
    const Shape_t sx = in[0]->shape();
    const Size_t maps = sx[0] * sx[1];
    const float *dy = out[0]->get_grad_pointer<float>(this->ctx_);
    float *dx = grad_wr(in[0], this->ctx_, true, accum[0]);
    nb200_check(nb200_global_average_pooling_backward_f32(dy, dx, maps, in[0]->size() / maps, accum[0], st),
                "GlobalAveragePooling backward");
  }
};


// INQAffine / INQConvolution (src/nbla/function/generic/inq_affine.cpp, inq_convolution.cpp). The reference's
// setup_impl is reused as it is: it creates the inner Affine / Convolution through the registry under this
// context, i.e. AffineB200 / ConvolutionB200, and sizes the state. forward_impl runs the weight update on the
// device; only the selection step (a few iterations of a training run) is done on the host with the
// reference's own loop (std::sort's order among equal magnitudes and the mt19937 / bernoulli stream are then
// the same library's, hence identical), reading and writing the arrays through the CPU context, which nnabla
// synchronises in both directions.
struct InqState { // the members of the two reference classes the update works on
  const vector<int> &iterations;
  const string &selection_algorithm;
  int seed, num_bits, minibatch_counter;
  std::mt19937 &rgen;
  std::bernoulli_distribution &rdist;
  Variable &old_weights, &old_indicators;
};

void inq_weight_update(const Context &ctx, void *st, Variable *weights_var, Variable *indicators_var, InqState s,
                       const char *what) {
  const Size_t n = weights_var->size();
  {
    float *w = weights_var->cast_data_and_get_pointer<float>(ctx);
    const float *ow = s.old_weights.get_data_pointer<float>(ctx);
    const int *oi = s.old_indicators.get_data_pointer<int>(ctx);
    nb200_check(nb200_inq_restore_f32(w, ow, oi, n, st), what);
  }
  int fix_all = 0;
  const vector<int> &its = s.iterations;
  if (std::find(its.begin(), its.end(), s.minibatch_counter) != its.end()) {
    if (its.back() == s.minibatch_counter) {
      fix_all = 1;
    } else {
      const Context cpu({"cpu:float"}, "CpuCachedArray", "0");
      const float *weights = weights_var->get_data_pointer<float>(cpu);
      int *indicators = indicators_var->cast_data_and_get_pointer<int>(cpu);
      if (s.selection_algorithm == "largest_abs") { // inq_affine.cpp:118-139
        vector<size_t> indices(n);
        std::iota(begin(indices), end(indices), 0);
        std::sort(begin(indices), end(indices),
                  [&](size_t a, size_t b) { return std::abs(weights[a]) > std::abs(weights[b]); });
        int num_learnable = 0;
        for (Size_t i = 0; i < n; ++i)
          num_learnable += indicators[i] == 0;
        int num_fixed = 0;
        for (Size_t i = 0; i < n; ++i) {
          if (indicators[indices[i]] == 0) {
            indicators[indices[i]] = 1;
            num_fixed++;
          }
          if (num_fixed >= num_learnable / 2)
            break;
        }
      } else { // :140-147
        std::mt19937 &rgen = s.seed == -1 ? SingletonManager::get<RandomManager>()->get_rand_generator() : s.rgen;
        for (Size_t i = 0; i < n; ++i)
          if (indicators[i] == 0)
            indicators[i] = s.rdist(rgen);
      }
    }
  }
  float *w = weights_var->cast_data_and_get_pointer<float>(ctx);
  int *ind = indicators_var->cast_data_and_get_pointer<int>(ctx);
  float *ow = s.old_weights.cast_data_and_get_pointer<float>(ctx);
  int *oi = s.old_indicators.cast_data_and_get_pointer<int>(ctx);
  nb200_check(nb200_inq_quantize_f32(w, ind, ow, oi, n, s.num_bits, fix_all, st), what);
}

template <typename T, typename T1> class INQAffineB200 : public INQAffine<T, T1> {
public:
  using INQAffine<T, T1>::INQAffine;
  virtual vector<string> allowed_array_classes() { return device_array_classes(); }

protected:
  virtual void forward_impl(const Variables &in, const Variables &out) {
    B200_ENTER(st);
    inq_weight_update(this->ctx_, st, in[1], in[2],
                      InqState{this->inq_iterations_, this->selection_algorithm_, this->seed_, this->num_bits_,
                               this->minibatch_counter_, this->rgen_, this->rdist_, this->old_weights_,
                               this->old_indicators_},
                      "INQAffine");
    if (in.size() == 4)
      this->affine_->forward(Variables{in[0], in[1], in[3]}, out);
    else
      this->affine_->forward(Variables{in[0], in[1]}, out);
    this->minibatch_counter_++;
  }
};

template <typename T, typename T1> class INQConvolutionB200 : public INQConvolution<T, T1> {
public:
  using INQConvolution<T, T1>::INQConvolution;
  virtual vector<string> allowed_array_classes() { return device_array_classes(); }

protected:
  virtual void forward_impl(const Variables &in, const Variables &out) {
    B200_ENTER(st);
    inq_weight_update(this->ctx_, st, in[1], in[2],
                      InqState{this->inq_iterations_, this->selection_algorithm_, this->seed_, this->num_bits_,
                               this->minibatch_counter_, this->rgen_, this->rdist_, this->old_weights_,
                               this->old_indicators_},
                      "INQConvolution");
    if (in.size() == 4)
      this->convolution_->forward(Variables{in[0], in[1], in[3]}, out);
    else
      this->convolution_->forward(Variables{in[0], in[1]}, out);
    this->minibatch_counter_++;
  }
};

} // namespace

// ------------------------------------------------------------------- init
void init_b200() {
  static std::mutex m;
  std::lock_guard<std::mutex> lock(m);
  static volatile bool done = false;
  if (done)
    return;
  done = true;
  init_cpu();
  nb200_check(nb200_check_device(), "init_b200");
  install_write_tracking();
  register_b200_communicator();

  NBLA_REGISTER_BACKEND("b200", []() { return SingletonManager::get<B200>(); });
  NBLA_REGISTER_ARRAY_CREATOR(B200Array);
  SingletonManager::get<B200>()->register_array_class("B200Array");
  NBLA_REGISTER_ARRAY_CREATOR(B200CachedArray);
  SingletonManager::get<B200>()->register_array_class("B200CachedArray");
  // "B200CachedArray" first: Function::setup picks the first allowed class the context names.
  SingletonManager::get<B200>()->_set_array_classes({"B200CachedArray", "B200Array"});
  NBLA_REGISTER_ARRAY_SYNCHRONIZER(B200Array, B200CachedArray, synchronizer_default);
  NBLA_REGISTER_ARRAY_SYNCHRONIZER(B200CachedArray, B200Array, synchronizer_default);
  NBLA_REGISTER_ARRAY_SYNCHRONIZER(CpuArray, B200Array, synchronizer_cpu_to_b200);
  NBLA_REGISTER_ARRAY_SYNCHRONIZER(CpuArray, B200CachedArray, synchronizer_cpu_to_b200);
  NBLA_REGISTER_ARRAY_SYNCHRONIZER(CpuCachedArray, B200Array, synchronizer_cpu_to_b200);
  NBLA_REGISTER_ARRAY_SYNCHRONIZER(CpuCachedArray, B200CachedArray, synchronizer_cpu_to_b200);
  NBLA_REGISTER_ARRAY_SYNCHRONIZER(B200Array, CpuArray, synchronizer_b200_to_cpu);
  NBLA_REGISTER_ARRAY_SYNCHRONIZER(B200Array, CpuCachedArray, synchronizer_b200_to_cpu);
  NBLA_REGISTER_ARRAY_SYNCHRONIZER(B200CachedArray, CpuArray, synchronizer_b200_to_cpu);
  NBLA_REGISTER_ARRAY_SYNCHRONIZER(B200CachedArray, CpuCachedArray, synchronizer_b200_to_cpu);
  NBLA_REGISTER_ARRAY_GROUP(B200Array, b200);
  NBLA_REGISTER_ARRAY_GROUP(B200CachedArray, b200);

  typedef const vector<int> &ivec;
#define REG(NAME, ...)                                                                                       \
  {                                                                                                          \
    using NAME##_b200_float = NAME##B200<float>;                                                             \
    NBLA_REGISTER_FUNCTION_IMPL(NAME, NAME##_b200_float, "b200:float", ##__VA_ARGS__);                       \
  }
  REG(FixedPointQuantize, bool, int, float, bool);
  REG(BinarySigmoid);
  REG(BinaryTanh);
  REG(QuantizeLinear, const string &, bool, int);
  REG(DequantizeLinear);
  REG(Prune, float);
  REG(Pow2Quantize, bool, bool, int, int, bool);
  REG(MinMaxQuantize, float, bool, bool, bool, float);
  REG(BinaryWeightAffine, int, float);
  REG(BinaryConnectAffine, int, float);
  REG(BinaryWeightConvolution, int, ivec, ivec, ivec, int, float);
  REG(BinaryConnectConvolution, int, ivec, ivec, ivec, int, float);
  REG(Affine, int);
  REG(Convolution, int, ivec, ivec, ivec, int, bool);
  REG(BatchNormalization, ivec, float, float, bool, bool, bool);
  REG(ReLU, bool);
  REG(Add2, bool);
  REG(MaxPooling, ivec, ivec, bool, ivec, bool);
  REG(GlobalAveragePooling);
#undef REG
  {
    using INQAffine_b200 = INQAffineB200<float, int>;
    NBLA_REGISTER_FUNCTION_IMPL(INQAffine, INQAffine_b200, "b200:float", int, int, ivec, const string &, int);
    using INQConvolution_b200 = INQConvolutionB200<float, int>;
    NBLA_REGISTER_FUNCTION_IMPL(INQConvolution, INQConvolution_b200, "b200:float", int, ivec, ivec, ivec, int, int,
                                ivec, const string &, int);
  }
}

} // namespace nbla
