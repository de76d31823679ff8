// C ABI over the reference's own CPU functions ("cpu:float" context), built
// into oracle/_ref/libnnabla_ref.so by oracle/Makefile from the reference
// sources where they lie. It creates the function through the reference's
// registry (create_X -> FunctionRegistry::create, function_registry.hpp:179-184),
// runs Function::setup and Function::forward (src/nbla/function.cpp:27-72,
// :107-123) on Variables filled from caller buffers, and copies every input
// (several hot-path functions write their inputs: Wb/alpha in
// binary_weight_affine.cpp:92-103, qr_min/qr_max in min_max_quantize.cpp:159-178,
// :353-361) and every output back.
//
// TEST INFRASTRUCTURE ONLY: used to pin the C restatement in oracle/, to make
// the golden fixtures under tests/golden/, and as the timed CPU baseline.
#include <nbla/context.hpp>
#include <nbla/exception.hpp>
#include <nbla/function.hpp>
#include <nbla/variable.hpp>

#include <nbla/function/add2.hpp>
#include <nbla/function/affine.hpp>
#include <nbla/function/average_pooling.hpp>
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
#include <nbla/function/max_pooling.hpp>
#include <nbla/function/binary_sigmoid.hpp>
#include <nbla/function/binary_tanh.hpp>
#include <nbla/function/dequantize_linear.hpp>
#include <nbla/function/min_max_quantize.hpp>
#include <nbla/function/prune.hpp>
#include <nbla/function/quantize_linear.hpp>
#include <nbla/function/pow2_quantize.hpp>
#include <nbla/function/relu.hpp>
#include <nbla/function/sign.hpp>

#include <chrono>
#include <cstdint>
#include <cstring>
#include <memory>
#include <string>
#include <vector>

using namespace nbla;

static std::vector<std::vector<int>> split_vectors(const int32_t *iv,
                                                    const int32_t *iv_len,
                                                    int n_iv) {
  std::vector<std::vector<int>> ivs;
  const int32_t *p = iv;
  for (int i = 0; i < n_iv; ++i) {
    ivs.emplace_back(p, p + iv_len[i]);
    p += iv_len[i];
  }
  return ivs;
}

// Creates function `op` through the reference's registry. s: scalar arguments
// in the order of the reference constructor, each as a double (bool/int/float
// alike); ivs: the vector<int> arguments in constructor order.
static FunctionPtr make_function(const Context &ctx, const char *op,
                                 const double *s, int n_s,
                                 const std::vector<std::vector<int>> &ivs) {
  const int n_iv = (int)ivs.size();
  auto S = [&](int i) -> double {
    NBLA_CHECK(i < n_s, error_code::value, "missing scalar argument %d", i);
    return s[i];
  };
  auto V = [&](int i) -> const std::vector<int> & {
    NBLA_CHECK(i < n_iv, error_code::value, "missing vector argument %d", i);
    return ivs[i];
  };
  const std::string name(op);
  FunctionPtr f;
  if (name == "FixedPointQuantize")
    f = create_FixedPointQuantize(ctx, S(0) != 0, (int)S(1), (float)S(2),
                                  S(3) != 0);
  else if (name == "Pow2Quantize")
    f = create_Pow2Quantize(ctx, S(0) != 0, S(1) != 0, (int)S(2), (int)S(3),
                            S(4) != 0);
  else if (name == "MinMaxQuantize")
    f = create_MinMaxQuantize(ctx, (float)S(0), S(1) != 0, S(2) != 0,
                              S(3) != 0, (float)S(4));
  else if (name == "BinaryWeightAffine")
    f = create_BinaryWeightAffine(ctx, (int)S(0), (float)S(1));
  else if (name == "BinaryConnectAffine")
    f = create_BinaryConnectAffine(ctx, (int)S(0), (float)S(1));
  else if (name == "BinaryWeightConvolution")
    f = create_BinaryWeightConvolution(ctx, (int)S(0), V(0), V(1), V(2),
                                       (int)S(1), (float)S(2));
  else if (name == "BinaryConnectConvolution")
    f = create_BinaryConnectConvolution(ctx, (int)S(0), V(0), V(1), V(2),
                                        (int)S(1), (float)S(2));
  else if (name == "Sign")
    f = create_Sign(ctx, (float)S(0));
  else if (name == "Affine")
    f = create_Affine(ctx, (int)S(0));
  else if (name == "Convolution")
    f = create_Convolution(ctx, (int)S(0), V(0), V(1), V(2), (int)S(1),
                           S(2) != 0);
  else if (name == "BatchNormalization")
    f = create_BatchNormalization(ctx, V(0), (float)S(0), (float)S(1),
                                  S(2) != 0, S(3) != 0, S(4) != 0);
  else if (name == "ReLU")
    f = create_ReLU(ctx, S(0) != 0);
  else if (name == "MaxPooling")
    f = create_MaxPooling(ctx, V(0), V(1), S(0) != 0, V(2), S(1) != 0);
  else if (name == "AveragePooling")
    f = create_AveragePooling(ctx, V(0), V(1), S(0) != 0, V(2), S(1) != 0,
                              S(2) != 0);
  else if (name == "GlobalAveragePooling")
    f = create_GlobalAveragePooling(ctx);
  else if (name == "Add2")
    f = create_Add2(ctx, S(0) != 0);
  else if (name == "BinarySigmoid")
    f = create_BinarySigmoid(ctx);
  else if (name == "BinaryTanh")
    f = create_BinaryTanh(ctx);
  else if (name == "INQAffine") // scalars: base_axis, num_bits, selection (0 = largest_abs, 1 = random), seed; ivecs: inq_iterations
    f = create_INQAffine(ctx, (int)S(0), (int)S(1), ivs.at(0), S(2) != 0 ? "random" : "largest_abs", (int)S(3));
  else if (name == "INQConvolution") // scalars: base_axis, group, num_bits, selection, seed; ivecs: pad, stride, dilation, inq_iterations
    f = create_INQConvolution(ctx, (int)S(0), V(0), V(1), V(2), (int)S(1), (int)S(2), ivs.at(3),
                              S(3) != 0 ? "random" : "largest_abs", (int)S(4));
  else if (name == "QuantizeLinear") // scalars: round mode (0 = HALF_AWAY_FROM_ZERO, 1 = HALF_TO_EVEN), narrow_range, dtype
    f = create_QuantizeLinear(ctx, S(0) != 0 ? "HALF_TO_EVEN" : "HALF_AWAY_FROM_ZERO", S(1) != 0, (int)S(2));
  else if (name == "DequantizeLinear")
    f = create_DequantizeLinear(ctx);
  else if (name == "Prune")
    f = create_Prune(ctx, (float)S(0));
  else
    NBLA_ERROR(error_code::value, "unknown function %s", op);

  return f;
}

extern "C" {

struct nbref_tensor {
  float *data;      // host buffer (may be null when mode == 0)
  int32_t ndim;     // in: for inputs; out: for outputs
  int64_t shape[8]; // in: for inputs; out: for outputs
};

static thread_local std::string g_err;
const char *nbref_last_error() { return g_err.c_str(); }

// mode 0: setup only, report output shapes. mode 1: setup + forward, copy
// inputs and outputs back. `repeat` (>= 1) forwards are run and the mean
// wall time of Function::forward alone is stored in *forward_seconds.
//
// sargs: scalar arguments in the order of the reference constructor, each as a
// double (bool/int/float alike); iargs: the vector<int> arguments, flattened,
// with their lengths in iargs_len, in constructor order.
int nbref_forward(const char *op, const double *s, int n_s, const int32_t *iv,
                  const int32_t *iv_len, int n_iv, nbref_tensor *in, int n_in,
                  nbref_tensor *out, int n_out, int mode, int repeat,
                  double *forward_seconds) {
  try {
    Context ctx({"cpu:float"}, "CpuCachedArray", "0");
    const std::vector<std::vector<int>> ivs = split_vectors(iv, iv_len, n_iv);
    FunctionPtr f = make_function(ctx, op, s, n_s, ivs);

    std::vector<VariablePtr> vin, vout;
    Variables pin, pout;
    for (int i = 0; i < n_in; ++i) {
      Shape_t sh(in[i].shape, in[i].shape + in[i].ndim);
      vin.push_back(std::make_shared<Variable>(sh));
      pin.push_back(vin.back().get());
    }
    for (int i = 0; i < n_out; ++i) {
      vout.push_back(std::make_shared<Variable>());
      pout.push_back(vout.back().get());
    }
    f->setup(pin, pout);
    for (int i = 0; i < n_out; ++i) {
      const Shape_t sh = pout[i]->shape();
      NBLA_CHECK(sh.size() <= 8, error_code::value, "ndim > 8");
      out[i].ndim = (int32_t)sh.size();
      for (size_t d = 0; d < sh.size(); ++d)
        out[i].shape[d] = sh[d];
    }
    if (mode == 0)
      return 0;
    for (int i = 0; i < n_in; ++i) {
      float *p = pin[i]->cast_data_and_get_pointer<float>(ctx, true);
      std::memcpy(p, in[i].data, sizeof(float) * pin[i]->size());
    }
    for (int i = 0; i < n_out; ++i) // allocate before timing
      pout[i]->cast_data_and_get_pointer<float>(ctx, true);
    if (repeat < 1)
      repeat = 1;
    auto t0 = std::chrono::steady_clock::now();
    for (int r = 0; r < repeat; ++r)
      f->forward(pin, pout);
    auto t1 = std::chrono::steady_clock::now();
    if (forward_seconds)
      *forward_seconds =
          std::chrono::duration<double>(t1 - t0).count() / repeat;
    for (int i = 0; i < n_in; ++i) {
      const float *p = pin[i]->get_data_pointer<float>(ctx);
      std::memcpy(in[i].data, p, sizeof(float) * pin[i]->size());
    }
    for (int i = 0; i < n_out; ++i) {
      const float *p = pout[i]->get_data_pointer<float>(ctx);
      std::memcpy(out[i].data, p, sizeof(float) * pout[i]->size());
    }
    return 0;
  } catch (const std::exception &e) {
    g_err = e.what();
    return 1;
  }
}
// Setup + forward + backward. in[i].data / out[j].data as in nbref_forward
// (inputs and outputs are copied back after the forward); out_grad[j] is the
// gradient arriving at output j; in_grad[i] holds the initial gradient of
// input i (read when accum[i] != 0, otherwise the buffer is pre-filled with it
// anyway so that elements the reference leaves untouched are visible) and
// receives the gradient after Function::backward (src/nbla/function.cpp:125-
// 160) ran with the given propagate_down / accum flags.
int nbref_backward(const char *op, const double *s, int n_s, const int32_t *iv,
                   const int32_t *iv_len, int n_iv, nbref_tensor *in,
                   nbref_tensor *in_grad, int n_in, nbref_tensor *out,
                   nbref_tensor *out_grad, int n_out,
                   const int32_t *propagate_down, const int32_t *accum) {
  try {
    Context ctx({"cpu:float"}, "CpuCachedArray", "0");
    const std::vector<std::vector<int>> ivs = split_vectors(iv, iv_len, n_iv);
    FunctionPtr f = make_function(ctx, op, s, n_s, ivs);
    std::vector<VariablePtr> vin, vout;
    Variables pin, pout;
    for (int i = 0; i < n_in; ++i) {
      Shape_t sh(in[i].shape, in[i].shape + in[i].ndim);
      vin.push_back(std::make_shared<Variable>(sh));
      pin.push_back(vin.back().get());
    }
    for (int i = 0; i < n_out; ++i) {
      vout.push_back(std::make_shared<Variable>());
      pout.push_back(vout.back().get());
    }
    f->setup(pin, pout);
    for (int i = 0; i < n_out; ++i) {
      const Shape_t sh = pout[i]->shape();
      NBLA_CHECK(sh.size() <= 8, error_code::value, "ndim > 8");
      out[i].ndim = (int32_t)sh.size();
      for (size_t d = 0; d < sh.size(); ++d)
        out[i].shape[d] = sh[d];
    }
    for (int i = 0; i < n_in; ++i) {
      float *p = pin[i]->cast_data_and_get_pointer<float>(ctx, true);
      std::memcpy(p, in[i].data, sizeof(float) * pin[i]->size());
      float *g = pin[i]->cast_grad_and_get_pointer<float>(ctx, true);
      std::memcpy(g, in_grad[i].data, sizeof(float) * pin[i]->size());
    }
    f->forward(pin, pout);
    for (int i = 0; i < n_out; ++i) {
      float *g = pout[i]->cast_grad_and_get_pointer<float>(ctx, true);
      std::memcpy(g, out_grad[i].data, sizeof(float) * pout[i]->size());
    }
    std::vector<bool> pd(n_in), ac(n_in);
    for (int i = 0; i < n_in; ++i) {
      pd[i] = propagate_down[i] != 0;
      ac[i] = accum[i] != 0;
    }
    f->backward(pin, pout, pd, ac);
    for (int i = 0; i < n_in; ++i) {
      const float *p = pin[i]->get_data_pointer<float>(ctx);
      std::memcpy(in[i].data, p, sizeof(float) * pin[i]->size());
      const float *g = pin[i]->get_grad_pointer<float>(ctx);
      std::memcpy(in_grad[i].data, g, sizeof(float) * pin[i]->size());
    }
    for (int i = 0; i < n_out; ++i) {
      const float *p = pout[i]->get_data_pointer<float>(ctx);
      std::memcpy(out[i].data, p, sizeof(float) * pout[i]->size());
    }
    return 0;
  } catch (const std::exception &e) {
    g_err = e.what();
    return 1;
  }
}
}
