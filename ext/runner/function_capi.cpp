// C binding for single functions over the nnabla host library with the b200
// extension loaded: creates a function through nnabla's registry for a given backend
// ("cpu:float" or "b200:float"), feeds it from host buffers through
// nnabla's own Variable / SyncedArray machinery (so device arrays, the
// allocator and the synchronizers of the extension are exercised), runs
// setup + forward and copies inputs (several functions write theirs) and
// outputs back. The same graph runs on either backend by changing the
// context only, which is what the tests compare.
#include <nbla_b200/b200.hpp>

#include <nbla/exception.hpp>
#include <nbla/function.hpp>
#include <nbla/variable.hpp>

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
#include <nbla/function/max_pooling.hpp>
#include <nbla/function/binary_sigmoid.hpp>
#include <nbla/function/binary_tanh.hpp>
#include <nbla/function/dequantize_linear.hpp>
#include <nbla/function/min_max_quantize.hpp>
#include <nbla/function/prune.hpp>
#include <nbla/function/quantize_linear.hpp>
#include <nbla/function/pow2_quantize.hpp>
#include <nbla/function/relu.hpp>

#include <chrono>
#include <cstdint>
#include <cstring>
#include <memory>
#include <string>
#include <vector>

using namespace nbla;

#include "create_function.hpp"

namespace {
thread_local std::string g_err;
using nbla_b200_runner::create_function;
} // namespace

extern "C" {

struct nbext_tensor {
  float *data;
  int32_t ndim;
  int64_t shape[8];
};

const char *nbext_last_error() { return g_err.c_str(); }

int nbext_init() {
  try {
    init_b200();
    return 0;
  } catch (const std::exception &e) {
    g_err = e.what();
    return 1;
  }
}

// backend: "cpu:float" or "b200:float". prequant[i] > 0: input i is first
// passed through FixedPointQuantize(sign, 8, prequant[i]) on the same backend
// and the function consumes that function's output Variable (this is how the
// fixed-point tag reaches the contraction functions). Returns the name() of
// the created function in fname (for the tests' name check).
int nbext_forward(const char *backend, const char *op, const double *s, int n_s, const int32_t *iv,
                  const int32_t *iv_len, int n_iv, nbext_tensor *in, int n_in, const float *prequant,
                  nbext_tensor *out, int n_out, int mode, char *fname, int fname_len) {
  try {
    const std::string be(backend);
    Context ctx = be == "cpu:float" ? Context({"cpu:float"}, "CpuCachedArray", "0")
                                    : b200_context("0", be == "b200:half" ? "half" : "float");
    if (be != "cpu:float")
      init_b200();
    Context cpu({"cpu:float"}, "CpuCachedArray", "0");
    std::vector<std::vector<int>> ivs;
    const int32_t *p = iv;
    for (int i = 0; i < n_iv; ++i) {
      ivs.emplace_back(p, p + iv_len[i]);
      p += iv_len[i];
    }
    FunctionPtr f = create_function(op, ctx, s, n_s, ivs);
    if (fname && fname_len > 0) {
      std::strncpy(fname, f->name().c_str(), fname_len - 1);
      fname[fname_len - 1] = 0;
    }
    std::vector<VariablePtr> vin, vq, vout;
    std::vector<FunctionPtr> quantizers;
    Variables pin, pout;
    for (int i = 0; i < n_in; ++i) {
      Shape_t sh(in[i].shape, in[i].shape + in[i].ndim);
      vin.push_back(std::make_shared<Variable>(sh));
      if (prequant && prequant[i] > 0.f) {
        vq.push_back(std::make_shared<Variable>(sh));
        quantizers.push_back(create_FixedPointQuantize(ctx, true, 8, prequant[i], true));
        quantizers.back()->setup(Variables{vin.back().get()}, Variables{vq.back().get()});
        pin.push_back(vq.back().get());
      } else {
        vq.push_back(nullptr);
        quantizers.push_back(nullptr);
        pin.push_back(vin.back().get());
      }
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
    // Host data enters through a CPU array; the function's first device read triggers the synchronizer.
    for (int i = 0; i < n_in; ++i) {
      float *h = vin[i]->cast_data_and_get_pointer<float>(cpu, true);
      std::memcpy(h, in[i].data, sizeof(float) * vin[i]->size());
    }
    for (int i = 0; i < n_in; ++i)
      if (quantizers[i])
        quantizers[i]->forward(Variables{vin[i].get()}, Variables{vq[i].get()});
    for (int r = 0; r < mode; ++r) // mode = number of forward passes of the same function instance
      f->forward(pin, pout);
    for (int i = 0; i < n_in; ++i) {
      const float *h = pin[i]->get_data_pointer<float>(cpu);
      std::memcpy(in[i].data, h, sizeof(float) * pin[i]->size());
    }
    for (int i = 0; i < n_out; ++i) {
      const float *h = pout[i]->get_data_pointer<float>(cpu);
      std::memcpy(out[i].data, h, sizeof(float) * pout[i]->size());
    }
    return 0;
  } catch (const std::exception &e) {
    g_err = e.what();
    return 1;
  }
}

// Setup + forward + Function::backward on `backend`. in_grad[i] holds the
// initial gradient of input i and receives it after the backward; out_grad[j]
// is the gradient arriving at output j. Host data enters and leaves through
// CPU arrays, the device arrays are reached through the synchronizers.
int nbext_backward(const char *backend, const char *op, const double *s, int n_s, const int32_t *iv,
                   const int32_t *iv_len, int n_iv, nbext_tensor *in, nbext_tensor *in_grad, int n_in,
                   nbext_tensor *out, nbext_tensor *out_grad, int n_out, const int32_t *propagate_down,
                   const int32_t *accum) {
  try {
    const std::string be(backend);
    Context ctx = be == "cpu:float" ? Context({"cpu:float"}, "CpuCachedArray", "0")
                                    : b200_context("0", be == "b200:half" ? "half" : "float");
    if (be != "cpu:float")
      init_b200();
    Context cpu({"cpu:float"}, "CpuCachedArray", "0");
    std::vector<std::vector<int>> ivs;
    const int32_t *p = iv;
    for (int i = 0; i < n_iv; ++i) {
      ivs.emplace_back(p, p + iv_len[i]);
      p += iv_len[i];
    }
    FunctionPtr f = create_function(op, ctx, s, n_s, ivs);
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
    for (int i = 0; i < n_in; ++i) {
      float *h = pin[i]->cast_data_and_get_pointer<float>(cpu, true);
      std::memcpy(h, in[i].data, sizeof(float) * pin[i]->size());
      float *g = pin[i]->cast_grad_and_get_pointer<float>(cpu, true);
      std::memcpy(g, in_grad[i].data, sizeof(float) * pin[i]->size());
    }
    f->forward(pin, pout);
    for (int i = 0; i < n_out; ++i) {
      float *g = pout[i]->cast_grad_and_get_pointer<float>(cpu, true);
      std::memcpy(g, out_grad[i].data, sizeof(float) * pout[i]->size());
    }
    std::vector<bool> pd(n_in), ac(n_in);
    for (int i = 0; i < n_in; ++i) {
      pd[i] = propagate_down[i] != 0;
      ac[i] = accum[i] != 0;
    }
    f->backward(pin, pout, pd, ac);
    for (int i = 0; i < n_in; ++i) {
      const float *h = pin[i]->get_data_pointer<float>(cpu);
      std::memcpy(in[i].data, h, sizeof(float) * pin[i]->size());
      const float *g = pin[i]->get_grad_pointer<float>(cpu);
      std::memcpy(in_grad[i].data, g, sizeof(float) * pin[i]->size());
    }
    for (int i = 0; i < n_out; ++i) {
      const float *h = pout[i]->get_data_pointer<float>(cpu);
      std::memcpy(out[i].data, h, sizeof(float) * pout[i]->size());
    }
    return 0;
  } catch (const std::exception &e) {
    g_err = e.what();
    return 1;
  }
}
}
