// C binding for whole graphs over nnabla's own graph engine
// (CgVariable / CgFunction / connect(), src/nbla/computation_graph/computation_graph.cpp:59-123;
// CgVariable::forward, src/nbla/computation_graph/variable.cpp:939-957) with the
// b200 extension loaded. A graph is built function by function under one
// context, "cpu:float" or "b200:float"; the same sequence of calls builds it
// under either, so a graph moves between the backends by changing the context
// string only. It stands in for the nnabla Python package (Cython over
// libnnabla), which cannot be built without nnabla's code generator.
//
//   g   = nbg_create("b200:float", "0")
//   x   = nbg_variable(g, 4, shape, 0);  nbg_set_data(g, x, host_ptr)
//   y   = nbg_function(g, "Convolution", scalars, n, ivecs, lens, n_iv, inputs, n_in, 1, outs)
//   nbg_forward(g, y, /*clear_buffer=*/1, /*repeat=*/10, &seconds)
//   nbg_get_data(g, y, host_ptr)
#include "create_function.hpp"

#include <nbla_b200/b200.hpp>

#include <nbla/computation_graph/computation_graph.hpp>
#include <nbla/computation_graph/function.hpp>
#include <nbla/computation_graph/variable.hpp>
#include <nbla/exception.hpp>

#include <nnabla_b200.h>

#include <chrono>
#include <cstring>
#include <map>
#include <memory>
#include <string>
#include <vector>

using namespace nbla;

namespace {
thread_local std::string g_err;

struct Graph {
  std::string backend;
  Context ctx;
  Context cpu{{"cpu:float"}, "CpuCachedArray", "0"};
  std::vector<CgVariablePtr> vars;
  bool on_device() const { return backend != "cpu:float"; }
  void device_sync() const {
    if (on_device())
      nb200_check(nb200_device_synchronize(), "nb200_device_synchronize");
  }
};

CgVariablePtr var_of(Graph *g, int id) {
  NBLA_CHECK(id >= 0 && id < (int)g->vars.size(), error_code::value, "unknown variable id %d", id);
  return g->vars[id];
}

template <typename F> int guarded(F &&f) {
  try {
    f();
    return 0;
  } catch (const std::exception &e) {
    g_err = e.what();
    return 1;
  }
}
} // namespace

extern "C" {

const char *nbg_last_error() { return g_err.c_str(); }

void *nbg_create(const char *backend, const char *device_id) {
  try {
    std::unique_ptr<Graph> g(new Graph());
    g->backend = backend;
    g->ctx = nbla_b200_runner::context_for(backend, device_id ? device_id : "0");
    return g.release();
  } catch (const std::exception &e) {
    g_err = e.what();
    return nullptr;
  }
}

void nbg_destroy(void *h) { delete static_cast<Graph *>(h); }

// A leaf variable of the given shape. Returns its id, or -1.
int nbg_variable(void *h, int ndim, const int64_t *shape, int need_grad) {
  Graph *g = static_cast<Graph *>(h);
  int id = -1;
  guarded([&] {
    g->vars.push_back(std::make_shared<CgVariable>(Shape_t(shape, shape + ndim), need_grad != 0));
    id = (int)g->vars.size() - 1;
  });
  return id;
}

int nbg_num_variables(void *h) { return (int)static_cast<Graph *>(h)->vars.size(); }

int nbg_shape(void *h, int id, int64_t *shape, int *ndim) {
  Graph *g = static_cast<Graph *>(h);
  return guarded([&] {
    const Shape_t s = var_of(g, id)->variable()->shape();
    NBLA_CHECK(s.size() <= 8, error_code::value, "ndim > 8");
    *ndim = (int)s.size();
    for (size_t d = 0; d < s.size(); ++d)
      shape[d] = s[d];
  });
}

// Host data into a variable: written through a CPU array, so the first device
// read goes through the extension's synchronizer (and is cached afterwards).
int nbg_set_data(void *h, int id, const float *data) {
  Graph *g = static_cast<Graph *>(h);
  return guarded([&] {
    VariablePtr v = var_of(g, id)->variable();
    float *p = v->cast_data_and_get_pointer<float>(g->cpu, true);
    std::memcpy(p, data, sizeof(float) * v->size());
  });
}

int nbg_get_data(void *h, int id, float *data) {
  Graph *g = static_cast<Graph *>(h);
  return guarded([&] {
    VariablePtr v = var_of(g, id)->variable();
    const float *p = v->get_data_pointer<float>(g->cpu);
    std::memcpy(data, p, sizeof(float) * v->size());
  });
}

int nbg_set_persistent(void *h, int id, int persistent) {
  Graph *g = static_cast<Graph *>(h);
  return guarded([&] { var_of(g, id)->set_persistent(persistent != 0); });
}

// Creates function `op` under the graph's context and connects it to the
// given inputs. The ids of its n_out outputs are written to out_ids.
int nbg_function(void *h, const char *op, const double *s, int n_s, const int32_t *iv, const int32_t *iv_len, int n_iv,
                 const int32_t *in_ids, int n_in, int n_out, int32_t *out_ids) {
  Graph *g = static_cast<Graph *>(h);
  return guarded([&] {
    std::vector<std::vector<int>> ivs;
    const int32_t *p = iv;
    for (int i = 0; i < n_iv; ++i) {
      ivs.emplace_back(p, p + iv_len[i]);
      p += iv_len[i];
    }
    FunctionPtr f = nbla_b200_runner::create_function(op, g->ctx, s, n_s, ivs);
    std::vector<CgVariablePtr> ins;
    for (int i = 0; i < n_in; ++i)
      ins.push_back(var_of(g, in_ids[i]));
    std::vector<CgVariablePtr> outs = connect(std::make_shared<CgFunction>(f), ins, n_out);
    for (int i = 0; i < n_out; ++i) {
      g->vars.push_back(outs[i]);
      out_ids[i] = (int)g->vars.size() - 1;
    }
  });
}

// Runs CgVariable::forward `repeat` times and waits for the device. *seconds
// (may be NULL) receives the wall time per forward pass, device work included.
int nbg_forward(void *h, int id, int clear_buffer, int repeat, double *seconds) {
  Graph *g = static_cast<Graph *>(h);
  return guarded([&] {
    CgVariablePtr v = var_of(g, id);
    g->device_sync();
    const auto t0 = std::chrono::steady_clock::now();
    for (int r = 0; r < repeat; ++r)
      v->forward(clear_buffer != 0, false);
    g->device_sync();
    const double dt = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
    if (seconds)
      *seconds = dt / (repeat > 0 ? repeat : 1);
  });
}

// CgVariable::backward from variable `id` with the initial gradient `grad` (host data of the variable's
// shape; NULL: the gradient array the variable already holds) and waits for the device. Gradients of
// leaf variables created with need_grad accumulate, as nnabla's do: zero them first (nbg_zero_grad).
int nbg_backward(void *h, int id, const float *grad, int clear_buffer, double *seconds) {
  Graph *g = static_cast<Graph *>(h);
  return guarded([&] {
    CgVariablePtr v = var_of(g, id);
    NdArrayPtr g0;
    if (grad) {
      g0 = NdArray::create(v->variable()->shape());
      float *p = g0->cast(dtypes::FLOAT, g->cpu, true)->pointer<float>();
      std::memcpy(p, grad, sizeof(float) * v->variable()->size());
    }
    g->device_sync();
    const auto t0 = std::chrono::steady_clock::now();
    v->backward(g0, clear_buffer != 0);
    g->device_sync();
    if (seconds)
      *seconds = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
  });
}

int nbg_zero_grad(void *h, int id) {
  Graph *g = static_cast<Graph *>(h);
  return guarded([&] { var_of(g, id)->variable()->grad()->zero(); });
}

int nbg_get_grad(void *h, int id, float *data) {
  Graph *g = static_cast<Graph *>(h);
  return guarded([&] {
    VariablePtr v = var_of(g, id)->variable();
    const float *p = v->get_grad_pointer<float>(g->cpu);
    std::memcpy(data, p, sizeof(float) * v->size());
  });
}

// Per-function times of one forward pass, the way nnabla's GraphProfiler takes
// them (python/src/nnabla/utils/profiler.py): the device is synchronised
// before and after every function. Up to `capacity` entries of `names`
// (64 bytes each) and `ms` are filled in execution order; *count receives the
// number of functions executed.
int nbg_profile(void *h, int id, int clear_buffer, char *names, double *ms, int capacity, int *count) {
  Graph *g = static_cast<Graph *>(h);
  return guarded([&] {
    CgVariablePtr v = var_of(g, id);
    int n = 0;
    std::chrono::steady_clock::time_point t0;
    auto pre = [&](const CgFunctionPtr &) {
      g->device_sync();
      t0 = std::chrono::steady_clock::now();
    };
    auto post = [&](const CgFunctionPtr &f) {
      g->device_sync();
      const double dt = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
      if (n < capacity) {
        std::strncpy(names + 64 * n, f->function()->name().c_str(), 63);
        names[64 * n + 63] = 0;
        ms[n] = dt * 1e3;
      }
      ++n;
    };
    v->forward(clear_buffer != 0, false, nullptr, pre, post);
    *count = n;
  });
}

// Counters the extension keeps about the paths its functions took (see b200.hpp).
long long nbg_counter(const char *name) { return b200_counter(name); }
void nbg_reset_counters() { b200_reset_counters(); }
}
