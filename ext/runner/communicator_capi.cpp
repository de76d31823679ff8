// C binding for nnabla's Communicator interface with the b200 extension loaded:
// creates the MultiProcessDataParallelCommunicator registered for a backend
// (create_MultiProcessDataParallelCommunicatorCommunicator, include/nbla/communicator_registry.hpp)
// and runs its collectives on host buffers, which travel through nnabla's own
// NdArray / SyncedArray machinery like any other data.
#include "create_function.hpp"

#include <nbla_b200/b200.hpp>

#include <nbla/communicator/multi_process_data_parallel_communicator.hpp>
#include <nbla/exception.hpp>
#include <nbla/nd_array.hpp>

#include <cstring>
#include <memory>
#include <string>
#include <vector>

using namespace nbla;

namespace {
thread_local std::string g_err;
struct Comm {
  Context ctx;
  Context cpu{{"cpu:float"}, "CpuCachedArray", "0"};
  std::shared_ptr<Communicator> comm;
};
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

const char *nbc_last_error() { return g_err.c_str(); }

void *nbc_create(const char *backend, const char *device_id) {
  try {
    std::unique_ptr<Comm> c(new Comm());
    c->ctx = nbla_b200_runner::context_for(backend, device_id ? device_id : "0");
    c->comm = create_MultiProcessDataParallelCommunicatorCommunicator(c->ctx);
    return c.release();
  } catch (const std::exception &e) {
    g_err = e.what();
    return nullptr;
  }
}
void nbc_destroy(void *h) { delete static_cast<Comm *>(h); }
int nbc_init(void *h) {
  return guarded([&] { static_cast<Comm *>(h)->comm->init(); });
}
int nbc_rank(void *h) { return static_cast<Comm *>(h)->comm->rank(); }
int nbc_size(void *h) { return static_cast<Comm *>(h)->comm->size(); }
int nbc_barrier(void *h) {
  return guarded([&] { static_cast<Comm *>(h)->comm->barrier(); });
}
int nbc_new_group(void *h, const char *name, const int32_t *ranks, int n) {
  return guarded([&] {
    static_cast<Comm *>(h)->comm->new_group({std::string(name), std::vector<int>(ranks, ranks + n)});
  });
}

// op: 0 all_reduce(arrays), 1 reduce(arrays -> rank `root`), 2 bcast(arrays from rank `root`),
// 3 all_gather(arrays[0] -> arrays[1..]), 4 reduce_scatter(arrays[1..] -> arrays[0]),
// 5 the all_reduce_callback with pack_size = `root` elements, run as at the end of a backward pass.
// Every array is a host buffer of sizes[i] floats, read before and written after the collective.
int nbc_collective(void *h, int op, float **arrays, const int64_t *sizes, int n, int root, int division, int inplace,
                   const char *group) {
  Comm *c = static_cast<Comm *>(h);
  return guarded([&] {
    std::vector<NdArrayPtr> nd;
    for (int i = 0; i < n; ++i) {
      nd.push_back(std::make_shared<NdArray>(Shape_t{sizes[i]}));
      float *p = nd.back()->cast(dtypes::FLOAT, c->cpu, true)->pointer<float>();
      std::memcpy(p, arrays[i], sizeof(float) * sizes[i]);
    }
    const std::string g(group ? group : "world");
    switch (op) {
    case 0: c->comm->all_reduce(nd, division != 0, inplace != 0, g); break;
    case 1: c->comm->reduce(nd, root, division != 0, inplace != 0, g); break;
    case 2: c->comm->bcast(nd, root, inplace != 0, g); break;
    case 3: c->comm->all_gather(nd[0], std::vector<NdArrayPtr>(nd.begin() + 1, nd.end()), g); break;
    case 4: c->comm->reduce_scatter(std::vector<NdArrayPtr>(nd.begin() + 1, nd.end()), nd[0], division != 0, g); break;
    case 5: c->comm->all_reduce_callback(nd, (size_t)root, division != 0, g, 1.0f, false)->on_finish_backward(); break;
    default: NBLA_ERROR(error_code::value, "unknown collective %d", op);
    }
    for (int i = 0; i < n; ++i) {
      const float *p = nd[i]->get(dtypes::FLOAT, c->cpu)->const_pointer<float>();
      std::memcpy(arrays[i], p, sizeof(float) * sizes[i]);
    }
  });
}

// The bucket plan of the packed all-reduce (no device needed): writes the bucket start indices
// and the end index to `starts` (capacity `cap`); returns how many were written, or -1.
int nbc_plan_buckets(const int64_t *sizes, int n, int64_t pack_size, int64_t *starts, int cap) {
  std::vector<size_t> s(sizes, sizes + n);
  const std::vector<size_t> plan = b200_plan_buckets(s, (size_t)pack_size);
  if ((int)plan.size() > cap)
    return -1;
  for (size_t i = 0; i < plan.size(); ++i)
    starts[i] = (int64_t)plan[i];
  return (int)plan.size();
}
}
