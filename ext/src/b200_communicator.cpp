// MultiProcessDataParallelCommunicator for the "b200" backend: nnabla's
// Communicator interface (include/nbla/communicator.hpp:39-293,
// include/nbla/communicator/multi_process_data_parallel_communicator.hpp) over
// NCCL, one process per GPU.
//
// The core only declares the interface (the CPU class raises "not
// implemented", src/nbla/communicator/multi_process_data_parallel_communicator.cpp);
// a backend supplies the collectives. nnabla's CUDA extension bootstraps through
// MPI; there is no MPI here, so ranks come from the environment a launcher sets
// (RANK / WORLD_SIZE / LOCAL_RANK as torchrun does, or OMPI_COMM_WORLD_*), and
// the NCCL unique id of a group travels through a file that its first rank
// writes and the others poll with a deadline (NNABLA_B200_COMM_DIR, default
// /tmp; the name carries MASTER_PORT so that concurrent jobs do not meet).
// NCCL itself is loaded at run time (dlopen), so the extension still loads on
// a machine without it.
//
// Collectives run on the backend's stream of the device, in stream order with
// the functions that produce and consume the arrays. Lists are either reduced
// array by array (inplace) or packed into one buffer, reduced once and
// unpacked, as the interface's `inplace` flag asks.
#include <nbla_b200/b200.hpp>

#include <nbla/communicator/multi_process_data_parallel_communicator.hpp>
#include <nbla/computation_graph/variable.hpp>
#include <nbla/exception.hpp>
#include <nbla/nd_array.hpp>
#include <nbla/singleton_manager.hpp>

#include <nnabla_b200.h>

#include <dlfcn.h>
#include <unistd.h>

#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <numeric>
#include <thread>

namespace nbla {

namespace {

// ---- the part of NCCL's C API that is used (types as in nccl.h) ----------------
typedef struct ncclComm *ncclComm_t;
typedef struct {
  char internal[128];
} ncclUniqueId;
enum { ncclSuccess = 0 };
enum { ncclFloat32 = 7 };
enum { ncclSum = 0 };

struct Nccl {
  int (*GetUniqueId)(ncclUniqueId *);
  int (*CommInitRank)(ncclComm_t *, int, ncclUniqueId, int);
  int (*CommDestroy)(ncclComm_t);
  int (*AllReduce)(const void *, void *, size_t, int, int, ncclComm_t, void *);
  int (*Reduce)(const void *, void *, size_t, int, int, int, ncclComm_t, void *);
  int (*Broadcast)(const void *, void *, size_t, int, int, ncclComm_t, void *);
  int (*AllGather)(const void *, void *, size_t, int, ncclComm_t, void *);
  int (*ReduceScatter)(const void *, void *, size_t, int, int, ncclComm_t, void *);
  const char *(*GetErrorString)(int);
};

const Nccl &nccl() {
  static Nccl api;
  static bool loaded = false;
  static std::mutex m;
  std::lock_guard<std::mutex> lock(m);
  if (loaded)
    return api;
  void *h = nullptr;
  for (const char *name : {"libnccl.so.2", "libnccl.so"}) {
    h = dlopen(name, RTLD_NOW | RTLD_GLOBAL);
    if (h)
      break;
  }
  NBLA_CHECK(h != nullptr, error_code::target_specific, "NCCL (libnccl.so.2) could not be loaded: %s", dlerror());
  auto sym = [&](const char *n) {
    void *p = dlsym(h, n);
    NBLA_CHECK(p != nullptr, error_code::target_specific, "NCCL symbol %s is missing", n);
    return p;
  };
  api.GetUniqueId = reinterpret_cast<decltype(api.GetUniqueId)>(sym("ncclGetUniqueId"));
  api.CommInitRank = reinterpret_cast<decltype(api.CommInitRank)>(sym("ncclCommInitRank"));
  api.CommDestroy = reinterpret_cast<decltype(api.CommDestroy)>(sym("ncclCommDestroy"));
  api.AllReduce = reinterpret_cast<decltype(api.AllReduce)>(sym("ncclAllReduce"));
  api.Reduce = reinterpret_cast<decltype(api.Reduce)>(sym("ncclReduce"));
  api.Broadcast = reinterpret_cast<decltype(api.Broadcast)>(sym("ncclBroadcast"));
  api.AllGather = reinterpret_cast<decltype(api.AllGather)>(sym("ncclAllGather"));
  api.ReduceScatter = reinterpret_cast<decltype(api.ReduceScatter)>(sym("ncclReduceScatter"));
  api.GetErrorString = reinterpret_cast<decltype(api.GetErrorString)>(sym("ncclGetErrorString"));
  loaded = true;
  return api;
}

void nccl_check(int rc, const char *what) {
  if (rc != ncclSuccess)
    NBLA_ERROR(error_code::target_specific, "%s: %s", what, nccl().GetErrorString(rc));
}

int env_int(std::initializer_list<const char *> names, int fallback) {
  for (const char *n : names) {
    const char *v = std::getenv(n);
    if (v && *v)
      return std::atoi(v);
  }
  return fallback;
}

// The id of a group goes through a file: written whole under a temporary name
// and renamed, so a reader never sees half of it.
string id_path(const string &group) {
  const char *dir = std::getenv("NNABLA_B200_COMM_DIR");
  const char *port = std::getenv("MASTER_PORT");
  const char *job = std::getenv("NNABLA_B200_COMM_JOB");
  return string(dir && *dir ? dir : "/tmp") + "/nnabla_b200_nccl_" + (job ? job : (port ? port : "0")) + "_" + group;
}

void publish_id(const string &path, const ncclUniqueId &id) {
  const string tmp = path + ".tmp" + std::to_string((long)getpid());
  {
    std::ofstream f(tmp, std::ios::binary | std::ios::trunc);
    f.write(id.internal, sizeof(id.internal));
    NBLA_CHECK(f.good(), error_code::io, "cannot write %s", tmp.c_str());
  }
  NBLA_CHECK(std::rename(tmp.c_str(), path.c_str()) == 0, error_code::io, "cannot publish %s", path.c_str());
}

ncclUniqueId fetch_id(const string &path, double timeout_s) {
  const auto t0 = std::chrono::steady_clock::now();
  for (;;) {
    std::ifstream f(path, std::ios::binary);
    ncclUniqueId id;
    if (f.read(id.internal, sizeof(id.internal)) && f.gcount() == (std::streamsize)sizeof(id.internal))
      return id;
    const double waited = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
    NBLA_CHECK(waited < timeout_s, error_code::runtime,
               "the first rank of the group did not publish %s within %.0f s", path.c_str(), timeout_s);
    std::this_thread::sleep_for(std::chrono::milliseconds(20));
  }
}

} // namespace

/** Splits `sizes` (elements per array, in order) into consecutive buckets of at most `pack_size`
    elements; an array larger than pack_size gets a bucket of its own. Returns the index of the
    first array of every bucket plus the end index. What all_reduce_callback packs by. */
vector<size_t> b200_plan_buckets(const vector<size_t> &sizes, size_t pack_size) {
  vector<size_t> starts{0};
  size_t used = 0;
  for (size_t i = 0; i < sizes.size(); ++i) {
    if (used > 0 && used + sizes[i] > pack_size) {
      starts.push_back(i);
      used = 0;
    }
    used += sizes[i];
  }
  starts.push_back(sizes.size());
  return starts;
}

template <typename T> class MultiProcessDataParallelCommunicatorB200 : public MultiProcessDataParallelCommunicator<T> {
  std::unordered_map<string, ncclComm_t> comms_;
  int group_serial_ = 0;
  double timeout_s_ = 60.0;

  void *stream() { return b200_stream(this->ctx_.device_id); }

  ncclComm_t comm_of(const string &group) {
    auto it = comms_.find(group);
    NBLA_CHECK(it != comms_.end(), error_code::value, "group %s does not exist or this rank is not a member",
               group.c_str());
    return it->second;
  }
  int group_size(const string &group) { return (int)this->groups_[group].size(); }
  int group_rank(const string &group, int world_rank) {
    const vector<int> &r = this->groups_[group];
    auto it = std::find(r.begin(), r.end(), world_rank);
    NBLA_CHECK(it != r.end(), error_code::value, "rank %d is not in group %s", world_rank, group.c_str());
    return (int)(it - r.begin());
  }

  void make_comm(const string &group, const vector<int> &ranks) {
    const string path = id_path(group + "_" + std::to_string(group_serial_++));
    ncclUniqueId id;
    if (this->rank_ == ranks.front()) {
      nccl_check(nccl().GetUniqueId(&id), "ncclGetUniqueId");
      publish_id(path, id);
    } else {
      id = fetch_id(path, timeout_s_);
    }
    b200_stream(this->ctx_.device_id); // makes the device current
    ncclComm_t c = nullptr;
    const int me = (int)(std::find(ranks.begin(), ranks.end(), this->rank_) - ranks.begin());
    nccl_check(nccl().CommInitRank(&c, (int)ranks.size(), id, me), "ncclCommInitRank");
    comms_[group] = c;
  }

  float *dev(const NdArrayPtr &a, bool write_only = false) {
    return a->cast(get_dtype<T>(), this->ctx_, write_only)->template pointer<float>();
  }

  // Packs the arrays into one buffer (device-to-device copies in stream order).
  NdArrayPtr pack(const vector<NdArrayPtr> &list, size_t first, size_t last) {
    Size_t total = 0;
    for (size_t i = first; i < last; ++i)
      total += list[i]->size();
    NdArrayPtr big = make_shared<NdArray>(Shape_t{total});
    float *p = dev(big, true);
    for (size_t i = first; i < last; ++i) {
      nb200_check(nb200_memcpy_d2d(p, dev(list[i]), list[i]->size() * sizeof(float), stream()), "pack");
      p += list[i]->size();
    }
    return big;
  }
  void unpack(const NdArrayPtr &big, const vector<NdArrayPtr> &list, size_t first, size_t last) {
    const float *p = dev(big);
    for (size_t i = first; i < last; ++i) {
      nb200_check(nb200_memcpy_d2d(dev(list[i]), p, list[i]->size() * sizeof(float), stream()), "unpack");
      p += list[i]->size();
    }
  }
  void divide(float *p, size_t n, const string &group) {
    nb200_check(nb200_scale_f32(p, n, 1.0f / (float)group_size(group), stream()), "division");
  }

public:
  explicit MultiProcessDataParallelCommunicatorB200(const Context &ctx)
      : MultiProcessDataParallelCommunicator<T>(ctx) {}
  virtual ~MultiProcessDataParallelCommunicatorB200() {
    for (auto &kv : comms_)
      if (kv.second)
        nccl().CommDestroy(kv.second);
  }
  virtual string name() { return "MultiProcessDataParallelCommunicatorB200"; }
  vector<string> allowed_array_classes() { return SingletonManager::get<B200>()->array_classes(); }

  virtual void init() {
    NBLA_CHECK(!this->initialized_, error_code::value, "Communicator was already initialized.");
    this->rank_ = env_int({"RANK", "OMPI_COMM_WORLD_RANK", "PMI_RANK"}, 0);
    this->size_ = env_int({"WORLD_SIZE", "OMPI_COMM_WORLD_SIZE", "PMI_SIZE"}, 1);
    this->local_rank_ = env_int({"LOCAL_RANK", "OMPI_COMM_WORLD_LOCAL_RANK"}, this->rank_);
    timeout_s_ = env_int({"NNABLA_B200_COMM_TIMEOUT"}, 60);
    NBLA_CHECK(this->rank_ >= 0 && this->rank_ < this->size_, error_code::value, "rank %d of %d", this->rank_,
               this->size_);
    vector<int> all(this->size_);
    std::iota(all.begin(), all.end(), 0);
    this->groups_["world"] = all;
    make_comm("world", all);
    this->initialized_ = true;
  }

  virtual void barrier() {
    // a one-element all-reduce, then the host waits for the stream
    NdArrayPtr one = make_shared<NdArray>(Shape_t{1});
    float *p = dev(one, true);
    nb200_check(nb200_fill_f32(p, 1, 0.f, stream()), "barrier");
    nccl_check(nccl().AllReduce(p, p, 1, ncclFloat32, ncclSum, comm_of("world"), stream()), "ncclAllReduce");
    nb200_check(nb200_stream_synchronize(stream()), "barrier");
  }

  virtual string new_group(pair<string, vector<int>> name_ranks_pair) {
    const string &group = name_ranks_pair.first;
    vector<int> ranks = name_ranks_pair.second;
    NBLA_CHECK(this->groups_.find(group) == this->groups_.end(), error_code::value, "group %s already exists",
               group.c_str());
    NBLA_CHECK(!ranks.empty(), error_code::value, "a group needs at least one rank");
    std::sort(ranks.begin(), ranks.end());
    for (int r : ranks)
      NBLA_CHECK(r >= 0 && r < this->size_, error_code::value, "rank %d is outside the world of %d", r, this->size_);
    this->groups_[group] = ranks;
    if (std::find(ranks.begin(), ranks.end(), this->rank_) != ranks.end())
      make_comm(group, ranks);
    else
      ++group_serial_; // every rank counts groups alike, so that the file names agree
    return group;
  }

  virtual void all_reduce(const vector<NdArrayPtr> &list, bool division, bool inplace, const string &group) {
    if (!this->find_self(group))
      return;
    if (inplace) {
      for (const NdArrayPtr &a : list)
        all_reduce(a, division, true, group);
      return;
    }
    NdArrayPtr big = pack(list, 0, list.size());
    all_reduce(big, division, true, group);
    unpack(big, list, 0, list.size());
  }
  virtual void all_reduce(NdArrayPtr a, bool division, bool inplace, const string &group) {
    if (!this->find_self(group))
      return;
    float *p = dev(a);
    nccl_check(nccl().AllReduce(p, p, a->size(), ncclFloat32, ncclSum, comm_of(group), stream()), "ncclAllReduce");
    if (division)
      divide(p, a->size(), group);
  }

  virtual void reduce(const vector<NdArrayPtr> &list, int dst, bool division, bool inplace, const string &group) {
    if (!this->find_self(group))
      return;
    if (inplace) {
      for (const NdArrayPtr &a : list)
        reduce(a, dst, division, true, group);
      return;
    }
    NdArrayPtr big = pack(list, 0, list.size());
    reduce(big, dst, division, true, group);
    if (this->rank_ == dst)
      unpack(big, list, 0, list.size());
  }
  virtual void reduce(NdArrayPtr a, int dst, bool division, bool inplace, const string &group) {
    if (!this->find_self(group))
      return;
    float *p = dev(a);
    nccl_check(nccl().Reduce(p, p, a->size(), ncclFloat32, ncclSum, group_rank(group, dst), comm_of(group), stream()),
               "ncclReduce");
    if (division && this->rank_ == dst)
      divide(p, a->size(), group);
  }

  virtual void bcast(const vector<NdArrayPtr> &list, int src, bool inplace, const string &group) {
    if (!this->find_self(group))
      return;
    if (inplace) {
      for (const NdArrayPtr &a : list)
        bcast(a, src, true, group);
      return;
    }
    NdArrayPtr big = pack(list, 0, list.size());
    bcast(big, src, true, group);
    unpack(big, list, 0, list.size());
  }
  virtual void bcast(NdArrayPtr a, int src, bool inplace, const string &group) {
    if (!this->find_self(group))
      return;
    float *p = dev(a);
    nccl_check(nccl().Broadcast(p, p, a->size(), ncclFloat32, group_rank(group, src), comm_of(group), stream()),
               "ncclBroadcast");
  }

  virtual void all_gather(NdArrayPtr a, const vector<NdArrayPtr> &list, const string &group) {
    if (!this->find_self(group))
      return;
    const int n = group_size(group);
    NBLA_CHECK((int)list.size() == n, error_code::value, "all_gather needs one receiving array per rank of the group");
    NdArrayPtr big = make_shared<NdArray>(Shape_t{a->size() * n});
    nccl_check(nccl().AllGather(dev(a), dev(big, true), a->size(), ncclFloat32, comm_of(group), stream()),
               "ncclAllGather");
    for (const NdArrayPtr &r : list)
      NBLA_CHECK(r->size() == a->size(), error_code::value, "receiving arrays must have the size of the sent one");
    unpack(big, list, 0, list.size());
  }

  virtual void reduce_scatter(const vector<NdArrayPtr> &list, NdArrayPtr a, bool division, const string &group) {
    if (!this->find_self(group))
      return;
    NBLA_CHECK((int)list.size() == group_size(group), error_code::value,
               "reduce_scatter needs one array per rank of the group");
    for (const NdArrayPtr &r : list)
      NBLA_CHECK(r->size() == a->size(), error_code::value, "the arrays must have the size of the receiving one");
    NdArrayPtr big = pack(list, 0, list.size());
    float *out = dev(a, true);
    nccl_check(nccl().ReduceScatter(dev(big), out, a->size(), ncclFloat32, ncclSum, comm_of(group), stream()),
               "ncclReduceScatter");
    if (division)
      divide(out, a->size(), group);
  }

  // allreduce() over the parameters registered with add_context_and_parameters: their gradients.
  virtual void allreduce(bool division, bool inplace) {
    vector<NdArrayPtr> grads;
    for (auto &per_device : this->device_func_named_param_)
      for (auto &kv : per_device)
        grads.push_back(kv.second->grad());
    all_reduce(grads, division, inplace, "world");
  }

  // Gradients all-reduced in buckets of at most pack_size values when the backward pass ends.
  struct Callback : public CommunicatorBackwardCallback {
    MultiProcessDataParallelCommunicatorB200 *self;
    vector<NdArrayPtr> list;
    size_t pack_size;
    bool division;
    string group;
    float scale_grad;
    virtual void on_finish_backward() {
      vector<size_t> sizes;
      for (const NdArrayPtr &a : list)
        sizes.push_back((size_t)a->size());
      const vector<size_t> starts = b200_plan_buckets(sizes, pack_size);
      for (size_t b = 0; b + 1 < starts.size(); ++b) {
        NdArrayPtr big = self->pack(list, starts[b], starts[b + 1]);
        float *p = self->dev(big);
        if (scale_grad != 1.0f)
          nb200_check(nb200_scale_f32(p, big->size(), scale_grad, self->stream()), "scale_grad");
        self->all_reduce(big, division, true, group);
        if (scale_grad != 1.0f)
          nb200_check(nb200_scale_f32(p, big->size(), 1.0f / scale_grad, self->stream()), "scale_grad");
        self->unpack(big, list, starts[b], starts[b + 1]);
      }
    }
  };
  virtual CommunicatorBackwardCallbackPtr all_reduce_callback(const vector<NdArrayPtr> &list, size_t pack_size,
                                                              bool division, const string &group, float scale_grad,
                                                              bool keep_dtype) {
    auto cb = make_shared<Callback>();
    cb->self = this;
    cb->list = list;
    cb->pack_size = pack_size;
    cb->division = division;
    cb->group = group;
    cb->scale_grad = scale_grad;
    return cb;
  }
  virtual CommunicatorBackwardCallbackPtr all_reduce_callback(NdArrayPtr a, size_t pack_size, bool division,
                                                              const string &group, float scale_grad, bool keep_dtype) {
    return all_reduce_callback(vector<NdArrayPtr>{a}, pack_size, division, group, scale_grad, keep_dtype);
  }
};

void register_b200_communicator() {
  typedef MultiProcessDataParallelCommunicatorB200<float> comm_b200_float;
  NBLA_REGISTER_COMMUNICATOR_IMPL(MultiProcessDataParallelCommunicator, comm_b200_float, "b200:float");
}

} // namespace nbla
