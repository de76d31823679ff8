// Backend, memory and array classes of the "b200" nnabla extension.
#include <nbla_b200/b200.hpp>

#include <nbla/array/cpu_array.hpp>
#include <nbla/array_registry.hpp>
#include <nbla/exception.hpp>
#include <nbla/memory/caching_allocator_with_buckets.hpp>
#include <nbla/memory/naive_allocator.hpp>
#include <nbla/singleton_manager-internal.hpp>
#include <nbla/synced_array.hpp>

#include <nnabla_b200.h>

#include <map>
#include <memory>
#include <mutex>
#include <string>
#include <unordered_map>

namespace nbla {

void nb200_check(int status, const char *what) {
  if (status == NB200_OK)
    return;
  const error_code code = status == NB200_EVALUE      ? error_code::value
                          : status == NB200_EMEMORY   ? error_code::memory
                          : status == NB200_ENOTIMPL  ? error_code::not_implemented
                                                      : error_code::target_specific;
  NBLA_ERROR(code, "%s: %s", what, nb200_last_error());
}

static size_t bytes_of(Size_t size, dtypes dtype) { return (size_t)size * sizeof_dtype(dtype); }

static int device_index(const string &device_id) { return device_id.empty() ? 0 : std::stoi(device_id); }

static void use_device(const string &device_id) {
  nb200_check(nb200_set_device(device_index(device_id)), "nb200_set_device");
}

void *b200_stream(const string &device_id) {
  static std::mutex m;
  static void *streams[64];
  const int dev = device_index(device_id);
  NBLA_CHECK(dev >= 0 && dev < 64, error_code::value, "device index %d out of range", dev);
  nb200_check(nb200_set_device(dev), "nb200_set_device");
  std::lock_guard<std::mutex> lock(m);
  if (streams[dev] == nullptr)
    nb200_check(nb200_stream_create(&streams[dev]), "nb200_stream_create");
  return streams[dev];
}

namespace {
std::mutex g_counter_mutex;
std::map<string, long long> g_counters;
} // namespace
long long b200_counter(const string &name) {
  std::lock_guard<std::mutex> lock(g_counter_mutex);
  auto it = g_counters.find(name);
  return it == g_counters.end() ? 0 : it->second;
}
void b200_count(const char *name) {
  std::lock_guard<std::mutex> lock(g_counter_mutex);
  ++g_counters[name];
}
void b200_reset_counters() {
  std::lock_guard<std::mutex> lock(g_counter_mutex);
  g_counters.clear();
}

// ---- write generations through nnabla's SyncedArrayCallback hook -------------
namespace {
std::mutex g_gen_mutex;
std::unordered_map<const SyncedArray *, unsigned long long> g_generation;
unsigned long long g_serial = 0;

void on_synced_array_event(SyncedArrayPtr sa, const SyncedArrayCallbackTag tag, const dtypes, const Context &,
                           const bool, const bool, const bool) {
  if (tag == SyncedArrayCallbackTag::GET)
    return; // a read leaves the contents as they are
  std::lock_guard<std::mutex> lock(g_gen_mutex);
  if (tag == SyncedArrayCallbackTag::CLEAR) {
    g_generation.erase(sa.get()); // contents gone; a stamp of them can never match again
    return;
  }
  if (g_generation.size() > (1u << 20))
    g_generation.clear(); // arrays that died without a clear(); every stamp goes stale once
  g_generation[sa.get()] = ++g_serial;
}
} // namespace

void install_write_tracking() {
  SingletonManager::get<SyncedArrayCallback>()->set_callback_func(on_synced_array_event);
}

bool write_tracking_alive() {
  // A cast of a private one-element host array must move its generation: if it does not, another
  // component has replaced the hook.
  static SyncedArrayPtr probe = std::make_shared<SyncedArray>(1);
  static std::mutex m;
  std::lock_guard<std::mutex> lock(m);
  unsigned long long before = 0, after = 0;
  {
    std::lock_guard<std::mutex> l2(g_gen_mutex);
    auto it = g_generation.find(probe.get());
    before = it == g_generation.end() ? 0 : it->second;
  }
  probe->cast(dtypes::FLOAT, Context({"cpu:float"}, "CpuArray", ""), true);
  {
    std::lock_guard<std::mutex> l2(g_gen_mutex);
    auto it = g_generation.find(probe.get());
    after = it == g_generation.end() ? 0 : it->second;
  }
  return after != 0 && after != before;
}

DataStamp data_stamp(const Variable *v) {
  SyncedArrayPtr a = const_cast<Variable *>(v)->data()->array();
  DataStamp s;
  s.array = a.get();
  s.count = a->modification_count();
  {
    std::lock_guard<std::mutex> lock(g_gen_mutex);
    auto it = g_generation.find(a.get());
    s.generation = it == g_generation.end() ? 0 : it->second;
  }
  s.valid = s.generation != 0 && write_tracking_alive();
  return s;
}

Context b200_context(const string &device_id, const string &type_config) {
  // "half": the backend list an nnabla extension gives for that type config. No function is registered under
  // "b200:half", so the registry's query (function_registry.hpp:57-72) goes on to "b200:float": the half
  // configuration runs the float implementations (fp32 arrays) rather than failing.
  if (type_config == "half")
    return Context({"b200:half", "b200:float"}, "B200CachedArray", device_id);
  NBLA_CHECK(type_config == "float", error_code::value, "Unknown data type config is given %s", type_config.c_str());
  return Context({"b200:float"}, "B200CachedArray", device_id);
}

// ---------------------------------------------------------------- B200Memory
B200Memory::B200Memory(size_t bytes, const string &device_id) : Memory(bytes, device_id) {}
B200Memory::B200Memory(size_t bytes, const string &device_id, void *ptr) : Memory(bytes, device_id) { ptr_ = ptr; }

B200Memory::~B200Memory() {
  if (!ptr_)
    return;
  NBLA_FORCE_ASSERT(!prev(), "freeing a device block that was split off another block");
  nb200_set_device(device_index(this->device_id()));
  nb200_free(ptr_);
}

bool B200Memory::alloc_impl() {
  if (nb200_set_device(device_index(this->device_id())) != NB200_OK)
    return false;
  void *p = nullptr;
  if (nb200_malloc(&p, this->bytes()) != NB200_OK)
    return false; // the allocator retries after freeing its caches
  ptr_ = p;
  return true;
}

shared_ptr<Memory> B200Memory::divide_impl(size_t second_start) {
  // The right part starts second_start bytes into this block; this object keeps the left part.
  void *right = static_cast<void *>(static_cast<uint8_t *>(ptr_) + second_start);
  return shared_ptr<Memory>(new B200Memory(this->bytes() - second_start, this->device_id(), right));
}

void B200Memory::merge_next_impl(Memory *from) {} // this block already starts the merged range
void B200Memory::merge_prev_impl(Memory *from) { ptr_ = from->pointer(); }

// ---------------------------------------------------------------------- B200
B200::B200() {
  naive_allocator_ = std::make_shared<NaiveAllocator<B200Memory>>();
  caching_allocator_ = std::make_shared<CachingAllocatorWithBuckets<B200Memory>>();
}
B200::~B200() {}
vector<string> B200::array_classes() const { return array_classes_; }
void B200::_set_array_classes(const vector<string> &a) { array_classes_ = a; }
void B200::register_array_class(const string &name) { array_classes_.push_back(name); }
shared_ptr<Allocator> B200::caching_allocator() { return caching_allocator_; }
shared_ptr<Allocator> B200::naive_allocator() { return naive_allocator_; }
void B200::free_unused_host_caches() {}
void B200::device_synchronize(const string &device) {
  use_device(device);
  nb200_check(nb200_device_synchronize(), "nb200_device_synchronize");
}
void B200::default_stream_synchronize(const string &device) {
  nb200_check(nb200_stream_synchronize(b200_stream(device)), "nb200_stream_synchronize");
}
void B200::create_lms_streams(int device) {}

NBLA_INSTANTIATE_SINGLETON(, B200);

// ----------------------------------------------------------------- B200Array
B200Array::B200Array(const Size_t size, dtypes dtype, const Context &ctx, const AllocatorMemoryPtr mem,
                     const Size_t offset)
    : Array(size, dtype, ctx,
            mem ? mem
                : SingletonManager::get<B200>()->naive_allocator()->alloc(Array::size_as_bytes(size, dtype),
                                                                          ctx.device_id),
            offset) {}
B200Array::~B200Array() {}

Context B200Array::filter_context(const Context &ctx) { return Context({}, "B200Array", ctx.device_id); }

void B200Array::zero() {
  void *st = b200_stream(this->ctx_.device_id);
  nb200_check(nb200_memset_zero(this->pointer<void>(), Array::size_as_bytes(this->size_, this->dtype_), st),
              "nb200_memset_zero");
}

void B200Array::fill(float value) {
  void *st = b200_stream(this->ctx_.device_id);
  if (this->dtype_ == dtypes::FLOAT) {
    nb200_check(nb200_fill_f32(this->pointer<float>(), this->size_, value, st), "nb200_fill_f32");
    return;
  }
  // Other element types: fill on the host with the reference's own typed fill, then upload.
  CpuArray host(this->size_, this->dtype_, Context({"cpu:float"}, "CpuArray", ""));
  host.fill(value);
  nb200_check(nb200_memcpy_h2d(this->pointer<void>(), host.const_pointer<void>(),
                               Array::size_as_bytes(this->size_, this->dtype_), st),
              "nb200_memcpy_h2d");
  nb200_check(nb200_stream_synchronize(st), "nb200_stream_synchronize"); // `host` goes away on return
}

void B200Array::copy_from(const Array *src) {
  NBLA_CHECK(src->size() == this->size_, error_code::unclassified, "Size mismatch.");
  void *st = b200_stream(this->ctx_.device_id);
  if (src->dtype() == this->dtype_) {
    nb200_check(nb200_memcpy_d2d(this->pointer<void>(), src->const_pointer<void>(),
                                 Array::size_as_bytes(this->size_, this->dtype_), st),
                "nb200_memcpy_d2d");
    return;
  }
  // A copy that changes the element type (the reference's arrays convert through the 15 x 15
  // switch of include/nbla/array.hpp): down to the host, the reference's own typed copy, up again.
  const Context cpu({"cpu:float"}, "CpuArray", "");
  CpuArray from(src->size(), src->dtype(), cpu), to(this->size_, this->dtype_, cpu);
  nb200_check(nb200_memcpy_d2h(from.pointer<void>(), src->const_pointer<void>(),
                               Array::size_as_bytes(src->size(), src->dtype()), st),
              "nb200_memcpy_d2h");
  nb200_check(nb200_stream_synchronize(st), "nb200_stream_synchronize");
  to.copy_from(&from);
  nb200_check(nb200_memcpy_h2d(this->pointer<void>(), to.const_pointer<void>(),
                               Array::size_as_bytes(this->size_, this->dtype_), st),
              "nb200_memcpy_h2d");
  nb200_check(nb200_stream_synchronize(st), "nb200_stream_synchronize");
}

B200CachedArray::B200CachedArray(const Size_t size, dtypes dtype, const Context &ctx, const AllocatorMemoryPtr mem,
                                 const Size_t offset)
    : B200Array(size, dtype, ctx,
                mem ? mem
                    : SingletonManager::get<B200>()->caching_allocator()->alloc(Array::size_as_bytes(size, dtype),
                                                                                ctx.device_id),
                offset) {}
B200CachedArray::~B200CachedArray() {}
Context B200CachedArray::filter_context(const Context &ctx) { return Context({}, "B200CachedArray", ctx.device_id); }

// ------------------------------------------------------------ synchronizers
// SyncedArray::sync copies head -> requested array in one call and the two may
// differ in dtype (src/nbla/synced_array.cpp:372-381): conversions run on the
// host with the reference's own typed copy, transfers are raw byte copies.
void synchronizer_cpu_to_b200(Array *src, Array *dst, const int async_flags) {
  const Array *host = src;
  std::unique_ptr<CpuArray> converted;
  if (src->dtype() != dst->dtype()) {
    converted.reset(new CpuArray(src->size(), dst->dtype(), Context({"cpu:float"}, "CpuArray", "")));
    converted->copy_from(src);
    host = converted.get();
  }
  void *st = b200_stream(dst->context().device_id);
  nb200_check(nb200_memcpy_h2d(dst->pointer<void>(), host->const_pointer<void>(),
                               bytes_of(dst->size(), dst->dtype()), st),
              "nb200_memcpy_h2d");
  // AsyncFlag::ASYNC (include/nbla/common.hpp:45): the caller orders later work itself and keeps the
  // source alive. A converted staging copy lives only until return, so that case always waits.
  if (!(async_flags & AsyncFlag::ASYNC) || converted)
    nb200_check(nb200_stream_synchronize(st), "nb200_stream_synchronize");
}

void synchronizer_b200_to_cpu(Array *src, Array *dst, const int async_flags) {
  void *st = b200_stream(src->context().device_id);
  if (src->dtype() == dst->dtype()) {
    nb200_check(nb200_memcpy_d2h(dst->pointer<void>(), src->const_pointer<void>(),
                                 bytes_of(src->size(), src->dtype()), st),
                "nb200_memcpy_d2h");
    if (!(async_flags & AsyncFlag::ASYNC))
      nb200_check(nb200_stream_synchronize(st), "nb200_stream_synchronize");
    return;
  }
  CpuArray staged(src->size(), src->dtype(), Context({"cpu:float"}, "CpuArray", ""));
  nb200_check(nb200_memcpy_d2h(staged.pointer<void>(), src->const_pointer<void>(),
                               bytes_of(src->size(), src->dtype()), st),
              "nb200_memcpy_d2h");
  nb200_check(nb200_stream_synchronize(st), "nb200_stream_synchronize");
  dst->copy_from(&staged);
}

// -------------------------------------------------------------- fixed-point tags
namespace {
struct FxpTag {
  DataStamp stamp;
  float delta;
  NdArrayPtr codes;
};
std::mutex g_tag_mutex;
std::unordered_map<const SyncedArray *, FxpTag> g_tags;
} // namespace

void fxp_tag_set(const Variable *v, float delta, const NdArrayPtr &codes) {
  const DataStamp s = data_stamp(v);
  std::lock_guard<std::mutex> lock(g_tag_mutex);
  if (g_tags.size() > 4096)
    g_tags.clear(); // tags of arrays long gone; the live ones are set again by their next forward
  if (s.valid)
    g_tags[s.array] = FxpTag{s, delta, codes};
  else
    g_tags.erase(s.array);
}

void fxp_tag_set(const Variable *v, float delta) { fxp_tag_set(v, delta, nullptr); }

NdArrayPtr fxp_tag_codes(const Variable *v) {
  const DataStamp s = data_stamp(v);
  std::lock_guard<std::mutex> lock(g_tag_mutex);
  auto it = g_tags.find(s.array);
  if (it == g_tags.end() || it->second.stamp != s)
    return nullptr;
  return it->second.codes;
}

float fxp_tag_get(const Variable *v) {
  const DataStamp s = data_stamp(v);
  std::lock_guard<std::mutex> lock(g_tag_mutex);
  auto it = g_tags.find(s.array);
  if (it == g_tags.end())
    return 0.0f;
  if (it->second.stamp != s) {
    g_tags.erase(it);
    return 0.0f;
  }
  return it->second.delta;
}

} // namespace nbla

// ---- C entry points for the extension's Python package -------------------------
// (ext/python/nnabla_ext/b200/__init__.py loads this library with ctypes)
extern "C" {
static thread_local std::string g_ext_error;
const char *nnabla_ext_b200_last_error() { return g_ext_error.c_str(); }
int nnabla_ext_b200_init() {
  try {
    nbla::init_b200();
    return 0;
  } catch (const std::exception &e) {
    g_ext_error = e.what();
    return 1;
  }
}
// clear_memory_cache() of an extension package (python/src/nnabla_ext/cpu/__init__.py:17-45):
// returns the caching allocator's unused blocks to the device.
int nnabla_ext_b200_clear_memory_cache() {
  try {
    nbla::SingletonManager::get<nbla::B200>()->caching_allocator()->free_unused_caches();
    return 0;
  } catch (const std::exception &e) {
    g_ext_error = e.what();
    return 1;
  }
}
int nnabla_ext_b200_device_synchronize(int device) {
  try {
    nbla::SingletonManager::get<nbla::B200>()->device_synchronize(std::to_string(device));
    return 0;
  } catch (const std::exception &e) {
    g_ext_error = e.what();
    return 1;
  }
}
}
